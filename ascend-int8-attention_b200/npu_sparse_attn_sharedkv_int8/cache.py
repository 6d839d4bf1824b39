"""Frozen-scale INT8 shared-KV cache writes on the caller's CUDA stream.

Counterpart of the reference's prepared writer (npu_sparse_attn_sharedkv_int8/cache.py:16-71):
`PreparedCacheWrite(cache, updates, slots, inverse_scale)`, `_rebind_same_geometry`, `run`, the
same attributes and the same error texts, over `launch_cache_write` of libsharedkv_cuda.so.
"""
import ctypes

import torch

from .runtime import Kernels, check, current_stream, native_launcher

ROW = 512                        # channels of a cache row = bytes of an INT8 row
_POINTERS = ("cache", "updates", "slots", "inverseScale")
_STRIDES = ("pageStride", "updateStride", "slotStride", "slotColumnStride")
_COUNTS = ("tokens", "pages", "pageSize", "int64Slots", "pairedSlots")


class _Args(ctypes.Structure):
    """CacheWriteArgs of the C ABI: eight 64-bit words, five 32-bit words, 88 bytes with padding
    (csrc/kernels/cache_write.h:4-8 of the reference)."""
    _fields_ = [(n, ctypes.c_uint64) for n in _POINTERS + _STRIDES] + [(n, ctypes.c_uint32) for n in _COUNTS]


def _advisory_blocks(rows):
    """`blocks` of the reference launcher (cache.py:42); the CUDA library sizes its own grid."""
    return min(48, -(-rows // 8))


def _require(ok, message):
    if not ok:
        raise ValueError(message)


def _check_cache(cache):
    shaped = cache.dtype == torch.int8 and cache.ndim == 4 and tuple(cache.shape[-2:]) == (1, ROW)
    _require(cache.device.type == "cuda" and shaped, "Expected INT8 CUDA cache[pages,page_size,1,512]")
    pages, page_size = cache.shape[:2]
    strided = cache.stride(1) == ROW and cache.stride(-1) == 1 and cache.stride(0) >= page_size * ROW
    _require(pages > 0 and page_size > 0 and strided, "Invalid cache strides or empty page storage")


def _check_updates(updates):
    shaped = updates.ndim in (2, 3) and updates.shape[-1] == ROW and (updates.ndim == 2 or updates.shape[1] == 1)
    rows_ok = shaped and updates.stride(-1) == 1 and (updates.shape[0] <= 1 or updates.stride(0) >= ROW)
    _require(updates.dtype == torch.bfloat16 and rows_ok, "Expected BF16 updates[T,512] or [T,1,512] with contiguous rows")


def _check_slots(slots, rows):
    shaped = slots.ndim == 1 or (slots.ndim == 2 and slots.shape[1] == 2)
    _require(slots.dtype in (torch.int32, torch.int64) and shaped and slots.shape[0] == rows,
             "Expected INT32/INT64 slots[T] or slots[T,2]")


class PreparedCacheWrite:
    """BF16 rows times a frozen inverse scale, rounded half-even, clamped to +-127 and scattered
    into INT8 pages.

    A slot is a flat physical row id (INT32 or INT64) or a [page, offset] pair.  Rows whose slot is
    negative or outside the cache are skipped; the valid slots of one call must be distinct.
    `run()` neither allocates nor reads anything back, and does not synchronise.
    """

    def __init__(self, cache, updates, slots, inverse_scale):
        _check_cache(cache)
        _check_updates(updates)
        _check_slots(slots, updates.shape[0])
        _require(inverse_scale.dtype == torch.float32 and tuple(inverse_scale.shape) == (ROW,) and inverse_scale.is_contiguous(),
                 "Expected frozen contiguous FP32 inverse_scale[512]")
        _require(all(t.device == cache.device for t in (updates, slots, inverse_scale)),
                 "Cache, updates, slots and scale must be on the same GPU")
        self.cache, self.updates, self.slots, self.inverse_scale = cache, updates, slots, inverse_scale
        paired = slots.ndim == 2
        self.args = _Args()
        self.args.inverseScale = inverse_scale.data_ptr()
        self.args.pageStride = cache.stride(0)
        self.args.updateStride = max(updates.stride(0), ROW)       # a single row may report any stride
        self.args.slotStride = slots.stride(0)
        self.args.slotColumnStride = slots.stride(1) if paired else 0
        self.args.pages, self.args.pageSize = cache.shape[0], cache.shape[1]
        self.args.int64Slots, self.args.pairedSlots = int(slots.dtype == torch.int64), int(paired)
        self._bind(cache, updates, slots)
        self.kernels = Kernels()
        self.launch = self.kernels.lib.launch_cache_write
        self.native = native_launcher()
        self.argument_address = ctypes.addressof(self.args)
        self.device_index = cache.device.index
        if self.kernels.lib.sharedkv_cache_args_size() != ctypes.sizeof(_Args):
            raise RuntimeError("Native library ABI changed; rebuild libsharedkv_cuda.so")

    def _bind(self, cache, updates, slots):
        for name, tensor in (("cache", cache), ("updates", updates), ("slots", slots)):
            setattr(self.args, name, tensor.data_ptr())
        self.args.tokens = updates.shape[0]
        self.blocks = _advisory_blocks(updates.shape[0])

    def _rebind_same_geometry(self, cache, updates, slots):
        """Serving fast path (cache.py:57-62): other pointers, possibly another row count, the same
        layouts; nothing is validated again."""
        self.cache, self.updates, self.slots = cache, updates, slots
        self._bind(cache, updates, slots)

    def run(self):
        if not self.blocks:
            return self.cache
        if self.native is not None:
            self.native.cache_write(self.argument_address, self.blocks, self.device_index)
        else:
            with torch.cuda.device(self.cache.device):
                status = self.launch(self.blocks, current_stream(self.device_index), ctypes.byref(self.args))
            check(status, "cache-write launch")
        return self.cache
