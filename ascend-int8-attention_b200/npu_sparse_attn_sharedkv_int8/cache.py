"""Frozen-scale INT8 shared-KV cache writes on the caller's CUDA stream.

Mirror of the reference's prepared writer (npu_sparse_attn_sharedkv_int8/cache.py:16-71):
same constructor arguments, validation messages, attributes and rebind/run protocol.
The kernel is `launch_cache_write` of libsharedkv_cuda.so.
"""
import ctypes

import torch

from .runtime import Kernels, check, current_stream, native_launcher


class _Args(ctypes.Structure):
    """CacheWriteArgs, 88 bytes (csrc/kernels/cache_write.h:4-8 of the reference)."""
    _fields_ = [(name, ctypes.c_uint64) for name in (
        "cache updates slots inverseScale pageStride updateStride slotStride slotColumnStride").split()] + [
        (name, ctypes.c_uint32) for name in "tokens pages pageSize int64Slots pairedSlots".split()]


def _blocks(rows):
    # advisory only: the library sizes its own grid; kept because callers read `.blocks`
    return min(48, (rows + 7) // 8)


class PreparedCacheWrite:
    """Quantize BF16 rows with a frozen inverse scale and scatter them into INT8 pages.

    Negative or out-of-range destinations are skipped; valid slots of one call must be
    unique.  Slots are INT32/INT64 flat physical ids or [page, offset] pairs.  run()
    performs no host read, no allocation and no synchronisation.
    """

    def __init__(self, cache, updates, slots, inverse_scale):
        device = cache.device
        if device.type != "cuda" or cache.dtype != torch.int8 or cache.ndim != 4 or cache.shape[-2:] != (1, 512):
            raise ValueError("Expected INT8 CUDA cache[pages,page_size,1,512]")
        if (not cache.shape[0] or not cache.shape[1] or cache.stride(1) != 512 or cache.stride(-1) != 1
                or cache.stride(0) < cache.shape[1] * 512):
            raise ValueError("Invalid cache strides or empty page storage")
        if (updates.dtype != torch.bfloat16 or updates.ndim not in (2, 3) or updates.shape[-1] != 512
                or (updates.ndim == 3 and updates.shape[1] != 1) or updates.stride(-1) != 1
                or (updates.shape[0] > 1 and updates.stride(0) < 512)):
            raise ValueError("Expected BF16 updates[T,512] or [T,1,512] with contiguous rows")
        if (slots.dtype not in (torch.int32, torch.int64) or slots.ndim not in (1, 2)
                or (slots.ndim == 2 and slots.shape[1] != 2) or slots.shape[0] != updates.shape[0]):
            raise ValueError("Expected INT32/INT64 slots[T] or slots[T,2]")
        if inverse_scale.dtype != torch.float32 or inverse_scale.shape != (512,) or not inverse_scale.is_contiguous():
            raise ValueError("Expected frozen contiguous FP32 inverse_scale[512]")
        if any(t.device != device for t in (updates, slots, inverse_scale)):
            raise ValueError("Cache, updates, slots and scale must be on the same GPU")
        self.cache, self.updates, self.slots, self.inverse_scale = cache, updates, slots, inverse_scale
        self.blocks = _blocks(updates.shape[0])
        self.args = _Args(cache.data_ptr(), updates.data_ptr(), slots.data_ptr(), inverse_scale.data_ptr(),
                          cache.stride(0), max(updates.stride(0), 512), slots.stride(0),
                          slots.stride(1) if slots.ndim == 2 else 0,
                          updates.shape[0], cache.shape[0], cache.shape[1], slots.dtype == torch.int64, slots.ndim == 2)
        self.kernels = Kernels()
        self.launch = self.kernels.lib.launch_cache_write
        self.native = native_launcher()
        self.argument_address = ctypes.addressof(self.args)
        self.device_index = device.index
        if self.kernels.lib.sharedkv_cache_args_size() != ctypes.sizeof(_Args):
            raise RuntimeError("Native library ABI changed; rebuild libsharedkv_cuda.so")

    def _rebind_same_geometry(self, cache, updates, slots):
        """Serving fast path: new pointers and row count, same row layout."""
        self.cache, self.updates, self.slots = cache, updates, slots
        self.args.cache, self.args.updates, self.args.slots = cache.data_ptr(), updates.data_ptr(), slots.data_ptr()
        self.args.tokens = updates.shape[0]
        self.blocks = _blocks(updates.shape[0])

    def run(self):
        if self.blocks:
            if self.native is not None:
                self.native.cache_write(self.argument_address, self.blocks, self.device_index)
                return self.cache
            with torch.cuda.device(self.cache.device):
                check(self.launch(self.blocks, current_stream(self.device_index), ctypes.byref(self.args)),
                      "cache-write launch")
        return self.cache
