"""Prepared INT8 shared-KV decode attention (C4 / C128) for CUDA.

Mirror of the reference's prepared operator (npu_sparse_attn_sharedkv_int8/attention.py:20-257):
the same constructor signature, validation rules and messages, the 200-byte argument
struct, attribute names, `_rebind_same_geometry` and `run`.  What differs is below the
struct: one CUDA kernel family decides tiling and KV splitting on the device, so the
host-side tile / group / split planning of the Ascend build has no work to do here and
the corresponding keyword arguments only select what that kernel already does.
"""
import ctypes

import torch

from . import c8_attention
from .runtime import Kernels, native_launcher


class _Args(ctypes.Structure):
    """SharedKVArgs, 200 bytes (csrc/kernels/c8/args.h:7-14 of the reference)."""
    _fields_ = [(name, ctypes.c_uint64) for name in (
        "q ori cmp oriScale cmpScale oriTable cmpTable indices cuQ seqLens sinks "
        "out workspace lse oriStride cmpStride partial oriIndices").split()] + [
        (name, ctypes.c_uint32) for name in (
            "tokens heads batch oriBlock cmpBlock oriTableWidth cmpTableWidth ratio window topk splits oriTopk oriPages").split()
    ] + [("softmaxScale", ctypes.c_float)]


class PreparedAttention:
    """Retains all input/output storage; run() contains no allocation or readback.

    Protocol: BF16 Q[T,8,512], INT8 cache[P,32,1,512] (any page stride), frozen FP32
    per-channel scales for the original and compressed caches, symmetric zero offsets.
    """

    def __init__(self, case, ori_scale, cmp_scale=None, *, output=None, splits=None, tile_size=None, query_group=None,
                 max_seq_len=None, return_lse=False, lse_output=None, scratch_allocator=None,
                 adaptive_splits=False, trim_cube_tails=None, dynamic_c4=None, dynamic_c128=None,
                 dynamic_grouped_c128=None, implementation="auto"):
        if implementation not in ("auto", "v65", "fallback"):
            raise ValueError("implementation must be auto, v65 or fallback")
        if case.q.device.type != "cuda" or case.q.dtype != torch.bfloat16 or case.q.ndim != 3 or case.q.shape[-1] != 512:
            raise ValueError("Expected BF16 Q[T,H,512] on a CUDA device")
        tokens, heads, _ = case.q.shape
        if not heads or heads > 128 or not case.q.is_contiguous():
            raise ValueError("Expected 1..128 heads and contiguous Q")
        if case.ratio not in (1, 4, 128) or case.window <= 0:
            raise ValueError("Expected SWA/C4/C128 and a positive window")
        device = case.q.device

        def check_cache(cache, table, scale):
            if cache is None or cache.dtype != torch.int8 or cache.ndim != 4 or cache.shape[-2:] != (1, 512):
                raise ValueError("Expected INT8 cache[P,B,1,512]")
            if (cache.shape[0] == 0 or cache.shape[1] == 0 or cache.shape[0] * cache.shape[1] >= 2**31
                    or cache.stride(1) != 512 or cache.stride(-1) != 1 or cache.stride(0) < cache.shape[1] * 512):
                raise ValueError("Invalid page stride or empty cache")
            if (table is None or table.ndim != 2 or table.shape[0] != case.seq_lens.numel()
                    or table.dtype != torch.int32 or not table.is_contiguous()):
                raise ValueError("Expected contiguous INT32 block table[B,num_pages]")
            if scale is None or scale.shape != (512,) or scale.dtype != torch.float32 or not scale.is_contiguous():
                raise ValueError("Expected frozen contiguous FP32 scale[512]")
            if any(x.device != device for x in (cache, table, scale)):
                raise ValueError("All inputs must be on the same GPU")

        check_cache(case.ori, case.ori_block_table, ori_scale)
        if case.ratio != 1:
            check_cache(case.cmp, case.cmp_block_table, cmp_scale)
        if case.ratio == 4:
            ix = case.cmp_indices
            if (ix is None or ix.ndim != 3 or ix.shape[:2] != (tokens, 1) or ix.shape[2] == 0
                    or ix.dtype != torch.int32 or not ix.is_contiguous()):
                raise ValueError("C4 requires contiguous INT32 indices[T,1,topk]")
        if case.cu_q.shape != (case.seq_lens.numel() + 1,) or case.seq_lens.ndim != 1 or case.sink.shape != (heads,):
            raise ValueError("Invalid sequence metadata or sink shape")
        for x, dtype in [(case.cu_q, torch.int32), (case.seq_lens, torch.int32), (case.sink, torch.float32)]:
            if x.dtype != dtype or x.device != device or not x.is_contiguous():
                raise ValueError("Invalid metadata dtype, device or contiguity")
        if case.cmp_indices is not None and case.cmp_indices.device != device:
            raise ValueError("Indices must be on the same GPU")
        if case.ori_indices is not None:
            raise ValueError("Explicit original slots (ori_indices) are outside the C4/C128 decode path built for CUDA")

        self.case = case
        self.scales = ori_scale, cmp_scale
        self.out = output if output is not None else torch.empty_like(case.q)
        if (self.out.shape != case.q.shape or self.out.device != device or self.out.dtype != torch.bfloat16
                or not self.out.is_contiguous()):
            raise ValueError("Invalid output buffer")
        self.lse = lse_output if lse_output is not None else (
            torch.empty((tokens, heads), dtype=torch.float32, device=device) if return_lse else None)
        if self.lse is not None and (self.lse.shape != (tokens, heads) or self.lse.dtype != torch.float32
                                     or self.lse.device != device or not self.lse.is_contiguous()):
            raise ValueError("Invalid FP32 LSE[T,H] output buffer")
        # The kernel always works on 128-key tiles, one query token per task, and splits KV on
        # the device; the planning keywords are accepted only where they agree with that.
        if tile_size not in (None, 128):
            raise ValueError("The CUDA kernels use 128-key tiles; tile_size must be None or 128")
        if query_group not in (None, 1):
            raise ValueError("The CUDA kernels process one query token per task; query_group must be None or 1")
        if splits is not None and (not isinstance(splits, int) or not 1 <= splits <= 24):
            raise ValueError("Expected 1..24 KV partitions")
        if adaptive_splits or trim_cube_tails or dynamic_grouped_c128:
            raise ValueError("Host-selected Ascend tile plans have no CUDA counterpart; leave them unset")
        self.query_group, self.tile_size, self.splits = 1, 128, 1
        self.adaptive_splits = self.trim_cube_tails = self.dynamic_grouped_c128 = False
        self.dynamic_c4, self.dynamic_c128 = case.ratio == 4, case.ratio == 128
        self.max_seq_len = max_seq_len
        self.workspace = self.partial = None
        if tokens == 0:
            self.blocks = 0
            return
        ptr = lambda t: t.data_ptr() if t is not None else 0
        self.args = _Args(
            *map(ptr, (case.q, case.ori, case.cmp, ori_scale, cmp_scale,
                       case.ori_block_table, case.cmp_block_table, case.cmp_indices,
                       case.cu_q, case.seq_lens, case.sink, self.out, None)),
            ptr(self.lse), case.ori.stride(0), case.cmp.stride(0) if case.cmp is not None else 0, 0, 0,
            tokens, heads, case.seq_lens.numel(), case.ori.shape[1],
            case.cmp.shape[1] if case.cmp is not None else 0, case.ori_block_table.shape[1],
            case.cmp_block_table.shape[1] if case.cmp is not None else 0,
            case.ratio, case.window, case.cmp_indices.shape[-1] if case.cmp_indices is not None else 0, 1,
            0, case.ori.shape[0], case.softmax_scale,
        )
        self.blocks = c8_attention.CORES
        self.kernels = Kernels()
        self.native = native_launcher()
        self.argument_address = ctypes.addressof(self.args)
        self.device_index = device.index
        self.variant = -1
        if implementation == "fallback" or (implementation == "auto" and not c8_attention.enabled()):
            raise ValueError("No legacy INT8 kernels exist in the CUDA build: SHAREDKV_C8_DECODE=0 and "
                             "implementation='fallback' cannot be honoured")
        if not c8_attention.supported(self):
            raise ValueError("This geometry is outside the CUDA C4/C128 decode kernels: need 8 heads, window 128, "
                             "32-row pages, ratio 4 (top-k <= 1024) or ratio 128")
        selected = c8_attention.prepare(self, scratch_allocator=scratch_allocator)
        self.__dict__.update(selected.__dict__)

    def _rebind_same_geometry(self, case, *, output=None, lse_output=None):
        """Internal serving fast path; the adapter checks the geometry key."""
        self.case = case
        if output is not None:
            self.out, self.lse = output, lse_output
        if not self.blocks:
            return
        if output is not None:
            self.args.out = output.data_ptr()
            self.args.lse = lse_output.data_ptr() if lse_output is not None else 0
        for name, tensor in (("q", case.q), ("ori", case.ori), ("cmp", case.cmp),
                             ("oriTable", case.ori_block_table), ("cmpTable", case.cmp_block_table),
                             ("indices", case.cmp_indices), ("cuQ", case.cu_q),
                             ("seqLens", case.seq_lens), ("sinks", case.sink)):
            setattr(self.args, name, tensor.data_ptr() if tensor is not None else 0)

    def run(self):
        if self.blocks == 0:
            return self.out
        if self.native is not None:
            self.native.attention(self.argument_address, self.blocks, self.variant, self.device_index)
            return self.out
        c8_attention.launch_raw(self)
        return self.out
