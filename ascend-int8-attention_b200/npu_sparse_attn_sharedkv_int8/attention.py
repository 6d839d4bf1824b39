"""Prepared INT8 shared-KV decode attention (C4 / C128) for CUDA.

Counterpart of the reference's prepared operator (npu_sparse_attn_sharedkv_int8/attention.py:20-257):
the same constructor signature, attribute names, error texts, 200-byte argument struct,
`_rebind_same_geometry` and `run`.  Below the struct everything differs: one CUDA kernel family
decides tiling and KV splitting on the device, so the host-side tile / group / split planning of
the Ascend build has nothing to do here and its keyword arguments are accepted only where they
agree with what that kernel does.
"""
import ctypes

import torch

from . import c8_attention
from .runtime import Kernels, native_launcher

DIM = 512
_POINTER_FIELDS = ("q", "ori", "cmp", "oriScale", "cmpScale", "oriTable", "cmpTable", "indices", "cuQ", "seqLens",
                   "sinks", "out", "workspace", "lse", "oriStride", "cmpStride", "partial", "oriIndices")
_COUNT_FIELDS = ("tokens", "heads", "batch", "oriBlock", "cmpBlock", "oriTableWidth", "cmpTableWidth", "ratio",
                 "window", "topk", "splits", "oriTopk", "oriPages")
# argument-struct pointer <- attribute of the case, for everything a rebind may replace
_CASE_POINTERS = (("q", "q"), ("ori", "ori"), ("cmp", "cmp"), ("oriTable", "ori_block_table"),
                  ("cmpTable", "cmp_block_table"), ("indices", "cmp_indices"), ("cuQ", "cu_q"),
                  ("seqLens", "seq_lens"), ("sinks", "sink"), ("oriIndices", "ori_indices"))


class _Args(ctypes.Structure):
    """SharedKVArgs of the C ABI: 18 64-bit words, 13 32-bit words and one float, 200 bytes
    (csrc/kernels/c8/args.h:7-14 of the reference)."""
    _fields_ = ([(n, ctypes.c_uint64) for n in _POINTER_FIELDS] + [(n, ctypes.c_uint32) for n in _COUNT_FIELDS]
                + [("softmaxScale", ctypes.c_float)])


def _address(tensor):
    return 0 if tensor is None else tensor.data_ptr()


def _require(ok, message):
    if not ok:
        raise ValueError(message)


def _check_kv(cache, table, scale, batch, device):
    """One cache kind: INT8 pages, its block table and its frozen scale."""
    _require(cache is not None and cache.dtype == torch.int8 and cache.ndim == 4 and tuple(cache.shape[-2:]) == (1, DIM),
             "Expected INT8 cache[P,B,1,512]")
    pages, page_rows = cache.shape[:2]
    _require(pages > 0 and page_rows > 0 and pages * page_rows < 2 ** 31 and cache.stride(1) == DIM
             and cache.stride(-1) == 1 and cache.stride(0) >= page_rows * DIM, "Invalid page stride or empty cache")
    _require(table is not None and table.ndim == 2 and table.shape[0] == batch and table.dtype == torch.int32
             and table.is_contiguous(), "Expected contiguous INT32 block table[B,num_pages]")
    _require(scale is not None and tuple(scale.shape) == (DIM,) and scale.dtype == torch.float32 and scale.is_contiguous(),
             "Expected frozen contiguous FP32 scale[512]")
    _require(all(t.device == device for t in (cache, table, scale)), "All inputs must be on the same GPU")


def _check_case(case, ori_scale, cmp_scale):
    """Everything the constructor refuses about the inputs; returns (tokens, heads, device)."""
    q = case.q
    _require(q.device.type == "cuda" and q.dtype == torch.bfloat16 and q.ndim == 3 and q.shape[-1] == DIM,
             "Expected BF16 Q[T,H,512] on a CUDA device")
    tokens, heads, _ = q.shape
    _require(0 < heads <= 128 and q.is_contiguous(), "Expected 1..128 heads and contiguous Q")
    _require(case.ratio in (1, 4, 128) and case.window > 0, "Expected SWA/C4/C128 and a positive window")
    device, batch = q.device, case.seq_lens.numel()
    _check_kv(case.ori, case.ori_block_table, ori_scale, batch, device)
    if case.ratio > 1:
        _check_kv(case.cmp, case.cmp_block_table, cmp_scale, batch, device)
    picks = case.cmp_indices
    if case.ratio == 4:
        _require(picks is not None and picks.ndim == 3 and tuple(picks.shape[:2]) == (tokens, 1) and picks.shape[2] > 0
                 and picks.dtype == torch.int32 and picks.is_contiguous(), "C4 requires contiguous INT32 indices[T,1,topk]")
    _require(tuple(case.cu_q.shape) == (batch + 1,) and case.seq_lens.ndim == 1 and tuple(case.sink.shape) == (heads,),
             "Invalid sequence metadata or sink shape")
    for tensor, dtype in ((case.cu_q, torch.int32), (case.seq_lens, torch.int32), (case.sink, torch.float32)):
        _require(tensor.dtype == dtype and tensor.device == device and tensor.is_contiguous(),
                 "Invalid metadata dtype, device or contiguity")
    _require(picks is None or picks.device == device, "Indices must be on the same GPU")
    slots = case.ori_indices
    _require(slots is None or (slots.ndim == 3 and tuple(slots.shape[:2]) == (tokens, 1) and slots.shape[-1] > 0
                               and slots.dtype == torch.int32 and slots.device == device and slots.is_contiguous()),
             "Original physical slots must be contiguous INT32[T,1,K] on the query device")
    return tokens, heads, device


class PreparedAttention:
    """Holds every input and output tensor of one attention call; `run()` allocates nothing, reads
    nothing back and launches on the current stream.

    Protocol: BF16 Q[T,8,512], INT8 cache[P,32,1,512] (any page stride), frozen FP32 per-channel
    scales for the original and compressed caches, symmetric zero offsets.
    """

    def __init__(self, case, ori_scale, cmp_scale=None, *, output=None, splits=None, tile_size=None, query_group=None,
                 max_seq_len=None, return_lse=False, lse_output=None, scratch_allocator=None,
                 adaptive_splits=False, trim_cube_tails=None, dynamic_c4=None, dynamic_c128=None,
                 dynamic_grouped_c128=None, implementation="auto"):
        _require(implementation in ("auto", "v65", "fallback"), "implementation must be auto, v65 or fallback")
        tokens, heads, device = _check_case(case, ori_scale, cmp_scale)
        self.case, self.scales = case, (ori_scale, cmp_scale)
        self._bind_outputs(output, lse_output, return_lse, tokens, heads, device)
        # 128-key tiles, KV split on the device: the planning keywords of the reference are accepted
        # only where they say the same.  query_group = 2 or 4 (attention.py:96-100,186-190 of the reference)
        # selects the paired-query kernel: two adjacent tokens of a request share their tiles, and a group
        # of four is two pairs on the group's tiling.
        _require(tile_size in (None, 128), "The CUDA kernels use 128-key tiles; tile_size must be None or 128")
        _require(query_group in (None, 1, 2, 4), "Expected query_group 1, 2 or 4")
        # grouped C4 walks every compressed row of a context, so it is for short contexts only (attention.py:89-98)
        short_c4 = (case.ratio == 4 and isinstance(max_seq_len, int) and 0 < max_seq_len <= 1024
                    and case.cmp_indices is not None and case.cmp_indices.shape[-1] <= 1024)
        _require(query_group in (None, 1) or (heads == 8 and (case.ratio == 128 or short_c4)),
                 "Query grouping requires eight heads; C4 also requires a max_seq_len bound <= 1024 and top-k <= 1024")
        _require(query_group in (None, 1) or case.ori_indices is None, "Explicit original slots require ungrouped queries")
        _require(splits is None or (isinstance(splits, int) and 1 <= splits <= 24), "Expected 1..24 KV partitions")
        _require(not (adaptive_splits or trim_cube_tails or dynamic_grouped_c128),
                 "Host-selected Ascend tile plans have no CUDA counterpart; leave them unset")
        self.query_group, self.tile_size, self.splits = query_group or 1, 128, 1
        self.adaptive_splits = self.trim_cube_tails = self.dynamic_grouped_c128 = False
        general = case.ratio == 1 or case.ori_indices is not None      # the reference's compatibility entry (variant 0)
        self.dynamic_c4 = case.ratio == 4 and not general and self.query_group == 1
        self.dynamic_c128 = case.ratio == 128 and not general and self.query_group == 1
        _require(max_seq_len is None or (isinstance(max_seq_len, int) and max_seq_len > 0
                                         and (case.ori_indices is not None
                                              or max_seq_len <= case.ori_block_table.shape[1] * case.ori.shape[1])
                                         and (case.ratio == 1 or max_seq_len // case.ratio
                                              <= case.cmp_block_table.shape[1] * case.cmp.shape[1])),
                 "max_seq_len exceeds what the block tables can address")
        self.max_seq_len = max_seq_len
        self.workspace = self.partial = None
        self.blocks = 0
        if tokens == 0:
            return
        self.args = self._arguments(case, ori_scale, cmp_scale, tokens, heads)
        self.blocks = c8_attention.CORES
        self.kernels = Kernels()
        self.native = native_launcher()
        self.argument_address = ctypes.addressof(self.args)
        self.device_index = device.index
        self.variant = -1
        _require(implementation != "fallback" and (implementation != "auto" or c8_attention.enabled()),
                 "No legacy INT8 kernels exist in the CUDA build: SHAREDKV_C8_DECODE=0 and "
                 "implementation='fallback' cannot be honoured")
        _require(c8_attention.supported(self),
                 "This geometry is outside the CUDA decode kernels: need 8 heads, window 128, 32-row pages, "
                 "ratio 1, ratio 4 (top-k <= 1024) or ratio 128")
        self.__dict__.update(c8_attention.prepare(self, scratch_allocator=scratch_allocator).__dict__)

    def _bind_outputs(self, output, lse_output, return_lse, tokens, heads, device):
        q = self.case.q
        self.out = torch.empty_like(q) if output is None else output
        _require(self.out.shape == q.shape and self.out.dtype == torch.bfloat16 and self.out.device == device
                 and self.out.is_contiguous(), "Invalid output buffer")
        self.lse = lse_output
        if self.lse is None and return_lse:
            self.lse = torch.empty((tokens, heads), dtype=torch.float32, device=device)
        _require(self.lse is None or (tuple(self.lse.shape) == (tokens, heads) and self.lse.dtype == torch.float32
                                      and self.lse.device == device and self.lse.is_contiguous()),
                 "Invalid FP32 LSE[T,H] output buffer")

    def _arguments(self, case, ori_scale, cmp_scale, tokens, heads):
        args = _Args()
        for field, attribute in _CASE_POINTERS:
            setattr(args, field, _address(getattr(case, attribute)))
        args.oriScale, args.cmpScale = _address(ori_scale), _address(cmp_scale)
        args.out, args.lse = self.out.data_ptr(), _address(self.lse)
        args.oriStride, args.oriBlock, args.oriPages = case.ori.stride(0), case.ori.shape[1], case.ori.shape[0]
        args.oriTableWidth = case.ori_block_table.shape[1]
        if case.cmp is not None:
            args.cmpStride, args.cmpBlock = case.cmp.stride(0), case.cmp.shape[1]
            args.cmpTableWidth = case.cmp_block_table.shape[1]
        args.tokens, args.heads, args.batch = tokens, heads, case.seq_lens.numel()
        args.ratio, args.window, args.splits = case.ratio, case.window, 1
        args.topk = case.cmp_indices.shape[-1] if case.cmp_indices is not None else 0
        args.oriTopk = case.ori_indices.shape[-1] if case.ori_indices is not None else 0
        args.softmaxScale = case.softmax_scale
        return args

    def _rebind_same_geometry(self, case, *, output=None, lse_output=None):
        """Serving fast path (attention.py:233-247): other tensors of the same shapes, strides and
        dtypes; the caller has compared the geometry, nothing is validated again."""
        self.case = case
        if output is not None:
            self.out, self.lse = output, lse_output
        if not self.blocks:
            return
        if output is not None:
            self.args.out, self.args.lse = output.data_ptr(), _address(lse_output)
        for field, attribute in _CASE_POINTERS:
            setattr(self.args, field, _address(getattr(case, attribute)))

    def run(self):
        if self.blocks:
            if self.native is None:
                c8_attention.launch_raw(self)
            else:
                self.native.attention(self.argument_address, self.blocks, self.variant, self.device_index)
        return self.out
