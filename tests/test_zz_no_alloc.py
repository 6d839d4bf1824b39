"""The workspace-free attention entry (`sharedkv_attention_static_scratch`) against the regular one.

The entry keeps its scratch in a fixed array inside the library, shared by every call on the
device, so the checks are: same bits as the workspace-taking launch, on two calls in a row (the
second call meets whatever the first one left in the array), for both layer kinds; the caller's
argument struct is not modified; more query rows than the stated limit are refused.
"""
import ctypes
import re

import pytest
import torch

from tests.support import PAGE_STRIDE, load_case, to_device
from tests.conftest import ROOT

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def entry():
    from npu_sparse_attn_sharedkv_int8 import runtime
    lib = runtime._library()
    fn = lib.sharedkv_attention_static_scratch
    fn.argtypes, fn.restype = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int
    return runtime, fn


def max_tokens():
    header = (ROOT / "include" / "sharedkv_c_abi.h").read_text()
    return int(re.search(r"#define\s+SHAREDKV_STATIC_SCRATCH_MAX_TOKENS\s+(\d+)u", header).group(1))


@pytest.mark.parametrize("name", ("config0_c4", "mixed_c128", "real_c4", "real_c128"))
def test_same_bits_as_the_workspace_entry_twice_in_a_row(name):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    runtime, static_scratch = entry()
    case, ori_scale, cmp_scale, _ = load_case(name)
    op = PreparedAttention(to_device(case, DEVICE, stride=PAGE_STRIDE, offset=16384), ori_scale.to(DEVICE),
                           cmp_scale.to(DEVICE), return_lse=True)
    expected, expected_lse = op.run().clone(), op.lse.clone()
    torch.cuda.synchronize()

    # a copy of the arguments that points at other outputs and at NO workspace
    out, lse = torch.full_like(expected, 7.0), torch.full_like(expected_lse, 7.0)
    args = type(op.args).from_buffer_copy(op.args)
    args.out, args.lse, args.workspace = out.data_ptr(), lse.data_ptr(), 0
    before = bytes(args)
    for call in range(2):
        out.fill_(7.0)
        lse.fill_(7.0)
        status = static_scratch(op.variant, runtime.current_stream(0), ctypes.byref(args))
        runtime.check(status, "static-scratch launch")
        torch.cuda.synchronize()
        assert torch.equal(out, expected), (name, call)
        assert torch.equal(lse, expected_lse), (name, call)
    assert bytes(args) == before


def test_alternating_layer_kinds_share_the_array():
    """C4 then C128 then C4 on one stream: each launch rebuilds what it reads from the array."""
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    runtime, static_scratch = entry()
    ops, wanted = [], []
    for name in ("config0_c4", "mixed_c128"):
        case, ori_scale, cmp_scale, _ = load_case(name)
        op = PreparedAttention(to_device(case, DEVICE), ori_scale.to(DEVICE), cmp_scale.to(DEVICE))
        wanted.append(op.run().clone())
        ops.append(op)
    torch.cuda.synchronize()
    outs = []
    for k in (0, 1, 0):
        out = torch.zeros_like(wanted[k])
        args = type(ops[k].args).from_buffer_copy(ops[k].args)
        args.out, args.workspace = out.data_ptr(), 0
        runtime.check(static_scratch(ops[k].variant, runtime.current_stream(0), ctypes.byref(args)), "launch")
        outs.append((k, out))
    torch.cuda.synchronize()
    for k, out in outs:
        assert torch.equal(out, wanted[k])


@pytest.mark.parametrize("ratio", (4, 128))
def test_the_largest_accepted_call(ratio):
    """As many query rows as the entry accepts (the item list and the partial states then reach the
    top of their areas in the array), many of them split over several CTAs: same bits as the
    workspace-taking launch, twice in a row; the array's status word stays clear."""
    from types import SimpleNamespace
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    from npu_sparse_attn_sharedkv_int8.reference import SharedKVCase
    runtime, static_scratch = entry()
    tokens, pages = max_tokens(), 512
    g = torch.Generator().manual_seed(99 + ratio)
    queries = torch.randint(1, 4, (tokens,), generator=g)
    cu = torch.cat((torch.zeros(1, dtype=torch.int64), torch.cumsum(queries, 0)))
    batch = int((cu <= tokens).sum()) - 1
    cu = cu[:batch + 1].clone()
    cu[-1] = tokens                                         # the last request takes what is left
    lengths = torch.randint(200, 9000, (batch,), generator=g, dtype=torch.int32)
    lengths = torch.maximum(lengths, (cu[1:] - cu[:-1]).to(torch.int32))
    case = SharedKVCase(
        q=torch.randn(tokens, 8, 512, generator=g).bfloat16(),
        ori=torch.randint(-127, 128, (pages, 32, 1, 512), generator=g, dtype=torch.int8),
        ori_block_table=torch.randint(0, pages, (batch, 282), generator=g, dtype=torch.int32),
        cu_q=cu.to(torch.int32), seq_lens=lengths, sink=torch.linspace(-2, 2, 8),
        cmp=torch.randint(-127, 128, (pages, 32, 1, 512), generator=g, dtype=torch.int8),
        cmp_block_table=torch.randint(0, pages, (batch, 71), generator=g, dtype=torch.int32),
        cmp_indices=torch.randint(-1, 2300, (tokens, 1, 1024), generator=g, dtype=torch.int32) if ratio == 4 else None,
        ratio=ratio)
    scale = (torch.rand(512, generator=g) * 0.02 + 0.005).to(DEVICE)
    op = PreparedAttention(case.to(DEVICE), scale, scale, return_lse=True)
    expected, expected_lse = op.run().clone(), op.lse.clone()
    torch.cuda.synchronize()
    out, lse = torch.empty_like(expected), torch.empty_like(expected_lse)
    args = type(op.args).from_buffer_copy(op.args)
    args.out, args.lse, args.workspace = out.data_ptr(), lse.data_ptr(), 0
    assert args.tokens == tokens
    for call in range(2):
        out.fill_(7.0)
        lse.fill_(7.0)
        runtime.check(static_scratch(op.variant, runtime.current_stream(0), ctypes.byref(args)), "static-scratch launch")
        torch.cuda.synchronize()
        assert torch.equal(out, expected) and torch.equal(lse, expected_lse), call
    assert runtime._library().sharedkv_static_scratch_status(runtime.current_stream(0)) == 0


def test_more_rows_than_the_limit_are_refused():
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    runtime, static_scratch = entry()
    case, ori_scale, cmp_scale, _ = load_case("config0_c4")
    op = PreparedAttention(to_device(case, DEVICE), ori_scale.to(DEVICE), cmp_scale.to(DEVICE))
    args = type(op.args).from_buffer_copy(op.args)
    args.tokens = max_tokens() + 1
    status = static_scratch(op.variant, runtime.current_stream(0), ctypes.byref(args))
    assert status == -34
    with pytest.raises(RuntimeError, match="beyond"):
        runtime.check(status, "static-scratch launch")
    assert static_scratch(op.variant, runtime.current_stream(0), None) == -22
    assert static_scratch(99, runtime.current_stream(0), ctypes.byref(args)) == -2       # the variant is checked first
    torch.cuda.synchronize()
