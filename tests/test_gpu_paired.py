"""Paired-query kernel (query_group = 2) on the GPU against the reference's grouped arithmetic.

The reference's tiled oracle with query_group = 2 (reference.py:229-234,243-249,300-301) tiles the
union of two adjacent tokens' windows from its first row and walks the later token's compressed
prefix; on a ratio-4 layer every token attends the rows its own top-k list names, a row named n
times with log(n) added to its logits.  The paired kernel follows that tiling and never splits an
item, so its results are held to the reference's own device band (rtol 0.008, atol 0.0003 on BF16
output, 2e-5 on LSE; reference tests/npu/test_attention.py:102-103) against the golden `out_g2` and
against the oracle.
"""
from dataclasses import replace
import math

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import PAGE_STRIDE, bf16, error_metrics, load_case, strided_pages, to_device

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def prepared(case, ori_scale, cmp_scale, group=2, **kw):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    return PreparedAttention(case, ori_scale.to(DEVICE), cmp_scale.to(DEVICE), query_group=group, return_lse=True, **kw)


def assert_device_band(out, lse, expected, expected_lse):
    torch.testing.assert_close(lse, expected_lse, rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(out.float(), expected.float(), rtol=0.008, atol=0.0003)


def test_golden_grouped_case():
    case, ori_scale, cmp_scale, z = load_case("grouped_c128")
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale)
    assert op.variant == 7 and op.query_group == 2
    op.workspace[1024:].fill_(0xA5)
    out = op.run()
    torch.cuda.synchronize()
    from npu_sparse_attn_sharedkv_int8 import c8_attention
    c8_attention.workspace_status(op)
    assert_device_band(out.cpu(), op.lse.cpu(), bf16(z["out_g2"]), torch.from_numpy(z["lse_g2"]))
    m = error_metrics(out.cpu().float(), bf16(z["out_g1"]).float())          # the same keys as the ungrouped walk
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
    again = op.run().clone()
    torch.cuda.synchronize()
    assert torch.equal(again, out)


@pytest.mark.parametrize("name,bound,variant", [("grouped_c128", None, 3), ("grouped_c4_short", 1024, 4)])
def test_golden_cases_in_groups_of_four(name, bound, variant):
    """query_group = 4: the tiling of four adjacent tokens, walked as two pairs."""
    case, ori_scale, cmp_scale, z = load_case(name)
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, group=4, max_seq_len=bound)
    assert op.variant == variant and op.query_group == 4
    out = op.run()
    torch.cuda.synchronize()
    assert_device_band(out.cpu(), op.lse.cpu(), bf16(z["out_g4"]), torch.from_numpy(z["lse_g4"]))


def random_case(seed):
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    g = torch.Generator().manual_seed(7000 + seed)
    pick = lambda options: options[int(torch.randint(len(options), (1,), generator=g))]
    batch = int(torch.randint(1, 7, (1,), generator=g))
    queries = [int(torch.randint(1, 10, (1,), generator=g)) for _ in range(batch)]
    top = pick((70000, 40000, 9000, 300))
    lengths = [max(q, int(math.exp(float(torch.rand(1, generator=g)) * math.log(top)))) for q in queries]
    if seed % 4 == 0:
        lengths[0] = queries[0]                       # positions 0 .. q - 1: windows shorter than a tile
    if seed % 4 == 1:
        lengths[-1] = 127 + queries[-1] // 2          # the window union crosses the 128-row mark inside the request
    if seed % 4 == 2:
        lengths[0] = 16384 + queries[0] // 2          # a compressed tile appears between the tokens of one request
    source = make_case(query_lengths=tuple(queries), seq_lens=tuple(lengths), heads=8, ratio=128, topk=1024, seed=seed)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    stride = pick((16384, PAGE_STRIDE, 16384 + 512, 16384 + 48))
    return case, oq.scale, cq.scale, stride, (16 if stride % 512 else 1024)


@pytest.mark.parametrize("seed", range(16))
def test_random_geometry(seed):
    case, ori_scale, cmp_scale, stride, offset = random_case(seed)
    dev = case.to(DEVICE)
    dev = replace(dev, ori=strided_pages(case.ori, DEVICE, stride, offset), cmp=strided_pages(case.cmp, DEVICE, stride, offset))
    group = 4 if seed % 2 else 2
    op = prepared(dev, ori_scale, cmp_scale, group=group)
    out = op.run()
    torch.cuda.synchronize()
    expected, expected_lse = oracle.attention_tiled(case, ori_scale, cmp_scale, query_group=group, return_lse=True)
    assert_device_band(out.cpu(), op.lse.cpu(), expected, expected_lse)


def test_chunked_prefill_chunk_with_a_dead_request():
    """48 + 33 query tokens behind long contexts, then a request that is turned into padding after
    the call was prepared (as a captured serving graph meets it): its rows come back as zeros."""
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    source = make_case(query_lengths=(48, 33, 7), seq_lens=(33000, 20000, 900), heads=8, ratio=128, topk=1024, seed=5)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    expected, expected_lse = oracle.attention_tiled(case, oq.scale, cq.scale, query_group=2, return_lse=True)
    dev = case.to(DEVICE)
    op = prepared(dev, oq.scale, cq.scale)
    out = op.run()
    torch.cuda.synchronize()
    assert_device_band(out.cpu(), op.lse.cpu(), expected, expected_lse)
    dev.seq_lens[2:] = 0
    dev.cu_q[3:] = -1
    op.out.fill_(3.0)
    op.lse.fill_(3.0)
    out = op.run()
    torch.cuda.synchronize()
    assert_device_band(out[:81].cpu(), op.lse[:81].cpu(), expected[:81], expected_lse[:81])
    assert not out[81:].any() and not op.lse[81:].any()


@pytest.mark.parametrize("tokens,length", [(4096, 65536), (16384, 16384)])
def test_prefill_capacity(tokens, length):
    """One request with as many query tokens as the reference serves on one core (tests/npu/
    test_capacity.py:41-51 of the reference: chunk4096_long, prefill16384): the one-token walk, pairs and
    groups of four against the oracle on 24 sampled tokens each (device band for the grouped
    plans, acceptance band for the one-token walk, whose pieces the sample does not follow), and
    against one another on every token (acceptance band)."""
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    source = make_case(query_lengths=(tokens,), seq_lens=(length,), heads=8, ratio=128, topk=1024, seed=tokens)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    dev = case.to(DEVICE)
    g = torch.Generator().manual_seed(1)
    sample = sorted(set([0, 1, 2, 3, 126, 127, 128, 129, tokens - 2, tokens - 1] + torch.randint(0, tokens, (14,), generator=g).tolist()))
    outputs = {}
    for group in (1, 2, 4):
        op = PreparedAttention(dev, oq.scale.to(DEVICE), cq.scale.to(DEVICE), query_group=group, return_lse=True)
        out = op.run()
        torch.cuda.synchronize()
        outputs[group] = out.cpu().float()
        expected, expected_lse = oracle.attention_tiled(case, oq.scale, cq.scale, query_group=group, return_lse=True, only_tokens=sample)
        if group == 1:
            m = error_metrics(outputs[group][sample], expected.float())
            assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
            torch.testing.assert_close(op.lse.cpu()[sample], expected_lse, rtol=1e-4, atol=1e-4)
        else:
            assert_device_band(out.cpu()[sample], op.lse.cpu()[sample], expected, expected_lse)
    for group in (2, 4):
        m = error_metrics(outputs[group], outputs[1])
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (group, m)


def test_golden_grouped_c4_case_with_duplicate_selections():
    """Contexts of 700, 1024, 131 and 9 tokens, 5 + 2 + 3 + 1 query tokens, top-k lists that name some
    rows two and three times (and so drop others)."""
    case, ori_scale, cmp_scale, z = load_case("grouped_c4_short")
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, max_seq_len=1024)
    assert op.variant == 8 and op.query_group == 2
    out = op.run()
    torch.cuda.synchronize()
    from npu_sparse_attn_sharedkv_int8 import c8_attention
    c8_attention.workspace_status(op)
    assert_device_band(out.cpu(), op.lse.cpu(), bf16(z["out_g2"]), torch.from_numpy(z["lse_g2"]))
    again = op.run().clone()
    torch.cuda.synchronize()
    assert torch.equal(again, out)


def random_sparse_case(seed):
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    g = torch.Generator().manual_seed(9000 + seed)
    pick = lambda options: options[int(torch.randint(len(options), (1,), generator=g))]
    batch = int(torch.randint(1, 6, (1,), generator=g))
    queries = [int(torch.randint(1, 8, (1,), generator=g)) for _ in range(batch)]
    lengths = [max(q, int(torch.randint(1, 1025, (1,), generator=g))) for q in queries]
    if seed % 3 == 0:
        lengths[0] = 1024
    topk = pick((1024, 256, 64))
    source = make_case(query_lengths=tuple(queries), seq_lens=tuple(lengths), heads=8, ratio=4, topk=topk, seed=seed)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    idx = case.cmp_indices.clone()
    style = seed % 4
    if style == 1:
        idx[:, :, ::5] = -1                                    # holes
    elif style == 2:
        idx[:, :, 3::7] = 2 ** 30                              # out of range
        idx[:, :, 1::9] = idx[:, :, 0::9][:, :, :idx[:, :, 1::9].shape[-1]]      # duplicates
    elif style == 3:
        idx[:, :, topk // 2:] = idx[:, :, :topk - topk // 2]   # every named row named again
    case = replace(case, cmp_indices=idx.contiguous())
    stride = pick((16384, PAGE_STRIDE, 16384 + 48))
    return case, oq.scale, cq.scale, stride, (16 if stride % 512 else 1024)


@pytest.mark.parametrize("seed", range(12))
def test_random_grouped_c4_geometry(seed):
    case, ori_scale, cmp_scale, stride, offset = random_sparse_case(seed)
    dev = case.to(DEVICE)
    dev = replace(dev, ori=strided_pages(case.ori, DEVICE, stride, offset), cmp=strided_pages(case.cmp, DEVICE, stride, offset))
    group = 4 if seed % 2 else 2
    op = prepared(dev, ori_scale, cmp_scale, group=group, max_seq_len=int(case.seq_lens.max()))
    out = op.run()
    torch.cuda.synchronize()
    expected, expected_lse = oracle.attention_tiled(case, ori_scale, cmp_scale, query_group=group, return_lse=True)
    assert_device_band(out.cpu(), op.lse.cpu(), expected, expected_lse)


def test_grouped_c4_beyond_its_context_bound_is_reported():
    """The raw entry on a 2051-token context: the launch completes, the workspace status says
    SHAREDKV_ERANGE.  (PreparedAttention does not let such a call through.)"""
    import ctypes
    from npu_sparse_attn_sharedkv_int8 import c8_attention, runtime
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    case, ori_scale, cmp_scale, _ = load_case("grouped_c4")
    op = PreparedAttention(to_device(case, DEVICE), ori_scale.to(DEVICE), cmp_scale.to(DEVICE))
    lib = c8_attention.library()
    runtime.check(lib.launch_sharedkv_paired_sparse(0, runtime.current_stream(0), ctypes.byref(op.args)), "launch")
    torch.cuda.synchronize()
    assert lib.sharedkv_workspace_status(op.workspace.data_ptr(), runtime.current_stream(0)) == -34
    with pytest.raises(RuntimeError):
        c8_attention.workspace_status(op)


def test_graph_replay_and_a_workspace_shared_with_the_one_token_kernel():
    """A captured graph that launches the one-token kernel and the paired kernel in turn on ONE
    workspace (a serving scratch pool hands the same buffer to launches of different plans): the
    paired launch leaves the split-K tickets of the workspace as it found them, and replays give the
    bits of the first run."""
    import ctypes
    from npu_sparse_attn_sharedkv_int8 import c8_attention
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    case, ori_scale, cmp_scale, z = load_case("grouped_c128")
    dev = to_device(case, DEVICE)
    shared = torch.empty(c8_attention.workspace_bytes(case.q.shape[0]) + 256, dtype=torch.uint8, device=DEVICE)
    shared = shared[(-shared.data_ptr()) % 256:][:c8_attention.workspace_bytes(case.q.shape[0])]
    pool = lambda name, shape, dtype, device: shared
    single = PreparedAttention(dev, ori_scale.to(DEVICE), cmp_scale.to(DEVICE), return_lse=True, scratch_allocator=pool)
    paired = prepared(dev, ori_scale, cmp_scale, scratch_allocator=pool)
    assert single.workspace.data_ptr() == paired.workspace.data_ptr()
    for op in (single, paired, single, paired):
        op.run()
    torch.cuda.synchronize()
    first = single.out.clone(), paired.out.clone(), paired.lse.clone()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream(device=DEVICE)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for op in (paired, single, paired, single):
                op.run()
    torch.cuda.synchronize()
    for _ in range(3):
        single.out.fill_(1.0)
        paired.out.fill_(1.0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(single.out, first[0]) and torch.equal(paired.out, first[1]) and torch.equal(paired.lse, first[2])
    c8_attention.workspace_status(paired)
    assert_device_band(paired.out.cpu(), paired.lse.cpu(), bf16(z["out_g2"]), torch.from_numpy(z["lse_g2"]))

    # the workspace-free entry takes the paired variant as well
    from npu_sparse_attn_sharedkv_int8 import runtime
    static_scratch = runtime._library().sharedkv_attention_static_scratch
    static_scratch.argtypes, static_scratch.restype = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int
    out = torch.full_like(paired.out, 7.0)
    args = type(paired.args).from_buffer_copy(paired.args)
    args.out, args.lse, args.workspace = out.data_ptr(), 0, 0
    runtime.check(static_scratch(7, runtime.current_stream(0), ctypes.byref(args)), "static-scratch launch")
    torch.cuda.synchronize()
    assert torch.equal(out, first[1])


def test_selection_rules():
    case, ori_scale, cmp_scale, _ = load_case("grouped_c4")
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    for bound in (None, 2051):              # grouped C4 needs a context bound of at most 1024 tokens
        with pytest.raises(ValueError, match="Query grouping requires"):
            PreparedAttention(to_device(case, DEVICE), ori_scale.to(DEVICE), cmp_scale.to(DEVICE), query_group=2, max_seq_len=bound)
    case, ori_scale, cmp_scale, _ = load_case("grouped_c128")
    with pytest.raises(ValueError, match="Expected query_group"):
        PreparedAttention(to_device(case, DEVICE), ori_scale.to(DEVICE), cmp_scale.to(DEVICE), query_group=3)
