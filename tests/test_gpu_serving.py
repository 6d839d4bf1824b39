"""Serving-shaped checks of the decode path on the GPU.

* CUDA-graph replay with a live batch that changes between replays (the reference's
  tests/npu/test_dynamic.py:33-65): the live shape is derived on the device at every replay and
  rows past it are zeroed.
* Workload-sized parity: a synthetic serving batch (contexts up to 1M tokens, both layer kinds)
  is run on the GPU; sampled requests are extracted as small CPU cases and compared with the
  oracle inside the acceptance band (max-abs 2e-2, mean-abs 2e-3); the whole batch is checked
  through two size-independent properties: bit-identical repeat launches, and bit-identical
  output when Q is doubled and the softmax scale halved (the query's absmax scale doubles
  exactly, so codes and logits do not change).
"""
from dataclasses import replace
from types import SimpleNamespace

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import bf16, error_metrics, load_case, to_device

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def prepared(case, ori_scale, cmp_scale, **kw):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    return PreparedAttention(case, ori_scale.to(DEVICE), cmp_scale.to(DEVICE), **kw)


@pytest.mark.parametrize("name", ("config0_c4", "mixed_c128"))
def test_graph_replay_follows_the_live_batch(name):
    case, ori_scale, cmp_scale, z = load_case(name)
    dev = to_device(case, DEVICE)
    op = prepared(dev, ori_scale, cmp_scale, return_lse=True)
    expected, expected_lse = bf16(z["out_s1"]).float(), torch.from_numpy(z["lse_s1"])
    batch = case.seq_lens.numel()
    assert batch >= 2
    boundaries = case.cu_q.tolist()

    op.run()                                     # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream(device=DEVICE)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            op.run()
    torch.cuda.synchronize()

    full_lens, full_cu = dev.seq_lens.clone(), dev.cu_q.clone()
    for live in (batch, batch - 1, batch):
        dev.seq_lens.copy_(full_lens)
        dev.cu_q.copy_(full_cu)
        if live < batch:                         # trailing requests become padding
            dev.seq_lens[live:] = 0
            dev.cu_q[live + 1:] = -1
        op.out.fill_(3.0)
        op.lse.fill_(3.0)
        graph.replay()
        torch.cuda.synchronize()
        tokens = boundaries[live]
        out, lse = op.out.cpu().float(), op.lse.cpu()
        m = error_metrics(out[:tokens], expected[:tokens])
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (live, m)
        torch.testing.assert_close(lse[:tokens], expected_lse[:tokens], rtol=2e-5, atol=2e-5)
        assert not out[tokens:].any() and not lse[tokens:].any(), live      # padded rows are cleared


def test_an_all_padding_batch_writes_zeros():
    case, ori_scale, cmp_scale, _ = load_case("config0_c4")
    dev = to_device(case, DEVICE)
    op = prepared(dev, ori_scale, cmp_scale, return_lse=True)
    dev.seq_lens.zero_()
    op.out.fill_(5.0)
    op.lse.fill_(5.0)
    op.run()
    torch.cuda.synchronize()
    assert not op.out.any() and not op.lse.any()


@pytest.fixture(scope="module")
def serving_batch():
    from npu_sparse_attn_sharedkv_int8 import synthetic
    lengths = synthetic.log_uniform_lengths(160, 4096, 1 << 20, seed=7)
    lengths[0], lengths[1], lengths[2] = 1 << 20, 4096, 4099          # the extremes are always present
    work = synthetic.build("box", DEVICE, lengths, ratios=[4, 128], seed=11, max_context=1 << 20)
    yield work
    del work
    torch.cuda.empty_cache()


@pytest.mark.parametrize("layer_index", (0, 1))
def test_serving_batch_against_the_oracle_and_its_invariants(serving_batch, layer_index):
    from npu_sparse_attn_sharedkv_int8 import synthetic
    work = serving_batch
    layer = work.layers[layer_index]
    case = work.case(layer_index)
    op = prepared(case, layer.ori_scale, layer.cmp_scale, return_lse=True)
    out = op.run().clone()
    lse = op.lse.clone()
    torch.cuda.synchronize()

    # sampled requests against the CPU oracle (longest, shortest and a spread in between)
    order = torch.argsort(work.seq_lens_host).tolist()
    sample = sorted({order[0], order[1], order[len(order) // 3], order[len(order) // 2], order[-2], order[-1], 0, 1, 2})
    small, ori_scale, cmp_scale, ids = synthetic.extract_requests(work, layer_index, sample)
    expected, expected_lse = oracle.attention_tiled(small, ori_scale, cmp_scale, return_lse=True)
    m = error_metrics(out[ids.to(DEVICE)].cpu().float(), expected.float())
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
    torch.testing.assert_close(lse[ids.to(DEVICE)].cpu(), expected_lse, rtol=1e-4, atol=1e-4)

    # repeat launches are bit-identical (the split-K merge order is fixed by piece number)
    again = op.run()
    torch.cuda.synchronize()
    assert torch.equal(again, out)

    # Q * 2 with softmax_scale / 2: the same codes, the same logits, the same bits
    doubled = replace(case, q=(case.q.float() * 2).bfloat16(), softmax_scale=case.softmax_scale / 2)
    twin = prepared(doubled, layer.ori_scale, layer.cmp_scale, return_lse=True)
    assert torch.equal(twin.run(), out)
    torch.cuda.synchronize()
    assert torch.equal(twin.lse, lse)

    # every output row is a convex combination of dequantised rows plus the sink's share: finite, bounded
    bound = float((127 * torch.maximum(layer.ori_scale, layer.cmp_scale)).max())
    assert torch.isfinite(out.float()).all() and float(out.float().abs().max()) <= bound * 1.01


@pytest.mark.parametrize("ratio", (4, 128))
def test_many_query_tokens_per_request(ratio):
    """Chunked-prefill shapes run through the decode kernel as they are: every token is an
    independent query with its own causal position (the reference serves up to 16 384 tokens per
    request on this core, tests/npu/test_capacity.py:41-51).  A 300-token and a 17-token chunk."""
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    source = make_case(query_lengths=(300, 17), seq_lens=(2500, 4300), heads=8, ratio=ratio, topk=1024, seed=5)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    op = prepared(case.to(DEVICE), oq.scale, cq.scale, return_lse=True)
    out = op.run()
    torch.cuda.synchronize()
    expected, expected_lse = oracle.attention_tiled(case, oq.scale, cq.scale, return_lse=True)
    m = error_metrics(out.cpu().float(), expected.float())
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
    torch.testing.assert_close(op.lse.cpu(), expected_lse, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("ratio", (4, 128))
def test_twelve_thousand_requests_in_one_launch(ratio):
    """More requests than the work split keeps in shared memory (it then reads cuQ from global
    memory), sixteen tokens per planning thread, thousands of one- and two-tile items per CTA."""
    from npu_sparse_attn_sharedkv_int8.reference import SharedKVCase
    batch, pages = 12000, 512
    g = torch.Generator().manual_seed(77)
    lengths = torch.randint(1, 400, (batch,), generator=g, dtype=torch.int32)
    # requests share a small pool of pages (reads may alias), so the case stays small on the host
    case = SharedKVCase(
        q=torch.randn(batch, 8, 512, generator=g).bfloat16(),
        ori=torch.randint(-127, 128, (pages, 32, 1, 512), generator=g, dtype=torch.int8),
        ori_block_table=torch.randint(0, pages, (batch, 13), generator=g, dtype=torch.int32),
        cu_q=torch.arange(batch + 1, dtype=torch.int32), seq_lens=lengths, sink=torch.linspace(-2, 2, 8),
        cmp=torch.randint(-127, 128, (pages, 32, 1, 512), generator=g, dtype=torch.int8),
        cmp_block_table=torch.randint(0, pages, (batch, 4), generator=g, dtype=torch.int32),
        cmp_indices=torch.randint(-1, 110, (batch, 1, 1024), generator=g, dtype=torch.int32) if ratio == 4 else None,
        ratio=ratio)
    scale = SimpleNamespace(scale=torch.rand(512, generator=g) * 0.02 + 0.005)
    oq = cq = scale
    op = prepared(case.to(DEVICE), oq.scale, cq.scale, return_lse=True)
    out = op.run().cpu()
    torch.cuda.synchronize()
    lse = op.lse.cpu()
    for first in (0, 5000, batch - 40):                 # three slices of forty requests against the oracle
        rows = slice(first, first + 40)
        part = replace(case, q=case.q[rows], ori_block_table=case.ori_block_table[rows], cmp_block_table=case.cmp_block_table[rows],
                       cu_q=torch.arange(41, dtype=torch.int32), seq_lens=case.seq_lens[rows],
                       cmp_indices=case.cmp_indices[rows] if case.cmp_indices is not None else None)
        expected, expected_lse = oracle.attention_tiled(part, oq.scale, cq.scale, return_lse=True)
        m = error_metrics(out[rows].float(), expected.float())
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (first, m)
        torch.testing.assert_close(lse[rows], expected_lse, rtol=1e-4, atol=1e-4)
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("ratio", (4, 128))
@pytest.mark.parametrize("batch,queries", [(65, 1), (513, 1), (65, 5)])
@pytest.mark.parametrize("offset", (1, 15))
def test_metadata_views_at_odd_offsets(ratio, batch, queries, offset):
    """seqLens and cuQ as views 4 and 60 bytes into larger INT32 tensors (the reference's
    tests/npu/test_metadata_views.py:20-57: batches of 65 and 513, one and five query tokens, contexts
    of a few tokens): a captured launch replayed three times over a poisoned workspace, results
    against the oracle, the words around the views untouched."""
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    length = max(3, queries) if ratio == 4 else 127
    source = make_case(query_lengths=(queries,) * batch, seq_lens=(length,) * batch, heads=8, ratio=ratio, topk=1024,
                       seed=batch + queries + offset)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    dev = case.to(DEVICE)
    storage = []
    for name in ("seq_lens", "cu_q"):
        original = getattr(dev, name)
        raw = torch.full((offset + original.numel() + 16,), -777, dtype=torch.int32, device=DEVICE)
        view = raw[offset:offset + original.numel()]
        view.copy_(original)
        dev = replace(dev, **{name: view})
        storage.append((raw, original.numel()))
    op = prepared(dev, oq.scale, cq.scale, return_lse=True)
    assert op.args.seqLens % 16 != 0 and op.args.cuQ % 16 != 0
    initial = bytes(op.args)
    op.run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream(device=DEVICE)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            op.run()
    torch.cuda.synchronize()
    expected, expected_lse = oracle.attention_tiled(case, oq.scale, cq.scale, return_lse=True)
    for _ in range(3):
        op.workspace[1024:].fill_(0xA5)
        op.out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        m = error_metrics(op.out.cpu().float(), expected.float())
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
        torch.testing.assert_close(op.lse.cpu(), expected_lse, rtol=1e-4, atol=1e-4)
        assert bytes(op.args) == initial
    for raw, size in storage:
        assert (raw[:offset] == -777).all() and (raw[offset + size:] == -777).all()


def test_two_streams_at_once():
    """Two prepared operators with their own workspaces, launched back to back on two streams so
    that their persistent kernels compete for the SMs: no CTA ever waits for another CTA, so the
    launches interleave or serialise but both finish with the right answer."""
    streams = [torch.cuda.Stream(device=DEVICE) for _ in range(2)]
    jobs = []
    for name, stream in zip(("config0_c4", "mixed_c128"), streams):
        case, ori_scale, cmp_scale, z = load_case(name)
        with torch.cuda.stream(stream):
            op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
        jobs.append((op, stream, bf16(z["out_s1"]).float()))
    torch.cuda.synchronize()
    for _ in range(20):
        for op, stream, _ in jobs:
            with torch.cuda.stream(stream):
                op.run()
    torch.cuda.synchronize()
    for op, _, expected in jobs:
        m = error_metrics(op.out.cpu().float(), expected)
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
