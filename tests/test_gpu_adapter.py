"""The serving adapter on a GPU: compact page views from the planner, cache writes and attention
through LayerRuntime, two streams, graph replay.  Follows the reference's adapter test
(tests/npu/test_adapter.py:33-191), with the CPU oracle as the arbiter."""
from dataclasses import dataclass, replace
from types import SimpleNamespace

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import device_tile_parts, error_metrics

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"
LAYERS = 38                     # 38 x 16 384 B = 622 592 B per block, the reference's compact geometry


@dataclass(frozen=True)
class Spec:
    dtype: torch.dtype = torch.int8
    page_size_bytes: int = 16384
    head_size: int = 512
    num_kv_heads: int = 1
    block_size: int = 32


def groups():
    specs = {f"layer{i}": Spec() for i in range(LAYERS)}
    return [SimpleNamespace(layer_names=list(specs), kv_cache_spec=SimpleNamespace(kv_cache_specs=specs))]


@pytest.fixture()
def adapter(tmp_path, monkeypatch):
    from npu_sparse_attn_sharedkv_int8 import vllm_adapter
    yield vllm_adapter, tmp_path, monkeypatch
    vllm_adapter.load_scales.cache_clear()


def build(adapter_fixture, ratio, batch=2, queries=3, length=700):
    """BF16 case -> calibrated scales on disk -> compact INT8 page views filled through the adapter."""
    from npu_sparse_attn_sharedkv_int8 import cache_layout
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    vllm_adapter, tmp_path, monkeypatch = adapter_fixture
    source = make_case(query_lengths=(queries,) * batch, seq_lens=(length,) * batch, heads=8, ratio=ratio, topk=1024, seed=991)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    path = tmp_path / f"scales{ratio}.pt"
    torch.save({"protocol": "sharedkv-c8-v1", "scales": {"unit.ori": oq.scale, "unit.cmp": cq.scale}}, path)
    monkeypatch.setenv("SHAREDKV_SCALES", str(path))
    vllm_adapter.load_scales.cache_clear()
    state = vllm_adapter.LayerRuntime(SimpleNamespace(swa_cache_layer=SimpleNamespace(prefix="unit.swa_cache"),
                                                      head_dim=512, turboquant=None))
    dev = source.to(DEVICE)
    backings, writes = [], []
    for kind, layer in (("ori", "layer1"), ("cmp", "layer5")):
        tensor = getattr(source, kind)
        blocks = tensor.shape[0]
        g = groups()
        count, descriptors = cache_layout.cache_config(SimpleNamespace(parallel_config=None), g, 0, override_num_blocks=blocks)
        raw = cache_layout.allocate(g, count, descriptors, DEVICE)
        for t in raw.values():
            t.fill_(73)                        # sentinel in every byte of the backing
        view = cache_layout.reshape(g, count, raw)[layer][0]
        assert view.stride(0) == 622592 and view.shape == (blocks, 32, 1, 512)
        setattr(dev, kind, view)
        updates = tensor.reshape(-1, 1, 512).to(DEVICE)
        slots = torch.arange(updates.shape[0], dtype=torch.int32, device=DEVICE)
        writes.append((view, updates, slots, kind))
        backings.append((raw, layer))
    quantized = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    return state, dev, writes, backings, quantized, (oq, cq), source


def call(dev, ratio, **extra):
    return dict(ori_kv=dev.ori, cmp_kv=dev.cmp, ori_block_table=dev.ori_block_table, cmp_block_table=dev.cmp_block_table,
                cmp_sparse_indices=dev.cmp_indices, cu_seqlens_q=dev.cu_q, seqused_kv=dev.seq_lens, sinks=dev.sink,
                metadata=None, cmp_ratio=ratio, ori_mask_mode=4, cmp_mask_mode=3, ori_win_left=127, ori_win_right=0,
                softmax_scale=dev.softmax_scale, layout_q="TND", layout_kv="PA_ND", return_softmax_lse=True, **extra)


def expect(quantized, scales, q=None):
    case = quantized if q is None else replace(quantized, q=q)
    ctas = min(torch.cuda.get_device_properties(0).multi_processor_count, 160)
    return oracle.attention_tiled(case, scales[0].scale, scales[1].scale, return_lse=True,
                                  tile_parts=device_tile_parts(case, ctas))


@pytest.mark.parametrize("ratio", (4, 128))
def test_layer_runtime_writes_attends_and_replays(adapter, ratio):
    vllm_adapter = adapter[0]
    state, dev, writes, backings, quantized, scales, source = build(adapter, ratio)
    kw = call(dev, ratio)

    def run(query):
        for w in writes:
            state.write(*w)
        return state.attention(query, **kw)

    for factor in (1.0, -0.75):
        query = (dev.q * factor).bfloat16().contiguous()
        out, lse = run(query)
        torch.cuda.synchronize()
        want, want_lse = expect(quantized, scales, (source.q * factor).bfloat16())
        m = error_metrics(out.cpu().float(), want.float())
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
        torch.testing.assert_close(out.cpu().float(), want.float(), rtol=0.008, atol=0.0003)
        assert lse.shape == (*query.shape[:2], 1)
        torch.testing.assert_close(lse.cpu().squeeze(-1), want_lse, rtol=2e-5, atol=2e-5)
    assert len(state.attention_ops) == 1 and len(state.writers) == 2          # same geometry: operators are reused

    # cache contents are the reference quantizer's codes, and nothing outside the two layers' pages was touched
    for (view, _, _, kind), (raw, layer) in zip(writes, backings):
        torch.testing.assert_close(view.cpu(), getattr(quantized, kind), rtol=0, atol=0)
        pages = raw["layer0"].view(-1)[:view.shape[0] * 622592].view(-1, 622592).cpu()
        offset = 16384 * int(layer.removeprefix("layer"))
        assert (pages[:, :offset] == 73).all() and (pages[:, offset + 16384:] == 73).all()

    # a second stream gets its own scratch and its own prepared operators
    side = torch.cuda.Stream(device=DEVICE)
    side.wait_stream(torch.cuda.current_stream())
    main_key = vllm_adapter.stream_key(torch.device(DEVICE))
    with torch.cuda.stream(side):
        assert vllm_adapter.stream_key(torch.device(DEVICE)) != main_key
        out_side, _ = run(dev.q)
        side.synchronize()
    want, want_lse = expect(quantized, scales)
    torch.testing.assert_close(out_side.cpu().float(), want.float(), rtol=0.008, atol=0.0003)
    assert len(state.attention_ops) == 2

    # graph capture: the captured launch keeps its argument values although the operator object is reused
    query = dev.q.clone()
    graph = torch.cuda.CUDAGraph()
    capture = torch.cuda.Stream(device=DEVICE)
    capture.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(capture):
        run(query)                                           # warm the prepared operators of this stream
        capture.synchronize()
        with torch.cuda.graph(graph, stream=capture):
            out, lse = run(query)
    torch.cuda.synchronize()
    state.attention((-query).contiguous(), **kw)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu().float(), want.float(), rtol=0.008, atol=0.0003)
    torch.testing.assert_close(lse.cpu().squeeze(-1), want_lse, rtol=2e-5, atol=2e-5)
    assert state.captured_ops
    _, empty = state.attention(query, **{**kw, "return_softmax_lse": False})
    assert empty.shape == (0,) and empty.dtype == torch.float32 and empty.device == query.device
    assert all(op.case is None and op.out is None for op in state.attention_ops.values())


def test_explicit_original_slots_through_the_adapter(adapter):
    """The serving stack's draft layers name their original rows by physical slot
    (`ori_sparse_indices`, vllm_adapter.py:154 of the reference): the adapter hands them to the kernels
    through the general launcher; holes and out-of-range slots are masked."""
    state, dev, writes, _, quantized, scales, source = build(adapter, 4)
    for w in writes:
        state.write(*w)
    g = torch.Generator().manual_seed(41)
    total = quantized.ori.shape[0] * 32
    slots = torch.randint(0, total, (dev.q.shape[0], 1, 200), generator=g, dtype=torch.int32)
    slots[:, :, ::7] = -1
    slots[:, :, 3::11] = total + 1
    out, lse = state.attention(dev.q, **{**call(dev, 4), "ori_sparse_indices": slots.to(DEVICE)})
    torch.cuda.synchronize()
    case = replace(quantized, ori_indices=slots)
    ctas = min(torch.cuda.get_device_properties(0).multi_processor_count, 160)
    want, want_lse = oracle.attention_tiled(case, scales[0].scale, scales[1].scale, return_lse=True,
                                            tile_parts=device_tile_parts(case, ctas))
    torch.testing.assert_close(out.cpu().float(), want.float(), rtol=0.008, atol=0.0003)
    torch.testing.assert_close(lse.cpu().squeeze(-1), want_lse, rtol=2e-5, atol=2e-5)
    plain, _ = oracle.attention_tiled(case, scales[0].scale, scales[1].scale, return_lse=True)
    m = error_metrics(out.cpu().float(), plain.float())
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m


def test_operator_cache_is_bounded_and_calls_are_validated(adapter):
    vllm_adapter = adapter[0]
    state, dev, writes, _, _, _, _ = build(adapter, 4, batch=1, queries=1, length=300)
    for w in writes:
        state.write(*w)
    kw = call(dev, 4)
    for tokens in range(1, 12):                     # eleven query geometries through one layer
        q = dev.q[:1].repeat(tokens, 1, 1).contiguous()
        cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEVICE)
        idx = dev.cmp_indices[:1].repeat(tokens, 1, 1).contiguous()
        state.attention(q, **{**kw, "cu_seqlens_q": cu, "cmp_sparse_indices": idx})
    torch.cuda.synchronize()
    assert len(state.attention_ops) == vllm_adapter.PREPARED_PER_LAYER
    with pytest.raises(ValueError):
        state.attention(dev.q, **{**kw, "layout_q": "BSND"})
    with pytest.raises(ValueError):
        state.attention(dev.q, **{**kw, "cmp_mask_mode": 0})
    with pytest.raises(ValueError):
        state.write(writes[0][0], writes[0][1], writes[0][2][:-1], "ori")
    state.write(writes[0][0], writes[0][1][:0], writes[0][2][:0], "ori")        # no rows: nothing to do
