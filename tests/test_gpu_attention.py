"""Decode attention on the GPU, through the C ABI, against the golden vectors and the oracle.

Gates
  * BF16 output vs the reference CPU path (128-key tiles, one partial state):
    max-abs <= 2e-2 and mean-abs <= 2e-3 (the acceptance band of this build), and the
    tighter band the reference uses for its own device (rtol 0.008, atol 0.0003; LSE 2e-5;
    reference tests/npu/test_attention.py:102-103);
  * query codes and INT32 QK accumulators: exact; INT32 PV accumulators: exact for the
    P codes the kernel produced; P codes themselves are compared with the oracle's where the
    token was processed as one piece (they depend on exp() to the last bit).
"""
import ctypes
from dataclasses import replace

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import (ATTENTION_CASES, GROUPED_CASES, PAGE_STRIDE, SLOT_CASES, bf16, device_tile_parts, error_metrics, load_case,
                           to_device)

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def prepared(case, ori_scale, cmp_scale, **kw):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    return PreparedAttention(case, ori_scale.to(DEVICE), None if cmp_scale is None else cmp_scale.to(DEVICE), **kw)


def sm_count():
    return torch.cuda.get_device_properties(0).multi_processor_count


def check_against_reference(out, lse, z, case=None, scales=None, ctas=None):
    """Acceptance band against the reference's default configuration (one running state per
    token); the reference's own device band against the oracle dealt the same tile pieces as
    the launch (the reference's tests do the same through their `layout()` helper)."""
    expected, expected_lse = bf16(z["out_s1"]).float(), torch.from_numpy(z["lse_s1"])
    m = error_metrics(out.float(), expected)
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, m
    torch.testing.assert_close(lse, expected_lse, rtol=2e-5, atol=2e-5)
    if case is not None and ctas != 1:
        parts = device_tile_parts(case, ctas or min(sm_count(), 160))
        expected, expected_lse = oracle.attention_tiled(case, *scales, return_lse=True, tile_parts=parts)
        expected = expected.float()
        torch.testing.assert_close(lse, expected_lse, rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(out.float(), expected, rtol=0.008, atol=0.0003)
    return m


@pytest.mark.parametrize("name", ATTENTION_CASES + SLOT_CASES)
def test_golden_cases(name):
    case, ori_scale, cmp_scale, z = load_case(name)
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
    op.workspace[1024:].fill_(0xA5)                      # only the head of a workspace (cleared once, at prepare) has to be clean
    out = op.run()
    torch.cuda.synchronize()
    check_against_reference(out.cpu(), op.lse.cpu(), z, case, (ori_scale, cmp_scale))
    again = op.run().clone()
    torch.cuda.synchronize()
    assert torch.equal(again, out)                      # deterministic across launches


@pytest.mark.parametrize("name", GROUPED_CASES)
def test_chunked_prefill_shapes_against_the_grouped_reference(name):
    """Several query tokens per request.  The kernel walks every token by itself (the arithmetic of
    query_group = 1: bit-level bands against that reference output); the reference's grouped plans
    (query_group 2 and 4, which share tiles between adjacent tokens and re-tile the window union)
    attend the same keys, so their outputs are matched inside the acceptance band too."""
    case, ori_scale, cmp_scale, z = load_case(name)
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
    out = op.run()
    torch.cuda.synchronize()
    check_against_reference(out.cpu(), op.lse.cpu(), z, case, (ori_scale, cmp_scale))
    for group in (2, 4):
        m = error_metrics(out.cpu().float(), bf16(z[f"out_g{group}"]).float())
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (group, m)
        torch.testing.assert_close(op.lse.cpu(), torch.from_numpy(z[f"lse_g{group}"]), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("stride,offset", [(PAGE_STRIDE, 16384), (16384 + 48, 16)])
@pytest.mark.parametrize("name", ("config0_c4", "mixed_c128", "real_c4", "slots_swa"))
def test_page_stride_and_offset_views(name, stride, offset):
    """Compact-layout views (whole-row strides: TMA row gather) and strides that are not a
    multiple of 512 bytes (cp.async row gather)."""
    case, ori_scale, cmp_scale, z = load_case(name)
    dev = to_device(case, DEVICE, stride=stride, offset=offset)
    op = prepared(dev, ori_scale, cmp_scale, return_lse=True)
    out = op.run()
    torch.cuda.synchronize()
    check_against_reference(out.cpu(), op.lse.cpu(), z, case, (ori_scale, cmp_scale))


class Debug(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in "tileInfo validMask qkAcc pCodes pvAcc qCodes counter".split()] + [
        ("maxTiles", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


def run_debug(op, max_tiles, ctas=0):
    from npu_sparse_attn_sharedkv_int8 import runtime
    tokens = op.case.q.shape[0]
    dev = op.case.q.device
    buffers = dict(
        tileInfo=torch.full((max_tiles, 4), -1, dtype=torch.int32, device=dev),
        validMask=torch.zeros((max_tiles, 4), dtype=torch.int32, device=dev),
        qkAcc=torch.zeros((max_tiles, 128, 16), dtype=torch.int32, device=dev),
        pCodes=torch.zeros((max_tiles, 128, 16), dtype=torch.int8, device=dev),
        pvAcc=torch.zeros((max_tiles, 512, 16), dtype=torch.int32, device=dev),
        qCodes=torch.zeros((tokens, 2, 16, 512), dtype=torch.int8, device=dev),
        counter=torch.zeros(1, dtype=torch.int32, device=dev))
    dbg = Debug(*[buffers[n].data_ptr() for n in "tileInfo validMask qkAcc pCodes pvAcc qCodes counter".split()],
                max_tiles, ctas)
    lib = runtime._library()
    runtime.check(lib.sharedkv_attention_debug(op.variant, runtime.current_stream(0), ctypes.byref(op.args),
                                                ctypes.byref(dbg)), "debug launch")
    torch.cuda.synchronize()
    return {k: v.cpu() for k, v in buffers.items()}


@pytest.mark.parametrize("legacy_gather", [False, True])
@pytest.mark.parametrize("name,ctas", [("config0_c4", 1), ("holes_c4", 1), ("short_c4", 1), ("mixed_c128", 1),
                                       ("real_c128", 1), ("config0_c4", 0), ("mixed_c128", 0), ("short_c4", 5),
                                       ("slots_swa", 1), ("slots_swa", 0), ("slots_c4", 1), ("slots_c4", 3)])
def test_integer_stages_are_exact(name, ctas, legacy_gather):
    case, ori_scale, cmp_scale, z = load_case(name)
    trace = oracle.Trace()
    oracle.attention_tiled(case, ori_scale, cmp_scale, trace=trace)
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
    dump = run_debug(op, max_tiles=len(trace.tiles) + 64, ctas=ctas | (0x80000000 if legacy_gather else 0))
    out, lse = op.out.cpu(), op.lse.cpu()
    check_against_reference(out, lse, z, case, (ori_scale, cmp_scale), ctas=ctas or None)

    # query codes, both planes, for every cache kind the token has a tile of
    used = {(t.token, t.kind) for t in trace.tiles}
    for (token, kind), (alpha, hi, lo) in trace.q_codes.items():
        if (token, kind) not in used:
            continue
        got = dump["qCodes"][token, kind].int()
        assert torch.equal(got[:8], hi) and torch.equal(got[8:], lo), (token, kind)

    count = int(dump["counter"][0])
    by_key = {(t.token, t.kind, t.tile): t for t in trace.tiles}
    seen, p_total, p_differs = set(), 0, 0
    for rec in range(count):
        token, kind, tile, part = dump["tileInfo"][rec].tolist()
        want = by_key.get((token, kind, tile))
        words = dump["validMask"][rec].numpy().view("uint32")
        valid = torch.tensor([(int(words[i // 32]) >> (i % 32)) & 1 for i in range(128)], dtype=torch.bool)
        if want is None:                       # slots past the packed selections: a tile with no key
            assert not valid.any()
            continue
        seen.add((token, kind, tile))
        assert torch.equal(valid[:want.rows], want.keep) and not valid[want.rows:].any()
        rows = torch.nonzero(valid).flatten()
        qk = dump["qkAcc"][rec]
        assert torch.equal(qk[rows, :8].T, want.qk_hi[:, want.keep]), (token, kind, tile)
        assert torch.equal(qk[rows, 8:].T, want.qk_lo[:, want.keep]), (token, kind, tile)
        codes = dump["pCodes"][rec].int()
        assert not codes[~valid].any()                     # padded keys carry zero weight
        kv = torch.zeros(128, 512, dtype=torch.int32)
        kv[:want.rows] = want.kv
        p_hi, p_lo = codes[:, :8].T.contiguous(), codes[:, 8:].T.contiguous()
        pv = dump["pvAcc"][rec]
        assert torch.equal(pv[:, :8].T, p_hi @ kv), (token, kind, tile)
        assert torch.equal(pv[:, 8:].T, p_lo @ kv), (token, kind, tile)
        if ctas == 1:                                      # one running state per token, as in the oracle
            p_total += want.rows * 16
            p_differs += int((p_hi[:, :want.rows] != want.p_hi).sum() + (p_lo[:, :want.rows] != want.p_lo).sum())
            assert int((p_hi[:, :want.rows] - want.p_hi).abs().max()) <= 1
    assert seen == set(by_key)
    if ctas == 1:
        assert p_differs <= max(2, p_total // 200), (p_differs, p_total)


@pytest.mark.parametrize("name", ATTENTION_CASES + SLOT_CASES)
def test_production_kernel_gives_the_bits_of_the_instrumented_kernel(name):
    """The integer-stage proofs above run the kernel instantiation that dumps its intermediates;
    the instantiation that serving and the benchmark launch is another binary.  Same grid, same
    work split, same arithmetic: its output and LSE must be the same bits."""
    case, ori_scale, cmp_scale, _ = load_case(name)
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
    out, lse = op.run().clone(), op.lse.clone()
    torch.cuda.synchronize()
    op.out.fill_(9.0)
    op.lse.fill_(9.0)
    run_debug(op, max_tiles=256)
    assert torch.equal(op.out, out) and torch.equal(op.lse, lse)


def test_a_wait_that_runs_out_ends_the_kernel_and_sets_the_status_word():
    """Every wait inside the kernel is bounded.  The test entry can make one barrier arrival go
    missing under a wait limit of about a millisecond: the warp that waits for it gives up, all
    roles return, the CTA frees its tensor memory, the kernel ends, and the workspace's status word
    says so until the workspace is initialised again.  Nothing hangs and the context stays usable:
    the next ordinary launch is correct."""
    from npu_sparse_attn_sharedkv_int8 import c8_attention, runtime
    case, ori_scale, cmp_scale, z = load_case("unit_c4")
    op = prepared(to_device(case, DEVICE), ori_scale, cmp_scale, return_lse=True)
    lib = runtime._library()
    stream = runtime.current_stream(0)
    assert lib.sharedkv_workspace_status(op.workspace.data_ptr(), stream) == 0
    run_debug(op, max_tiles=64, ctas=1 | 0x40000000)
    assert lib.sharedkv_workspace_status(op.workspace.data_ptr(), stream) == -110
    with pytest.raises(RuntimeError, match="ran out"):
        c8_attention.workspace_status(op)
    # sticky: an ordinary launch does not clear it ...
    out = op.run()
    torch.cuda.synchronize()
    check_against_reference(out.cpu(), op.lse.cpu(), z, case, (ori_scale, cmp_scale))
    assert lib.sharedkv_workspace_status(op.workspace.data_ptr(), stream) == -110
    # ... initialising the workspace does
    assert lib.sharedkv_workspace_init(op.workspace.data_ptr(), stream) == 0
    out = op.run()
    torch.cuda.synchronize()
    check_against_reference(out.cpu(), op.lse.cpu(), z, case, (ori_scale, cmp_scale))
    assert lib.sharedkv_workspace_status(op.workspace.data_ptr(), stream) == 0


def test_rebind_and_streams():
    # reference tests/npu/test_queue.py:39-56: rapid pointer rebinding on two streams
    case, ori_scale, cmp_scale, z = load_case("real_c4")
    dev = to_device(case, DEVICE)
    op = prepared(dev, ori_scale, cmp_scale)
    factors = (1.0, -0.75, 0.5, -1.25)
    expected = [oracle.attention_tiled(replace(case, q=(case.q * f).bfloat16()), ori_scale, cmp_scale).float() for f in factors]
    for auxiliary in (False, True):
        stream = torch.cuda.Stream(device=DEVICE) if auxiliary else torch.cuda.current_stream()
        stream.wait_stream(torch.cuda.current_stream())
        outputs = []
        with torch.cuda.stream(stream):
            for index in range(16):
                query = (dev.q * factors[index % 4]).bfloat16()
                output = torch.empty_like(query)
                op._rebind_same_geometry(replace(dev, q=query), output=output)
                op.run()
                outputs.append((query, output))
            stream.synchronize()
        for index, (_, output) in enumerate(outputs):
            torch.testing.assert_close(output.cpu().float(), expected[index % 4], rtol=0.008, atol=0.0003)


def test_contract_violations():
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    case, ori_scale, cmp_scale, _ = load_case("unit_c4")
    dev = to_device(case, DEVICE)
    scales = ori_scale.to(DEVICE), cmp_scale.to(DEVICE)
    with pytest.raises(ValueError):
        PreparedAttention(case, ori_scale, cmp_scale)                         # CPU tensors
    with pytest.raises(ValueError):
        PreparedAttention(replace(dev, q=dev.q.float()), *scales)
    with pytest.raises(ValueError):
        PreparedAttention(replace(dev, cmp_indices=dev.cmp_indices.long()), *scales)
    with pytest.raises(ValueError):
        PreparedAttention(replace(dev, window=64), *scales)
    with pytest.raises(ValueError):
        PreparedAttention(dev, scales[0], scales[1][:256])
    with pytest.raises(ValueError):
        PreparedAttention(dev, *scales, implementation="fallback")
    with pytest.raises(ValueError):
        PreparedAttention(dev, *scales, tile_size=512)
    with pytest.raises(ValueError):                                      # explicit slots: INT32 [T, 1, K] on the query device
        PreparedAttention(replace(dev, ori_indices=torch.zeros((dev.q.shape[0], 1, 8), dtype=torch.int64, device=DEVICE)), *scales)
    with pytest.raises(ValueError):
        PreparedAttention(replace(dev, ori_indices=torch.zeros((dev.q.shape[0], 8), dtype=torch.int32, device=DEVICE)), *scales)
    empty = replace(dev, q=dev.q[:0], cmp_indices=dev.cmp_indices[:0])
    op = PreparedAttention(empty, *scales)
    assert op.blocks == 0 and op.run().shape == (0, 8, 512)
