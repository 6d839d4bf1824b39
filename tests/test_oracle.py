"""The CPU oracle against vectors produced by the reference's own Python functions.

Bit-exact: the oracle uses the same tensor library for round/exp/log as the reference,
so BF16 outputs and FP32 log-sum-exps must be identical, for every split count stored.
"""
import math

import numpy as np
import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import ATTENTION_CASES, GROUPED_CASES, SLOT_CASES, GOLDEN, bf16, load_case


def test_rounding_and_clipping_known_answer():
    # reference tests/unit/test_reference.py:22-27
    row = torch.zeros(1, 512)
    row[0, :8] = torch.tensor([-200.0, -127.0, -1.5, -0.5, 0.5, 1.5, 127.0, 200.0])
    codes = oracle.quantize_rows(row, oracle.inverse_scale(torch.ones(512)))
    assert codes[0, :8].tolist() == [-127, -127, -2, 0, 0, 2, 127, 127]
    assert codes.dtype == torch.int8


def test_writer_codes_match_reference():
    z = np.load(GOLDEN / "writer.npz")
    inv = oracle.inverse_scale(torch.from_numpy(z["scale"]))
    assert torch.equal(inv, torch.from_numpy(z["inverse_scale"]))
    assert torch.equal(oracle.quantize_rows(bf16(z["rows"]), inv), torch.from_numpy(z["codes"]))
    unit = oracle.inverse_scale(torch.ones(512))
    assert torch.equal(oracle.quantize_rows(torch.from_numpy(z["kat_rows"]), unit), torch.from_numpy(z["kat_codes"]))
    assert torch.equal(oracle.quantize_rows(bf16(z["tie_rows"]), unit), torch.from_numpy(z["tie_codes"]))


def test_writer_slot_rules():
    inv = torch.full((512,), 10.0)
    cache = torch.zeros(3, 32, 1, 512, dtype=torch.int8)
    rows = torch.arange(1, 8).float().reshape(7, 1).expand(7, 512) / 10
    slots = torch.tensor([0, 33, -1, 95, 96, 2 ** 31 - 1, 64], dtype=torch.int64)
    oracle.write_cache(cache, rows, slots, inv)
    flat = cache.reshape(96, 512)[:, 0]
    assert flat[0] == 1 and flat[33] == 2 and flat[95] == 4 and flat[64] == 7
    assert int((flat != 0).sum()) == 4          # -1, slot 96 (page 3 of 3) and the huge slot were skipped
    pairs = torch.tensor([[0, 1], [2, 31], [-1, 0], [1, 32], [1, -1], [3, 0]], dtype=torch.int32)
    cache.zero_()
    oracle.write_cache(cache, rows[:6], pairs, inv)
    assert cache[0, 1, 0, 0] == 1 and cache[2, 31, 0, 0] == 2 and int((cache[:, :, 0, 0] != 0).sum()) == 2


def test_joint_softmax_known_answer_and_random_row():
    # reference tests/unit/test_reference.py:50-56: out == 10 exactly, lse == ln 3
    q = torch.zeros(2, 512)
    caches = [torch.full((1, 512), v, dtype=torch.int8) for v in (10, 20)]
    out, lse = oracle.attention_joint_row(q, caches, [torch.ones(512)] * 2, torch.zeros(2), 1.0)
    assert torch.equal(out.float(), torch.full_like(q, 10.0))
    torch.testing.assert_close(lse, torch.full((2,), math.log(3)), rtol=1e-6, atol=1e-6)
    z = np.load(GOLDEN / "joint.npz")
    assert torch.equal(out, bf16(z["kat_out"])) and torch.equal(lse, torch.from_numpy(z["kat_lse"]))
    scale = torch.from_numpy(z["scale"])
    out, lse = oracle.attention_joint_row(bf16(z["q"]), [torch.from_numpy(z["c0"]), torch.from_numpy(z["c1"])],
                                          [scale, scale], torch.linspace(-2, 2, 8), 512 ** -0.5)
    assert torch.equal(out, bf16(z["out"])) and torch.equal(lse, torch.from_numpy(z["lse"]))


@pytest.mark.parametrize("name", ATTENTION_CASES)
def test_tiled_attention_reproduces_reference_bit_for_bit(name):
    case, ori_scale, cmp_scale, z = load_case(name)
    for splits in (1, 2, 3):
        out, lse = oracle.attention_tiled(case, ori_scale, cmp_scale, tile_size=128, splits=splits, return_lse=True)
        assert torch.equal(out, bf16(z[f"out_s{splits}"])), (name, splits)
        assert torch.equal(lse, torch.from_numpy(z[f"lse_s{splits}"])), (name, splits)


@pytest.mark.parametrize("name", GROUPED_CASES)
def test_query_groups_reproduce_reference_bit_for_bit(name):
    """reference.py:229-234,243-249,300-301: adjacent query tokens of a request share the union of their
    windows and (C128) the longest prefix; a grouped C4 token walks every compressed row with a
    log(multiplicity) bias for the rows its top-k list names, duplicates included."""
    case, ori_scale, cmp_scale, z = load_case(name)
    for group in (1, 2, 4):
        out, lse = oracle.attention_tiled(case, ori_scale, cmp_scale, tile_size=128, query_group=group, return_lse=True)
        assert torch.equal(out, bf16(z[f"out_g{group}"])), (name, group)
        assert torch.equal(lse, torch.from_numpy(z[f"lse_g{group}"])), (name, group)
    # grouping only re-tiles the same keys: the three results agree far inside the acceptance band
    for group in (2, 4):
        diff = (bf16(z[f"out_g{group}"]).float() - bf16(z["out_g1"]).float()).abs()
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3


@pytest.mark.parametrize("name", SLOT_CASES)
def test_explicit_original_slots_reproduce_reference_bit_for_bit(name):
    """reference.py:235-239,285: the caller names the original rows by physical slot; negative and
    out-of-range entries are masked in place, duplicates count twice; ratio 1 has no compressed kind."""
    case, ori_scale, cmp_scale, z = load_case(name)
    assert case.ori_indices is not None and (case.ratio == 1) == (case.cmp is None)
    for splits in (1, 2):
        out, lse = oracle.attention_tiled(case, ori_scale, cmp_scale, tile_size=128, splits=splits, return_lse=True)
        assert torch.equal(out, bf16(z[f"out_s{splits}"])), (name, splits)
        assert torch.equal(lse, torch.from_numpy(z[f"lse_s{splits}"])), (name, splits)


@pytest.mark.parametrize("name", ("unit_c4", "unit_c128", "short_c4", "mixed_c128"))
def test_float64_attention_reproduces_reference(name):
    case, ori_scale, cmp_scale, z = load_case(name)
    out, lse = oracle.attention_float64(case, ori_scale, cmp_scale)
    assert torch.equal(out, torch.from_numpy(z["out_fp64"]))
    assert torch.equal(lse, torch.from_numpy(z["lse_fp64"]))


@pytest.mark.parametrize("name", ("unit_c4", "unit_c128", "real_c4", "real_c128"))
def test_integer_oracle_close_to_float64(name):
    # reference tests/unit/test_reference.py:59-71: relative L2 < 0.01, LSE within 2e-4
    case, ori_scale, cmp_scale, z = load_case(name)
    out, lse = oracle.attention_tiled(case, ori_scale, cmp_scale, return_lse=True)
    expected = torch.from_numpy(z["out_fp64"])
    assert float((out.float() - expected).norm() / expected.norm()) < 0.01
    torch.testing.assert_close(lse, torch.from_numpy(z["lse_fp64"]), rtol=2e-4, atol=2e-4)


def test_padding_indices_do_not_contribute():
    # reference tests/unit/test_reference.py:74-82
    case, ori_scale, cmp_scale, _ = load_case("unit_c4")
    expected = oracle.attention_tiled(case, ori_scale, cmp_scale)
    indices = case.cmp_indices.clone()
    indices[indices < 0] = 2 ** 30
    case.cmp_indices = indices
    assert torch.equal(oracle.attention_tiled(case, ori_scale, cmp_scale), expected)


def test_trace_is_consistent_with_outputs():
    case, ori_scale, cmp_scale, _ = load_case("short_c4")
    trace = oracle.Trace()
    oracle.attention_tiled(case, ori_scale, cmp_scale, trace=trace)
    assert len(trace.tiles) and len(trace.q_codes) == 2 * case.q.shape[0]
    for tile in trace.tiles[:8]:
        alpha, hi, lo = trace.q_codes[(tile.token, tile.kind)]
        qk_hi, qk_lo, pv_hi, pv_lo = oracle.accumulate_from_codes(tile.kv, hi, lo, tile.p_hi, tile.p_lo)
        assert torch.equal(qk_hi, tile.qk_hi) and torch.equal(qk_lo, tile.qk_lo)
        assert torch.equal(pv_hi, tile.pv_hi) and torch.equal(pv_lo, tile.pv_lo)
        assert int(hi.abs().max()) <= 127 and int(lo.abs().max()) <= 64


def test_kv_row_accounting():
    case, *_ = load_case("config0_c4")
    assert oracle.kv_rows_attended(case) == 2 * 1152          # 1024 selected + 128 window rows per query
    case, *_ = load_case("mixed_c128")
    # windows: 100, 129 (two tokens share 127 rows), 128, 128; compressed: 0, 128, 312, 1
    assert oracle.kv_rows_attended(case) == (100 + 129 + 128 + 128) + (0 + 16500 // 128 + 40000 // 128 + 1)
