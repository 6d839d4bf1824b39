"""Cache writer on the GPU, through the C ABI, against the oracle: INT8 codes bit-exact."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import GOLDEN, PAGE_STRIDE, bf16

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def writer(*args):
    from npu_sparse_attn_sharedkv_int8.cache import PreparedCacheWrite
    return PreparedCacheWrite(*args)


def lognormal_rows(count, seed):
    g = torch.Generator().manual_seed(seed)
    sigma = torch.exp(torch.randn(512, generator=g) * 0.5)
    return (torch.randn(count, 512, generator=g) * sigma).bfloat16()


def test_golden_rows_and_ties():
    z = np.load(GOLDEN / "writer.npz")
    for rows, inv, codes in ((bf16(z["rows"]), torch.from_numpy(z["inverse_scale"]), torch.from_numpy(z["codes"])),
                             (bf16(z["tie_rows"]), torch.ones(512), torch.from_numpy(z["tie_codes"]))):
        pages = (rows.shape[0] + 31) // 32
        cache = torch.zeros(pages, 32, 1, 512, dtype=torch.int8, device=DEVICE)
        slots = torch.arange(rows.shape[0], dtype=torch.int32, device=DEVICE)
        writer(cache, rows.to(DEVICE), slots, inv.to(DEVICE)).run()
        torch.cuda.synchronize()
        assert torch.equal(cache.cpu().reshape(-1, 512)[:rows.shape[0]], codes)


def test_reference_example_four_slots_two_pages():
    # reference examples/cache_write.py:17-24
    from npu_sparse_attn_sharedkv_int8 import CacheQuantization
    values = torch.linspace(-1, 1, 4 * 512).reshape(4, 512).bfloat16()
    quantizer = CacheQuantization.calibrate([values])
    cache = torch.zeros((2, 32, 1, 512), dtype=torch.int8, device=DEVICE)
    slots = torch.tensor([0, 31, 32, 63], dtype=torch.int32, device=DEVICE)
    writer(cache, values.to(DEVICE), slots, quantizer.inverse_scale.to(DEVICE)).run()
    torch.cuda.synchronize()
    actual = cache.reshape(-1, 512)[slots.long()].cpu()
    assert torch.equal(actual, oracle.quantize_rows(values, oracle.inverse_scale(quantizer.scale)))


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("paired", [False, True])
@pytest.mark.parametrize("stride,offset", [(16384, 0), (PAGE_STRIDE, 16384), (16384 + 16, 48)])
def test_scatter_forms_strides_and_skips(dtype, paired, stride, offset):
    pages, rows = 40, 700
    g = torch.Generator().manual_seed(pages + rows + paired)
    updates = lognormal_rows(rows, 21)
    scale = (updates.float().abs().amax(0) * 1.1 / 127).clamp_min(1e-8)
    inv = oracle.inverse_scale(scale)
    flat = torch.randperm(pages * 32, generator=g)[:rows]
    flat[::17] = -1
    flat[5::29] = pages * 32 + torch.arange(len(flat[5::29]))          # past the last page: skipped
    slots = torch.stack((torch.div(flat, 32, rounding_mode="floor"), flat % 32), 1) if paired else flat
    if paired:
        slots[flat < 0] = torch.tensor([-1, 0])
        slots[7::31, 1] = 32                                            # offset outside the page: skipped
    slots = slots.to(dtype)
    raw = torch.full((pages * stride + offset + 64,), 77, dtype=torch.int8, device=DEVICE)
    view = raw[offset:].as_strided((pages, 32, 1, 512), (stride, 512, 512, 1))
    expected_raw = raw.cpu().clone()
    expected = expected_raw[offset:].as_strided((pages, 32, 1, 512), (stride, 512, 512, 1))
    oracle.write_cache(expected, updates, slots, inv)
    writer(view, updates.to(DEVICE), slots.to(DEVICE), inv.to(DEVICE)).run()
    torch.cuda.synchronize()
    assert torch.equal(raw.cpu(), expected_raw)          # payload exact, and nothing outside the rows touched


def test_unaligned_rows_take_the_scalar_path():
    rows = 130
    backing = torch.zeros(rows * 520 + 3, dtype=torch.bfloat16, device=DEVICE)
    updates = backing[3:].as_strided((rows, 512), (520, 1))           # rows start on odd 2-byte offsets
    source = lognormal_rows(rows, 5)
    updates.copy_(source.to(DEVICE))
    inv = oracle.inverse_scale((source.float().abs().amax(0) / 127).clamp_min(1e-8))
    cache = torch.zeros(5, 32, 1, 512, dtype=torch.int8, device=DEVICE)
    slots = torch.arange(rows, dtype=torch.int64, device=DEVICE)
    writer(cache, updates, slots, inv.to(DEVICE)).run()
    torch.cuda.synchronize()
    assert torch.equal(cache.cpu().reshape(-1, 512)[:rows], oracle.quantize_rows(source, inv))


def test_rebinding_with_varying_row_counts():
    # reference tests/npu/test_queue.py:58-74
    cache = torch.zeros((4, 32, 1, 512), dtype=torch.int8, device=DEVICE)
    updates = torch.zeros((1, 1, 512), dtype=torch.bfloat16, device=DEVICE)
    slots = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    inverse = torch.full((512,), 10.0, device=DEVICE)
    op = writer(cache, updates, slots, inverse)
    expected = torch.zeros((128, 512), dtype=torch.int8)
    for index in range(32):
        count = index % 3 + 1
        value = (index % 19 - 9) / 10
        updates = torch.full((count, 1, 512), value, dtype=torch.bfloat16, device=DEVICE)
        slots = torch.arange(index * 3, index * 3 + count, dtype=torch.int32, device=DEVICE)
        op._rebind_same_geometry(cache, updates, slots)
        op.run()
        expected[index * 3:index * 3 + count] = (torch.tensor(value).bfloat16().float() * 10).round().to(torch.int8)
        op.updates = op.slots = None
    torch.cuda.synchronize()
    assert torch.equal(cache.cpu().view(128, 512), expected)


@pytest.mark.parametrize("rows,ratio", [(65536, 1), (16384, 4)])
def test_writer_workload_size_round_trip(rows, ratio):
    """65 536 rows into the original cache and 16 384 into the ratio-4 compressed cache through a
    random slot mapping: codes equal the oracle's on a sample, every row lands exactly once
    (checksum of checksums), and dequantized values stay within half a quantization step."""
    updates = lognormal_rows(rows, 31 + ratio)
    scale = (updates.float().abs().amax(0) * 1.1 / 127).clamp_min(1e-8)
    inv = oracle.inverse_scale(scale)
    pages = rows // 32 + 64
    g = torch.Generator().manual_seed(rows)
    slots = torch.randperm(pages * 32, generator=g)[:rows].to(torch.int32)
    cache = torch.zeros(pages, 32, 1, 512, dtype=torch.int8, device=DEVICE)
    writer(cache, updates.to(DEVICE), slots.to(DEVICE), inv.to(DEVICE)).run()
    torch.cuda.synchronize()
    landed = cache.cpu().reshape(-1, 512)[slots.long()]
    sample = torch.randperm(rows, generator=g)[:4096]
    assert torch.equal(landed[sample], oracle.quantize_rows(updates[sample], inv))
    assert int(landed.long().sum()) == int(cache.long().sum())              # nothing written elsewhere
    error = (landed.float() * scale - updates.float()).abs()
    assert bool((error <= scale * 0.5 + 1e-6).all())


def test_contract_violations_raise_value_error():
    cache = torch.zeros(2, 32, 1, 512, dtype=torch.int8, device=DEVICE)
    rows = torch.zeros(4, 512, dtype=torch.bfloat16, device=DEVICE)
    slots = torch.zeros(4, dtype=torch.int32, device=DEVICE)
    inv = torch.ones(512, device=DEVICE)
    with pytest.raises(ValueError):
        writer(cache.cpu(), rows.cpu(), slots.cpu(), inv.cpu())
    with pytest.raises(ValueError):
        writer(cache, rows.float(), slots, inv)
    with pytest.raises(ValueError):
        writer(cache, rows, slots[:3], inv)
    with pytest.raises(ValueError):
        writer(cache, rows, slots.float(), inv)
    with pytest.raises(ValueError):
        writer(cache, rows, slots, inv[:256])
    with pytest.raises(ValueError):
        writer(cache.view(2, 32, 512), rows, slots, inv)
