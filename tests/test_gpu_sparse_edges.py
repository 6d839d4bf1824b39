"""C4 decode with damaged top-k selections, after the reference's own edge-case test
(tests/npu/test_sparse_edges.py:30-76 of the reference): one query token per request, contexts that
end just behind a tile or page boundary, and selections with duplicates, holes, out-of-range entries,
no entry at all, more entries than the context has rows, and a single entry in the last slot (alone,
or named twice: the key then counts twice).  Acceptance band against the oracle: max-abs 2e-2,
mean-abs 2e-3 on BF16 output, LSE 1e-4.
"""
from dataclasses import replace

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import error_metrics

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"
MODES = ("duplicates", "holes", "empty", "extended_duplicates", "single", "one_key_duplicates", "permutation")


def damaged(indices, mode, batch, length):
    out = torch.full_like(indices, -1)
    rows = length // 4
    extent = min(1024, rows)
    if mode == "duplicates":
        out[:, :, :extent] = torch.arange(extent).div(2, rounding_mode="floor").reshape(1, 1, -1)
    elif mode == "permutation":
        out[:, :, :extent] = torch.randperm(extent, generator=torch.Generator().manual_seed(length)).reshape(1, 1, -1)
    elif mode == "extended_duplicates":
        out[:, :, ::2] = torch.arange(512).remainder(rows).reshape(1, 1, -1)
    elif mode == "holes":
        out[:, :, :extent:3] = torch.arange((extent + 2) // 3).reshape(1, 1, -1)
        out[:, :, 1:extent:7] = rows + 3                                   # beyond the context
    elif mode in ("single", "one_key_duplicates"):
        selected = torch.arange(batch).remainder(rows).reshape(batch, 1).to(out.dtype)
        out[:, :, 1023] = selected
        if mode == "one_key_duplicates":
            out[:, :, 0] = selected
    return out


@pytest.mark.parametrize("batch,length", [(7, 129), (13, 513), (25, 513), (73, 517), (97, 1023), (25, 4 * 513), (33, 4 * 928), (49, 4 * 1025)])
def test_damaged_selections(batch, length):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    source = make_case(query_lengths=(1,) * batch, seq_lens=(length,) * batch, heads=8, ratio=4, topk=1024, seed=batch + length)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    dev = case.to(DEVICE)
    op = PreparedAttention(dev, oq.scale.to(DEVICE), cq.scale.to(DEVICE), return_lse=True)
    for mode in MODES:
        indices = damaged(case.cmp_indices, mode, batch, length)
        dev.cmp_indices.copy_(indices)
        op.out.fill_(float("nan"))
        out = op.run()
        torch.cuda.synchronize()
        expected, expected_lse = oracle.attention_tiled(replace(case, cmp_indices=indices), oq.scale, cq.scale, return_lse=True)
        m = error_metrics(out.cpu().float(), expected.float())
        assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (mode, m)
        torch.testing.assert_close(op.lse.cpu(), expected_lse, rtol=1e-4, atol=1e-4)
