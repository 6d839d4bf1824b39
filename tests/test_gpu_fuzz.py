"""Randomised geometries against the CPU oracle: ragged batches, one to four query tokens per
request, contexts from one token to several thousand, top-k widths that are not tile multiples,
selections with holes / out-of-range entries / duplicates, page strides that do and do not allow
the TMA row gather.  Acceptance band: max-abs 2e-2, mean-abs 2e-3 on BF16 output; LSE 1e-4."""
from dataclasses import replace
import math

import pytest
import torch

from oracle import sharedkv_oracle as oracle
from tests.support import error_metrics, strided_pages

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def random_case(seed, force_topk=None, min_length=0):
    from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, make_case
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda options: options[int(torch.randint(len(options), (1,), generator=g))]
    ratio = 4 if force_topk else pick((4, 128))
    batch = int(torch.randint(1, 7, (1,), generator=g))
    queries = [int(torch.randint(1, 5, (1,), generator=g)) for _ in range(batch)]
    top = pick((9000, 600, 40)) if ratio == 4 else pick((40000, 9000, 300))
    lengths = [max(q, int(math.exp(float(torch.rand(1, generator=g)) * math.log(top)))) for q in queries]
    lengths = [max(v, min_length) for v in lengths]
    if seed % 5 == 0 and not min_length:
        lengths[0] = queries[0]                                  # a request that consists of its query tokens only
    topk = force_topk or (pick((1024, 1000, 256, 64)) if ratio == 4 else 1024)
    source = make_case(query_lengths=tuple(queries), seq_lens=tuple(lengths), heads=8, ratio=ratio, topk=topk, seed=seed)
    oq, cq = CacheQuantization.calibrate([source.ori]), CacheQuantization.calibrate([source.cmp])
    case = replace(source, ori=oq.quantize(source.ori), cmp=cq.quantize(source.cmp))
    if ratio == 4:
        idx = case.cmp_indices.clone()
        style = seed % 4
        if style == 1:
            idx[:, :, ::5] = -1
        elif style == 2:
            idx[:, :, 3::7] = 2 ** 30
            idx[:, :, 1::9] = idx[:, :, 0::9][:, :, :idx[:, :, 1::9].shape[-1]]
        elif style == 3:
            idx = idx[:, :, torch.randperm(idx.shape[-1], generator=g)]
        case = replace(case, cmp_indices=idx.contiguous())
    stride = pick((16384, 622592, 16384 + 512, 16384 + 48))
    return case, oq.scale, cq.scale, stride, (16 if stride % 512 else 1024)


@pytest.mark.parametrize("seed,topk", [(s, None) for s in range(24)] + [(30, 1000), (31, 64), (32, 130), (33, 1), (34, 1023), (35, -1000), (36, -200), (37, -129)])
def test_random_geometry(seed, topk):
    from npu_sparse_attn_sharedkv_int8.attention import PreparedAttention
    # a negative width asks for contexts long enough that the selection is not packed (holes keep their slots)
    case, ori_scale, cmp_scale, stride, offset = random_case(seed, abs(topk) if topk else None, 4200 if topk and topk < 0 else 0)
    dev = case.to(DEVICE)
    dev = replace(dev, ori=strided_pages(case.ori, DEVICE, stride, offset), cmp=strided_pages(case.cmp, DEVICE, stride, offset))
    op = PreparedAttention(dev, ori_scale.to(DEVICE), cmp_scale.to(DEVICE), return_lse=True)
    out = op.run()
    torch.cuda.synchronize()
    expected, expected_lse = oracle.attention_tiled(case, ori_scale, cmp_scale, return_lse=True)
    m = error_metrics(out.cpu().float(), expected.float())
    assert m["max_abs"] <= 2e-2 and m["mean_abs"] <= 2e-3, (seed, m)
    torch.testing.assert_close(op.lse.cpu(), expected_lse, rtol=1e-4, atol=1e-4)
