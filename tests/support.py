"""Helpers shared by the tests: golden cases as tensors, comparison metrics, device staging."""
from dataclasses import replace
from pathlib import Path

import numpy as np
import torch

from npu_sparse_attn_sharedkv_int8.reference import CacheQuantization, SharedKVCase

GOLDEN = Path(__file__).resolve().parent / "golden"
ATTENTION_CASES = ("unit_c4", "unit_c128", "config0_c4", "holes_c4", "short_c4", "mixed_c128", "real_c4", "real_c128")
SLOT_CASES = ("slots_swa", "slots_c4")       # explicit original slots: a ratio-1 layer and a C4 layer
GROUPED_CASES = ("grouped_c128", "grouped_c4", "grouped_c4_short")      # several query tokens per request; outputs for query_group 1, 2 and 4
PAGE_STRIDE = 622592          # the non-unit page stride the reference's device tests use (tests/support/serving_shapes.py:19)


def bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def load_case(name):
    """Returns (case, ori_scale, cmp_scale, arrays) for a golden attention case."""
    z = np.load(GOLDEN / f"{name}.npz")
    t = lambda key: torch.from_numpy(z[key].copy())
    optional = lambda key: t(key) if key in z else None
    case = SharedKVCase(
        q=bf16(z["q"]), ori=t("ori"), ori_block_table=t("ori_table"), cu_q=t("cu_q"), seq_lens=t("seq_lens"),
        sink=t("sink"), cmp=optional("cmp"), cmp_block_table=optional("cmp_table"), cmp_indices=optional("cmp_indices"),
        ratio=int(z["ratio"]), softmax_scale=float(z["softmax_scale"]), ori_indices=optional("ori_indices"))
    return case, t("ori_scale"), optional("cmp_scale"), z


def strided_pages(cache, device, stride=PAGE_STRIDE, offset=0):
    """Copy cache[P,32,1,512] into a backing whose pages are `stride` bytes apart, starting
    `offset` bytes in, and return the strided view (what a compact page allocator hands out)."""
    pages = cache.shape[0]
    raw = torch.zeros(pages * stride + offset, dtype=torch.int8, device=device)
    view = raw[offset:].as_strided(cache.shape, (stride, 512, 512, 1))
    view.copy_(cache.to(device))
    return view


def to_device(case, device, *, stride=None, offset=0):
    dev = case.to(device)
    if stride is not None:
        dev = replace(dev, ori=strided_pages(case.ori, device, stride, offset),
                      cmp=strided_pages(case.cmp, device, stride, offset) if case.cmp is not None else None)
    return dev


def error_metrics(actual, expected):
    a, b = actual.double(), expected.double()
    diff = (a - b).abs()
    return dict(max_abs=float(diff.max()) if diff.numel() else 0.0, mean_abs=float(diff.mean()) if diff.numel() else 0.0,
                rel_l2=float(torch.linalg.vector_norm(a - b) / torch.linalg.vector_norm(b).clamp_min(1e-30)))


def synthetic_scale(rows):
    return CacheQuantization((rows.float().reshape(-1, 512).abs().amax(0) * 1.1 / 127).clamp_min(1e-8))


ITEM_COST = 1                 # the kernel's kItemCost


def device_tile_parts(case, ctas):
    """Which piece each 128-key tile of each token belongs to when the flat tile list of a
    launch is cut into `ctas` contiguous ranges of equal cost (the CUDA kernel's work-split rule): a C4
    token with at least one compressed row has 1 + ceil(topk / 128) tiles, a C128 token
    1 + ceil(rows / 128), a token that sees no compressed row has 1."""
    counts = []
    slots = getattr(case, "ori_indices", None)
    original = -(-slots.shape[-1] // 128) if slots is not None else 1      # explicit slots: one tile per 128 entries
    for batch in range(case.seq_lens.numel()):
        first, last = int(case.cu_q[batch]), int(case.cu_q[batch + 1])
        for token in range(first, last):
            position = int(case.seq_lens[batch]) - last + token
            rows = (position + 1) // case.ratio if position >= 0 else 0
            if case.ratio == 1:
                counts.append(original)
            elif case.ratio == 4:
                counts.append(original + (-(-case.cmp_indices.shape[-1] // 128) if rows else 0))
            else:
                counts.append(original + -(-rows // 128))
    # ranges are cut in units of cost: a token's tiles plus ITEM_COST units in front of its first tile
    total = sum(counts) + ITEM_COST * len(counts)
    quota = max(1, -(-total // ctas))
    parts, start = {}, 0
    for token, n in enumerate(counts):
        start += ITEM_COST
        parts[token] = [(start + j) // quota - start // quota for j in range(n)]
        start += n
    return parts
