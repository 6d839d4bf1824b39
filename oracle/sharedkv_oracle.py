"""CPU oracle for the INT8 shared-KV path.  TEST INFRASTRUCTURE ONLY.

This module restates, in independent code, the arithmetic of the reference
project's CPU path (file paths are relative to the reference checkout):

* frozen-scale cache quantization        npu_sparse_attn_sharedkv_int8/reference.py:48-56
* writer slot rules                      csrc/kernels/cache_write.cpp:51-65
* row selection (window + compressed)    npu_sparse_attn_sharedkv_int8/reference.py:224-253
* query dual-residual encode             npu_sparse_attn_sharedkv_int8/reference.py:274-279
* tiled online softmax with P residuals  npu_sparse_attn_sharedkv_int8/reference.py:268-322
* single-softmax ("joint") row           npu_sparse_attn_sharedkv_int8/reference.py:175-207
* FP64 float attention                   npu_sparse_attn_sharedkv_int8/reference.py:129-139

It is the checker used by the tests, by the smoke entry and by the timed CPU
baseline of the benchmark.  Nothing on the product path may import it.

Parity pin: `tests/golden/*.npz` hold inputs and outputs produced by the
reference's own `tiled_quantized_reference`, `sharedkv_reference`,
`joint_quantized_row` and `CacheQuantization.quantize`; `tests/test_oracle.py`
requires this restatement to reproduce them bit for bit (FP32/BF16 outputs
compared with `torch.equal`), together with the known-answer vectors of the
reference's unit tests (tests/unit/test_reference.py:22-27, :50-56, :74-82).

Besides the outputs, the tiled oracle can record every intermediate the CUDA
kernel can be asked to dump (query codes, INT32 QK accumulators, P codes,
INT32 PV accumulators) so that integer stages are compared exactly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
import math

import torch

DIM = 512
INV127 = 1.0 / 127          # a Python double; torch multiplies FP32 tensors by float32(INV127)
MASKED = -1e30


# --------------------------------------------------------------------------- cache codes

def inverse_scale(scale: torch.Tensor) -> torch.Tensor:
    """FP32(1 / FP64(scale))   (reference.py:48-50)."""
    return scale.double().reciprocal().float()


def quantize_rows(rows: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    """round-half-even(FP32(x) * inv) clamped to +-127 as INT8   (reference.py:52-53)."""
    return torch.round(rows.float() * inv).clamp(-127, 127).to(torch.int8)


def dequantize_rows(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return codes.float() * scale


def write_cache(cache: torch.Tensor, updates: torch.Tensor, slots: torch.Tensor,
                inv: torch.Tensor) -> torch.Tensor:
    """Scatter quantized rows into cache[pages, page_size, 1, 512] (any page stride).

    Slot rules of the device writer (cache_write.cpp:53-63): a negative first
    component skips the row; flat slots split as page = slot // page_size,
    offset = slot % page_size; rows whose page >= pages or whose offset is
    outside [0, page_size) are skipped.
    """
    pages, page_size = cache.shape[0], cache.shape[1]
    codes = quantize_rows(updates.reshape(updates.shape[0], DIM), inv)
    slots = slots.long()
    for row in range(updates.shape[0]):
        if slots.ndim == 2:
            page, offset = int(slots[row, 0]), int(slots[row, 1])
            if page < 0:
                continue
        else:
            first = int(slots[row])
            if first < 0:
                continue
            page, offset = first // page_size, first % page_size
        if page >= pages or offset < 0 or offset >= page_size:
            continue
        cache[page, offset, 0, :] = codes[row]
    return cache


# --------------------------------------------------------------------------- selection

def _paged_rows(cache, table, batch, logical):
    block = cache.shape[1]
    pages = table[batch, logical // block].long()
    return cache[pages, logical % block, 0, :]


def _slot_rows(cache, slots):
    """Rows named by physical slot, no block-table lookup   (reference.py:88-90)."""
    block = cache.shape[1]
    return cache[slots // block, slots % block, 0, :]


@dataclass
class Selection:
    """What one query token attends to (before tiling)."""
    token: int
    batch: int
    position: int
    ori_index: torch.Tensor          # logical original rows, ascending; or the caller's physical slots, in list order
    cmp_index: torch.Tensor | None   # logical compressed rows in slot order (may hold invalid entries)
    cmp_valid: torch.Tensor | None   # which cmp_index entries take part
    ori_valid: torch.Tensor | None = None   # which ori_index entries take part
    ori_explicit: bool = False       # ori_index holds physical slots
    cmp_bias: torch.Tensor | None = None    # log(multiplicity) per cmp_index entry (grouped C4 only)


def select(case, batch: int, token: int, query_group: int = 1) -> Selection:
    """Row selection of reference.py:224-253: the window, or the caller's own physical slots of the
    original cache (:235-239; holes keep their place and are masked).

    With query_group > 1 (:229-234, 243-249) adjacent query tokens of a request share their tiles:
    the original rows are the union of the group's windows, tiled from the union's first row, with the
    token's own window as validity; a C128 token walks the prefix of the group's last token; a C4
    token walks ALL compressed rows of the group's last token, each weighted by how often its own
    top-k list names it (a bias of log(multiplicity) on the logit), rows it does not name masked."""
    first, last = int(case.cu_q[batch]), int(case.cu_q[batch + 1])
    length = int(case.seq_lens[batch])
    position = length - last + token
    group_first = first + (token - first) // query_group * query_group
    group_last = min(last, group_first + query_group) - 1
    first_pos, last_pos = length - last + group_first, length - last + group_last
    explicit = getattr(case, "ori_indices", None) is not None
    if explicit:
        if query_group != 1:
            raise ValueError("Explicit original slots require ungrouped queries")
        ori = case.ori_indices[token, 0].long()
        ori_valid = (ori >= 0) & (ori < case.ori.shape[0] * case.ori.shape[1])
    else:
        ori = torch.arange(max(0, first_pos + 1 - case.window), last_pos + 1)
        ori_valid = (ori >= max(0, position + 1 - case.window)) & (ori <= position)
    cmp_index = cmp_valid = cmp_bias = None
    if case.ratio != 1:
        count = (position + 1) // case.ratio
        if case.ratio == 4:
            cmp_index = case.cmp_indices[token, 0].long()
        else:
            cmp_index = torch.arange((last_pos + 1) // case.ratio)
        cmp_valid = (cmp_index >= 0) & (cmp_index < count)
        if case.ratio == 4 and query_group > 1:
            multiplicity = torch.bincount(cmp_index[cmp_valid], minlength=(last_pos + 1) // 4).float()
            cmp_index = torch.arange(multiplicity.numel())
            cmp_valid = multiplicity > 0
            cmp_bias = multiplicity.clamp_min(1).log()
        elif case.ratio == 4 and count < cmp_index.numel() <= 1024:
            # short contexts: the valid entries are packed to the front, order kept
            cmp_index = cmp_index[cmp_valid]
            cmp_valid = torch.ones_like(cmp_index, dtype=torch.bool)
    return Selection(token, batch, position, ori, cmp_index, cmp_valid, ori_valid, explicit, cmp_bias)


def tokens_of(case):
    for batch in range(case.seq_lens.numel()):
        for token in range(int(case.cu_q[batch]), int(case.cu_q[batch + 1])):
            yield batch, token


# --------------------------------------------------------------------------- query encode

def encode_query(q_row: torch.Tensor, scale: torch.Tensor):
    """Fold the cache scale into Q and split it into two INT8 code planes.

    Returns (alpha[H], hi[H,512] int32, lo[H,512] int32)   (reference.py:274-279).
    """
    folded = q_row.float() * scale
    alpha = (folded.abs().amax(-1) * INV127).clamp_min(1e-12)
    normalized = (folded * alpha.reciprocal()[:, None]).clamp(-127, 127)
    hi = normalized.round().int()
    lo = ((normalized - hi.float()) * 127).round().int()
    return alpha, hi, lo


def encode_weights(weights: torch.Tensor):
    """P dual-residual codes: hi = rint(127 w), lo = rint((127 w - hi) 127)   (reference.py:309-312)."""
    hi = (weights * 127).round().int()
    lo = ((weights * 127 - hi.float()) * 127).round().int()
    return hi, lo


# --------------------------------------------------------------------------- tiled attention

@dataclass
class TileTrace:
    token: int
    kind: int            # 0 original window, 1 compressed
    tile: int            # tile number within the kind
    part: int            # split the tile was dealt to
    rows: int            # slots in the tile (<= tile_size)
    keep: torch.Tensor   # bool[rows]
    kv: torch.Tensor     # int32[rows,512]; invalid rows are zero
    qk_hi: torch.Tensor  # int32[H,rows]
    qk_lo: torch.Tensor
    logits: torch.Tensor
    p_hi: torch.Tensor   # int32[H,rows]
    p_lo: torch.Tensor
    pv_hi: torch.Tensor  # int32[H,512]
    pv_lo: torch.Tensor


@dataclass
class Trace:
    q_codes: dict = field(default_factory=dict)   # (token, kind) -> (alpha, hi, lo)
    tiles: list = field(default_factory=list)


def attention_tiled(case, ori_scale, cmp_scale=None, *, tile_size=128, splits=1, query_group=1,
                    return_lse=False, trace: Trace | None = None, tile_parts=None, only_tokens=None):
    """Online-softmax INT8 attention, tile by tile   (reference.py:210-323).

    Tiles are numbered original-first then compressed and dealt round-robin
    to `splits` partial states; every state starts at max = sink, and only
    state 0 starts with the sink's unit in its denominator.

    `tile_parts` (token -> list of state numbers, one per tile) replaces the
    round-robin deal by an explicit one, so that the oracle can follow a device
    that cuts a token's tiles into contiguous pieces; tiles beyond the list go to
    the last state named.  The merge formula is the same.

    `only_tokens` (a collection of query token numbers) restricts the walk to those tokens, in
    increasing order; the results then have one row per listed token (sampling a large launch).
    """
    heads = case.q.shape[1]
    outputs, lses = [], []
    wanted = None if only_tokens is None else set(int(t) for t in only_tokens)
    for batch, token in tokens_of(case):
        if wanted is not None and token not in wanted:
            continue
        sel = select(case, batch, token, query_group)
        groups = [(case.ori, case.ori_block_table, sel.ori_index, sel.ori_valid, ori_scale)]
        if case.ratio != 1:
            groups.append((case.cmp, case.cmp_block_table, sel.cmp_index, sel.cmp_valid, cmp_scale))
        deal = tile_parts[token] if tile_parts is not None else None
        if deal is not None:
            splits = max(deal) + 1
        maximum = case.sink.repeat(splits, 1)
        denominator = torch.zeros(splits, heads)
        denominator[0].fill_(1)
        numerator = torch.zeros(splits, heads, DIM)
        tile_number = 0
        for kind, (cache, table, index, valid, scale) in enumerate(groups):
            alpha, q_hi, q_lo = encode_query(case.q[token], scale)
            if trace is not None:
                trace.q_codes[(token, kind)] = (alpha, q_hi, q_lo)
            for start in range(0, index.numel(), tile_size):
                part = tile_number % splits if deal is None else deal[min(tile_number, len(deal) - 1)]
                tile_number += 1
                ix, keep = index[start:start + tile_size], valid[start:start + tile_size]
                kv = torch.zeros((ix.numel(), DIM), dtype=torch.int32)
                kv[keep] = (_slot_rows(cache, ix[keep]) if kind == 0 and sel.ori_explicit
                            else _paged_rows(cache, table, batch, ix[keep])).int()
                qk_hi, qk_lo = q_hi @ kv.T, q_lo @ kv.T
                dots = qk_hi.float()
                dots += qk_lo.float() * INV127
                logits = dots * (alpha[:, None] * case.softmax_scale)
                if kind == 1 and sel.cmp_bias is not None:
                    logits += sel.cmp_bias[ix]                      # duplicate selections count as often as they are named
                logits[:, ~keep] = MASKED
                new_max = torch.maximum(maximum[part], logits.amax(-1))
                rescale = torch.exp(maximum[part] - new_max)
                weights = torch.exp(logits - new_max[:, None])
                denominator[part] = denominator[part] * rescale + weights.sum(-1)
                p_hi, p_lo = encode_weights(weights)
                pv_hi, pv_lo = p_hi @ kv, p_lo @ kv
                dots = pv_hi.float()
                dots += pv_lo.float() * INV127
                pv = dots * scale * INV127
                numerator[part] = numerator[part] * rescale[:, None] + pv
                maximum[part] = new_max
                if trace is not None:
                    trace.tiles.append(TileTrace(token, kind, start // tile_size, part, ix.numel(), keep.clone(),
                                                 kv, qk_hi, qk_lo, logits.clone(), p_hi, p_lo, pv_hi, pv_lo))
        top = maximum.amax(0)
        factors = torch.exp(maximum - top)
        num = (numerator * factors[:, :, None]).sum(0)
        den = (denominator * factors).sum(0)
        outputs.append((num / den[:, None]).bfloat16())
        lses.append(top + den.log())
    out = torch.stack(outputs) if outputs else torch.empty((0, heads, DIM), dtype=torch.bfloat16)
    if return_lse:
        return out, (torch.stack(lses) if lses else torch.empty((0, heads)))
    return out


def accumulate_from_codes(kv: torch.Tensor, q_hi, q_lo, p_hi, p_lo):
    """Exact INT32 products for codes produced elsewhere (for example dumped by the
    CUDA kernel): returns (qk_hi, qk_lo, pv_hi, pv_lo)."""
    kv = kv.int()
    return q_hi.int() @ kv.T, q_lo.int() @ kv.T, p_hi.int() @ kv, p_lo.int() @ kv


# --------------------------------------------------------------------------- joint row / float

def attention_joint_row(q_row, caches, scales, sink, softmax_scale):
    """One softmax over both cache kinds   (reference.py:175-207, without logit biases)."""
    logits = []
    for kv, scale in zip(caches, scales):
        alpha, hi, lo = encode_query(q_row, scale)
        dot = (hi @ kv.int().T).float() + (lo @ kv.int().T).float() * INV127
        logits.append(dot * (alpha[:, None] * softmax_scale))
    scores = torch.cat(logits, dim=-1)
    top = torch.maximum(scores.amax(-1), sink)
    weights = torch.exp(scores - top[:, None])
    den = torch.exp(sink - top) + weights.sum(-1)
    p_hi, p_lo = encode_weights(weights)
    out = torch.zeros(q_row.shape[0], DIM)
    offset = 0
    for kv, scale in zip(caches, scales):
        end = offset + len(kv)
        dot = (p_hi[:, offset:end] @ kv.int()).float()
        dot += (p_lo[:, offset:end] @ kv.int()).float() * INV127
        out += dot * (scale * INV127)
        offset = end
    return (out / den[:, None]).bfloat16(), top + den.log()


def attention_float64(case, ori_scale=None, cmp_scale=None):
    """FP64 softmax attention over the selected rows with the sink in the denominator
    (reference.py:129-139).  With scales given, INT8 caches are first dequantized in FP32 (code * scale), as
    the reference's tests do (tests/unit/test_reference.py:64-66)."""
    outputs, lses = [], []
    for batch, token in tokens_of(case):
        first, last = int(case.cu_q[batch]), int(case.cu_q[batch + 1])
        position = int(case.seq_lens[batch]) - last + token
        if getattr(case, "ori_indices", None) is not None:
            slots = case.ori_indices[token, 0].long()
            rows = _slot_rows(case.ori, slots[(slots >= 0) & (slots < case.ori.shape[0] * case.ori.shape[1])])
        else:
            ori_ix = torch.arange(max(0, position - case.window + 1), position + 1)
            rows = _paged_rows(case.ori, case.ori_block_table, batch, ori_ix)
        rows = (dequantize_rows(rows, ori_scale) if ori_scale is not None else rows).double()
        if case.ratio != 1:
            count = (position + 1) // case.ratio
            if case.ratio == 4 and case.cmp_indices is not None:
                ix = case.cmp_indices[token, 0].long()
                ix = ix[(ix >= 0) & (ix < count)]
            else:
                ix = torch.arange(count)
            more = _paged_rows(case.cmp, case.cmp_block_table, batch, ix)
            more = (dequantize_rows(more, cmp_scale) if cmp_scale is not None else more).double()
            rows = torch.cat((rows, more), 0)
        logits = case.q[token].double() @ rows.T * case.softmax_scale
        lse = torch.logsumexp(torch.cat((logits, case.sink.double()[:, None]), -1), -1)
        outputs.append((torch.exp(logits - lse[:, None]) @ rows).float())
        lses.append(lse.float())
    return torch.stack(outputs), torch.stack(lses)


# --------------------------------------------------------------------------- work accounting

def kv_rows_attended(case) -> int:
    """Unique KV rows one launch must fetch: per request the union of its tokens'
    windows plus the compressed rows (C4: valid top-k entries per token; C128: the
    longest prefix any of its tokens sees).  512 bytes each."""
    total = 0
    for batch in range(case.seq_lens.numel()):
        first, last = int(case.cu_q[batch]), int(case.cu_q[batch + 1])
        if last <= first or int(case.seq_lens[batch]) <= 0:
            continue
        length = int(case.seq_lens[batch])
        lo_pos, hi_pos = length - (last - first), length - 1
        total += hi_pos - max(0, lo_pos + 1 - case.window) + 1
        if case.ratio == 128:
            total += (hi_pos + 1) // 128
        elif case.ratio == 4:
            for token in range(first, last):
                count = (length - last + token + 1) // 4
                ix = case.cmp_indices[token, 0]
                total += int(((ix >= 0) & (ix < count)).sum())
    return total
