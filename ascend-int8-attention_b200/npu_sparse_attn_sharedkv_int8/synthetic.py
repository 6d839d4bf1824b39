"""Seeded synthetic serving workloads for the decode path, resident on one GPU.

The reference measures on private real activations resampled into serving geometries
(tests/support/serving_shapes.py of the reference); none of that data is public, so the
benchmarks and the large parity tests of this build use synthetic state with the same
shapes and value distributions:

* per-channel spread sigma_c = exp(N(0, 0.5^2)), rows ~ N(0, sigma_c^2) in BF16,
  scale = 1.1 * absmax_c / 127 per cache kind, codes produced by the writer kernel;
* block-32 pages; every layer of a cache kind shares block ids and sits at its own
  16 384-byte offset inside a common page stride (the compact page layout of the
  reference's cache_layout.packed_layout), so page strides are non-unit;
* page tables are random permutations of the block pool; only the window pages of the
  original cache are allocated; table rows have full model-capacity width;
* C4 selections: top-k 1024 distinct rows, uniform over the rows a token may see.

Large pools are filled by tiling one block of quantized rows (`PATTERN_ROWS` rows): DRAM
traffic does not depend on the values, and the parity checks compare the kernel with the
CPU oracle on whatever the pool holds.
"""
from dataclasses import dataclass, field
import math

import torch

from .cache import PreparedCacheWrite
from .reference import CacheQuantization, SharedKVCase

PAGE = 32
ROW = 512
PAGE_BYTES = PAGE * ROW
PATTERN_ROWS = 1 << 18          # 128 MiB of INT8 rows


@dataclass
class Layer:
    ratio: int
    ori: torch.Tensor            # INT8 [blocks, 32, 1, 512], strided view
    cmp: torch.Tensor
    ori_scale: torch.Tensor      # FP32 [512] on the device
    cmp_scale: torch.Tensor
    cmp_indices: torch.Tensor | None
    q: torch.Tensor              # BF16 [tokens, 8, 512]


@dataclass
class Workload:
    name: str
    device: torch.device
    queries: int                             # query tokens per request
    seq_lens_host: torch.Tensor              # INT64 [requests]
    cu_q: torch.Tensor
    seq_lens: torch.Tensor
    sink: torch.Tensor
    ori_table: torch.Tensor
    cmp_tables: dict                         # ratio -> INT32 [requests, width]
    layers: list = field(default_factory=list)
    pools: list = field(default_factory=list)   # keeps the backings alive
    kv_bytes_resident: int = 0

    @property
    def requests(self):
        return int(self.seq_lens_host.numel())

    @property
    def tokens(self):
        return self.requests * self.queries

    def case(self, layer_index):
        layer = self.layers[layer_index]
        return SharedKVCase(q=layer.q, ori=layer.ori, ori_block_table=self.ori_table, cu_q=self.cu_q,
                            seq_lens=self.seq_lens, sink=self.sink, cmp=layer.cmp,
                            cmp_block_table=self.cmp_tables[layer.ratio], cmp_indices=layer.cmp_indices,
                            ratio=layer.ratio)

    def kv_rows(self, layer_index):
        """Algorithmic KV rows one launch of this layer reads: per request the union of its
        tokens' windows, plus the compressed rows (C4: top-k per token; C128: the prefix)."""
        ratio = self.layers[layer_index].ratio
        s, t = self.seq_lens_host, self.queries
        window = torch.minimum(s, torch.full_like(s, 127 + t))
        if ratio == 128:
            compressed = s // 128
        else:
            compressed = sum(torch.clamp((s - t + i + 1) // 4, max=1024) for i in range(t))
        return int((window + compressed).sum())


def _pattern(device, seed):
    """One block of quantized rows and its scale, produced by the writer kernel."""
    g = torch.Generator(device=device).manual_seed(seed)
    sigma = torch.exp(torch.randn(ROW, generator=g, device=device) * 0.5)
    chunk = 1 << 15
    codes = torch.empty((PATTERN_ROWS // PAGE, PAGE, 1, ROW), dtype=torch.int8, device=device)
    first = (torch.randn(chunk, ROW, generator=g, device=device) * sigma).bfloat16()
    # absmax over the first chunk with headroom stands in for the calibrated scale of the whole block
    quant = CacheQuantization((first.float().abs().amax(0).cpu() * 1.1 / 127).clamp_min(1e-8))
    inverse = quant.inverse_scale.to(device)
    for start in range(0, PATTERN_ROWS, chunk):
        rows = first if start == 0 else (torch.randn(chunk, ROW, generator=g, device=device) * sigma).bfloat16()
        slots = torch.arange(start, start + chunk, dtype=torch.int32, device=device)
        PreparedCacheWrite(codes, rows, slots, inverse).run()
    torch.cuda.synchronize(device)
    return codes.view(-1), quant.scale.to(device)


def _fill(pool, pattern):
    flat = pool.view(-1)
    step = pattern.numel()
    for start in range(0, flat.numel(), step):
        end = min(flat.numel(), start + step)
        flat[start:end].copy_(pattern[:end - start])


def _table(block_counts, width, generator, device):
    """Random-permutation page table: request b owns block_counts[b] distinct block ids."""
    counts = torch.as_tensor(block_counts, dtype=torch.int64)
    total = int(counts.sum())
    order = torch.randperm(max(total, 1), generator=generator, device=device).to(torch.int32)
    offsets = (torch.cumsum(counts, 0) - counts).to(device)
    columns = torch.arange(width, device=device)
    live = columns[None, :] < counts.to(device)[:, None]
    table = torch.zeros((counts.numel(), width), dtype=torch.int32, device=device)
    table[live] = order[(offsets[:, None] + columns[None, :])[live]]
    return table, max(total, 1)


def build(name, device, seq_lens, *, ratios, queries=1, seed=0, stride_slots=None, slot_offset=0,
          max_context=None):
    """Device-resident state for one decode step over `len(ratios)` attention layers.

    seq_lens       context length of every request (host integers), query tokens included
    ratios         compression ratio of each layer, e.g. [4, 128, 4, 128, ...]
    stride_slots   16 384-byte slots per physical block in each pool (>= layers of the kind);
                   the default packs exactly the layers of a kind into a block
    slot_offset    first slot used by the layers (a non-zero payload offset inside the block)
    """
    device = torch.device(device)
    s = torch.as_tensor(seq_lens, dtype=torch.int64)
    requests, t = s.numel(), queries
    g = torch.Generator(device=device).manual_seed(seed)
    capacity = max_context or int(s.max())
    pattern, scale = _pattern(device, seed + 1)
    work = Workload(name=name, device=device, queries=t, seq_lens_host=s,
                    cu_q=torch.arange(0, requests * t + 1, t, dtype=torch.int32, device=device),
                    seq_lens=s.to(torch.int32).to(device), sink=torch.linspace(-2, 2, 8, device=device),
                    ori_table=None, cmp_tables={})

    def pool(blocks, layers_of_kind):
        slots = max(stride_slots or 0, layers_of_kind + slot_offset)
        backing = torch.empty((blocks, slots * PAGE_BYTES), dtype=torch.int8, device=device)
        _fill(backing, pattern)
        work.pools.append(backing)
        work.kv_bytes_resident += backing.numel()
        return backing, slots

    def view(backing, slots, index):
        blocks = backing.shape[0]
        return backing.view(-1)[(slot_offset + index) * PAGE_BYTES:].as_strided(
            (blocks, PAGE, 1, ROW), (slots * PAGE_BYTES, ROW, ROW, 1))

    # original cache: only the pages the window (and this step's queries) can touch
    first_page = torch.clamp(s - t - 127, min=0) // PAGE
    last_page = (s - 1) // PAGE
    ori_counts = last_page - first_page + 1
    width = math.ceil(capacity / PAGE)
    ori_ids, ori_blocks = _table(ori_counts, int(ori_counts.max()), g, device)
    work.ori_table = torch.zeros((requests, width), dtype=torch.int32, device=device)
    columns = torch.arange(int(ori_counts.max()), device=device)
    live = columns[None, :] < ori_counts.to(device)[:, None]
    target = first_page.to(device)[:, None] + columns[None, :]
    work.ori_table[torch.arange(requests, device=device)[:, None].expand_as(target)[live], target[live]] = ori_ids[live]
    ori_pool, ori_slots = pool(ori_blocks, len(ratios))

    pools = {}
    for ratio in sorted(set(ratios)):
        rows = s // ratio
        counts = torch.clamp((rows + PAGE - 1) // PAGE, min=1)
        table_width = max(1, math.ceil(capacity / (ratio * PAGE)))
        work.cmp_tables[ratio], blocks = _table(counts, table_width, g, device)
        pools[ratio] = pool(blocks, sum(1 for r in ratios if r == ratio))

    used = {ratio: 0 for ratio in pools}
    for index, ratio in enumerate(ratios):
        backing, slots = pools[ratio]
        cmp = view(backing, slots, used[ratio])
        used[ratio] += 1
        indices = None
        if ratio == 4:
            indices = torch.full((requests * t, 1, 1024), -1, dtype=torch.int32, device=device)
            for b in range(requests):
                for local in range(t):
                    count = int(s[b] - t + local + 1) // 4
                    if count <= 0:
                        continue
                    chosen = torch.randperm(count, generator=g, device=device)[:1024]
                    indices[b * t + local, 0, :chosen.numel()] = chosen.to(torch.int32)
        q = torch.randn((requests * t, 8, ROW), generator=g, device=device).bfloat16()
        work.layers.append(Layer(ratio, view(ori_pool, ori_slots, index), cmp, scale, scale, indices, q))
    torch.cuda.synchronize(device)
    return work


def extract_requests(work, layer_index, requests):
    """CPU copy of what `requests` need from one layer, as an equivalent small case.

    Attention depends on the selected rows and their slot order, not on absolute positions
    (rotary embedding is applied before the cache), so every C4 request is re-based to a
    context whose compressed cache holds exactly its selected rows in ascending logical
    order (selections are renumbered by rank), while C128 requests keep their length.
    Returns (case, ori_scale, cmp_scale, token_ids) with token_ids indexing the workload's rows.
    """
    layer = work.layers[layer_index]
    ratio, t = layer.ratio, work.queries
    ori_pages, cmp_pages, ori_rows, cmp_rows, lengths, token_ids, picks = [], [], [], [], [], [], []
    cmp_table = work.cmp_tables[ratio]
    for b in requests:
        length = int(work.seq_lens_host[b])
        tokens = list(range(b * t, b * t + t))
        token_ids.extend(tokens)
        first = max(0, length - t - 127)
        logical = torch.arange(first, length, device=work.device)
        pages = work.ori_table[b, logical // PAGE].long()
        window = layer.ori[pages, logical % PAGE, 0].cpu()
        if ratio == 128:
            count = length // 128
            logical = torch.arange(count, device=work.device)
            pages = cmp_table[b, logical // PAGE].long()
            rows = layer.cmp[pages, logical % PAGE, 0].cpu()
            new_length = length
            selection = None
        elif length < 4096 + t:
            # short context: keep it as it is (the packed / in-place slot rules depend on the row count)
            count = length // 4
            logical = torch.arange(max(count, 1), device=work.device)
            pages = cmp_table[b, logical // PAGE].long()
            rows = layer.cmp[pages, logical % PAGE, 0].cpu()
            new_length = length
            selection = layer.cmp_indices[b * t:b * t + t, 0].cpu()
        else:
            chosen = layer.cmp_indices[b * t:b * t + t, 0].long()
            valid = chosen >= 0
            unique = torch.unique(chosen[valid])
            pages = cmp_table[b, unique // PAGE].long()
            rows = layer.cmp[pages, unique % PAGE, 0].cpu()
            rank = torch.searchsorted(unique, chosen.clamp_min(0))
            selection = torch.where(valid, rank, torch.full_like(rank, -1)).cpu().to(torch.int32)
            # a context long enough that every renumbered row is visible to every token of the request
            new_length = max(4 * int(unique.numel()) + t, 4096 + t)
        lengths.append(new_length)
        ori_rows.append((window, new_length - window.shape[0], new_length))
        cmp_rows.append(rows)
        picks.append(selection)
    batch = len(requests)
    ori_width = math.ceil(max(lengths) / PAGE)
    cmp_width = max(1, math.ceil(max(r.shape[0] for r in cmp_rows) / PAGE))
    ori_table = torch.zeros((batch, ori_width), dtype=torch.int32)
    cmp_table_cpu = torch.zeros((batch, cmp_width), dtype=torch.int32)
    ori_store, cmp_store = [], []
    for i in range(batch):
        window, start, end = ori_rows[i]
        for page in range(start // PAGE, (end - 1) // PAGE + 1):
            block = torch.zeros(PAGE, ROW, dtype=torch.int8)
            lo, hi = max(start, page * PAGE), min(end, (page + 1) * PAGE)
            block[lo - page * PAGE:hi - page * PAGE] = window[lo - start:hi - start]
            ori_table[i, page] = len(ori_store)
            ori_store.append(block)
        rows = cmp_rows[i]
        for page in range(max(1, math.ceil(rows.shape[0] / PAGE))):
            block = torch.zeros(PAGE, ROW, dtype=torch.int8)
            part = rows[page * PAGE:(page + 1) * PAGE]
            block[:part.shape[0]] = part
            cmp_table_cpu[i, page] = len(cmp_store)
            cmp_store.append(block)
    ids = torch.tensor(token_ids)
    case = SharedKVCase(
        q=layer.q[ids.to(work.device)].cpu(), ori=torch.stack(ori_store).view(-1, PAGE, 1, ROW), ori_block_table=ori_table,
        cu_q=torch.arange(0, batch * t + 1, t, dtype=torch.int32), seq_lens=torch.tensor(lengths, dtype=torch.int32),
        sink=work.sink.cpu(), cmp=torch.stack(cmp_store).view(-1, PAGE, 1, ROW), cmp_block_table=cmp_table_cpu,
        cmp_indices=torch.cat(picks).view(-1, 1, 1024) if ratio == 4 else None, ratio=ratio)
    return case, layer.ori_scale.cpu(), layer.cmp_scale.cpu(), ids


def log_uniform_lengths(count, low, high, seed):
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(count, generator=g, dtype=torch.float64)
    return torch.round(torch.exp(math.log(low) + u * (math.log(high) - math.log(low)))).to(torch.int64)


def uniform_lengths(count, low, high, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(low, high + 1, (count,), generator=g, dtype=torch.int64)
