"""Compact page layout: every cache layer of a block lives at a fixed offset inside one common
per-block stride of a single backing allocation.

Mirror of the reference's planner (npu_sparse_attn_sharedkv_int8/cache_layout.py:24-159).  The
planning functions are pure and duck-typed: a *group* is any object with `layer_names` and
`kv_cache_spec.kv_cache_specs` (name -> spec); a *spec* has `dtype`, `page_size_bytes` and, where
they apply, `head_size`, `scale_dim`, `scale_dtype`, `block_size`, `num_kv_heads`,
`max_memory_usage_pages(config)`.  vLLM's own KVCacheGroupSpec / KVCacheSpec objects fit, and so
do plain dataclasses, which is what the tests use.

The views `reshape` returns are what the attention and writer kernels consume:
INT8 [blocks, rows per block, heads, 512] with `stride(0)` = the common stride in bytes, starting
`offset` bytes into the backing.  A stride that is a whole number of 512-byte rows keeps the
decode kernel on its TMA row-gather path.
"""
from dataclasses import dataclass, replace
import logging
import math

import torch

ROW_BYTES = 512
_installed = False


@dataclass(frozen=True)
class BackingTensor:
    """Where one layer's pages sit inside the shared backing (the fields the reference adds to
    its cache-tensor descriptors, cache_layout.py:108-111)."""
    size: int
    layers: tuple
    offset: int
    layer_stride: int
    block_stride: int


def _specs_of(group):
    spec = group.kv_cache_spec
    inner = getattr(spec, "kv_cache_specs", None)
    return inner if inner is not None else {name: spec for name in group.layer_names}


def _element_size(dtype):
    return torch.empty((), dtype=dtype).element_size()


def _round_up(value, multiple):
    return -(-value // multiple) * multiple


def uses_compact(groups):
    """True when any layer is an INT8 D=512 shared-KV cache of a DeepSeek-V4 model
    (cache_layout.py:24-29): the three conditions of the reference, `model_version` included."""
    for group in groups:
        if group is None or getattr(group, "kv_cache_spec", None) is None:
            continue
        for spec in _specs_of(group).values():
            if (spec.dtype == torch.int8 and getattr(spec, "head_size", None) == 512
                    and getattr(spec, "model_version", None) == "deepseek_v4"):
                return True
    return False


def group_specs(grouped_specs, make_group=None):
    """Split over-full state groups so that no group needs more bytes per block than the larger of
    the two attention groups, rounded up to the largest page (cache_layout.py:32-62).  The first
    two groups (C4 with its indexer, C128) are kept whole.  Each input is a mapping-bearing
    object (`.kv_cache_specs`, `.page_size_bytes`); `make_group(names, specs)` builds an output
    group and defaults to a plain (names, specs) pair."""
    make_group = make_group or (lambda names, specs: (list(names), dict(specs)))
    largest = max(spec.page_size_bytes for group in grouped_specs for spec in group.kv_cache_specs.values())
    budget = _round_up(max(grouped_specs[0].page_size_bytes, grouped_specs[1].page_size_bytes), largest)
    result = []
    for group in grouped_specs:
        chunk, used = {}, 0
        for name, spec in group.kv_cache_specs.items():
            # FP32 compressor states need no padding inside a common stride
            if spec.dtype == torch.float32 and getattr(spec, "page_size_padded", None) is not None:
                spec = replace(spec, page_size_padded=None)
            if chunk and used + spec.page_size_bytes > budget:
                result.append(make_group(chunk.keys(), chunk))
                chunk, used = {}, 0
            chunk[name] = spec
            used += spec.page_size_bytes
        if chunk:
            result.append(make_group(chunk.keys(), chunk))
    return result


def packed_layout(groups):
    """(stride, {layer name: byte offset}): within a group the layers are packed largest first,
    each aligned to its element size (and scale element size), INT8 D=512 layers to whole
    512-byte rows; groups overlay each other because a block id belongs to one group at a time;
    the stride is the largest group extent rounded up to 512 bytes (cache_layout.py:65-85)."""
    offsets, extent = {}, 0
    for group in groups:
        specs = _specs_of(group)
        cursor = 0
        for name in sorted(group.layer_names, key=lambda n: -specs[n].page_size_bytes):
            spec = specs[name]
            alignment = _element_size(spec.dtype)
            if getattr(spec, "scale_dim", 0):
                alignment = math.lcm(alignment, _element_size(spec.scale_dtype))
            if spec.dtype == torch.int8 and getattr(spec, "head_size", None) == 512:
                alignment = math.lcm(alignment, ROW_BYTES)
            if name in offsets:
                raise ValueError(f"Cache layer appears in multiple groups: {name}")
            offsets[name] = _round_up(cursor, alignment)
            cursor = offsets[name] + spec.page_size_bytes
        extent = max(extent, cursor)
    return _round_up(extent, ROW_BYTES), offsets


def pool_bytes_per_block(groups):
    return packed_layout(groups)[0]


def max_memory_usage(config, groups):
    """Bytes the pool needs for the model's maximum length (cache_layout.py:92-93)."""
    return pool_bytes_per_block(groups) * sum(group.kv_cache_spec.max_memory_usage_pages(config) for group in groups)


def cache_config(config, groups, available_memory, override_num_blocks=None):
    """(number of blocks, one BackingTensor per layer) for `available_memory` bytes
    (cache_layout.py:96-112).  Pipeline- and context-parallel serving are refused as in the
    reference."""
    parallel = getattr(config, "parallel_config", None)
    for name in ("pipeline_parallel_size", "decode_context_parallel_size", "prefill_context_parallel_size"):
        if getattr(parallel, name, 1) != 1:
            raise ValueError("Compact C8 pages are integrated for single-stage, non-context-parallel serving")
    stride, offsets = packed_layout(groups)
    blocks = available_memory // stride
    if override_num_blocks is not None:
        blocks = override_num_blocks
    size = blocks * stride
    return blocks, [BackingTensor(size=size, layers=(name,), offset=offset, layer_stride=0, block_stride=stride)
                    for name, offset in offsets.items()]


def allocate(groups, num_blocks, descriptors, device, alignment=2 * 1024 * 1024):
    """One INT8 backing for all layers; returns {layer name: backing[offset:]} after checking the
    descriptors against the layout (cache_layout.py:115-137).  The backing starts on an
    `alignment` boundary."""
    stride, offsets = packed_layout(groups)
    size = stride * num_blocks
    seen = {}
    for descriptor in descriptors:
        if (len(descriptor.layers) != 1 or descriptor.layer_stride != 0 or descriptor.block_stride != stride
                or descriptor.size != size):
            raise ValueError("Invalid compact C8 backing descriptor")
        name = descriptor.layers[0]
        if name in seen or descriptor.offset != offsets.get(name):
            raise ValueError("Invalid compact C8 layer offset")
        seen[name] = descriptor.offset
    if set(seen) != set(offsets):
        raise ValueError("Compact C8 descriptor/spec coverage differs")
    raw = torch.zeros(size + alignment, dtype=torch.int8, device=device)
    shift = (-raw.data_ptr()) % alignment
    backing = raw[shift:shift + size]
    logging.getLogger(__name__).info("Compact INT8 sharedKV: %d blocks, %d bytes/block, %d groups, one %d-byte backing",
                                     num_blocks, stride, len(groups), size)
    return {name: backing[offset:] for name, offset in seen.items()}


def page_view(raw, shape, dtype, stride_bytes):
    """View of one layer: `shape` = [blocks, rows, heads, width] of `dtype`, consecutive blocks
    `stride_bytes` apart, rows contiguous inside a block (the role of the runner's
    `_adjust_kv_layout`, cache_layout.py:159)."""
    element = _element_size(dtype)
    if stride_bytes % element or raw.data_ptr() % element:
        raise ValueError("Page stride and offset must be multiples of the element size")
    blocks, rows, heads, width = shape
    if rows * heads * width * element > stride_bytes:
        raise ValueError("A block's payload exceeds the common stride")
    needed = (blocks - 1) * stride_bytes + rows * heads * width * element if blocks else 0
    available = raw.numel() * raw.element_size()
    if available < needed:
        raise ValueError("Backing too small for the requested view")
    typed = raw.view(torch.int8)[:available // element * element].view(dtype)
    return typed.as_strided((blocks, rows, heads, width), (stride_bytes // element, heads * width, width, 1))


def reshape(groups, num_blocks, raw):
    """{layer name: [views]}: the cache view of every layer, followed by its scale view where the
    spec has a `scale_dim` (cache_layout.py:140-166)."""
    stride = pool_bytes_per_block(groups)
    result = {}
    for group in groups:
        specs = _specs_of(group)
        for name in group.layer_names:
            spec = specs[name]
            rows = getattr(spec, "storage_block_size", None) or spec.block_size
            views = [page_view(raw[name], (num_blocks, rows, spec.num_kv_heads, spec.head_size), spec.dtype, stride)]
            if getattr(spec, "scale_dim", 0):
                payload = rows * spec.num_kv_heads * spec.head_size * _element_size(spec.dtype)
                views.append(page_view(raw[name][payload:], (num_blocks, rows, spec.num_kv_heads, spec.scale_dim),
                                       spec.scale_dtype, stride))
            result[name] = views
    if set(result) != {name for group in groups for name in group.layer_names}:
        raise ValueError("Compact C8 runner views do not cover the cache specifications")
    return result


def install(planner=None, runner=None):
    """Hook the planner into a serving stack (cache_layout.py:169-206).  The reference wraps
    vllm-ascend's DeepSeek-V4 planner functions and the NPU model runner; CUDA vLLM has neither,
    so the objects to wrap are passed in: `planner` with `pool_bytes_per_block(groups)` and
    `max_memory_usage(config, groups)` attributes, `runner` (a class) with
    `_allocate_kv_cache_tensors(self, config)`.  Non-compact groups keep the original behaviour."""
    global _installed
    if _installed:
        return
    if planner is None or runner is None:
        raise RuntimeError("No CUDA serving stack exposes the DeepSeek-V4 cache planner hooks this module wraps; "
                           "pass install(planner=..., runner=...) or call the planning functions directly")
    old_pool, old_max = planner.pool_bytes_per_block, planner.max_memory_usage
    old_allocate = runner._allocate_kv_cache_tensors
    planner.pool_bytes_per_block = lambda groups: (
        pool_bytes_per_block(groups) if uses_compact(groups) else old_pool(groups))
    planner.max_memory_usage = lambda config, groups: (
        max_memory_usage(config, groups) if uses_compact(groups) else old_max(config, groups))

    def allocate_hook(self, config):
        if not uses_compact(config.kv_cache_groups):
            return old_allocate(self, config)
        return allocate(config.kv_cache_groups, config.num_blocks, config.kv_cache_tensors, self.device)

    runner._allocate_kv_cache_tensors = allocate_hook
    _installed = True
