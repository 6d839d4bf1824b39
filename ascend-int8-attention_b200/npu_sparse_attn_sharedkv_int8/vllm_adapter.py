"""Serving-side runtime of the INT8 shared-KV layers on CUDA: frozen scales, per-stream scratch,
and a small cache of prepared operators per attention layer.

Mirror of the reference's adapter (npu_sparse_attn_sharedkv_int8/vllm_adapter.py:28-214): the same
module functions (`stream_key`, `geometry`, `scratch_allocator`, `load_scales`, `check_device`,
`runtime`, `install`) and the same `LayerRuntime.write` / `LayerRuntime.attention` calling
convention, so that a D=512 sparse-attention layer of a serving stack hands its cache writes and
its attention call to the CUDA kernels without knowing about prepared operators.

What is CUDA-specific: stream identity is the raw `cudaStream_t`; capture is detected with
`torch.cuda.is_current_stream_capturing`; the device check asks for compute capability 10.x.
`install()` needs a serving stack that exposes the layer hooks the reference patches; plain CUDA
vLLM has no such sparse shared-KV layer, so `install()` says so instead of patching anything.
"""
from collections import OrderedDict
from functools import lru_cache
import logging
import math
import os

import torch

from .attention import PreparedAttention
from .cache import PreparedCacheWrite
from .reference import SharedKVCase
from .runtime import current_stream, native_launcher

SCALE_PROTOCOL = "sharedkv-c8-v1"
PREPARED_PER_LAYER = 8                 # prepared attention operators kept per layer (vllm_adapter.py:181-182)

_scratch = {}
_log = logging.getLogger("vllm.sharedkv_c8")


def stream_key(device):
    """Identity of the current stream of `device`: the raw stream handle (vllm_adapter.py:28-32)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    return int(current_stream(index) or 0)


def geometry(tensor):
    """What a prepared operator depends on besides the pointer (vllm_adapter.py:35-38)."""
    if tensor is None:
        return None
    return tensor.shape, tensor.stride(), tensor.dtype, tensor.device


def scratch_allocator(name, shape, dtype, device):
    """Growth-only scratch per (device, stream, name, dtype) (vllm_adapter.py:41-49).

    The layers of a model run one after the other on one stream and may share scratch; another
    stream gets its own.  Capacities are powers of two and superseded buffers are kept alive,
    because a captured graph may still point at them.
    """
    elements = math.prod(shape)
    generations = _scratch.setdefault((device, stream_key(device), name, dtype), [])
    newest = generations[-1] if generations else None
    if newest is None or newest.numel() < elements:
        capacity = 1 << max(elements - 1, 0).bit_length()
        newest = torch.empty(capacity, dtype=dtype, device=device)
        generations.append(newest)
    return newest[:elements].view(shape)


@lru_cache(maxsize=1)
def load_scales():
    """Frozen per-channel scales from the file named by SHAREDKV_SCALES (vllm_adapter.py:52-63):
    {"protocol": "sharedkv-c8-v1", "scales": {"<layer prefix>.<ori|cmp>": FP32[512] > 0}}."""
    location = os.environ.get("SHAREDKV_SCALES", "")
    if location == "":
        raise ValueError("INT8 mode requires SHAREDKV_SCALES containing frozen calibrated scales")
    stored = torch.load(location, map_location="cpu", weights_only=True)
    if stored.get("protocol") != SCALE_PROTOCOL:
        raise ValueError("Wrong shared-KV scale protocol")
    table = stored["scales"]
    for name, vector in table.items():
        shaped = tuple(vector.shape) == (512,) and vector.dtype == torch.float32
        if not (shaped and bool(torch.isfinite(vector).all()) and bool((vector > 0).all())):
            raise ValueError(f"Invalid scale vector: {name}")
    return table


@lru_cache(maxsize=16)
def check_device(device):
    """The kernels are sm_100a only (the reference pins its own part, vllm_adapter.py:66-71)."""
    major, _ = torch.cuda.get_device_capability(device)
    if major != 10:
        raise ValueError("This adapter needs an sm_100 GPU (B200): the kernels are built for sm_100a only")
    if native_launcher() is None:
        raise RuntimeError("Build the native library with csrc/build.sh before serving")


class LayerRuntime:
    """Per-layer state: scales on the device, cache writers and prepared attention operators keyed
    by everything but the pointers (vllm_adapter.py:74-214)."""

    def __init__(self, impl):
        if impl.head_dim != 512 or getattr(impl, "turboquant", None) is not None:
            raise ValueError("INT8 shared-KV requires ordinary D=512 DSA")
        parallel = getattr(getattr(impl, "vllm_config", None), "parallel_config", None)
        context_parallel = [getattr(parallel, f"{phase}_context_parallel_size", 1) for phase in ("decode", "prefill")]
        if context_parallel != [1, 1]:
            raise ValueError("Context-parallel cache writers have not been integrated")
        self.impl = impl
        self.prefix = impl.swa_cache_layer.prefix.removesuffix(".swa_cache")      # key prefix in the scale file
        self.scales, self.writers = {}, {}                   # kind -> (scale, inverse); geometry -> prepared writer
        self.attention_ops = OrderedDict()                   # geometry -> prepared attention, least recent first
        self.captured_ops, self.captured_ids = [], set()     # operators whose launches sit in a captured graph
        self.reported_caches = set()
        self.empty_lse = self.plan = None

    def scale(self, kind, device):
        """(scale, inverse scale) of this layer's `kind` cache on `device`; the inverse is rounded
        from the FP64 reciprocal as the cache writer expects (reference.py:48-50)."""
        pair = self.scales.get(kind)
        if pair is None:
            check_device(device)
            name = f"{self.prefix}.{kind}"
            frozen = load_scales().get(name)
            if frozen is None:
                raise ValueError(f"Missing real-model calibration for {name}")
            inverse = frozen.to(torch.float64).reciprocal().to(torch.float32)
            pair = self.scales[kind] = (frozen.to(device), inverse.to(device))
        return pair

    def write(self, cache, updates, slots, kind):
        """Quantize `updates` with the layer's frozen scale and scatter them into `cache`."""
        rows = 0 if updates is None else updates.shape[0]
        if rows == 0:
            return
        if slots.shape[0] != rows:
            raise ValueError("Cache-write slot/update lengths differ")
        # a prepared writer is reused while everything but the pointers and the row count stays the same
        layout = (kind, stream_key(cache.device), geometry(cache),
                  updates.shape[1:], updates.stride(), updates.dtype, updates.device,
                  slots.shape[1:], slots.stride(), slots.dtype, slots.device)
        writer = self.writers.get(layout)
        if writer is not None:
            writer._rebind_same_geometry(cache, updates, slots)
        else:
            writer = self.writers[layout] = PreparedCacheWrite(cache, updates, slots, self.scale(kind, cache.device)[1])
        writer.run()
        # the launch is queued: same-stream lifetimes protect the tensors, no need to pin activations here
        writer.updates = writer.slots = None
        if kind not in self.reported_caches:
            self.reported_caches.add(kind)
            _log.info("Standalone INT8 sharedKV cache %s.%s: shape=%s dtype=%s page_stride=%d bytes",
                      self.prefix, kind, tuple(cache.shape), cache.dtype, cache.stride(0))

    @staticmethod
    def _case_from_call(q, kw):
        """Translate the serving stack's keyword protocol into a SharedKVCase, refusing what the
        kernels do not implement."""
        if (kw.get("layout_q"), kw.get("layout_kv")) != ("TND", "PA_ND"):
            raise ValueError("Expected TND / PA_ND shared-KV layout")
        explicit = kw.get("ori_sparse_indices")
        if kw.get("ori_mask_mode", 4) != 4 or (explicit is None and kw.get("ori_win_right", 0) != 0):
            raise ValueError("Unsupported original window mask")
        ratio = max(1, kw.get("cmp_ratio", 1))
        if ratio > 1 and kw.get("cmp_mask_mode", 3) != 3:
            raise ValueError("Compressed cache must use causal masking")
        return SharedKVCase(
            q=q, ori=kw["ori_kv"], ori_block_table=kw["ori_block_table"], cu_q=kw["cu_seqlens_q"],
            seq_lens=kw["seqused_kv"], sink=kw["sinks"], cmp=kw.get("cmp_kv"),
            cmp_block_table=kw.get("cmp_block_table"), cmp_indices=kw.get("cmp_sparse_indices"),
            ratio=ratio, window=kw["ori_win_left"] + 1, softmax_scale=kw["softmax_scale"], ori_indices=explicit)

    def _operator(self, case, output, lse):
        """Prepared operator for this geometry on this stream: the newest PREPARED_PER_LAYER are kept.
        The kernel derives tiling and KV splits on the device, so the key holds no length bound."""
        shapes = tuple(geometry(v) if isinstance(v, torch.Tensor) else v for v in vars(case).values())
        key = (shapes, lse is not None, stream_key(case.q.device))
        op = self.attention_ops.get(key)
        if op is not None:
            self.attention_ops.move_to_end(key)
            op._rebind_same_geometry(case, output=output, lse_output=lse)
            return op
        device = case.q.device
        op = PreparedAttention(case, self.scale("ori", device)[0], self.scale("cmp", device)[0] if case.ratio > 1 else None,
                               return_lse=lse is not None, output=output, lse_output=lse, scratch_allocator=scratch_allocator)
        self.attention_ops[key] = op
        while len(self.attention_ops) > PREPARED_PER_LAYER:
            self.attention_ops.popitem(last=False)
        return op

    def attention(self, q, **kw):
        """The sparse shared-KV attention call of the serving stack (vllm_adapter.py:133-214):
        returns (output, lse[T, H, 1]), or (output, empty FP32 tensor) when no LSE was asked for."""
        case = self._case_from_call(q, kw)
        output = torch.empty_like(q)
        lse = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device) if kw.get("return_softmax_lse", False) else None
        op = self._operator(case, output, lse)
        if torch.cuda.is_current_stream_capturing() and id(op) not in self.captured_ids:
            self.captured_ids.add(id(op))
            self.captured_ops.append(op)
        result = op.run()
        # outputs belong to the caller (or to the graph's pool); keep only geometry and scratch
        op.case = op.out = op.lse = None
        if lse is not None:
            return result, lse.unsqueeze(-1)
        if self.empty_lse is None:
            self.empty_lse = torch.empty(0, dtype=torch.float32, device=q.device)
        return result, self.empty_lse


def runtime(impl):
    """The LayerRuntime attached to an attention implementation object (vllm_adapter.py:217-222)."""
    state = getattr(impl, "_sharedkv_int8_runtime", None)
    if state is None:
        state = LayerRuntime(impl)
        impl._sharedkv_int8_runtime = state
    return state


def install(attention_impl=None, cache_layers=(), *, planner=None, runner=None):
    """Route a serving stack's D=512 sparse shared-KV layers through this package.

    The reference patches vllm-ascend's DSA classes in place (vllm_adapter.py:225-277).  CUDA vLLM
    ships no such layer, so the classes to patch are passed in: `attention_impl` needs
    `get_kv_plan()` returning a dataclass with a `sparse_attn_op` field and a
    `_write_kv_cache(cache, kv, slot_mapping, *, quantize)` method; every class in `cache_layers`
    needs `get_kv_cache_spec(config)` returning a dataclass with `head_size`, `dtype` and (where
    the stack pads pages) `page_size_padded`.  SHAREDKV_COMPACT_PAGES=1 also installs the compact
    page planner (cache_layout.install), which needs the stack's `planner` and `runner` objects;
    without compact pages an INT8 layer keeps the BF16 pool's page size as padding, as in the
    reference (vllm_adapter.py:258-262).
    """
    from dataclasses import fields, replace
    load_scales()            # fail before weight loading if the calibration file is absent
    if attention_impl is None:
        raise RuntimeError("No CUDA serving stack exposes the sparse shared-KV layer hooks this adapter patches; "
                           "pass the implementation class to install(attention_impl=..., cache_layers=...) "
                           "or use LayerRuntime directly")
    compact_pages = os.environ.get("SHAREDKV_COMPACT_PAGES") == "1"
    if compact_pages:
        from .cache_layout import install as install_cache_layout
        install_cache_layout(planner, runner)
    original_plan = attention_impl.get_kv_plan

    def get_plan(self):
        state = runtime(self)
        if state.plan is None:
            state.plan = replace(original_plan(self), sparse_attn_op=state.attention)
        return state.plan

    def write(self, cache, kv, slot_mapping, *, quantize):
        return runtime(self).write(cache, kv, slot_mapping, "cmp" if quantize else "ori")

    attention_impl.get_kv_plan = get_plan
    attention_impl._write_kv_cache = write
    for cls in cache_layers:
        original_spec = cls.get_kv_cache_spec

        def spec(self, config, _original=original_spec):
            old = _original(self, config)
            if old is None:
                return None
            if old.head_size != 512 or old.dtype != torch.bfloat16:
                raise ValueError("INT8 plugin expects the ordinary BF16 D=512 cache specification")
            changes = {"dtype": torch.int8}
            if any(f.name == "page_size_padded" for f in fields(old)):
                changes["page_size_padded"] = None if compact_pages else old.page_size_bytes
            return replace(old, **changes)

        cls.get_kv_cache_spec = spec
