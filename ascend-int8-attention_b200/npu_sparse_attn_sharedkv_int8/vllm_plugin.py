"""Opt-in entry point for a serving stack's plugin loader.

Mirror of the reference's plugin module (npu_sparse_attn_sharedkv_int8/vllm_plugin.py:9-67):
`register()` does nothing unless SHAREDKV_INT8_MODE is set and accepts the same two modes.
"calibrate" wraps the attention implementation's cache writer with the calibration observer
(BF16 execution is left as it is); "int8" routes the stack's sparse shared-KV layers through
`vllm_adapter`.  In both modes a draft model that precomputes target-context KV outside the
attention forward (the reference's DSpark model, vllm_plugin.py:48-66) has that writer routed
through the same `_write_kv_cache`, so the rows are observed, or quantized, like all others.

The reference names vllm-ascend's classes; CUDA vLLM has no D=512 sparse shared-KV layer, so the
classes come from the environment, each as "package.module:Class":
  SHAREDKV_ATTENTION_IMPL   the attention implementation (get_kv_plan, _write_kv_cache)
  SHAREDKV_CACHE_LAYERS     comma-separated cache-owning layer classes (get_kv_cache_spec)
  SHAREDKV_DRAFT_MODEL      optional draft model class whose `_store_standard_swa_kv` is replaced
"""
from importlib import import_module
import os

_registered = False
_observer = None


def layer_prefix(impl):
    """Scale-file key prefix of an attention implementation object (vllm_plugin.py:9-10)."""
    return impl.swa_cache_layer.prefix.removesuffix(".swa_cache")


def _resolve(spec):
    module, _, name = spec.partition(":")
    if not module or not name:
        raise ValueError(f"Expected 'package.module:Class', got {spec!r}")
    return getattr(import_module(module), name)


def store_draft_context(self, shared_kv, slot_mapping, attn=None):
    """Replacement for a draft model's target-context KV writer (vllm_plugin.py:51-64): same slot
    conversion, but the scatter goes through the attention implementation's `_write_kv_cache`,
    i.e. through the observer in calibrate mode and through the INT8 writer in int8 mode."""
    if slot_mapping is None or slot_mapping.numel() == 0:
        return
    assert attn is not None
    layer = attn.dsa_attn.swa_cache_layer
    cache = getattr(layer, "kv_cache", None)
    if cache is None:
        return
    while isinstance(cache, (tuple, list)) and len(cache) == 1:
        cache = cache[0]
    impl = attn.dsa_attn.dsa_attn.impl
    if slot_mapping.ndim == 1:
        slot_mapping = impl.get_kv_plan().format_dsa_slot_mapping(slot_mapping, layer.block_size)
    impl._write_kv_cache(cache, shared_kv, slot_mapping, quantize=False)


def register():
    global _registered, _observer
    mode = os.environ.get("SHAREDKV_INT8_MODE", "")
    if not mode or _registered:
        return
    if mode not in ("calibrate", "int8"):
        raise ValueError(f"Unsupported SHAREDKV_INT8_MODE={mode!r}")
    directory = os.environ.get("SHAREDKV_CALIBRATION_DIR")
    if mode == "calibrate" and not directory:
        raise ValueError("calibrate mode requires SHAREDKV_CALIBRATION_DIR")
    implementation = os.environ.get("SHAREDKV_ATTENTION_IMPL")
    if not implementation:
        raise ValueError(f"SHAREDKV_INT8_MODE={mode} needs SHAREDKV_ATTENTION_IMPL=package.module:Class naming the "
                         "sparse shared-KV attention implementation to hook")
    implementation = _resolve(implementation)
    if mode == "calibrate":
        from .calibration import CacheObserver
        _observer = CacheObserver(directory)
        original_write = implementation._write_kv_cache

        def observed_write(self, cache, kv, slot_mapping, *, quantize):
            if getattr(self, "turboquant", None) is not None:
                raise ValueError("Shared-KV calibration requires the ordinary BF16 DSA path")
            _observer.observe(layer_prefix(self), "cmp" if quantize else "ori", cache, kv, slot_mapping)
            return original_write(self, cache, kv, slot_mapping, quantize=quantize)

        implementation._write_kv_cache = observed_write
    else:
        layers = [s for s in os.environ.get("SHAREDKV_CACHE_LAYERS", "").split(",") if s]
        from .vllm_adapter import install
        install(implementation, tuple(_resolve(s) for s in layers))
    draft = os.environ.get("SHAREDKV_DRAFT_MODEL")
    if draft:
        _resolve(draft)._store_standard_swa_kv = store_draft_context
    _registered = True
