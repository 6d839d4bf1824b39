"""Opt-in entry point for a serving stack's plugin loader.

Mirror of the reference's plugin module (npu_sparse_attn_sharedkv_int8/vllm_plugin.py:9-67):
`register()` does nothing unless SHAREDKV_INT8_MODE is set, accepts the same two modes, and in
"int8" mode routes the stack's sparse shared-KV layers through `vllm_adapter`.  The classes to
patch are looked up through SHAREDKV_ATTENTION_IMPL / SHAREDKV_CACHE_LAYERS
("package.module:Class", comma separated for the latter), because CUDA vLLM itself has no D=512
sparse shared-KV layer to name here; "calibrate" mode belongs to the calibration tooling, which
is outside this build.
"""
from importlib import import_module
import os

_registered = False


def layer_prefix(impl):
    """Scale-file key prefix of an attention implementation object (vllm_plugin.py:9-10)."""
    return impl.swa_cache_layer.prefix.removesuffix(".swa_cache")


def _resolve(spec):
    module, _, name = spec.partition(":")
    if not module or not name:
        raise ValueError(f"Expected 'package.module:Class', got {spec!r}")
    return getattr(import_module(module), name)


def register():
    global _registered
    mode = os.environ.get("SHAREDKV_INT8_MODE", "")
    if not mode or _registered:
        return
    if mode not in ("calibrate", "int8"):
        raise ValueError(f"Unsupported SHAREDKV_INT8_MODE={mode!r}")
    if mode == "calibrate":
        raise ValueError("SHAREDKV_INT8_MODE=calibrate: the calibration observer is not part of the CUDA build; "
                         "produce the sharedkv-c8-v1 scale file with the reference's tooling")
    implementation = os.environ.get("SHAREDKV_ATTENTION_IMPL")
    if not implementation:
        raise ValueError("SHAREDKV_INT8_MODE=int8 needs SHAREDKV_ATTENTION_IMPL=package.module:Class naming the "
                         "sparse shared-KV attention implementation to route through the INT8 kernels")
    layers = [s for s in os.environ.get("SHAREDKV_CACHE_LAYERS", "").split(",") if s]
    from .vllm_adapter import install
    install(_resolve(implementation), tuple(_resolve(s) for s in layers))
    _registered = True
