"""INT8 shared-KV decode attention and paged INT8 KV-cache writer for NVIDIA B200.

The import surface is that of the Ascend package of the same name
(npu_sparse_attn_sharedkv_int8/__init__.py:7-23 of the reference): four public names, looked up
on first use so that the data classes can be imported on a machine without CUDA.
"""
import importlib

__version__ = "0.1.0+b200"
__stage__ = "b200-sm100a"

# public name -> submodule that defines it
_HOME = {
    "CacheQuantization": "reference",
    "SharedKVCase": "reference",
    "PreparedAttention": "attention",
    "PreparedCacheWrite": "cache",
}
__all__ = sorted(_HOME)


def __getattr__(name):
    submodule = _HOME.get(name)
    if submodule is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(f"{__name__}.{submodule}"), name)
    globals()[name] = value            # later lookups bypass this hook
    return value


def __dir__():
    return sorted(set(globals()) | set(_HOME))
