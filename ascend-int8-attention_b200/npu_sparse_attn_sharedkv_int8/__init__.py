"""INT8 shared-KV decode attention and paged INT8 KV-cache writer for NVIDIA B200.

Same import surface as the Ascend package of the same name
(npu_sparse_attn_sharedkv_int8/__init__.py:7-23 of the reference): the four public
names are resolved lazily so that the data classes import without CUDA.
"""
from importlib import import_module

__version__ = "0.1.0+b200"
__stage__ = "b200-sm100a"

__all__ = ["CacheQuantization", "SharedKVCase", "PreparedAttention", "PreparedCacheWrite"]

_EXPORTS = {
    "CacheQuantization": ("reference", "CacheQuantization"),
    "SharedKVCase": ("reference", "SharedKVCase"),
    "PreparedAttention": ("attention", "PreparedAttention"),
    "PreparedCacheWrite": ("cache", "PreparedCacheWrite"),
}


def __getattr__(name):
    if name not in _EXPORTS:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    module, attribute = _EXPORTS[name]
    value = getattr(import_module(f".{module}", __name__), attribute)
    globals()[name] = value
    return value
