"""Loader for the C-ABI CUDA library and the host-bridge shim.

The reference loads two things here (npu_sparse_attn_sharedkv_int8/runtime.py:12-42):
a pybind11 "host launcher" module that looks up the framework's current stream in C++
(csrc/host/launch.cpp) and the device library through ctypes.  On CUDA one shared
library does both jobs; it has no tensor-framework dependency, so the current stream is
looked up here, in Python, and handed over as a raw ``cudaStream_t``.
"""
import ctypes
from functools import lru_cache
import os

import torch

from ._paths import native_path


class NativeError(RuntimeError):
    pass


def check(status, what):
    """Turn a non-zero library status into RuntimeError (csrc/host/launch.cpp:45 throws there)."""
    if status:
        text = _library().sharedkv_status_string(int(status)).decode()
        raise NativeError(f"{what} failed with status {int(status)}: {text}")


@lru_cache(maxsize=1)
def _library():
    lib = ctypes.CDLL(str(native_path()))
    u32, u64, i32, ptr = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int32, ctypes.c_void_p
    for name in ("sharedkv_attention_args_size", "sharedkv_cache_args_size", "sharedkv_attention_variant_count"):
        getattr(lib, name).argtypes, getattr(lib, name).restype = [], u32
    lib.sharedkv_workspace_bytes.argtypes, lib.sharedkv_workspace_bytes.restype = [u32], u64
    for name in ("launch_sharedkv", "launch_sharedkv_paired", "launch_sharedkv_paired_sparse", "launch_sharedkv_packed", "launch_sharedkv_packed_sparse", "launch_sharedkv_c8_sparse", "launch_sharedkv_c8_sparse_small", "launch_sharedkv_c8_dense",
                 "launch_cache_write"):
        getattr(lib, name).argtypes, getattr(lib, name).restype = [u32, ptr, ptr], ctypes.c_int
    lib.sharedkv_attention.argtypes, lib.sharedkv_attention.restype = [u64, u32, u32, i32, ptr], ctypes.c_int
    lib.sharedkv_cache_write.argtypes, lib.sharedkv_cache_write.restype = [u64, u32, i32, ptr], ctypes.c_int
    lib.sharedkv_attention_debug.argtypes = [u32, ptr, ptr, ptr]
    lib.sharedkv_attention_debug.restype = ctypes.c_int
    lib.sharedkv_status_string.argtypes, lib.sharedkv_status_string.restype = [ctypes.c_int], ctypes.c_char_p
    lib.sharedkv_workspace_init.argtypes, lib.sharedkv_workspace_init.restype = [ptr, ptr], ctypes.c_int
    lib.sharedkv_workspace_status.argtypes, lib.sharedkv_workspace_status.restype = [ptr, ptr], ctypes.c_int
    lib.sharedkv_attention_static_scratch.argtypes = [u32, ptr, ptr]
    lib.sharedkv_attention_static_scratch.restype = ctypes.c_int
    lib.sharedkv_static_scratch_status.argtypes, lib.sharedkv_static_scratch_status.restype = [ptr], ctypes.c_int
    return lib


def current_stream(device_index):
    return torch.cuda.current_stream(device_index if device_index is not None and device_index >= 0 else None).cuda_stream


class _HostBridge:
    """Same attribute names as the reference's pybind module (csrc/host/launch.cpp:105-115)."""

    def __init__(self, lib):
        self._owner = lib
        self.attention_args_size = lib.sharedkv_attention_args_size()
        self.cache_args_size = lib.sharedkv_cache_args_size()
        self.attention_variant_count = lib.sharedkv_attention_variant_count()

    def attention(self, argument_address, blocks, variant, device):
        check(self._owner.sharedkv_attention(argument_address, blocks, variant, device, current_stream(device)),
              "attention launch")

    def cache_write(self, argument_address, blocks, device):
        check(self._owner.sharedkv_cache_write(argument_address, blocks, device, current_stream(device)),
              "cache-write launch")

    # CUDA copies kernel arguments by value when the launch is enqueued, which is all the
    # reference's queued variants add (csrc/host/launch.cpp:60-96); they are the same calls here.
    attention_queued = attention
    cache_write_queued = cache_write

    @staticmethod
    def stream_id(device):
        return current_stream(device)


@lru_cache(maxsize=1)
def native_launcher():
    """The host bridge, or None when SHAREDKV_USE_CTYPES=1 asks for raw launcher symbols."""
    if os.environ.get("SHAREDKV_USE_CTYPES") == "1":
        return None
    return _HostBridge(_library())


class Kernels:
    """Handle on the device library (reference: runtime.py:39-42)."""

    def __init__(self):
        self.lib = _library()
