"""C4 / C128 decode route: ABI guard, scratch sizing and the three launcher symbols.

Counterpart of the reference's default route (npu_sparse_attn_sharedkv_int8/c8_attention.py).
Tiling, KV splitting and live-shape handling are decided on the device at every launch,
so nothing here depends on sequence lengths.
"""
import copy
import ctypes
from functools import lru_cache
import os
from types import SimpleNamespace

import torch

from .runtime import _library, check, current_stream, native_launcher

CORES = 148                 # persistent CTAs on a B200 (the reference: 24 AI cores); `blocks` is advisory
HEADS = 8
DIM = 512
MAX_SPLITS = CORES          # a token's KV may be spread over at most one piece per CTA
_MAX_CTAS = 160             # partial-result slots reserved by the library
_PARTIAL_FLOATS = HEADS * DIM + 16


def workspace_bytes(tokens):
    """Scratch bytes one launch with `tokens` query rows needs (plan, tickets, partial sums).
    Python restatement of sharedkv_workspace_bytes(); a unit test keeps the two equal."""
    plan = 1024 + 32 * (tokens + _MAX_CTAS) + 4 * tokens + 4 * tokens
    return (plan + 255) // 256 * 256 + _MAX_CTAS * 2 * _PARTIAL_FLOATS * 4


# Enough for 8192 query rows per launch; larger capacities use workspace_bytes(tokens).
WORKSPACE_BYTES = workspace_bytes(8192)


def enabled():
    value = os.environ.get('SHAREDKV_C8_DECODE', '1')
    if value not in ('0', '1'):
        raise ValueError('SHAREDKV_C8_DECODE must be 0 or 1')
    return value == '1'


def argument_type():
    from .attention import _Args
    return _Args


@lru_cache(maxsize=1)
def library():
    lib = _library()
    if lib.sharedkv_attention_args_size() != ctypes.sizeof(argument_type()):
        raise RuntimeError('C8 host/device argument ABI mismatch')
    return lib


def supported(entry):
    """The geometry the CUDA kernels implement: eight heads, window 128, 32-row pages,
    ratio 4 (top-k <= 1024, no explicit original slots) or ratio 128."""
    if not getattr(entry, 'blocks', 0) or not hasattr(entry, 'args'):
        return False
    p = entry.args
    if not isinstance(p, argument_type()):
        return False
    return (
        p.heads == HEADS
        and p.tokens > 0
        and p.batch > 0
        and p.ratio in (4, 128)
        and p.window == 128
        and p.oriBlock == p.cmpBlock == 32
        and not p.oriIndices
        and (p.ratio != 4 or 0 < p.topk <= 1024)
    )


def prepare(entry, *, scratch_allocator=None, shared_storage=False):
    """Bind scratch and the launcher to a validated entry; no device read-back.

    With shared_storage the caller has already placed a workspace of at least
    workspace_bytes(tokens) in entry.workspace (tests use that to put guard bands around it).
    """
    if getattr(entry, 'c8_dynamic', False) or not supported(entry):
        return entry
    p = entry.args
    need = workspace_bytes(p.tokens)
    allocate = scratch_allocator or (
        lambda name, shape, dtype, device: torch.empty(shape, dtype=dtype, device=device)
    )
    workspace = getattr(entry, 'workspace', None)
    if shared_storage:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            raise ValueError('C8 shared controls require a workspace of workspace_bytes(tokens) bytes')
    elif workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = allocate('workspace', (need,), torch.uint8, entry.case.q.device)
    if workspace.data_ptr() % 256:
        raise ValueError('Attention workspace must be 256-byte aligned')
    partial = getattr(entry, 'partial', None)
    if partial is None:
        partial = torch.empty(0, dtype=torch.float32, device=entry.case.q.device)

    out = copy.copy(entry)
    out.args = type(p).from_buffer_copy(p)
    out.args.workspace = workspace.data_ptr()
    out.args.partial = 0
    out.args.splits = 1
    out.workspace, out.partial = workspace, partial
    out.blocks, out.splits = CORES, 1
    out.argument_address = ctypes.addressof(out.args)
    out._c8_library = library()
    small = p.ratio == 4 and p.tokens < 24
    suffix = 'sparse_small' if small else ('sparse' if p.ratio == 4 else 'dense')
    out.launch = getattr(out._c8_library, 'launch_sharedkv_c8_' + suffix)
    out.variant = 22 if small else (20 if p.ratio == 4 else 21)
    out.native = native_host(os.environ.get('SHAREDKV_HOST_QUEUE') == '1')
    if out.native is not None and out.native.attention_args_size != ctypes.sizeof(type(p)):
        raise RuntimeError('C8 host/device argument ABI mismatch')
    out.c8_dynamic = True
    return out


def host_module():
    """The object playing the role of the reference's `sharedkv_c8_host` extension module."""
    return native_launcher()


@lru_cache(maxsize=2)
def native_host(queued=False):
    module = host_module()
    if module is None:
        return None
    return SimpleNamespace(
        attention=module.attention_queued if queued else module.attention,
        attention_args_size=module.attention_args_size,
        _owner=module,
    )


def launch_raw(entry):
    """ctypes path (SHAREDKV_USE_CTYPES=1): call the launcher symbol on the current stream."""
    with torch.cuda.device(entry.case.q.device):
        check(entry.launch(entry.blocks, current_stream(entry.device_index), ctypes.byref(entry.args)),
              'attention launch')
