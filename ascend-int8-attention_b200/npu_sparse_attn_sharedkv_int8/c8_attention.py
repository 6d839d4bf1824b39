"""C4 / C128 decode route on CUDA: ABI guard, scratch sizing, launcher selection.

Counterpart of the reference's default route (npu_sparse_attn_sharedkv_int8/c8_attention.py:16-138)
with the same module surface (`CORES HEADS DIM MAX_SPLITS WORKSPACE_BYTES enabled argument_type
library supported prepare host_module native_host`).  Tiling, KV splitting and the live shape are
decided on the device at every launch, so nothing here looks at sequence lengths.
"""
import copy
import ctypes
from functools import lru_cache
import os
from types import SimpleNamespace

import torch

from .runtime import _library, check, current_stream, native_launcher

CORES = 148                 # persistent CTAs on a B200 (24 AI cores in the reference); `blocks` is advisory
HEADS = 8
DIM = 512
MAX_SPLITS = CORES          # a token's KV may be spread over at most one piece per CTA
_MAX_CTAS = 160             # partial-result slots the library reserves
_PARTIAL_FLOATS = HEADS * DIM + 16
_VARIANTS = {"general": 0, "packed": 3, "packed_sparse": 4, "paired": 7, "paired_sparse": 8, "sparse": 20, "dense": 21, "sparse_small": 22}     # kernel ids of the host bridge
_PAIRED_MAX_BATCH = 11775   # requests whose cumulative counts the paired kernel keeps in shared memory
_SMALL_C4_TOKENS = 24       # below this the reference selects its "small" C4 image (c4_small.cpp:21)


def workspace_bytes(tokens):
    """Scratch bytes one launch with `tokens` query rows needs (work items, tickets, partial sums).
    Python restatement of sharedkv_workspace_bytes(); a unit test keeps the two equal."""
    plan = 1024 + 32 * (tokens + _MAX_CTAS) + 4 * tokens + 4 * tokens
    return (plan + 255) // 256 * 256 + _MAX_CTAS * 2 * _PARTIAL_FLOATS * 4


# Enough for 8192 query rows per launch; larger capacities use workspace_bytes(tokens).
WORKSPACE_BYTES = workspace_bytes(8192)


def enabled():
    """SHAREDKV_C8_DECODE switch of the reference (c8_attention.py:33-37): unset or "1" is on."""
    setting = os.environ.get("SHAREDKV_C8_DECODE", "1")
    if setting == "1":
        return True
    if setting == "0":
        return False
    raise ValueError("SHAREDKV_C8_DECODE must be 0 or 1")


def argument_type():
    from .attention import _Args
    return _Args


@lru_cache(maxsize=1)
def library():
    """The loaded CUDA library, after checking that it was built for this argument struct."""
    lib = _library()
    if lib.sharedkv_attention_args_size() != ctypes.sizeof(argument_type()):
        raise RuntimeError("C8 host/device argument ABI mismatch")
    return lib


def supported(entry):
    """True for the geometry the CUDA kernels implement: eight heads, window 128, 32-row pages;
    ratio 128, ratio 4 with at most 1024 selections per token, or ratio 1 (original cache only);
    with or without explicit original slots.  (The reference's C4/C128 route refuses explicit slots
    and ratio 1, c8_attention.py:56-74, and leaves them to its general kernel; here one kernel family
    serves both, through the general launcher.)"""
    args = getattr(entry, "args", None)
    if not getattr(entry, "blocks", 0) or not isinstance(args, argument_type()):
        return False
    if args.tokens == 0 or args.batch == 0 or (args.oriIndices and not args.oriTopk):
        return False
    if (args.heads, args.window, args.oriBlock) != (HEADS, 128, 32) or (args.ratio != 1 and args.cmpBlock != 32):
        return False
    if getattr(entry, "query_group", 1) in (2, 4) and (args.ratio not in (4, 128) or args.oriIndices or args.batch > _PAIRED_MAX_BATCH):
        return False
    return args.ratio in (1, 128) or (args.ratio == 4 and 0 < args.topk <= 1024)


def _launcher_name(args, query_group=1):
    if query_group in (2, 4):
        return ("paired" if query_group == 2 else "packed") + ("" if args.ratio == 128 else "_sparse")
    if args.ratio == 1 or args.oriIndices:
        return "general"
    if args.ratio == 128:
        return "dense"
    return "sparse_small" if args.tokens < _SMALL_C4_TOKENS else "sparse"


def prepare(entry, *, scratch_allocator=None, shared_storage=False):
    """A copy of a validated entry bound to scratch and to its launcher; nothing is read back.

    Scratch comes from `scratch_allocator(name, shape, dtype, device)` (serving passes its
    per-stream pool) or from torch.  With shared_storage the caller has already put a workspace of
    at least workspace_bytes(tokens) in entry.workspace (tests surround it with guard bands).
    Entries that are already prepared, or outside `supported`, are returned as they are.
    """
    if getattr(entry, "c8_dynamic", False) or not supported(entry):
        return entry
    device = entry.case.q.device
    need = workspace_bytes(entry.args.tokens)
    workspace = getattr(entry, "workspace", None)
    large_enough = workspace is not None and workspace.numel() * workspace.element_size() >= need
    if shared_storage and not large_enough:
        raise ValueError("C8 shared controls require a workspace of workspace_bytes(tokens) bytes")
    if not large_enough:
        workspace = (scratch_allocator("workspace", (need,), torch.uint8, device) if scratch_allocator
                     else torch.empty(need, dtype=torch.uint8, device=device))
    if workspace.data_ptr() % 256:
        raise ValueError("Attention workspace must be 256-byte aligned")
    # Split-K arrival counters and the status word at the head of the workspace start at zero; the
    # kernels keep them so from launch to launch, so this is the only clear a workspace ever gets
    # (stream-ordered, on the current stream, like every launch that will use it).
    with torch.cuda.device(device):
        check(library().sharedkv_workspace_init(workspace.data_ptr(), current_stream(device.index)), "workspace init")
    partial = getattr(entry, "partial", None)
    if partial is None:
        partial = torch.empty(0, dtype=torch.float32, device=device)       # kept for callers that read `.partial`

    bound = copy.copy(entry)
    bound.args = type(entry.args).from_buffer_copy(entry.args)
    bound.args.workspace, bound.args.partial, bound.args.splits = workspace.data_ptr(), 0, 1
    bound.workspace, bound.partial = workspace, partial
    bound.blocks, bound.splits = CORES, 1
    bound.argument_address = ctypes.addressof(bound.args)
    name = _launcher_name(bound.args, getattr(bound, "query_group", 1))
    bound._c8_library = library()
    bound.launch = getattr(bound._c8_library, "launch_sharedkv" if name == "general" else
                           "launch_sharedkv_" + name if name.startswith(("paired", "packed")) else "launch_sharedkv_c8_" + name)
    bound.variant = _VARIANTS[name]
    bound.native = native_host(os.environ.get("SHAREDKV_HOST_QUEUE") == "1")
    if bound.native is not None and bound.native.attention_args_size != ctypes.sizeof(type(bound.args)):
        raise RuntimeError("C8 host/device argument ABI mismatch")
    bound.c8_dynamic = True
    return bound


def host_module():
    """The object playing the role of the reference's `sharedkv_c8_host` extension module."""
    return native_launcher()


@lru_cache(maxsize=2)
def native_host(queued=False):
    """attention / attention_queued of the host bridge behind one name (c8_attention.py:131-138)."""
    module = host_module()
    if module is None:
        return None
    call = module.attention_queued if queued else module.attention
    return SimpleNamespace(attention=call, attention_args_size=module.attention_args_size, _owner=module)


def workspace_status(entry):
    """Synchronises the current stream and raises RuntimeError if a wait inside a decode kernel that
    used this entry's workspace ever ran out (its outputs are then invalid).  Diagnostic only."""
    with torch.cuda.device(entry.case.q.device):
        check(library().sharedkv_workspace_status(entry.workspace.data_ptr(), current_stream(entry.device_index)),
              "attention kernel")


def launch_raw(entry):
    """ctypes path (SHAREDKV_USE_CTYPES=1): call the launcher symbol on the current stream."""
    with torch.cuda.device(entry.case.q.device):
        status = entry.launch(entry.blocks, current_stream(entry.device_index), ctypes.byref(entry.args))
    check(status, "attention launch")
