"""The drop-in boundary without a GPU: the C-ABI library loads and exports every symbol the
header declares, struct layouts match the reference's, and the Python mirror keeps the
reference's policy and validation behaviour (reference tests/npu/test_policy.py:18-34)."""
import ctypes
import os
from pathlib import Path
import re
from types import SimpleNamespace
from unittest.mock import patch

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def library():
    from npu_sparse_attn_sharedkv_int8 import runtime
    return runtime._library()


def test_every_declared_symbol_is_exported():
    header = (ROOT / "include" / "sharedkv_c_abi.h").read_text()
    names = re.findall(r"SHAREDKV_API\s+[\w\s\*]+?\b(\w+)\s*\(", header)
    assert len(names) >= 12
    lib = library()
    for name in names:
        assert hasattr(lib, name), name


def test_struct_layouts_match_the_reference_abi():
    from npu_sparse_attn_sharedkv_int8.attention import _Args as AttentionArgs
    from npu_sparse_attn_sharedkv_int8.cache import _Args as CacheArgs
    lib = library()
    assert ctypes.sizeof(AttentionArgs) == 200 == lib.sharedkv_attention_args_size()
    assert ctypes.sizeof(CacheArgs) == 88 == lib.sharedkv_cache_args_size()
    assert AttentionArgs.tokens.offset == 144 and AttentionArgs.softmaxScale.offset == 196
    assert AttentionArgs.oriStride.offset == 112 and AttentionArgs.oriIndices.offset == 136
    assert CacheArgs.tokens.offset == 64 and CacheArgs.pairedSlots.offset == 80
    assert lib.sharedkv_attention_variant_count() == 23


def test_workspace_formula_matches_library():
    from npu_sparse_attn_sharedkv_int8 import c8_attention
    lib = library()
    for tokens in (1, 7, 64, 2048, 8192, 100000):
        assert lib.sharedkv_workspace_bytes(tokens) == c8_attention.workspace_bytes(tokens)
    assert c8_attention.WORKSPACE_BYTES == c8_attention.workspace_bytes(8192)


def test_host_side_rejections_need_no_gpu():
    lib = library()
    null = ctypes.c_void_p(0)
    assert lib.launch_cache_write(0, null, null) == -22
    assert lib.launch_sharedkv_c8_sparse(0, null, null) == -22
    assert lib.launch_sharedkv_c8_dense(0, null, null) == -22
    assert lib.sharedkv_attention(0, 0, 20, -1, null) == -22
    from npu_sparse_attn_sharedkv_int8.attention import _Args
    args = _Args(tokens=4, batch=1, heads=8, ratio=4, window=128, oriBlock=32, cmpBlock=32, topk=1024)
    assert lib.sharedkv_attention(ctypes.addressof(args), 0, 99, -1, null) == -2          # unknown variant
    assert lib.launch_sharedkv(0, null, None) == -22
    args.ratio = 2
    assert lib.sharedkv_attention(ctypes.addressof(args), 0, 0, -1, null) == -22         # general entry: ratio 1, 4 or 128 only
    args.ratio = 4
    args.oriIndices = 4
    assert lib.sharedkv_attention(ctypes.addressof(args), 0, 20, -1, null) == -22        # the C4 entry takes no explicit slots
    assert lib.sharedkv_attention(ctypes.addressof(args), 0, 20, -1, null) == -22         # null pointers
    assert b"variant" in lib.sharedkv_status_string(-2)
    assert b"invalid" in lib.sharedkv_status_string(-22)
    empty = _Args()
    assert lib.launch_sharedkv_c8_sparse(0, null, ctypes.byref(empty)) == 0               # zero tokens: nothing to do


def test_route_selector_and_abi_guard():
    from npu_sparse_attn_sharedkv_int8 import c8_attention
    from npu_sparse_attn_sharedkv_int8.attention import _Args
    with patch.dict(os.environ, {}, clear=True):
        assert c8_attention.enabled()
    for flag, expected in (("0", False), ("1", True)):
        with patch.dict(os.environ, SHAREDKV_C8_DECODE=flag):
            assert c8_attention.enabled() is expected
    with patch.dict(os.environ, SHAREDKV_C8_DECODE="typo"), pytest.raises(ValueError):
        c8_attention.enabled()
    valid = dict(heads=8, tokens=48, batch=8, ratio=4, window=128, oriBlock=32, cmpBlock=32, oriIndices=0, topk=1024)
    assert c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**valid)))
    for key, value in (("tokens", 0), ("batch", 0), ("heads", 16), ("ratio", 2), ("window", 129), ("oriBlock", 64),
                       ("cmpBlock", 64), ("oriIndices", 1), ("topk", 2048)):       # explicit slots need oriTopk > 0
        assert not c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**(valid | {key: value}))))
    # beyond the reference's C4 / C128 route (its general kernel's territory): the same CUDA kernels serve
    # ratio-1 layers (no compressed cache, so its block size is not looked at) and explicit original slots
    assert c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**(valid | dict(ratio=1, cmpBlock=0, topk=0)))))
    assert c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**(valid | dict(oriIndices=1, oriTopk=300)))))
    for batch, tokens in ((9, 49), (23, 138), (128, 768), (1024, 8192)):
        assert c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**(valid | dict(batch=batch, tokens=tokens)))))
    assert c8_attention.supported(SimpleNamespace(blocks=24, args=_Args(**(valid | dict(ratio=128, topk=0)))))


def test_cpu_tensors_are_rejected_not_emulated():
    from npu_sparse_attn_sharedkv_int8 import PreparedAttention, PreparedCacheWrite
    from tests.support import load_case
    case, ori_scale, cmp_scale, _ = load_case("unit_c4")
    with pytest.raises(ValueError, match="CUDA"):
        PreparedAttention(case, ori_scale, cmp_scale)
    cache = torch.zeros(2, 32, 1, 512, dtype=torch.int8)
    with pytest.raises(ValueError, match="CUDA"):
        PreparedCacheWrite(cache, torch.zeros(4, 512, dtype=torch.bfloat16), torch.zeros(4, dtype=torch.int32), torch.ones(512))


def test_missing_library_fails_loudly(tmp_path):
    from npu_sparse_attn_sharedkv_int8 import _paths
    with patch.object(_paths, "NATIVE_DIR", tmp_path), pytest.raises(RuntimeError, match="Missing native library"):
        _paths.native_path()


def test_frozen_scale_contract():
    from npu_sparse_attn_sharedkv_int8 import CacheQuantization
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        scale = torch.ones(512)
        scale[17] = bad
        with pytest.raises(ValueError):
            CacheQuantization(scale)
    quant = CacheQuantization.calibrate([torch.ones(3, 512)])
    before = quant.quantize(torch.linspace(-1, 1, 512).reshape(1, 512))
    quant.quantize(torch.full((2, 512), 1000.0))
    assert torch.equal(quant.quantize(torch.linspace(-1, 1, 512).reshape(1, 512)), before)
    tensors = {"layer.kv_cache_scale": torch.ones(512), "layer.kv_cache_offset": torch.zeros(512)}
    assert torch.equal(CacheQuantization.from_msmodelslim(tensors, "layer").scale, torch.ones(512))
    tensors["layer.kv_cache_offset"][0] = 1
    with pytest.raises(ValueError, match="nonzero offsets"):
        CacheQuantization.from_msmodelslim(tensors, "layer")


def test_request_sharding_is_balanced_and_complete():
    import bench
    lengths = bench.box_lengths(2048)
    for ranks in (1, 2, 4, 8):
        shards = bench.shard(lengths, ranks)
        assert sorted(i for s in shards for i in s) == list(range(2048))
        loads = [int((lengths[torch.tensor(s)] // 4 + lengths[torch.tensor(s)] // 128 + 256).sum()) for s in shards]
        assert max(loads) <= 1.02 * (sum(loads) / ranks)


def _two_rank_worker(rank, world, port, results):
    import torch.distributed as dist
    import bench
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        lengths = bench.box_lengths(256, seed=0)
        mine = bench.shard(lengths, world)[rank]
        # every rank derives the same partition on its own: no exchange is needed to agree on it
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        cost = int((lengths[torch.tensor(mine)] // 4 + lengths[torch.tensor(mine)] // 128 + 256).sum())
        total_ms, counts = bench.combine_ranks(10.0 + rank, [len(mine), cost], torch.device("cpu"), world)
        results[rank] = (gathered, total_ms, counts, cost)
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_requests_and_combine_timings():
    """World size 2 on the gloo backend: the ranks' request shards are disjoint, complete and
    balanced, and the whole-job figures are the slowest rank's time and the summed counts."""
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_two_rank_worker, args=(2, port, results), nprocs=2, join=True)
    assert set(results.keys()) == {0, 1}
    gathered, total_ms, counts, _ = results[0]
    assert results[1][0] == gathered
    assert sorted(gathered[0] + gathered[1]) == list(range(256)) and not set(gathered[0]) & set(gathered[1])
    assert total_ms == 11.0 and results[1][1] == 11.0
    assert counts[0] == 256 and counts[1] == results[0][3] + results[1][3]
    costs = [results[0][3], results[1][3]]
    assert max(costs) / min(costs) < 1.02


def test_work_split_invariants_on_the_host(tmp_path):
    """The device planner's arithmetic (csrc/work_split.h) compiled for the host and checked over
    22 000 random workloads: every tile of every live token in exactly one item, unique workspace
    entries below tokens + 160, no colliding partial-state slots or tickets, nobody beyond its quota
    (reference precedent: tests/cpp/test_schedule.cpp:35-107)."""
    import shutil
    import subprocess
    compiler = shutil.which("g++")
    if compiler is None:
        pytest.skip("no host C++ compiler")
    binary = tmp_path / "test_work_split"
    subprocess.run([compiler, "-std=c++17", "-O2", "-I", str(ROOT / "ascend-int8-attention_b200" / "csrc"),
                    str(ROOT / "tests" / "cpp" / "test_work_split.cpp"), "-o", str(binary)], check=True)
    done = subprocess.run([str(binary), "22000"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert "work split ok: 22000 workloads" in done.stdout


def test_paired_work_split_invariants_on_the_host(tmp_path):
    """The paired kernel's plan and tiling (csrc/work_split.h: pair_*) compiled for the host: every live
    token in exactly one item of one or two adjacent tokens, a CTA's items consecutive, owners below
    the grid, nobody more than one item over its quota, and the tiles of an item offering each token
    exactly the rows it may see (reference.py:229-234,243-245 with query_group = 2)."""
    import shutil
    import subprocess
    compiler = shutil.which("g++")
    if compiler is None:
        pytest.skip("no host C++ compiler")
    binary = tmp_path / "test_pair_split"
    subprocess.run([compiler, "-std=c++17", "-O2", "-I", str(ROOT / "ascend-int8-attention_b200" / "csrc"),
                    str(ROOT / "tests" / "cpp" / "test_pair_split.cpp"), "-o", str(binary)], check=True)
    done = subprocess.run([str(binary), "22000"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert "pair split ok: 22000 workloads" in done.stdout
