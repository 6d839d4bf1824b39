"""Calibration tooling and the plugin's calibrate mode, on the CPU with stand-in serving classes
(reference: npu_sparse_attn_sharedkv_int8/calibration.py:17-73, vllm_plugin.py:28-66,
docs/kv-cache.md:51-66)."""
from types import SimpleNamespace

import pytest
import torch

from npu_sparse_attn_sharedkv_int8 import calibration, vllm_adapter, vllm_plugin
from tests.fakes import FakeAttentionImpl, FakeDraftModel


def test_observer_collects_only_behind_the_marker_and_only_valid_slots(tmp_path):
    observer = calibration.CacheObserver(tmp_path, save_interval=1e9)
    cache = torch.zeros(4, 32, 1, 512, dtype=torch.bfloat16)
    rows = torch.randn(6, 512).bfloat16()
    slots = torch.tensor([0, 5, -1, 127, 128, 64])                   # -1 and 128 are not written by the cache writer
    observer.observe("l0", "ori", cache, rows, slots)                # no marker: nothing is recorded
    assert not observer.stats and not list(tmp_path.glob("rank_*.pt"))
    observer.marker.touch()
    observer.observe("l0", "ori", cache, rows, slots)
    observer.observe("l0", "ori", cache, rows[:2] * 3, torch.tensor([[1, 2], [9, 0]]))      # pair form; page 9 is out of range
    valid = torch.tensor([True, True, False, True, False, True])
    expected = torch.maximum(rows[valid].float().abs().amax(0), (rows[0] * 3).float().abs())
    assert torch.equal(observer.stats["l0.ori"][0], expected) and int(observer.stats["l0.ori"][1]) == 5
    observer.observe("l0", "cmp", cache, None, slots)                # empty updates are ignored
    with pytest.raises(ValueError):
        observer.observe("l0", "ori", cache, torch.zeros(2, 256), slots[:2])
    observer.marker.unlink()
    observer.observe("l0", "ori", cache, rows, slots)                # marker gone: the call flushes
    saved = torch.load(tmp_path / "rank_00.pt", weights_only=True)
    assert saved["version"] == 1 and saved["rank"] == 0 and saved["stats"]["l0.ori"]["rows"] == 5
    assert torch.equal(saved["stats"]["l0.ori"]["maximum"], expected)
    assert not list(tmp_path.glob("*.tmp.*"))                        # written through a rename


def test_merge_gives_a_scale_file_the_adapter_loads(tmp_path, monkeypatch):
    stats = []
    for rank in range(3):
        g = torch.Generator().manual_seed(rank)
        entry = {"l0.ori": {"maximum": torch.rand(512, generator=g) * 5, "rows": 10 + rank},
                 "l0.cmp": {"maximum": torch.rand(512, generator=g), "rows": 3}}
        if rank == 2:
            entry["l1.ori"] = {"maximum": torch.zeros(512), "rows": 1}         # all-zero channels hit the floor
        path = tmp_path / f"rank_{rank:02d}.pt"
        torch.save({"version": 1, "rank": rank, "pid": 1, "stats": entry}, path)
        stats.append(entry)
    payload = calibration.merge_ranks(sorted(tmp_path.glob("rank_*.pt")), margin=1.1, provenance={"model": "unit-test"},
                                      required_keys=["l0.ori", "l0.cmp"])
    top = torch.stack([s["l0.ori"]["maximum"] for s in stats]).amax(0)
    assert torch.equal(payload["scales"]["l0.ori"], (top * (1.1 / 127)).clamp_min(1e-8))
    assert payload["observed_rows_across_ranks"]["l0.ori"] == 33 and payload["margin"] == 1.1
    assert torch.equal(payload["scales"]["l1.ori"], torch.full((512,), 1e-8))
    assert set(payload["source_sha256"]) == {"rank_00.pt", "rank_01.pt", "rank_02.pt"}
    with pytest.raises(ValueError, match="required"):
        calibration.merge_ranks(sorted(tmp_path.glob("rank_*.pt")), required_keys=["l7.ori"])
    out = calibration.save_scales(payload, tmp_path / "scales.pt")
    monkeypatch.setenv("SHAREDKV_SCALES", str(out))
    vllm_adapter.load_scales.cache_clear()
    loaded = vllm_adapter.load_scales()
    assert set(loaded) == {"l0.ori", "l0.cmp", "l1.ori"} and torch.equal(loaded["l0.cmp"], payload["scales"]["l0.cmp"])
    vllm_adapter.load_scales.cache_clear()
    # the same rank twice (two nodes that both wrote rank_00.pt) is refused
    torch.save({"version": 1, "rank": 0, "pid": 2, "stats": stats[0]}, tmp_path / "rank_00_node2.pt")
    with pytest.raises(ValueError, match="twice"):
        calibration.merge_ranks(sorted(tmp_path.glob("rank_*.pt")))


def test_plugin_calibrate_mode_observes_writes_and_reroutes_the_draft_writer(tmp_path, monkeypatch):
    monkeypatch.setattr(vllm_plugin, "_registered", False)
    original_write, original_store = FakeAttentionImpl._write_kv_cache, FakeDraftModel._store_standard_swa_kv
    monkeypatch.setenv("SHAREDKV_INT8_MODE", "calibrate")
    monkeypatch.setenv("SHAREDKV_CALIBRATION_DIR", str(tmp_path))
    monkeypatch.setenv("SHAREDKV_ATTENTION_IMPL", "tests.fakes:FakeAttentionImpl")
    monkeypatch.setenv("SHAREDKV_DRAFT_MODEL", "tests.fakes:FakeDraftModel")
    try:
        vllm_plugin.register()
        (tmp_path / "collect").touch()
        impl = FakeAttentionImpl("model.layers.3.self_attn")
        cache = torch.zeros(2, 32, 1, 512, dtype=torch.bfloat16)
        rows = torch.randn(4, 512).bfloat16()
        impl._write_kv_cache(cache, rows, torch.tensor([[0, 1], [0, 2], [1, 0], [-1, 0]]), quantize=True)
        assert impl.writes == [((4, 512), (4, 2), True)]                       # BF16 execution is unchanged
        assert torch.equal(cache[0, 1, 0], rows[0])
        observer = vllm_plugin._observer
        assert int(observer.stats["model.layers.3.self_attn.cmp"][1]) == 3
        # the draft model's target-context rows take the same route (flat slots are converted first)
        impl.swa_cache_layer.kv_cache = [cache]
        attn = SimpleNamespace(dsa_attn=SimpleNamespace(swa_cache_layer=impl.swa_cache_layer,
                                                       dsa_attn=SimpleNamespace(impl=impl)))
        FakeDraftModel()._store_standard_swa_kv(rows[:2] * 2, torch.tensor([33, 40]), attn=attn)
        assert impl.writes[-1] == ((2, 512), (2, 2), False)
        assert int(observer.stats["model.layers.3.self_attn.ori"][1]) == 2
        assert torch.equal(cache[1, 1, 0], rows[0] * 2)
        FakeDraftModel()._store_standard_swa_kv(rows[:0], torch.zeros(0, dtype=torch.long), attn=attn)   # nothing to store
        observer.flush()
        assert (tmp_path / "rank_00.pt").exists()
    finally:
        FakeAttentionImpl._write_kv_cache, FakeDraftModel._store_standard_swa_kv = original_write, original_store
        monkeypatch.setattr(vllm_plugin, "_registered", False)
