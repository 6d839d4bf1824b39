"""Stand-ins for the serving stack's classes the plugin hooks (the reference patches vllm-ascend's
AscendDSAImpl and DeepseekV4DSparkModel; its device tests use SimpleNamespace fakes the same way,
tests/npu/test_adapter.py:77-92)."""
from dataclasses import dataclass
from types import SimpleNamespace

import torch


@dataclass(frozen=True)
class Plan:
    sparse_attn_op: object = None

    @staticmethod
    def format_dsa_slot_mapping(slots, block_size):
        return torch.stack((slots // block_size, slots % block_size), dim=1)


class FakeAttentionImpl:
    """Has what the plugin wraps: get_kv_plan and _write_kv_cache (a BF16 scatter)."""
    head_dim = 512
    turboquant = None

    def __init__(self, prefix="model.layers.0.self_attn"):
        self.swa_cache_layer = SimpleNamespace(prefix=prefix + ".swa_cache", block_size=32, kv_cache=None)
        self.writes = []

    def get_kv_plan(self):
        return Plan()

    def _write_kv_cache(self, cache, kv, slot_mapping, *, quantize):
        self.writes.append((tuple(kv.shape), tuple(slot_mapping.shape), quantize))
        pages, offsets = (slot_mapping[:, 0], slot_mapping[:, 1]) if slot_mapping.ndim == 2 else (
            slot_mapping // cache.shape[1], slot_mapping % cache.shape[1])
        keep = (pages >= 0) & (pages < cache.shape[0])
        cache[pages[keep].long(), offsets[keep].long(), 0] = kv.reshape(-1, 512)[keep].to(cache.dtype)


class FakeDraftModel:
    def _store_standard_swa_kv(self, shared_kv, slot_mapping, attn=None):
        raise AssertionError("the plugin should have replaced this writer")
