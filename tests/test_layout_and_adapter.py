"""Host-side logic of the serving glue: the compact page planner, the scale file loader and the
plugin switch.  No GPU is needed (tests/test_gpu_adapter.py drives the same objects on one)."""
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

from npu_sparse_attn_sharedkv_int8 import cache_layout, vllm_plugin


@dataclass(frozen=True)
class Spec:
    dtype: torch.dtype
    page_size_bytes: int
    head_size: int = 512
    num_kv_heads: int = 1
    block_size: int = 32
    scale_dim: int = 0
    scale_dtype: torch.dtype = torch.float32
    page_size_padded: int | None = None
    pages: int = 10
    model_version: str | None = "deepseek_v4"

    def max_memory_usage_pages(self, config):
        return self.pages


def group(specs):
    inner = SimpleNamespace(kv_cache_specs=specs, page_size_bytes=sum(s.page_size_bytes for s in specs.values()),
                            max_memory_usage_pages=lambda config: max(s.pages for s in specs.values()))
    return SimpleNamespace(layer_names=list(specs), kv_cache_spec=inner)


def serving_groups(layers=38):
    """`layers` INT8 D=512 caches of 16 384 bytes per block in one group (the reference's compact
    serving geometry: 38 x 16 384 = 622 592 bytes per block), an FP32 state group beside it."""
    attention = {f"model.layers.{i}.attn.cache": Spec(torch.int8, 16384) for i in range(layers)}
    states = {f"model.layers.{i}.state": Spec(torch.float32, 4160, head_size=65, block_size=16) for i in range(4)}
    return [group(attention), group(states)]


def test_packed_layout_gives_the_reference_serving_stride():
    groups = serving_groups()
    stride, offsets = cache_layout.packed_layout(groups)
    assert stride == 622592 == cache_layout.pool_bytes_per_block(groups)
    attention = sorted(v for k, v in offsets.items() if k.endswith("cache"))
    assert attention == [16384 * i for i in range(38)]                 # whole rows, no gaps, no overlap
    assert all(v % 512 == 0 for v in attention)
    states = sorted(v for k, v in offsets.items() if k.endswith("state"))
    assert states == [4160 * i for i in range(4)] and all(v % 4 == 0 for v in states)
    assert cache_layout.uses_compact(groups) and not cache_layout.uses_compact([groups[1]])
    assert cache_layout.max_memory_usage(None, groups) == stride * 20


def test_layout_matches_the_reference_planner_on_vllm_specs():
    """tests/golden/cache_layout.json holds what the reference's own uses_compact / packed_layout /
    group_specs (cache_layout.py:24-85 of the reference) returned for vLLM's real cache-spec
    objects; the same numbers fed to this build's duck-typed planner must give the same strides,
    offsets, compact decision and group split."""
    import json
    from pathlib import Path
    golden = json.loads((Path(__file__).resolve().parent / "golden" / "cache_layout.json").read_text())

    def spec_of(d):
        return Spec(getattr(torch, d["dtype"]), d["page_size_bytes"], head_size=d["head_size"],
                    num_kv_heads=d["num_kv_heads"], block_size=d["block_size"], page_size_padded=d["page_size_padded"],
                    model_version=d["model_version"])

    checked = 0
    for name, want in golden.items():
        if name == "group_specs":
            continue
        groups = [group({d["name"]: spec_of(d) for d in layers}) for layers in want["groups"]]
        stride, offsets = cache_layout.packed_layout(groups)
        assert stride == want["stride"] == cache_layout.pool_bytes_per_block(groups), name
        assert offsets == want["offsets"], name
        assert cache_layout.uses_compact(groups) == want["uses_compact"], name
        checked += 1
    assert checked >= 5 and golden["serving38"]["stride"] == 622592
    @dataclass(frozen=True)
    class PageSpec:
        """As vLLM's specs: the page size follows from the geometry unless a padded size is set."""
        dtype: torch.dtype
        head_size: int
        unpadded: int
        page_size_padded: int | None
        model_version: str | None

        @property
        def page_size_bytes(self):
            return self.unpadded if self.page_size_padded is None else self.page_size_padded

    def page_spec_of(d):
        made = PageSpec(getattr(torch, d["dtype"]), d["head_size"], d["unpadded_page_size_bytes"],
                        d["page_size_padded"], d["model_version"])
        assert made.page_size_bytes == d["page_size_bytes"]
        return made

    want = golden["group_specs"]
    inputs = []
    for layers in want["groups"]:
        specs = {d["name"]: page_spec_of(d) for d in layers}
        inputs.append(SimpleNamespace(kv_cache_specs=specs, page_size_bytes=sum(s.page_size_bytes for s in specs.values())))
    out = cache_layout.group_specs(inputs)
    assert [names for names, _ in out] == [[d["name"] for d in g] for g in want["split"]]
    for (names, specs), g in zip(out, want["split"]):
        for d in g:
            assert specs[d["name"]].page_size_bytes == d["page_size_bytes"]
            assert specs[d["name"]].page_size_padded == d["page_size_padded"]


def test_layout_orders_by_size_aligns_scales_and_rejects_duplicates():
    specs = {"small": Spec(torch.int8, 1000, head_size=100), "big": Spec(torch.int8, 16384),
             "scaled": Spec(torch.int8, 4100, head_size=128, scale_dim=1)}
    stride, offsets = cache_layout.packed_layout([group(specs)])
    assert offsets["big"] == 0 and offsets["scaled"] == 16384 and offsets["small"] == 16384 + 4100
    assert stride == -(-(16384 + 4100 + 1000) // 512) * 512
    with pytest.raises(ValueError):
        cache_layout.packed_layout([group({"x": Spec(torch.int8, 16384)}), group({"x": Spec(torch.int8, 16384)})])


def test_group_specs_splits_state_groups_at_the_attention_budget():
    c4 = SimpleNamespace(kv_cache_specs={"c4": Spec(torch.int8, 16384), "indexer": Spec(torch.int8, 4224, head_size=132)},
                         page_size_bytes=16384 + 4224)
    c128 = SimpleNamespace(kv_cache_specs={"c128": Spec(torch.int8, 16384)}, page_size_bytes=16384)
    states = SimpleNamespace(kv_cache_specs={f"s{i}": Spec(torch.float32, 16384, page_size_padded=32768) for i in range(5)},
                             page_size_bytes=5 * 16384)
    out = cache_layout.group_specs([c4, c128, states])
    sizes = [sum(s.page_size_bytes for s in specs.values()) for _, specs in out]
    assert [names for names, _ in out][:2] == [["c4", "indexer"], ["c128"]]
    assert all(size <= 32768 for size in sizes) and sum(len(n) for n, _ in out) == 8
    assert all(s.page_size_padded is None for _, specs in out for s in specs.values())


def test_cache_config_allocate_and_views_on_cpu():
    groups = serving_groups(layers=3)
    stride = cache_layout.pool_bytes_per_block(groups)
    config = SimpleNamespace(parallel_config=SimpleNamespace(pipeline_parallel_size=1))
    blocks, descriptors = cache_layout.cache_config(config, groups, available_memory=10 * stride + 17)
    assert blocks == 10 and len(descriptors) == 7 and all(d.block_stride == stride and d.size == 10 * stride for d in descriptors)
    raw = cache_layout.allocate(groups, blocks, descriptors, "cpu", alignment=4096)
    base = min(t.data_ptr() for t in raw.values())
    assert base % 4096 == 0
    views = cache_layout.reshape(groups, blocks, raw)
    _, offsets = cache_layout.packed_layout(groups)
    for name, (view, *rest) in views.items():
        spec = {**groups[0].kv_cache_spec.kv_cache_specs, **groups[1].kv_cache_spec.kv_cache_specs}[name]
        assert view.dtype == spec.dtype and view.shape == (10, spec.block_size, 1, spec.head_size)
        assert view.stride(0) * view.element_size() == stride and view.data_ptr() - base == offsets[name]
        assert not rest
    # writing one layer's pages leaves every other layer untouched
    target = views["model.layers.1.attn.cache"][0]
    target.fill_(7)
    assert int((views["model.layers.0.attn.cache"][0] != 0).sum()) == 0
    assert int((views["model.layers.2.attn.cache"][0] != 0).sum()) == 0
    with pytest.raises(ValueError):
        cache_layout.allocate(groups, blocks, descriptors[:-1], "cpu")
    with pytest.raises(ValueError):
        cache_layout.cache_config(SimpleNamespace(parallel_config=SimpleNamespace(pipeline_parallel_size=2)), groups, stride)
    with pytest.raises(RuntimeError):
        cache_layout.install()


def test_scale_file_contract(tmp_path, monkeypatch):
    from npu_sparse_attn_sharedkv_int8 import vllm_adapter
    good = {"protocol": "sharedkv-c8-v1", "scales": {"l0.ori": torch.full((512,), 0.01)}}
    for name, payload, ok in (("good.pt", good, True),
                              ("protocol.pt", {**good, "protocol": "other"}, False),
                              ("shape.pt", {**good, "scales": {"l0.ori": torch.ones(256)}}, False),
                              ("sign.pt", {**good, "scales": {"l0.ori": -torch.ones(512)}}, False)):
        path = tmp_path / name
        torch.save(payload, path)
        monkeypatch.setenv("SHAREDKV_SCALES", str(path))
        vllm_adapter.load_scales.cache_clear()
        if ok:
            assert set(vllm_adapter.load_scales()) == {"l0.ori"}
        else:
            with pytest.raises(ValueError):
                vllm_adapter.load_scales()
    monkeypatch.delenv("SHAREDKV_SCALES")
    vllm_adapter.load_scales.cache_clear()
    with pytest.raises(ValueError):
        vllm_adapter.load_scales()
    with pytest.raises(ValueError):      # D != 512 layers are refused before anything touches a device
        vllm_adapter.LayerRuntime(SimpleNamespace(swa_cache_layer=SimpleNamespace(prefix="l0.swa_cache"), head_dim=128))


def test_plugin_switch(monkeypatch):
    monkeypatch.delenv("SHAREDKV_INT8_MODE", raising=False)
    vllm_plugin.register()                                  # unset: nothing happens
    assert vllm_plugin.layer_prefix(SimpleNamespace(swa_cache_layer=SimpleNamespace(prefix="m.l3.swa_cache"))) == "m.l3"
    for mode in ("fp8", "calibrate"):
        monkeypatch.setenv("SHAREDKV_INT8_MODE", mode)
        with pytest.raises(ValueError):
            vllm_plugin.register()
    monkeypatch.setenv("SHAREDKV_INT8_MODE", "int8")
    monkeypatch.delenv("SHAREDKV_ATTENTION_IMPL", raising=False)
    with pytest.raises(ValueError):
        vllm_plugin.register()
