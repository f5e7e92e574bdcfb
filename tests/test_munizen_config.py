"""What needs no GPU of the Munizen design: reading its config.json, the order of its layer runs, the caches
its blocks ask for, tensor names, and the plain implementation's own consistency."""
import json
import os

import pytest
import torch

import plain_munizen as plain
from munizen_cases import CASES, attention_layer, config, delta_layer, write_model


def test_config_round_trip_and_registry(tmp_path):
    from carbon_engine_b200.config.munizen import MunizenConfig
    from carbon_engine_b200.config.registry import load_config
    for name, raw in CASES.items():
        folder = write_model(raw, str(tmp_path / name))
        arch, cfg = load_config(folder)
        assert arch.name == "Munizen" and cfg == MunizenConfig.from_dict(dict(raw))
        with open(os.path.join(folder, "config.json")) as fh:
            assert MunizenConfig.from_dict(json.load(fh)) == cfg
        assert list(cfg.layer_runs()) == plain.layer_runs(raw)
    assert MunizenConfig.from_dict(CASES["S"]).layer_runs() == (0, 1, 1, 1, 2)
    assert MunizenConfig.from_dict(CASES["Q"]).streams is None and MunizenConfig.from_dict(CASES["R"]).streams == 1


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].update(mask={"size": 4, "kind": "x"}), "mask"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "dense"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.pop("width"), "width"),
])
def test_config_errors_name_the_key(change, message):
    from carbon_engine_b200.config.base import ConfigError
    from carbon_engine_b200.config.munizen import MunizenConfig
    raw = json.loads(json.dumps(CASES["P"]))
    change(raw)
    with pytest.raises(ConfigError, match=message):
        MunizenConfig.from_dict(raw)


def test_schedule_caches_and_tensor_names():
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.munizen import MunizenConfig
    from carbon_engine_b200.config.registry import resolve_architecture
    from carbon_engine_b200.parts.base import BundleCacheSpec, PagedCacheSpec, StateCacheSpec
    raw = CASES["P"]
    cfg = MunizenConfig.from_dict(raw)
    model = resolve_architecture(raw).build_model(cfg, 256)
    assert [(c.block, c.cache) for c in model.schedule] == [(0, 0), (1, 1), (0, 2), (1, 3), (2, 4), (3, 5)]
    layout = dict(model.cache_layout())
    assert all(isinstance(s, BundleCacheSpec) and s.extra[0][1] == StateCacheSpec((48,), torch.float32) for s in layout.values())
    assert layout[0].main == StateCacheSpec((2, 24, 24), torch.float32) == layout[2].main
    # two key "heads" per key/value head (the two maps), values with a head count and size of their own
    assert layout[1].main == PagedCacheSpec(4, 16, 0, None, v_heads=2, v_head_dim=24)
    names = {s.name for s in model.all_tensor_specs()}
    assert {"embed", "head", "final.norm", "l0.shift", "l0.hc1.mix", "l1.hc2.in", "l1.mix.q.b", "l1.mix.lq2", "l0.mix.w2",
            "l0.mix.a.b", "l2.mlp.down", "l1.mix.o.b", "l3.norm2"} <= names
    assert "l0.norm2" not in names and "l0.hc2.in" not in names          # a layer without a feed-forward has neither
    assert model.streams == 2 and model.graph_safe


def test_a_size_left_to_the_checkpoint(tmp_path):
    """The rank of the decay's narrow projection is not in config.json: -1 takes the stored tensors' size."""
    from carbon_engine_b200.config.registry import load_config
    from carbon_engine_b200.weights.loader import WeightError, check_tensors
    from carbon_engine_b200.weights.safetensors_io import TensorDirectory
    folder = write_model(CASES["Q"], str(tmp_path / "Q"))
    path = os.path.join(folder, "config.json")
    raw = json.load(open(path))
    for layer in raw["layers"]:
        layer["mixer"].pop("rank", None)
    json.dump(raw, open(path, "w"))
    arch, cfg = load_config(folder)
    model = arch.build_model(cfg, 128)
    check_tensors(model.all_tensor_specs(), TensorDirectory(folder))
    model.load_weights(TensorDirectory(folder).get, torch.device("cpu"), torch.float32)
    delta = model.blocks[1].mixer
    assert delta.rank == 7 and delta.inp.out_features[-1] == 7 and delta.inp.weight.shape[0] == delta.inp.padded_out
    raw["layers"][1]["mixer"]["dim"] = 20                     # but a size that is given must fit
    json.dump(raw, open(path, "w"))
    arch, cfg = load_config(folder)
    with pytest.raises(WeightError, match="wrong shapes"):
        check_tensors(arch.build_model(cfg, 128).all_tensor_specs(), TensorDirectory(folder))


def test_cache_storage_holds_the_blocks_states_and_value_pools(tmp_path):
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.config.munizen import MunizenConfig
    from carbon_engine_b200.config.registry import resolve_architecture
    from carbon_engine_b200.parts.model import LayerCall
    cfg = MunizenConfig.from_dict(CASES["P"])
    model = resolve_architecture(CASES["P"]).build_model(cfg, 128)
    st = CacheStorage(model, torch.float32, torch.device("cpu"), 8, 10, 3, 128)
    assert len(st.groups) == 1
    a, d = st.view(LayerCall(1, 1)), st.view(LayerCall(0, 2))
    assert a.k_pool.shape == (10, 4, 8, 16) and a.v_pool.shape == (10, 2, 8, 24) and a.extra["shift"].shape == (3, 48)
    assert d.state.shape == (3, 2, 24, 24) and d.state.dtype == torch.float32 and d.extra["shift"].shape == (3, 48)
    d.state[1].fill_(2.0); d.extra["shift"][1].fill_(3.0)
    st.zero_state(1)
    assert float(d.state.abs().sum()) == 0.0 and float(d.extra["shift"].abs().sum()) == 0.0
    assert st.bytes_per_token() == 3 * (4 * 16 + 2 * 24) * 4         # three attention calls in the schedule, float32
    assert st.state_bytes() == 3 * 4 * (6 * 48 + 2 * 2 * 24 * 24 + 3 * 16 * 16)


def test_plain_recurrence_carries_its_state():
    """The plain delta rule over two halves, the state handed over, equals the whole; and the plain mask."""
    g = torch.Generator().manual_seed(0)
    H, d, W, L, T = 2, 6, 10, 3, 9
    m = {"heads": H, "dim": d}
    w = {f"x.{n}": torch.randn(H * d, W, generator=g, dtype=torch.float64) * 0.3 for n in ("r", "k", "v", "a", "g")}
    w.update({"x.w1": torch.randn(L, W, generator=g, dtype=torch.float64), "x.w2": torch.randn(H * d, L, generator=g, dtype=torch.float64),
              "x.w0": torch.randn(H * d, generator=g, dtype=torch.float64), "x.a.b": torch.randn(H * d, generator=g, dtype=torch.float64),
              "x.norm": torch.ones(H * d, dtype=torch.float64), "x.o": torch.randn(W, H * d, generator=g, dtype=torch.float64)})
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    whole = plain.general_delta(h, w, "x.", m, 1e-6)
    S = torch.zeros(H, d, d, dtype=torch.float64)
    parts = torch.cat([plain.general_delta(h[:4], w, "x.", m, 1e-6, S), plain.general_delta(h[4:], w, "x.", m, 1e-6, S)])
    assert torch.allclose(whole, parts, atol=1e-12)
    mask = plain.chunk_mask(7, 3)
    assert mask[5].tolist() == [False, False, False, True, True, True, False] and mask[3].tolist()[:4] == [False, False, False, True]
