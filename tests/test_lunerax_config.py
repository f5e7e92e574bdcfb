"""Lunerax on the CPU: the typed configuration, the model's tensors and caches, and the plain implementation's own
consistency (its recurrence and its windows, which the GPU tests then lean on)."""
import json

import numpy as np
import pytest
import torch

import plain_lunerax as plain
from lunerax_cases import CASES, attention, config, delta, latent, write_model


def build(raw, max_positions=256):
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.registry import resolve_architecture
    arch = resolve_architecture(raw)
    cfg = arch.parse_config(dict(raw))
    return cfg, arch.build_model(cfg, max_positions)


def test_config_round_trip_and_registry():
    from carbon_engine_b200.config.lunerax import LuneraxConfig
    for name, raw in CASES.items():
        cfg, model = build(raw)
        assert isinstance(cfg, LuneraxConfig) and cfg.architecture == "Lunerax"
        again = LuneraxConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())))
        assert again == cfg, name
        assert len(model.blocks) == len(raw["layers"])


@pytest.mark.parametrize("bad, text", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"].update(mask={"keep_first": 2}), "'mask'"),
    (lambda r: r["layers"][2]["mixer"].update(mask={"size": 4, "keep_first": 2}), "'mask'"),
    (lambda r: r.update(norm={"eps": 0.0}), "positive"),
    (lambda r: r["layers"][3]["mixer"].update(vdim=20), "v_mix"),
    (lambda r: r.update(token_side={"dim": 0}), "token_side"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts") if r["layers"][1]["mlp"] else r["layers"][0]["mlp"].update(kind="experts"), "mlp"),
])
def test_config_errors_name_the_key(bad, text):
    from carbon_engine_b200.config.base import ConfigError
    from carbon_engine_b200.config.lunerax import LuneraxConfig
    raw = json.loads(json.dumps(CASES["A"]))
    bad(raw)
    with pytest.raises(ConfigError, match=text):
        LuneraxConfig.from_dict(raw)


def test_tensors_caches_and_value_roles():
    from carbon_engine_b200.parts.base import BundleCacheSpec, PagedCacheSpec, StateCacheSpec
    cfg, model = build(CASES["A"])
    names = {s.name: s.shape for s in model.all_tensor_specs()}
    assert names["side.embed"] == (97, 5 * 5) and names["l0.mix.vmix"] == () and names["l3.mix.vmix"] == ()
    assert names["l1.mix.q.conv"] == (16, 4) and names["l1.mix.v.conv"] == (48, 4) and names["l1.mix.a2"] == (32, 5)
    assert names["l2.mix.dkv"] == (14 + 8, 40) and names["l2.mix.uk"] == (36, 14) and names["l4.mix.norm"] == (6,)
    assert "l3.mlp.gate" not in names and "l4.mlp.gate" in names and names["final.norm.b"] == (40,)
    roles = [getattr(b.mixer, "value_mix", None) for b in model.blocks]
    assert roles == ["source", None, None, "blend", None]
    layout = dict(model.cache_layout())
    assert layout[0] == PagedCacheSpec(2, 16, 0, None, v_heads=2, v_head_dim=24)          # kept first tokens: no page is given back
    assert layout[3] == PagedCacheSpec(2, 8, 7, None, v_heads=2, v_head_dim=24)           # a plain window
    assert layout[2] == PagedCacheSpec(1, 14 + 8, 9, None, v_heads=1, v_head_dim=0)       # one row per token, no value pool
    assert isinstance(layout[1], BundleCacheSpec) and layout[1].main == StateCacheSpec((4, 8, 12), torch.float32)
    assert layout[1].extra == (("conv", StateCacheSpec((3, 2 * 2 * 8 + 4 * 12), torch.float32)),)
    # ranks left to the checkpoint
    raw = json.loads(json.dumps(CASES["A"]))
    for k in ("a_rank", "g_rank"):
        del raw["layers"][1]["mixer"][k]
    _, model = build(raw)
    assert {s.name: s.shape for s in model.all_tensor_specs()}["l1.mix.a1"] == (-1, 40)


def test_random_model_folder_is_read_back_by_name(tmp_path):
    from carbon_engine_b200.weights.loader import check_tensors
    from carbon_engine_b200.weights.safetensors_io import TensorDirectory
    folder = write_model(CASES["C"], str(tmp_path / "C"))
    cfg, model = build(json.load(open(f"{folder}/config.json")))
    check_tensors(model.all_tensor_specs(), TensorDirectory(folder), model.all_ignorable_tensors())
    pcfg, w = plain.read_model(folder)
    assert set(w) == {s.name for s in model.all_tensor_specs()} and pcfg["token_side"]["dim"] == 11


def test_plain_window_keeps_first_tokens_and_plain_recurrence_hands_over():
    """The oracle's own mask, and its recurrence run in two halves from a handed-over state against one run."""
    assert plain.visible(30, 30, 5, 2) and plain.visible(30, 26, 5, 2) and not plain.visible(30, 25, 5, 2)
    assert plain.visible(30, 1, 5, 2) and not plain.visible(30, 2, 5, 2) and not plain.visible(3, 4, 5, 2)
    assert plain.visible(30, 2, 0, 0)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(9, 2, 4, generator=g, dtype=torch.float64)
    k, v = torch.randn(9, 1, 4, generator=g, dtype=torch.float64), torch.randn(9, 1, 3, generator=g, dtype=torch.float64)
    out = plain.masked_softmax_attention(q, k, v, 0.7, 2.0, 3, 1)
    s = 2.0 * torch.tanh(0.7 * (q[8, 1] @ k[[0, 6, 7, 8], 0].T) / 2.0)
    assert torch.allclose(out[8, 1], torch.softmax(s, 0) @ v[[0, 6, 7, 8], 0])
    x = torch.randn(7, 3, generator=g, dtype=torch.float64)
    taps = torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = plain.causal_conv_silu(x, taps)
    z = taps[:, 3] * x[5] + taps[:, 2] * x[4] + taps[:, 1] * x[3] + taps[:, 0] * x[2]
    assert torch.allclose(y[5], z * torch.sigmoid(z)) and torch.allclose(y[0], plain.silu(taps[:, 3] * x[0]))
