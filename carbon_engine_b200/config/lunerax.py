"""Typed configuration of the Lunerax architecture.

config.json names the design with ``"architecture": "Lunerax"`` and describes the model layer by layer:

* ``vocab``, ``width``: vocabulary and residual width; ``embedding`` = ``{"scale"}`` multiplies the embedding rows;
* ``layers``: a list of ``{"type", "mixer", "mlp"}``.  ``type`` is
  ``"attention"`` (softmax attention without rotation: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``,
  ``mask`` = ``{"size", "keep_first"}``, ``v_mix``),
  ``"latent_attention"`` (``heads``, ``dim``, ``rot_dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``,
  ``rot`` = ``{"dims", "base"}``, ``mask`` = ``{"size"}``) or
  ``"channel_delta"`` (the gated delta rule with a decay per key channel: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
  ``conv`` taps);  ``mlp`` is ``{"kind": "dense", "ff"}`` or null;
* ``norm`` = ``{"eps"}``: the epsilon of the layer norms and of the mixers' RMS norms;
* ``token_side`` = ``{"dim"}``: the per-layer token input's width (absent: none);
* ``logit_softcap``: the logits become cap * tanh(logits / cap) (absent: no cap).

What config.json does not give is taken from the stored tensors' shapes (the ranks of the delta rule's two narrow
projections), unless the mixer's entry names them (``a_rank``, ``g_rank``), which a model with random weights needs.
``max_position_embeddings`` and ``eos_token_id`` are optional additions of this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, token_id_list

ATTENTION, LATENT_ATTENTION, CHANNEL_DELTA = "attention", "latent_attention", "channel_delta"
DEFAULT_MAX_POSITIONS = 32768


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, got {v!r}")
    return v


def _float(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _mask(m: Dict[str, Any], where: str, allowed: Tuple[str, ...]) -> None:
    mask = m.get("mask")
    if mask is None:
        return
    if not isinstance(mask, dict) or not set(mask) <= set(allowed) or "size" not in mask:
        raise ConfigError(f"config.json: {where}'mask' must be an object with 'size'" +
                          (" and optionally 'keep_first'" if "keep_first" in allowed else "") + f", got {mask!r}")
    _int(mask, "size", where + "mask: ")
    if mask.get("keep_first") is not None:
        _int(mask, "keep_first", where + "mask: ", 0)


def _check_layer(i: int, layer: Any) -> Dict[str, Any]:
    where = f"layers[{i}]: "
    if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
        raise ConfigError(f"config.json: {where}an object with 'type', 'mixer' and 'mlp' is expected")
    kind, m = layer.get("type"), layer["mixer"]
    if kind == ATTENTION:
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} kv_heads")
        _int(m, "dim", where); _int(m, "vdim", where); _float(m, "scale", where)
        if m.get("softcap") is not None and _float(m, "softcap", where) < 0.0:
            raise ConfigError(f"config.json: {where}softcap must not be negative")
        _mask(m, where, ("size", "keep_first"))
    elif kind == LATENT_ATTENTION:
        for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            _int(m, key, where)
        _float(m, "scale", where)
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
        dims = _int(rot, "dims", where + "rot: ", 2)
        if dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most rot_dim={m['rot_dim']}")
        if _float(rot, "base", where + "rot: ") <= 0.0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        _mask(m, where, ("size",))
    elif kind == CHANNEL_DELTA:
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} kv_heads")
        _int(m, "dim", where); _int(m, "vdim", where); _int(m, "conv", where)
        for key in ("a_rank", "g_rank"):
            if m.get(key) is not None:
                _int(m, key, where)
    else:
        raise ConfigError(f"config.json: {where}unknown layer type {kind!r} ({ATTENTION}, {LATENT_ATTENTION}, {CHANNEL_DELTA})")
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense', got {mlp!r}")
        _int(mlp, "ff", where + "mlp: ")
    return {"type": kind, "mixer": copy.deepcopy(m), "mlp": copy.deepcopy(mlp)}


@dataclass(frozen=True)
class LuneraxConfig(ModelConfig):
    width: int = 0
    layers: Tuple[Dict[str, Any], ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    token_side_dim: int = 0

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "LuneraxConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        checked = tuple(_check_layer(i, layer) for i, layer in enumerate(layers))
        mixed = [l["mixer"] for l in checked if l["type"] == ATTENTION and l["mixer"].get("v_mix")]
        if len({m["kv_heads"] * m["vdim"] for m in mixed}) > 1:
            raise ConfigError("config.json: layers with 'v_mix' must agree in kv_heads * vdim (their values are blended)")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _float(norm, "eps", "norm: ")
        if eps <= 0.0:
            raise ConfigError(f"config.json: norm eps={eps} must be positive")
        scale = 1.0
        if raw.get("embedding") is not None:
            if not isinstance(raw["embedding"], dict):
                raise ConfigError("config.json: 'embedding' must be an object with 'scale'")
            scale = _float(raw["embedding"], "scale", "embedding: ")
        cap = 0.0
        if raw.get("logit_softcap") is not None:
            cap = _float(raw, "logit_softcap", "")
            if cap < 0.0:
                raise ConfigError("config.json: logit_softcap must not be negative")
        side = 0
        if raw.get("token_side") is not None:
            if not isinstance(raw["token_side"], dict):
                raise ConfigError("config.json: 'token_side' must be an object with 'dim'")
            side = _int(raw["token_side"], "dim", "token_side: ")
        max_pos = raw.get("max_position_embeddings")
        max_pos = DEFAULT_MAX_POSITIONS if max_pos is None else _int(raw, "max_position_embeddings", "")
        eos = token_id_list(raw.get("eos_token_id"))
        for t in raw.get("_generation_eos_token_ids", []):
            if t not in eos:
                eos.append(t)
        return cls(architecture="Lunerax", vocab_size=vocab, max_position_embeddings=max_pos, eos_token_ids=tuple(eos),
                   width=width, layers=checked, norm_eps=eps, embedding_scale=scale, logit_softcap=cap, token_side_dim=side)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Lunerax", "vocab": self.vocab_size, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale}}
        if self.logit_softcap > 0.0:
            out["logit_softcap"] = self.logit_softcap
        if self.token_side_dim > 0:
            out["token_side"] = {"dim": self.token_side_dim}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out


def sketch_config(vocab: int, width: int, n_layers: int, heads: int, kv_heads: int, head_dim: int, ff: int, window: int = 1024,
                  keep_first: int = 4, side_dim: int = 0, max_positions: int = DEFAULT_MAX_POSITIONS, eps: float = 1e-6,
                  rope_base: float = 10000.0, softcap: float = 30.0, logit_softcap: float = 30.0) -> LuneraxConfig:
    """A configuration of the usual proportions from a few sizes, for random-weight models (the command line's
    ``tiny-model``, measurements): layers go attention, delta rule, delta rule, latent attention and again; attention heads of
    ``head_dim`` for keys and values alike with blended values; delta heads of ``head_dim`` filling the width; latents of a
    quarter of the width (keys/values) and half of it (queries) with a rotated part of half a head."""
    delta_heads = max(1, width // head_dim)
    rot = max(2, head_dim // 4 * 2)
    kinds = (ATTENTION, CHANNEL_DELTA, CHANNEL_DELTA, LATENT_ATTENTION)
    layers = []
    for i in range(n_layers):
        kind = kinds[i % 4]
        if kind == ATTENTION:
            m = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                 "softcap": softcap, "mask": {"size": window, "keep_first": keep_first}, "v_mix": True}
        elif kind == CHANNEL_DELTA:
            m = {"heads": delta_heads, "kv_heads": delta_heads, "dim": head_dim, "vdim": head_dim, "conv": 4,
                 "a_rank": max(8, width // 32 * 2), "g_rank": max(8, width // 32 * 2)}
        else:
            m = {"heads": heads, "dim": head_dim, "rot_dim": rot, "vdim": head_dim, "q_rank": max(8, width // 16 * 8),
                 "kv_rank": max(8, width // 32 * 8), "scale": (head_dim + rot) ** -0.5, "rot": {"dims": rot, "base": rope_base},
                 "mask": {"size": window}}
        layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    raw = {"architecture": "Lunerax", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "embedding": {"scale": float(width) ** 0.5}, "logit_softcap": logit_softcap, "max_position_embeddings": max_positions}
    if side_dim > 0:
        raw["token_side"] = {"dim": side_dim}
    return LuneraxConfig.from_dict(raw)
