"""Typed configuration of the Munizen architecture.

config.json names the design with ``"architecture": "Munizen"`` and describes the model layer by layer:

* ``vocab``, ``width``: vocabulary and residual width;
* ``layers``: a list of ``{"type", "mixer", "mlp"}``; ``type`` is ``"attention"`` (differential attention:
  ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff``, ``rot`` = ``{"dims", "base"}``, ``mask`` =
  ``{"size"}``) or ``"general_delta"`` (``heads``, ``dim``); ``mlp`` is ``{"kind": "dense", "ff"}`` or null;
* ``loop`` = ``{"start", "stop", "times"}``: layers start..stop-1 run ``times`` times in a row with the same
  weights, each pass with a cache of its own (absent: every layer once);
* ``norm`` = ``{"eps", "groups"}``: the RMS norm's epsilon and the number of equal parts it is taken in;
* ``streams``: the number of residual streams (absent: an ordinary residual).

What config.json does not give is taken from the stored tensors' shapes (the rank of the decay's narrow
projection), unless the mixer's entry names it (``rank``), which a model with random weights needs.
``max_position_embeddings`` and ``eos_token_id`` are optional additions of this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, token_id_list

ATTENTION, GENERAL_DELTA = "attention", "general_delta"
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


def _check_layer(i: int, layer: Any, width: int) -> Dict[str, Any]:
    where = f"layers[{i}]: "
    if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
        raise ConfigError(f"config.json: {where}an object with 'type', 'mixer' and 'mlp' is expected")
    kind, m = layer.get("type"), layer["mixer"]
    if kind == ATTENTION:
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} kv_heads")
        _int(m, "dim", where); _int(m, "vdim", where); _float(m, "scale", where)
        diff = _float(m, "diff", where)
        if m.get("rot") is not None:
            if not isinstance(m["rot"], dict):
                raise ConfigError(f"config.json: {where}'rot' must be an object")
            dims = _int(m["rot"], "dims", where + "rot: ", 2)
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most dim={m['dim']}")
            if _float(m["rot"], "base", where + "rot: ") <= 0.0:
                raise ConfigError(f"config.json: {where}rot.base must be positive")
        if m.get("mask") is not None:
            if not isinstance(m["mask"], dict) or set(m["mask"]) != {"size"}:
                raise ConfigError(f"config.json: {where}'mask' must be {{\"size\": n}} (keys seen only inside the query's "
                                  f"block of n positions); got {m['mask']!r}")
            _int(m["mask"], "size", where + "mask: ")
        del diff
    elif kind == GENERAL_DELTA:
        _int(m, "heads", where); _int(m, "dim", where)
        if m.get("rank") is not None:
            _int(m, "rank", where)
    else:
        raise ConfigError(f"config.json: {where}unknown layer type {kind!r} ({ATTENTION}, {GENERAL_DELTA})")
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense', got {mlp!r}")
        _int(mlp, "ff", where + "mlp: ")
    return {"type": kind, "mixer": copy.deepcopy(m), "mlp": copy.deepcopy(mlp)}


@dataclass(frozen=True)
class MunizenConfig(ModelConfig):
    width: int = 0
    layers: Tuple[Dict[str, Any], ...] = ()
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    norm_eps: float = 1e-6
    norm_groups: int = 1
    streams: Optional[int] = None

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MunizenConfig":
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        checked = tuple(_check_layer(i, layer, width) for i, layer in enumerate(layers))
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            if not isinstance(lp, dict):
                raise ConfigError("config.json: 'loop' must be an object")
            start, stop, times = _int(lp, "start", "loop: ", 0), _int(lp, "stop", "loop: ", 0), _int(lp, "times", "loop: ", 1)
            if not start <= stop <= len(checked):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(checked)} layers")
            loop = (start, stop, times)
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps' and 'groups'")
        eps = _float(norm, "eps", "norm: ")
        groups = _int(norm, "groups", "norm: ") if norm.get("groups") is not None else 1
        if eps <= 0.0 or width % groups:
            raise ConfigError(f"config.json: norm eps={eps} must be positive and groups={groups} must divide width={width}")
        streams = _int(raw, "streams", "") if raw.get("streams") is not None else None
        if streams is not None and streams > 16:
            raise ConfigError(f"config.json: streams={streams}: at most 16 are supported")
        max_pos = raw.get("max_position_embeddings")
        max_pos = DEFAULT_MAX_POSITIONS if max_pos is None else _int(raw, "max_position_embeddings", "")
        eos = token_id_list(raw.get("eos_token_id"))
        for t in raw.get("_generation_eos_token_ids", []):
            if t not in eos:
                eos.append(t)
        return cls(architecture="Munizen", vocab_size=vocab, max_position_embeddings=max_pos, eos_token_ids=tuple(eos),
                   width=width, layers=checked, loop=loop, norm_eps=eps, norm_groups=groups, streams=streams)

    def layer_runs(self) -> Tuple[int, ...]:
        """The layers' indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Munizen", "vocab": self.vocab_size, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)),
                               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out
