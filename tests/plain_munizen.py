"""A plain, slow implementation of the Munizen decoder for tests: whole sequences, no cache, float64,
one function per mechanism, written from the design's equations.  It shares no code with the engine
(it reads config.json and model.safetensors with the plain reader of ``plain_qwen3``).

Notation: T tokens, W width, S residual streams, H query heads, G key/value heads, d the size of a
query/key map, dv the size of a value head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from plain_qwen3 import read_model  # noqa: F401  (a plain reader of a model folder, no engine code)

F = torch.float64


def grouped_rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, groups: int) -> torch.Tensor:
    """The last axis is cut into ``groups`` equal consecutive parts; each part is divided by
    sqrt(mean(part^2) + eps); the whole is multiplied by ``weight`` (if there is one)."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    y = parts.reshape(shape)
    return y if weight is None else y * weight


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h_t + (h_{t-1} - h_t) * mu with h_{-1} = 0; the previous row is the one before the replacement."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def rotate_half_partial(x: torch.Tensor, positions: torch.Tensor, rot_dims: int, base: float) -> torch.Tensor:
    """x [T, n, d]: the first ``rot_dims`` elements of every vector turn, element i with element
    i + rot_dims/2 by the angle position * base^(-2i/rot_dims); the rest pass."""
    half = rot_dims // 2
    freq = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:rot_dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., rot_dims:]], dim=-1)


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] True where query i may see key j: j <= i and both in the same block of ``size`` positions."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, o = a1 - lambda a2, unit-RMS per head times
    (1 - diff), a per-head sigmoid gate, and the output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_half_partial(q.reshape(T, 2 * H, d), pos, rot["dims"], rot["base"]).reshape(T, H, 2, d)
        k = rotate_half_partial(k.reshape(T, 2 * G, d), pos, rot["dims"], rot["base"]).reshape(T, G, 2, d)
    mask = chunk_mask(T, m["mask"]["size"]) if m.get("mask") else chunk_mask(T, T + 1)
    lam = math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) \
        + m["diff"]
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for z in range(2):
            s = (q[:, hd, z] @ k[:, g, z].T) * m["scale"]
            s = s.masked_fill(~mask, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps) * (1.0 - m["diff"])
        heads.append(o * gate[:, hd:hd + 1])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T + w[p + "o.b"]


def general_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                  state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """S_t = diag(decay_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T per head, o_t = S_t^T r_t."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
    decay = decay.reshape(T, H, d)
    a = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, d)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F) if state is None else state
    out = torch.zeros(T, H, d, dtype=F)
    for t in range(T):
        for hd in range(H):
            old = S[hd]
            S[hd] = decay[t, hd][:, None] * old - (a[t, hd] * u[t, hd])[:, None] * (u[t, hd] @ old)[None, :] \
                + k[t, hd][:, None] * v[t, hd][None, :]
            out[t, hd] = S[hd].T @ r[t, hd]
    out = out / torch.sqrt((out * out).mean(dim=-1, keepdim=True) + eps)
    y = out.reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def dense_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def hyper_read(xs: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """xs [S, T, W] -> sum_s in[s] xs[s]."""
    return torch.einsum("s,stw->tw", w_in, xs)


def hyper_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """new[t] = sum_s mix[s, t] old[s] + out[t] y, all streams at once from the old ones."""
    return torch.einsum("st,snw->tnw", mix, xs) + out[:, None, None] * y[None]


def layer_runs(cfg: dict) -> List[int]:
    """The indices of the layers in the order they run, looped span repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def mixer_of(layer: dict, h, w, p, eps):
    if layer["type"] == "attention":
        return differential_attention(h, w, p, layer["mixer"], eps)
    if layer["type"] == "general_delta":
        return general_delta(h, w, p, layer["mixer"], eps)
    raise ValueError(layer["type"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``trace`` receives the residual stream (the sum of the
    streams) after every layer run."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    S = cfg.get("streams")
    xs = torch.stack([x] * S) if S else None
    for i in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if sub == "mlp" and layer["mlp"] is None:
                continue
            u = hyper_read(xs, w[p + f"hc{q}.in"]) if S else x
            h = grouped_rms_norm(u, w[p + f"norm{q}"], eps, groups)
            if sub == "mixer":
                y = mixer_of(layer, token_shift(h, w[p + "shift"]), w, p + "mix.", eps)
            else:
                y = dense_mlp(h, w, p + "mlp.")
            if S:
                xs = hyper_write(xs, y, w[p + f"hc{q}.mix"], w[p + f"hc{q}.out"])
            else:
                x = x + y
        if trace is not None:
            trace.append(xs.sum(dim=0) if S else x.clone())
    x = xs.sum(dim=0) if S else x
    return grouped_rms_norm(x, w["final.norm"], eps, groups) @ w["head"].T
