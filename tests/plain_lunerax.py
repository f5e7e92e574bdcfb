"""A plain, slow implementation of the Lunerax design: whole sequences, float64, one function per mechanism.

It shares no code with the engine: it takes the configuration as the dict config.json holds and the weights
as a dict name -> tensor, runs one sequence from its first token, and keeps nothing between calls.  The tests
compare the engine's logits, residual streams and single mechanisms with it.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, size]: element i of the first ``dims`` turns with element i + dims/2 by the angle
    position * base^(-2i/dims); the rest passes unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    """May the query at position i see the key at position j?  window 0: every earlier key."""
    if j > i:
        return False
    if window <= 0:
        return True
    return i - j < window or j < keep_first


def masked_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: float,
                             window: int, keep_first: int) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence from position 0 -> [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap > 0.0:
            s = softcap * torch.tanh(s / softcap)
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = (j <= i) & ((i - j < window) | (j < keep_first)) if window > 0 else j <= i       # visible(i, j, ...) as a table
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def softcap_attention_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, shared: dict) -> torch.Tensor:
    """The 'attention' mixer: no rotation, capped scores, a window that keeps the first tokens, values blended
    with the values of the first layer that mixes them, an output gate."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{p}.q"].T).view(T, H, d)
    k = (h @ w[f"{p}.k"].T).view(T, G, d)
    v = (h @ w[f"{p}.v"].T).view(T, G, dv)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = w[f"{p}.vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    mask = m.get("mask") or {}
    o = masked_softmax_attention(q, k, v, m["scale"], float(m.get("softcap") or 0.0), int(mask.get("size", 0)),
                                 int(mask.get("keep_first", 0)))
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def latent_attention_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Latent attention: queries and keys/values through low-rank latents, one rotated key part shared by the heads."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[f"{p}.dq"].T, w[f"{p}.dq.norm"], eps)
    q = (cq @ w[f"{p}.uq"].T).view(T, H, d + dr)
    kv = h @ w[f"{p}.dkv"].T
    c = rms_norm(kv[:, :r], w[f"{p}.dkv.norm"], eps)
    k_rot = kv[:, r:].view(T, 1, dr)
    k_plain = (c @ w[f"{p}.uk"].T).view(T, H, d)
    v = (c @ w[f"{p}.uv"].T).view(T, H, dv)
    rot = m["rot"]
    q_rot = rotate_half_pairs(q[..., d:], pos, rot["dims"], rot["base"])
    k_rot = rotate_half_pairs(k_rot, pos, rot["dims"], rot["base"])
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, dr)], dim=-1)
    mask = m.get("mask") or {}
    o = masked_softmax_attention(qq, kk, v, m["scale"], 0.0, int(mask.get("size", 0)), 0)
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros((K - 1, C), dtype=F), x], dim=0)
    y = torch.zeros((T, C), dtype=F)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return silu(y)


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def channel_delta_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit(causal_conv_silu(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"]).view(T, G, d)) * d ** -0.5
    k = unit(causal_conv_silu(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"]).view(T, G, d))
    v = causal_conv_silu(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"]).view(T, H, dv)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)                                            # [T, H]
    a = (h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"]
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, d))
    gate = torch.sigmoid((h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T).view(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros((d, dv), dtype=F)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = rms_norm(out, w[f"{p}.norm"], eps) * gate
    return out.reshape(T, H * dv) @ w[f"{p}.o"].T


def dense_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def token_side(w: Dict[str, torch.Tensor], p: str, layer: int, dim: int, tokens: torch.Tensor, x: torch.Tensor,
               eps: float) -> torch.Tensor:
    """What a layer's per-token input adds to the residual x."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[f"{p}.gate"].T) * e
    return rms_norm(g @ w[f"{p}.proj"].T, w[f"{p}.norm"], eps)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the residual after every layer."""
    w = {k: v.to(F) if v.is_floating_point() else v for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"][tok] * float(cfg["embedding"]["scale"]) if cfg.get("embedding") else w["embed"][tok]
    shared: dict = {}
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = layer_norm(x, w[f"{p}.norm1"], w[f"{p}.norm1.b"], eps)
        if layer["type"] == "attention":
            y = softcap_attention_mixer(w, f"{p}.mix", m, h, shared)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(w, f"{p}.mix", m, h, eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta_mixer(w, f"{p}.mix", m, h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + dense_ff(w, f"{p}.mlp", layer_norm(x, w[f"{p}.norm2"], w[f"{p}.norm2.b"], eps))
        if side:
            x = x + token_side(w, f"{p}.side", i, int(side["dim"]), tok, x, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    z = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0.0 else z


def read_model(folder: str):
    """(config dict, weights dict) of a model folder: config.json and model.safetensors (an 8-byte little-endian header
    length, a JSON header name -> dtype, shape, data_offsets, then the data)."""
    import json
    import os
    import struct
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode())
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = {"F32": torch.float32, "BF16": torch.bfloat16, "I32": torch.int32}[meta["dtype"]]
        weights[name] = torch.frombuffer(bytearray(blob[8 + n + lo:8 + n + hi]), dtype=dt).reshape(meta["shape"]).clone()
    return cfg, weights
