"""The Lunerax decoder, put together from the package's parts.

Every layer is a pre-norm block with layer norms (weight and bias); its mixer is, as config.json lists them, softmax
attention without rotation (capped scores, a window that keeps first tokens, blended values, an output gate:
``parts/masked_attention.py``), latent attention (``parts/latent_attention.py``) or the gated delta rule with a decay per
key channel (``parts/gated_delta.py``); its feed-forward is gated with ReLU, or absent; after the sublayers a per-layer
token input adds into the residual (``parts/side_input.py``).  The embedding rows are scaled, the logits capped.
Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``l<i>.side.gate|proj|norm``, ``final.norm`` (+ ``.b``), ``head``.
"""
from __future__ import annotations

from ..config.lunerax import ATTENTION, LATENT_ATTENTION, LuneraxConfig
from ..config.registry import register_architecture
from ..parts.block import PreNormBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.model import DecoderModel
from ..parts.registry import build_part
from ..parts.side_input import SideTable, TokenSideInput


def build_lunerax(cfg: LuneraxConfig, max_positions: int) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: build_part("norm", "layernorm", width=W, eps=eps, name=name)
    side = cfg.token_side_dim
    table = SideTable(cfg.vocab_size, side * len(cfg.layers), "side.embed") if side > 0 else None
    rotations = {}            # one table per (rotated part, rotated elements, base)
    blocks = []
    mixes_values = False      # has a layer that blends values come by yet?  The first such layer is the source.
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        mask = m.get("mask") or {}
        if layer["type"] == ATTENTION:
            role = None
            if m.get("v_mix"):
                role, mixes_values = ("blend" if mixes_values else "source"), True
            mixer = build_part("mixer", "gated_window_attention", hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                               vdim=m["vdim"], prefix=f"{p}.mix", scale=m["scale"], softcap=m.get("softcap") or 0.0,
                               window=mask.get("size", 0), keep_first=mask.get("keep_first") or 0, value_mix=role)
        elif layer["type"] == LATENT_ATTENTION:
            key = (m["rot_dim"], m["rot"]["dims"], float(m["rot"]["base"]))
            if key not in rotations:
                rotations[key] = build_part("position", "rotary", head_dim=key[0], theta=key[2], max_positions=max_positions,
                                            rotary_dim=key[1])
            mixer = build_part("mixer", "latent_attention", hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                               vdim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"], prefix=f"{p}.mix", eps=eps,
                               position=rotations[key], scale=m["scale"], window=mask.get("size", 0))
        else:
            mixer = build_part("mixer", "channel_gated_delta", hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                               vdim=m["vdim"], taps=m["conv"], prefix=f"{p}.mix", eps=eps, decay_rank=m.get("a_rank") or -1,
                               gate_rank=m.get("g_rank") or -1)
        ffn = ffn_norm = None
        if layer["mlp"] is not None:
            ffn = build_part("feed_forward", "gated_mlp", hidden=W, intermediate=layer["mlp"]["ff"], prefix=f"{p}.mlp",
                             activation="relu", names=("gate", "up", "down"))
            ffn_norm = norm(f"{p}.norm2")
        after = TokenSideInput(W, side, i * side, table, f"{p}.side", eps) if table is not None else None
        blocks.append(PreNormBlock(norm(f"{p}.norm1"), mixer, ffn_norm, ffn, after))
    embedding = Embedding(cfg.vocab_size, W, "embed", scale=cfg.embedding_scale)
    head = LMHead(cfg.vocab_size, W, norm("final.norm"), "head", logit_cap=cfg.logit_softcap)
    return DecoderModel(cfg, embedding, blocks, head, extras=[table] if table is not None else [])


register_architecture("Lunerax", LuneraxConfig.from_dict, build_lunerax, model_types=("lunerax",), replace=True)
