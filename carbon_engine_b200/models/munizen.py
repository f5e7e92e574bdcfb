"""The Munizen decoder, put together from the package's parts.

Layers alternate, in the order config.json lists them, between differential attention
(``parts/diff_attention.py``) and the generalized delta rule (``parts/delta_rule.py``); a layer may have a
gated feed-forward or none.  Every layer is a pre-norm block with a group-wise RMS norm, a token shift in
front of the mixer, and, if the model has residual streams, a hyper-connection around every sublayer
(``parts/block.py:StreamBlock``).  A span of layers may run several times in a row with the same weights:
the schedule then names those blocks again, each time with a cache of its own.  Tensor names:
``embed``, ``l<i>.norm1|norm2|shift``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``, ``l<i>.hc1|hc2.in|out|mix``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.munizen import ATTENTION, MunizenConfig
from ..config.registry import register_architecture
from ..parts.block import StreamBlock
from ..parts.embedding import Embedding, LMHead
from ..parts.model import DecoderModel, LayerCall
from ..parts.registry import build_part
from ..parts.streams import HyperConnection, TokenShift


def build_munizen(cfg: MunizenConfig, max_positions: int) -> DecoderModel:
    W, eps, groups = cfg.width, cfg.norm_eps, cfg.norm_groups
    norm = lambda name: build_part("norm", "grouped_rmsnorm", width=W, eps=eps, name=name, groups=groups)
    rotations = {}            # one table per (head size, rotated elements, base)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        if layer["type"] == ATTENTION:
            position = None
            if m.get("rot") is not None:
                key = (m["dim"], m["rot"]["dims"], float(m["rot"]["base"]))
                if key not in rotations:
                    rotations[key] = build_part("position", "rotary", head_dim=m["dim"], theta=key[2],
                                                max_positions=max_positions, rotary_dim=key[1])
                position = rotations[key]
            mixer = build_part("mixer", "differential_attention", hidden=W, heads=m["heads"], kv_heads=m["kv_heads"],
                               dim=m["dim"], vdim=m["vdim"], prefix=f"{p}.mix", diff=m["diff"], eps=eps, position=position,
                               scale=m["scale"], chunk=m["mask"]["size"] if m.get("mask") else 0)
        else:
            mixer = build_part("mixer", "general_delta", hidden=W, heads=m["heads"], dim=m["dim"],
                               rank=m.get("rank") or -1, prefix=f"{p}.mix", eps=eps)
        ffn = ffn_norm = None
        if layer["mlp"] is not None:
            ffn = build_part("feed_forward", "gated_mlp", hidden=W, intermediate=layer["mlp"]["ff"], prefix=f"{p}.mlp",
                             names=("gate", "up", "down"))
            ffn_norm = norm(f"{p}.norm2")
        connections = None
        if cfg.streams is not None:
            connections = [HyperConnection(cfg.streams, f"{p}.hc{q}") for q in ((1, 2) if ffn is not None else (1,))]
        blocks.append(StreamBlock(W, norm(f"{p}.norm1"), mixer, ffn_norm, ffn, connections, TokenShift(W, f"{p}.shift")))
    embedding = Embedding(cfg.vocab_size, W, "embed")
    head = LMHead(cfg.vocab_size, W, norm("final.norm"), "head")
    schedule = [LayerCall(block, run, True) for run, block in enumerate(cfg.layer_runs())]
    return DecoderModel(cfg, embedding, blocks, head, schedule, streams=cfg.streams or 0)


register_architecture("Munizen", MunizenConfig.from_dict, build_munizen, model_types=("munizen",), replace=True)
