"""Small Lunerax configurations for the tests.

They differ from one another in every size and option: widths and vocabularies that are no powers of two; the order of
the three kinds of layer and which comes first; attention with and without a score cap, window, kept first tokens, gate
partners (one key head for all, one per query head, groups), key heads smaller, equal and larger than value heads, no,
one, two and three layers that blend values; latent attention with the rotated part turned whole or in part, latents
smaller and larger than a head, with and without a window; the delta rule with 1 to 5 taps, fewer key heads than value
heads, key size against value size; layers without a feed-forward; models without the per-layer token input, without
a logit cap, with an embedding scale of 1.
"""
from __future__ import annotations

from typing import Dict

from munizen_cases import Harness, rel_err  # noqa: F401  (the harness steps any architecture's folder)


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, softcap=5.0, window=11, keep_first=3, v_mix=False, ff=40):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first} if keep_first is not None else {"size": window}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads=3, dim=12, rot_dim=8, rot_dims=4, vdim=20, q_rank=10, kv_rank=14, scale=0.25, base=500.0, window=9, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dims, "base": base}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads=4, kv_heads=2, dim=8, vdim=12, conv=4, a_rank=5, g_rank=3, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "a_rank": a_rank, "g_rank": g_rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=40, vocab=97, eps=1e-5, scale=3.0, side=5, logit_cap=9.0, max_positions=1024):
    raw = {"architecture": "Lunerax", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "max_position_embeddings": max_positions}
    if scale is not None:
        raw["embedding"] = {"scale": scale}
    if side:
        raw["token_side"] = {"dim": side}
    if logit_cap:
        raw["logit_softcap"] = logit_cap
    return raw


CASES: Dict[str, dict] = {
    # all three kinds, two layers that blend values, the delta rule with grouped key heads, a part of the rotated part turned
    "A": config([attention(v_mix=True), delta(), latent(), attention(heads=2, kv_heads=2, dim=8, vdim=24, window=7, keep_first=0,
                                                                     v_mix=True, softcap=0, ff=None),
                 delta(heads=2, kv_heads=1, dim=20, vdim=6, conv=2, a_rank=2, g_rank=7, ff=30)]),
    # latent attention first and without a window, attention without a window, cap or blended values and one head,
    # one tap (no convolution state), no token input, no logit cap, embedding scale left out
    "B": config([latent(heads=1, dim=24, rot_dim=6, rot_dims=6, vdim=8, q_rank=32, kv_rank=40, window=0, ff=24),
                 delta(heads=1, kv_heads=1, dim=12, vdim=28, conv=1, a_rank=3, g_rank=3),
                 attention(heads=1, kv_heads=1, dim=20, vdim=12, softcap=0, window=0, ff=None)],
                width=36, vocab=131, eps=1e-6, scale=None, side=0, logit_cap=0),
    # the delta rule first, three layers that blend values (the middle one between other kinds), one key head for six,
    # a window longer than any test sequence, five taps, a wide token input
    "C": config([delta(heads=3, kv_heads=3, dim=16, vdim=16, conv=5, a_rank=4, g_rank=4, ff=50),
                 attention(heads=6, kv_heads=1, dim=8, vdim=16, window=4096, keep_first=2, v_mix=True, scale=0.5, softcap=2.5),
                 latent(heads=2, dim=8, rot_dim=4, rot_dims=2, vdim=8, q_rank=6, kv_rank=20, window=4096, ff=30),
                 attention(heads=2, kv_heads=1, dim=12, vdim=16, window=5, keep_first=9, v_mix=True),
                 attention(heads=3, kv_heads=1, dim=4, vdim=16, window=6, keep_first=1, v_mix=True, ff=None)],
                width=48, vocab=75, side=11, logit_cap=4.0, scale=1.0),
}
# Head sizes the tensor-core attention kernel takes (multiples of 16), with windows that cut through its tiles of 64 keys
CASES["T"] = config([attention(heads=4, kv_heads=2, dim=32, vdim=64, window=37, keep_first=5, v_mix=True, scale=0.18, softcap=6.0, ff=72),
                     latent(heads=4, dim=32, rot_dim=16, rot_dims=16, vdim=32, q_rank=24, kv_rank=48, window=70, scale=0.15),
                     delta(heads=2, kv_heads=2, dim=32, vdim=48, conv=3, a_rank=8, g_rank=8),
                     attention(heads=2, kv_heads=2, dim=16, vdim=64, window=100, keep_first=0, v_mix=True, scale=0.25, softcap=0)],
                    width=64, vocab=151, side=8)
# The head sizes of a mid-sized model: keys of 128, values wider than a slice of 128, a latent of 256 + 32, state heads of 64 x 128
CASES["V"] = config([latent(heads=4, dim=64, rot_dim=32, rot_dims=32, vdim=64, q_rank=96, kv_rank=256, window=90, scale=0.1, ff=384),
                     attention(heads=4, kv_heads=1, dim=128, vdim=144, window=50, keep_first=8, scale=0.09, softcap=12.0),
                     delta(heads=2, kv_heads=1, dim=64, vdim=128, conv=4, a_rank=16, g_rank=16)],
                    width=256, vocab=300, side=16)
#: one layer of one kind each, for looking at a mechanism alone
SINGLE = {
    "attention": config([attention(ff=None)], side=0, logit_cap=0),
    "attention_plain": config([attention(ff=None, softcap=0, window=0)], side=0, logit_cap=0),
    "latent": config([latent()], side=0, logit_cap=0),
    "delta": config([delta()], side=0, logit_cap=0),
    "delta_one_tap": config([delta(conv=1, heads=2, kv_heads=2, dim=36, vdim=5)], side=0, logit_cap=0),
    # more than 128 key channels (32 lanes a state column), and sizes that are no multiples of 4 (4-byte copies)
    "delta_wide_keys": config([delta(heads=1, kv_heads=1, dim=136, vdim=8, conv=2, a_rank=4, g_rank=4)], side=0, logit_cap=0),
    "delta_odd_sizes": config([delta(heads=2, kv_heads=1, dim=10, vdim=7, conv=3, a_rank=3, g_rank=2)], width=34, side=0, logit_cap=0),
    "feed_forward_and_side": config([attention(ff=56, heads=1, kv_heads=1)], side=7, logit_cap=3.0),
}


def write_model(raw: dict, folder: str, seed: int = 3) -> str:
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.lunerax import LuneraxConfig
    from carbon_engine_b200.weights.loader import write_random_model
    return write_random_model(LuneraxConfig.from_dict(dict(raw)), folder, seed=seed)
