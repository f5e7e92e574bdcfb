"""Small Munizen configurations for the tests, and a harness that steps the engine's runner.

The configurations differ from one another in every size and option: widths and vocabularies that are no
powers of two, group counts of the norm (1, 2, 3), residual streams (none, 1, 2, 4), head and group counts
(one key head for all, one per query head, groups of two and three), map sizes against value sizes (smaller,
equal, larger), the rotated part (none, a part, the whole map), the block size of the mask (small, larger
than any sequence, none), a loop (none, once, several times, over one layer or all), layers with and without
a feed-forward in both kinds, and either kind as the first layer.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, diff=0.25, scale=0.3, rot=(8, 10000.0), mask=7, ff=40):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(heads=2, dim=24, rank=5, ff=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "rank": rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=48, vocab=97, groups=3, eps=1e-5, streams=2, loop=None, max_positions=1024):
    raw = {"architecture": "Munizen", "vocab": vocab, "width": width, "layers": layers,
           "norm": {"eps": eps, "groups": groups}, "max_position_embeddings": max_positions}
    if streams is not None:
        raw["streams"] = streams
    if loop is not None:
        raw["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return raw


CASES: Dict[str, dict] = {
    # delta first, a looped pair, two streams, partial rotation, groups of two query heads, a small mask block
    "P": config([delta_layer(), attention_layer(), delta_layer(heads=3, dim=16, rank=3, ff=56), attention_layer(mask=19)],
                loop=(0, 2, 2)),
    # attention first, no streams, one norm group, every query head its own key head, map larger than the value
    # head, the whole map rotated, a mask block longer than any test sequence, no loop
    "Q": config([attention_layer(heads=3, kv_heads=3, dim=24, vdim=8, rot=(24, 500.0), mask=4096, diff=0.6, scale=0.21),
                 delta_layer(heads=1, dim=40, rank=7, ff=64)], width=40, vocab=131, groups=1, eps=1e-6, streams=None),
    # one stream, one key head for six query heads, no rotation and no mask, a loop of one pass over everything,
    # value head as large as the map, attention without a feed-forward
    "R": config([attention_layer(heads=6, kv_heads=1, dim=8, vdim=8, rot=None, mask=None, ff=None, diff=0.1, scale=0.5),
                 delta_layer(heads=2, dim=16, rank=2), delta_layer(heads=4, dim=8, rank=4, ff=30)],
                width=64, vocab=75, groups=2, streams=1, loop=(0, 3, 1)),
    # four streams, a loop of three passes over one attention layer in the middle, groups of three heads
    "S": config([delta_layer(heads=2, dim=32, rank=6), attention_layer(heads=6, kv_heads=2, dim=12, vdim=20, rot=(4, 77.0), mask=5),
                 delta_layer(heads=5, dim=12, rank=9)], width=60, vocab=211, groups=4, streams=4, loop=(1, 2, 3)),
}
# Head sizes the tensor-core attention kernel takes (multiples of 16): small maps with larger values and groups of two
# heads; and maps over 64 with values over 128 (the kernel's larger register layouts), one key head for all.
CASES["T"] = config([attention_layer(heads=4, kv_heads=2, dim=32, vdim=64, rot=(16, 10000.0), mask=37, scale=0.18, ff=72),
                     delta_layer(heads=2, dim=32, rank=8)], width=64, vocab=151, groups=2, streams=2, loop=(0, 2, 2))
CASES["U"] = config([delta_layer(heads=1, dim=48, rank=8), attention_layer(heads=2, kv_heads=1, dim=80, vdim=144, rot=(80, 3000.0),
                                                                           mask=100, scale=0.11, diff=0.45, ff=None)],
                    width=96, vocab=89, groups=3, streams=3)
# The head sizes of a mid-sized model: maps of 64, values of 128, state heads of 64.
CASES["V"] = config([delta_layer(heads=4, dim=64, rank=16), attention_layer(heads=4, kv_heads=2, dim=64, vdim=128, rot=(32, 1e6),
                                                                            mask=50, scale=0.125, ff=384)],
                    width=256, vocab=300, groups=2, streams=2)
#: one layer of one kind each, for looking at a mechanism alone
SINGLE = {
    "attention": config([attention_layer(ff=None)], streams=None, groups=1),
    "attention_windowless": config([attention_layer(ff=None, mask=None, rot=None)], streams=None, groups=1),
    "delta": config([delta_layer()], streams=None, groups=1),
    "streams": config([delta_layer(ff=40)], streams=3, groups=2),
}


def write_model(raw: dict, folder: str, seed: int = 3) -> str:
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.munizen import MunizenConfig
    from carbon_engine_b200.weights.loader import write_random_model
    return write_random_model(MunizenConfig.from_dict(dict(raw)), folder, seed=seed)


class Harness:
    """The engine's own model, cache storage and step function over a model folder."""

    def __init__(self, folder: str, dtype: str, page_size: int = 8, pages: int = 64, slots: int = 4,
                 max_step_tokens: int = 512, poison: bool = True, device: str = "cuda:0"):
        from carbon_engine_b200.cache.storage import CacheStorage
        from carbon_engine_b200.engine.engine import build_model, parse_dtype
        from carbon_engine_b200.engine.runner import ModelRunner
        self.dtype = parse_dtype(dtype)
        self.model, self.cfg, self.max_len = build_model(folder, self.dtype, torch.device(device))
        self.storage = CacheStorage(self.model, self.dtype, torch.device(device), page_size, pages, slots, self.max_len,
                                    poison=poison)
        self.runner = ModelRunner(self.model, self.storage, max_step_tokens)
        self._next = 0

    def open(self) -> int:
        self._next += 1
        self.runner.open_request(self._next)
        return self._next

    def close(self, rid: int) -> None:
        self.runner.close_request(rid)
        self.storage.manager.check()

    def step(self, entries: Sequence[tuple]) -> np.ndarray:
        """entries: (request, tokens, wanted places) -> float32 logits [wanted, vocab]."""
        from carbon_engine_b200.engine.batch import StepEntry
        out = self.runner.step([StepEntry(r, list(t), list(w)) for r, t, w in entries])
        self.runner.check_status()
        return out.float().cpu().numpy()

    def run(self, tokens: List[int], cuts: Optional[Sequence[int]] = None) -> np.ndarray:
        """One request alone, cut into portions of the given sizes (taken in turn; None: whole); all logits."""
        rid = self.open()
        rows, pos, k = [], 0, 0
        while pos < len(tokens):
            n = len(tokens) - pos if cuts is None else min(cuts[k % len(cuts)], len(tokens) - pos)
            k += 1
            rows.append(self.step([(rid, tokens[pos:pos + n], range(n))]))
            pos += n
        self.close(rid)
        return np.concatenate(rows)


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.abs(got - want).max() / np.abs(want).max())
