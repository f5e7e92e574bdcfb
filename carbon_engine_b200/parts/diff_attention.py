"""Differential attention over the paged cache.

Every query head has two maps: two query vectors of size ``dim`` (laid out [map 1, map 2] head by head),
and every key/value head two key vectors and ONE value vector of size ``vdim``.  Each map is a softmax
attention of its own over the same values, a1 and a2; the head's output is a1 - lam * a2 with
lam = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff (one number for the layer), brought to unit root mean square
over the head (no weight) and multiplied by (1 - diff); then by a per-head sigmoid gate computed from the
mixer's input; then the output projection.  q, k, v and the output projection may carry biases; q and k
are rotated over their first ``rotary_dim`` elements; scores are multiplied by ``scale``.

Visible keys: causal, optionally a window, optionally only the keys of the query's own block of ``chunk``
positions, blocks counted from position 0 of the sequence.

In the cache the two maps of a key head are two heads of the K pool; the V pool has its own head count and
head size (``PagedCacheSpec.v_heads`` / ``v_head_dim``).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, PagedCacheSpec, Part, TensorGetter, TensorSpec, register_init_kind
from .linear import ACCUM, STORE, STORE_F32, Linear
from .rope import PositionEncoding

register_init_kind("lambda_vec", 0.0, 0.1, True)


class DiffAttentionPlan:
    def __init__(self, tiles, n_tiles):
        self.tiles, self.n_tiles = tiles, n_tiles
        self.graph_key = None            # a decode step of B sequences is always B tiles


class DifferentialAttention(Mixer):
    graph_safe = True
    can_store = True
    plan_key = "differential_attention"
    TILE = 64               # query tokens a block of the tensor-core kernel takes

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, prefix: str, diff: float, eps: float,
                 position: Optional[PositionEncoding] = None, scale: Optional[float] = None, chunk: int = 0,
                 window: int = 0, bias: bool = True, page_size: Optional[int] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = hidden, heads, kv_heads, dim, vdim
        self.prefix, self.diff, self.eps, self.position = prefix, float(diff), float(eps), position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dim)
        self.chunk, self.window, self.page_size = int(chunk), int(window), page_size
        p = prefix
        b = (lambda n: f"{p}.{n}.b") if bias else (lambda n: None)
        # one product for q | k | v | gate logits; the row stride keeps 16-byte alignment
        self.qkvg = Linear(hidden, [heads * 2 * dim, kv_heads * 2 * dim, kv_heads * vdim, heads],
                           [f"{p}.q", f"{p}.k", f"{p}.v", f"{p}.g"], bias_names=[b("q"), b("k"), b("v"), None], pad_rows_to=8)
        self.o = Linear(heads * vdim, [hidden], [f"{p}.o"], bias_names=[b("o")])
        self.lam = 0.0

    def children(self) -> List[Part]:
        return [self.qkvg, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}.{n}", (self.dim,), "lambda_vec") for n in ("lq1", "lk1", "lq2", "lk2")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        v = {n: get(f"{self.prefix}.{n}").to(torch.float64) for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((v["lq1"] * v["lk1"]).sum())) - math.exp(float((v["lq2"] * v["lk2"]).sum())) + self.diff
        if self.position is not None and self.position.cos is None:
            self.position.prepare(device)

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(2 * self.kv_heads, self.dim, self.window, self.page_size,
                              v_heads=self.kv_heads, v_head_dim=self.vdim)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * (self.qkvg.padded_out + self.heads * self.vdim) * element_size

    def step_sections(self, max_tokens: int, max_seqs: int):
        return [("differential_attention.tiles", 2 * (max_seqs + max_tokens // self.TILE + 1))]

    def plan_step(self, ctx) -> "DiffAttentionPlan":
        """The step's tiles of up to 64 query tokens, (sequence, first token) pairs, of EVERY sequence: one-token
        sequences are tiles of one row (a query sees at most a mask block of keys, so there is nothing to split
        among blocks, and a block per sequence and head on the tensor-core kernel is the shortest way)."""
        tiles = ctx.bufs.host_section("differential_attention.tiles")
        n = 0
        for b in range(ctx.B):
            for q0 in range(0, ctx.h_q_start[b + 1] - ctx.h_q_start[b], self.TILE):
                tiles[2 * n], tiles[2 * n + 1] = b, q0
                n += 1
        return DiffAttentionPlan(ctx.bufs.dev_section("differential_attention.tiles"), n)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        qkvg = ctx.buffer((T, self.qkvg.padded_out))
        self.qkvg.forward(h, qkvg, STORE, add_bias=False)
        pos = self.position
        cos = pos.cos if pos is not None else None
        sin = pos.sin if pos is not None else None
        if cos is not None and ctx.max_position >= cos.shape[0]:
            raise ValueError(f"position {ctx.max_position} is beyond the rotary table ({cos.shape[0]}): raise max_seq_len")
        table = ctx.block_tables[cache.group]
        ops.bias_rope_kvwrite(qkvg, cache.k_pool, cache.v_pool, self.qkvg.bias, cos, sin, ctx.positions, ctx.seq_of_token,
                              ctx.seq_slot, table, ctx.status, 2 * H, 2 * G, G, d, dv,
                              pos.rotary_dim if cos is not None else 0, cache.page_size, write_kv=cache.writes)
        out = ctx.buffer((T, H * dv))
        self.attend(ctx, qkvg, out, cache, table)
        # stored, not added: the output bias is left to the caller, whose next kernel reads the output anyway
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32, add_bias=accumulate)
        return None if accumulate else self.o.bias

    def attend(self, ctx, qkvg: torch.Tensor, out: torch.Tensor, cache, table: torch.Tensor) -> None:
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        gate = qkvg[:, (2 * H + 2 * G) * d + G * dv:]
        prof = ops.profiling()
        if prof is not None:
            el, keys, pairs = qkvg.element_size(), 0, 0
            for b in range(ctx.B):
                n, before = ctx.h_q_start[b + 1] - ctx.h_q_start[b], ctx.h_ctx_before[b]
                first = before
                if self.chunk > 0:
                    first = max(first - first % self.chunk, 0)
                keys += before + n - (first if self.chunk > 0 else 0)
                for p in range(before, before + n):          # the keys position p sees
                    lo = max(0, p - self.window + 1) if self.window > 0 else 0
                    if self.chunk > 0:
                        lo = max(lo, p - p % self.chunk)
                    pairs += p - lo + 1
            prof.note_work((keys * G * (2 * d + dv) + ctx.T * H * (2 * d + dv)) * el, 4 * pairs * H * (d + dv))
        consts = (self.window, self.chunk, self.scale, self.lam, self.eps, 1.0 - self.diff)
        stride = qkvg.stride(0)
        if qkvg.dtype == torch.bfloat16 and ctx.fast_attention and ops.diff_attention_mma_supported(d, dv, stride):
            plan = ctx.plans[self.plan_key]
            ops.diff_attention_mma(qkvg, stride, cache.k_pool, cache.v_pool, gate, stride, out, ctx.positions, ctx.seq_slot,
                                   ctx.q_start, table, plan.tiles, plan.n_tiles, ctx.status, H, G, d, dv, cache.page_size,
                                   *consts)
            return
        ops.diff_attention(qkvg, stride, cache.k_pool, cache.v_pool, gate, stride, out, ctx.positions, ctx.seq_of_token,
                           ctx.seq_slot, table, ctx.status, H, G, d, dv, cache.page_size, *consts)
