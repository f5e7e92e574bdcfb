"""The generalized delta rule: a recurrent mixer with a matrix state per head.

Per head, with S [dim, dim] (key channel x value channel) carried from token to token in float32:

    S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t

r, k, v are projections of the mixer's input; w_t = exp(-exp(-1/2) sigmoid(W2 tanh(W1 h) + w0)) is a decay per
key channel through a narrow pair of matrices; a_t = sigmoid(Wa h + b) a removal rate per key channel;
u_t the key of unit length, k / sqrt(sum k^2 + 1e-6).  Decay and removal both read the old state.  Each
head's o is divided by its root mean square, the heads are concatenated and multiplied by a weight and by
sigmoid(Wg h), then projected.

The six projections of the input are one product into float32; the decay's second matrix is a product of
its own over tanh of the narrow projection; then three kernels: every token's decays, unit keys and rates
(parallel), the walk over each sequence's tokens of the step in order from the state of the request's slot
(a block per head, sequence and slice of value channels), and the norm, weight and gate (parallel).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, Part, StateCacheSpec, TensorGetter, TensorSpec, register_init_kind
from .linear import ACCUM, STORE_F32, Linear

register_init_kind("decay_bias", 0.0, 1.0, True)
register_init_kind("decay_lora", 0.0, 0.3, True)


class GeneralDeltaRule(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, dim: int, rank: int, prefix: str, eps: float):
        """``rank``: the width of the decay's narrow projection; -1 takes it from the stored tensors."""
        self.hidden, self.heads, self.dim, self.rank, self.prefix, self.eps = hidden, heads, dim, int(rank), prefix, float(eps)
        p, n = prefix, heads * dim
        self.inp = Linear(hidden, [n, n, n, n, n, self.rank], [f"{p}.{t}" for t in ("r", "k", "v", "a", "g", "w1")],
                          pad_rows_to=8)
        self.offsets = (0, n, 2 * n, 3 * n, 4 * n, 5 * n)
        self.decay = Linear(self.rank, [n], [f"{p}.w2"], init="decay_lora")
        self.o = Linear(n, [hidden], [f"{p}.o"])
        self.w0: Optional[torch.Tensor] = None
        self.a_bias: Optional[torch.Tensor] = None
        self.norm_w: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.inp, self.decay, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        p, n = self.prefix, self.heads * self.dim
        return [TensorSpec(f"{p}.w0", (n,), "decay_bias"), TensorSpec(f"{p}.a.b", (n,), "decay_bias"),
                TensorSpec(f"{p}.norm", (n,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        f32 = lambda name: get(f"{self.prefix}.{name}").to(device).to(torch.float32).contiguous()
        self.w0, self.a_bias, self.norm_w = f32("w0"), f32("a.b"), f32("norm")
        self.rank = self.decay.in_features = int(get(f"{self.prefix}.w2").shape[1])       # a rank of -1 is the stored tensors'

    def cache_spec(self) -> StateCacheSpec:
        return StateCacheSpec((self.heads, self.dim, self.dim), torch.float32)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        n = self.heads * self.dim
        return tokens * (self.inp.padded_out * 4 + 5 * n * 4 + max(self.rank, 0) * element_size + n * element_size)

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache, accumulate: bool = True) -> None:
        T = h.shape[0]
        proj = ctx.buffer((T, self.inp.padded_out), torch.float32)
        self.inp.forward(h, proj, STORE_F32)
        n = self.heads * self.dim
        th = ctx.buffer((T, self.rank))
        ops.tanh_cols(proj, self.offsets[5], self.rank, th)
        zz = ctx.buffer((T, n), torch.float32)
        self.decay.forward(th, zz, STORE_F32)
        prep, raw = ctx.buffer((T, 3 * n), torch.float32), ctx.buffer((T, n), torch.float32)
        out = ctx.buffer((T, n))
        prof = ops.profiling()
        if prof is not None:         # what the three kernels read and write once, the state of every sequence twice
            d = self.dim
            prof.note_work(T * n * 4 * (6 + 3 + 3 + 5 + 1 + 2) + T * n * out.element_size() + 2 * ctx.B * self.heads * d * d * 4,
                           8 * T * self.heads * d * d)
        ops.general_delta(proj, zz, self.w0, self.a_bias, self.norm_w, prep, raw, cache.state, out, ctx.seq_slot, ctx.q_start,
                          ctx.B, self.offsets[:5], self.heads, self.dim, self.eps)
        self.o.forward(out, x, ACCUM if accumulate else STORE_F32)
