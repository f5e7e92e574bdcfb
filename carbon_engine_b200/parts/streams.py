"""Parts around the residual: hyper-connections (a residual kept as several streams) and the token shift.

Hyper-connection of one sublayer, S streams x_1..x_S of a token: the sublayer reads
u = sum_s c_in[s] x_s (formed inside the norm kernel), and its output y goes back as
x_t <- sum_s mix[s, t] x_s + c_out[t] y for all t at once, from the old streams.  ``mix`` is stored
[from, to].  The three small tensors are held in float32.

Token shift: the normed row of a token is blended with the normed row of the token before it,
h_t + (h_{t-1} - h_t) * mu, element by element; h_{t-1} is the row BEFORE its own blend, zeros for the first
token of a sequence.  Between steps the last row of every sequence is kept in a per-request state.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Part, StateCacheSpec, TensorGetter, TensorSpec, register_init_kind

register_init_kind("stream_coef", 0.5, 0.2, True)
register_init_kind("shift", 0.5, 0.2, True)


class HyperConnection(Part):
    def __init__(self, streams: int, prefix: str):
        """Tensors ``prefix.in`` [S], ``prefix.out`` [S], ``prefix.mix`` [S, S]."""
        self.streams, self.prefix = int(streams), prefix
        self.c_in: Optional[torch.Tensor] = None
        self.c_out: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        S = self.streams
        return [TensorSpec(f"{self.prefix}.in", (S,), "stream_coef"), TensorSpec(f"{self.prefix}.out", (S,), "stream_coef"),
                TensorSpec(f"{self.prefix}.mix", (S, S), "stream_coef")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        f32 = lambda n: get(f"{self.prefix}.{n}").to(device).to(torch.float32).contiguous()
        self.c_in, self.c_out, self.mix = f32("in"), f32("out"), f32("mix")

    def write(self, x: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """``bias`` (float32 [width]): added to ``y`` on the way, for a sublayer that left its output bias to its caller."""
        ops.streams_write(x, y, self.mix, self.c_out, bias)


class TokenShift(Part):
    def __init__(self, width: int, name: str):
        self.width, self.name = int(width), name
        self.mu: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), "shift")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.mu = get(self.name).to(device).to(torch.float32).contiguous()

    def state_spec(self) -> StateCacheSpec:
        return StateCacheSpec((self.width,), torch.float32)

    def forward(self, ctx, h: torch.Tensor, out: torch.Tensor, state: torch.Tensor) -> None:
        """``h`` float32 [T, width] (the rows before the blend), ``out`` what the mixer reads, ``state``
        [slots, width]: read for the first token of every portion, then given every sequence's last row."""
        ops.token_shift(h, self.mu, state, out, ctx.positions, ctx.seq_of_token, ctx.seq_slot, ctx.q_start, save=True)
