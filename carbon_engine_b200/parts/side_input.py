"""A per-layer token input: every layer adds to the residual a small vector that depends on the token itself.

A table holds, for every token id, ``dim`` numbers per layer (the layers' slices side by side in one row).  After a
layer's sublayers, with x the residual and e the token's slice for this layer:

    g = gelu_tanh(W_gate x) * e;      y = W_proj g;      x <- x + y / sqrt(mean(y^2) + eps) * w

The gate product reads the residual itself (no norm in front); the norm of y is an RMS norm with a plain weight.
The table is a part of its own (:class:`SideTable`), loaded once and shared by the layers' :class:`TokenSideInput`.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Part, TensorGetter, TensorSpec, to_device
from .linear import STORE_F32, Linear


class SideTable(Part):
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = int(vocab), int(width), name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab, self.width), "embedding")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.weight = to_device(get(self.name), device, dtype)


class TokenSideInput(Part):
    def __init__(self, width: int, dim: int, offset: int, table: SideTable, prefix: str, eps: float):
        """``offset``: the first column of this layer's slice in the table's rows.  Tensors ``prefix.gate`` [dim, width],
        ``prefix.proj`` [width, dim], ``prefix.norm`` [width]."""
        if offset < 0 or offset + dim > table.width:
            raise ValueError(f"columns {offset}..{offset + dim} do not lie in a table {table.width} wide")
        self.width, self.dim, self.offset, self.table, self.prefix, self.eps = int(width), int(dim), int(offset), table, prefix, float(eps)
        self.gate = Linear(width, [dim], [f"{prefix}.gate"])
        self.proj = Linear(dim, [width], [f"{prefix}.proj"])
        self.norm_w: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.gate, self.proj]          # the table belongs to the model, not to one layer

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}.norm", (self.width,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.norm_w = get(f"{self.prefix}.norm").to(device).to(torch.float32).contiguous()

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * (self.width * (element_size + 4) + self.dim * (element_size + 4))

    def forward(self, ctx, x: torch.Tensor) -> None:
        """Adds this layer's side input into the float32 residual ``x`` [T, width]."""
        T = x.shape[0]
        if ctx.dtype == torch.float32:
            xa = x
        else:
            xa = ctx.buffer((T, self.width))
            ops.copy_cols(x, 0, self.width, xa)
        z = ctx.buffer((T, self.dim), torch.float32)
        self.gate.forward(xa, z, STORE_F32)
        g = ctx.buffer((T, self.dim))
        ops.side_gate(z, self.table.weight, ctx.tokens, g, self.offset, ctx.status)
        y = ctx.buffer((T, self.width), torch.float32)
        self.proj.forward(g, y, STORE_F32)
        ops.rmsnorm_add(y, self.norm_w, x, self.eps)
