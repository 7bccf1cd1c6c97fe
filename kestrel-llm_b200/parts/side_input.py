"""A per-layer input looked up by token: x <- x + norm(W_proj (gelu_tanh(W_gate x) * e)), where e
is the layer's part of a table row of the token, x is the residual stream after the layer's
sublayers, and the norm divides by the root mean square and multiplies by a plain weight.
The table is one part of the model (`TokenTable`), shared by the layers."""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from .base import Part, WeightSlot
from .linear import Linear


class TokenTable(Part):
    graph_safe = True

    def __init__(self, vocab: int, columns: int, dtype: torch.dtype, device, weight_name: str):
        self.weight = torch.empty((vocab, columns), dtype=dtype, device=device)
        self.weight_name = weight_name

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.weight_name, self.weight)]


class TokenSideInput(Part):
    graph_safe = True

    def __init__(self, width: int, dim: int, table: TokenTable, column0: int, eps: float, dtype: torch.dtype, device, prefix: str):
        self.width, self.dim, self.table, self.column0, self.eps = width, dim, table, int(column0), float(eps)
        self.dtype, self.prefix = dtype, prefix
        self.gate = Linear(width, dim, dtype, device)
        self.proj = Linear(dim, width, dtype, device)
        self.norm_w = torch.empty((width,), dtype=torch.float32, device=device)

    def weight_slots(self) -> List[WeightSlot]:
        p = self.prefix
        return [WeightSlot(p + "gate", self.gate.weight), WeightSlot(p + "proj", self.proj.weight), WeightSlot(p + "norm", self.norm_w, "norm")]

    def add_forward(self, residual: torch.Tensor, x: torch.Tensor, batch) -> None:
        """``x`` is the residual stream in the storage type; the result is added to ``residual``."""
        g = self.gate.forward(x)
        gated = torch.empty((x.shape[0], self.dim), dtype=self.dtype, device=x.device)
        ops.gelu_table_mul(g, self.table.weight, self.column0, batch.token_ids, gated)
        ops.add_normed(residual, self.proj.forward(gated), self.norm_w, self.eps)
