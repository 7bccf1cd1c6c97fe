"""Routed feed-forward: E small gated experts, of which each token uses ``top``.

Router logits z = W_r h + b in float32; the ``top`` largest are chosen and weighted by the
softmax over the chosen logits alone.  An expert with a clamp ``limit``:

    g = min(W_gate h, limit);  u = clamp(W_up h, -limit, limit);  y = W_down (g sigmoid(1.702 g) (u + 1))

The experts' matrices are stacked ([E, 2 ff, width] gate rows then up rows, [E, width, ff]), the
step's (token, choice) pairs are grouped by expert on the device, and two grouped products run
them; a token's result does not depend on the batch.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, WeightSlot
from .linear import Linear


class RoutedExperts(FeedForward):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, inner: int, experts: int, top: int, limit: float, dtype: torch.dtype, device, prefix: str,
                 router_bias: bool = True, expert_name: str = "e{}."):
        if not 1 <= top <= min(experts, 32):
            raise ValueError(f"top = {top} of {experts} experts: the router kernel takes 1 to min(experts, 32)")
        self.width, self.inner, self.experts, self.top, self.limit = width, inner, experts, top, float(limit)
        self.dtype, self.prefix, self.expert_name = dtype, prefix, expert_name
        self.router = Linear(width, experts, dtype, device)
        self.router_bias: Optional[torch.Tensor] = torch.empty((experts,), dtype=torch.float32, device=device) if router_bias else None
        self.w_gate_up = torch.empty((experts, 2 * inner, width), dtype=dtype, device=device)
        self.w_down = torch.empty((experts, width, inner), dtype=dtype, device=device)

    def weight_slots(self) -> List[WeightSlot]:
        p, ff = self.prefix, self.inner
        slots = [WeightSlot(p + "router", self.router.weight)]
        if self.router_bias is not None:
            slots.append(WeightSlot(p + "router.b", self.router_bias, "bias"))
        for e in range(self.experts):
            q = p + self.expert_name.format(e)
            slots += [WeightSlot(q + "gate", self.w_gate_up[e, :ff]), WeightSlot(q + "up", self.w_gate_up[e, ff:]),
                      WeightSlot(q + "down", self.w_down[e])]
        return slots

    def forward(self, x: torch.Tensor, batch) -> ops.Partials:
        ids, weights = ops.moe_route(self.router.forward(x), self.router_bias, self.top)
        return ops.Partials(ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit))
