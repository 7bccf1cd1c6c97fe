"""A recurrent mixer: the gated delta rule with one decay per head and key channel.

With h the mixer's input, G key heads of size d and H value heads of size dv (value head n
uses key head n // (H / G)):

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     short causal convolutions over time, per channel
    q <- q / sqrt(sum q^2 + 1e-6) * d^-1/2,   k <- k / sqrt(sum k^2 + 1e-6)   per head
    beta = sigmoid(W_b h)                                                  one per value head
    a = exp(-exp(A_log[n]) * softplus(W_a2 (W_a1 h) + dt_bias))            one per value head and key channel
    S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      per value head, S [d, dv] from zero
    y = W_o ( o / sqrt(mean(o^2) + eps) * w_norm * sigmoid(W_g2 (W_g1 h)) )

The state S and the last taps - 1 inputs of the convolutions live in the request's state slot,
in float32; everything between the products and the output norm is float32.  W_q, W_k, W_v,
W_b, W_a1 and W_g1 are one fused product.
"""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from .base import FixedStateSpec, Mixer, WeightSlot
from .linear import Linear


class ChannelDeltaMixer(Mixer):
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int, decay_rank: int,
                 gate_rank: int, norm_eps: float, dtype: torch.dtype, device, prefix: str):
        if heads % kv_heads:
            raise ValueError(f"{heads} value heads are not a multiple of {kv_heads} key heads")
        if key_dim > 256:
            raise ValueError(f"key size {key_dim}: the recurrence kernel holds up to 256 key channels a thread")
        if not 1 <= taps <= 9:
            raise ValueError(f"{taps} taps: the convolution kernel takes 1 to 9")
        self.width, self.H, self.G, self.d, self.dv, self.taps = width, heads, kv_heads, key_dim, value_dim, taps
        self.ra, self.rg = decay_rank, gate_rank
        self.eps, self.dtype, self.prefix = float(norm_eps), dtype, prefix
        qk, vv = kv_heads * key_dim, heads * value_dim
        self.C = 2 * qk + vv                                   # channels that pass a convolution: q | k | v
        self.col_v, self.col_beta = 2 * qk, self.C
        self.col_a1, self.col_g1 = self.C + heads, self.C + heads + decay_rank
        self.in_proj = Linear(width, self.C + heads + decay_rank + gate_rank, dtype, device)
        self.a2 = Linear(decay_rank, heads * key_dim, dtype, device)
        self.g2 = Linear(gate_rank, vv, dtype, device)
        self.out = Linear(vv, width, dtype, device)
        self.conv_w = torch.empty((self.C, taps), dtype=torch.float32, device=device)
        self.A_log = torch.empty((heads,), dtype=torch.float32, device=device)
        self.dt_bias = torch.empty((heads * key_dim,), dtype=torch.float32, device=device)
        self.norm_w = torch.empty((value_dim,), dtype=torch.float32, device=device)
        self.tail_off = heads * key_dim * value_dim             # the slot: S [H, d, dv], then the convolutions' tail [taps - 1, C]
        self.state_size = self.tail_off + (taps - 1) * self.C

    def cache_spec(self) -> FixedStateSpec:
        return FixedStateSpec((self.state_size,), torch.float32)

    def weight_slots(self) -> List[WeightSlot]:
        p, w, qk = self.prefix, self.in_proj.weight, self.G * self.d
        return [WeightSlot(p + "q", w[:qk]), WeightSlot(p + "k", w[qk:2 * qk]), WeightSlot(p + "v", w[2 * qk:self.C]),
                WeightSlot(p + "b", w[self.col_beta:self.col_a1]), WeightSlot(p + "a1", w[self.col_a1:self.col_g1]),
                WeightSlot(p + "g1", w[self.col_g1:]),
                WeightSlot(p + "q.conv", self.conv_w[:qk]), WeightSlot(p + "k.conv", self.conv_w[qk:2 * qk]),
                WeightSlot(p + "v.conv", self.conv_w[2 * qk:]),
                WeightSlot(p + "a2", self.a2.weight), WeightSlot(p + "g2", self.g2.weight), WeightSlot(p + "o", self.out.weight),
                WeightSlot(p + "A_log", self.A_log, "bias"), WeightSlot(p + "dt_bias", self.dt_bias, "bias"),
                WeightSlot(p + "norm", self.norm_w, "norm")]

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        T, dev, f32 = x.shape[0], x.device, torch.float32
        H, G, d, dv = self.H, self.G, self.d, self.dv
        fused = self.in_proj.forward(x)
        act = torch.empty((T, self.C), dtype=f32, device=dev)
        ops.delta_conv_silu(fused, self.conv_w, cache.state, self.tail_off, batch, act)
        a = self.a2.forward(ops.partial_columns(fused, self.col_a1, self.ra, self.dtype))
        g = self.g2.forward(ops.partial_columns(fused, self.col_g1, self.rg, self.dtype))
        qn = torch.empty((T, G * d), dtype=f32, device=dev)
        kn = torch.empty((T, G * d), dtype=f32, device=dev)
        decay = torch.empty((T, H * d), dtype=f32, device=dev)
        beta = torch.empty((T, H), dtype=f32, device=dev)
        ops.delta_gates(act, fused, self.col_beta, a, self.A_log, self.dt_bias, qn, kn, decay, beta, H, G, d)
        o = torch.empty((T, H * dv), dtype=f32, device=dev)
        ops.delta_scan(qn, kn, decay, act, self.col_v, beta, cache.state, batch, o, H, G, d, dv)
        y = torch.empty((T, H * dv), dtype=self.dtype, device=dev)
        ops.delta_out(o, self.norm_w, self.eps, g, y, H, dv)
        return self.out.forward(y)
