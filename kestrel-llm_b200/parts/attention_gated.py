"""Grouped-query softmax attention without rotation, over a window that keeps the first tokens
of a request, with values of their own size and a gate on every head's output.

q, k, v and the gate logits are one fused product of the mixer's input h.  q and k are divided by
their root mean square per head (no weight); score = q . k * scale with ``scale`` a parameter;
query i sees key j <= i if i - j < window or j < keep_first (window 0: every j <= i); the output
of head n is multiplied by sigmoid(gate logit n) before the output projection.  K (after the
norm) and V go to the request's pages; a mixer built with ``own_kv=False`` has no key and value
projections and attends over the pages that an earlier layer of the same step wrote, with its
own queries, mask and scale.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, WeightSlot
from .linear import Linear


class GatedWindowAttention(Mixer):
    force_plain = False        # tests: bfloat16 through the plain kernel too, the twin of the tensor-core one
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, v_head_dim: int, dtype: torch.dtype, device,
                 prefix: str, scale: float, norm_eps: float, window: int = 0, keep_first: int = 0, own_kv: bool = True,
                 head_gate: bool = True, cache_window: Optional[int] = None, cache_keep_first: Optional[int] = None,
                 names=("q", "k", "v", "g", "o")):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if max(head_dim, v_head_dim) > 256:
            raise ValueError(f"head sizes {head_dim} / {v_head_dim}: the attention kernels take sizes up to 256")
        self.width, self.heads, self.kv_heads, self.head_dim, self.v_head_dim = width, heads, kv_heads, head_dim, v_head_dim
        self.window, self.keep_first = int(window), int(keep_first) if window else 0
        # what the cache must hold: this layer's mask, widened by the layers that read its pages
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.own_kv, self.head_gate = own_kv, head_gate
        self.prefix, self.names, self.dtype = prefix, names, dtype
        self.q_cols = heads * head_dim
        self.kv_cols = kv_heads * (head_dim + v_head_dim) if own_kv else 0
        self.proj = Linear(width, self.q_cols + self.kv_cols + (heads if head_gate else 0), dtype, device)
        self.out = Linear(heads * v_head_dim, width, dtype, device)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.kv_heads, self.head_dim, self.cache_window, self.cache_keep_first, self.v_head_dim)

    def weight_slots(self) -> List[WeightSlot]:
        p, (nq, nk, nv, ng, no) = self.prefix, self.names
        w = self.proj.weight
        slots = [WeightSlot(p + nq, w[:self.q_cols])]
        if self.own_kv:
            k_end = self.q_cols + self.kv_heads * self.head_dim
            slots += [WeightSlot(p + nk, w[self.q_cols:k_end]), WeightSlot(p + nv, w[k_end:self.q_cols + self.kv_cols])]
        if self.head_gate:
            slots.append(WeightSlot(p + ng, w[self.q_cols + self.kv_cols:]))
        slots.append(WeightSlot(p + no, self.out.weight))
        return slots

    def forward(self, x: torch.Tensor, batch, cache) -> ops.Partials:
        if cache.writable != self.own_kv:
            raise ValueError("a mixer with key and value projections writes its cache layer; one without reads another's")
        T = x.shape[0]
        fused = self.proj.forward(x)
        q = torch.empty((T, self.q_cols), dtype=self.dtype, device=x.device)
        gate = torch.empty((T, self.heads), dtype=torch.float32, device=x.device) if self.head_gate else None
        table = batch.block_table(cache.group)
        ops.attn_prepare_ex(fused, None, None, True, self.norm_eps, batch.positions, batch.seq_of_token, table, cache.page_size,
                            cache.k, cache.v, q, gate, self.heads, self.kv_heads, self.head_dim, self.v_head_dim, self.own_kv)
        a = torch.empty((T, self.heads * self.v_head_dim), dtype=self.dtype, device=x.device)
        if self.dtype == torch.bfloat16 and not self.force_plain and \
                ops.attention_window_supported(self.head_dim, self.v_head_dim, self.heads, self.kv_heads):
            ops.attention_window(q, cache.k, cache.v, batch, table, cache.page_size, a, self.heads, self.kv_heads, self.head_dim,
                                 self.v_head_dim, self.window, self.keep_first, gate, self.scale)
        else:           # float32, and head sizes that are no multiple of 8
            ops.attention_plain_ex(q, cache.k, cache.v, batch.positions, batch.seq_of_token, table, cache.page_size, a, self.heads,
                                   self.kv_heads, self.head_dim, self.v_head_dim, self.window, self.keep_first, gate, self.scale)
        return self.out.forward(a)
