"""Softmax attention whose keys and values of all heads are expanded from one latent vector a
token, and only that vector is cached.

With h the mixer's input, H heads, d query/key dimensions and dv value dimensions a head:

    cq = rmsnorm(W_dq h) * w_q                  query latent, q_rank numbers
    q  = W_uq cq                                [H, d]
    c  = rmsnorm(W_dkv h) * w_kv                key/value latent, kv_rank numbers - what the cache keeps
    k_n = Uk_n c,  v_n = Uv_n c                 head n's rows of W_uk [H d, kv_rank] and W_uv [H dv, kv_rank]
    p   = softmax_j(q_n . k_nj * scale)         over the window: query i sees key j if 0 <= i - j < window (0: all)
    y   = W_o concat_n( sigmoid(W_g h)_n * sum_j p_j v_nj )

Heads are not rotated.  Since q_n . k_nj = (Uk_n^T q_n) . c_j and sum_j p_j v_nj = Uv_n sum_j p_j c_j,
attention runs over the cached latents themselves as ONE key/value head of size kv_rank shared by
all query heads (`PagedKVSpec.values_are_keys`): the queries are taken into the latent space by a
head-wise product before it, the mixed latents out of it by another one afterwards.  W_dq, W_dkv
and W_g are one fused product.  The gate may be absent (``head_gate=False``).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, WeightSlot
from .linear import Linear


class LatentAttention(Mixer):
    force_plain = False        # tests: bfloat16 through the plain attention kernel too
    graph_safe = True          # forward launches kernels over device tensors of the batch only

    def __init__(self, width: int, heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int, dtype: torch.dtype, device,
                 prefix: str, scale: float, norm_eps: float, window: int = 0, head_gate: bool = True,
                 names=("dq", "uq", "dkv", "uk", "uv", "g", "o")):
        if kv_rank > 256:
            raise ValueError(f"a cached latent of {kv_rank} numbers: the attention kernels take head sizes up to 256")
        self.width, self.heads, self.head_dim, self.v_head_dim = width, heads, head_dim, v_head_dim
        self.q_rank, self.kv_rank, self.window = q_rank, kv_rank, int(window)
        self.scale, self.norm_eps, self.head_gate = float(scale), float(norm_eps), head_gate
        self.prefix, self.names, self.dtype = prefix, names, dtype
        self.down = Linear(width, q_rank + kv_rank + (heads if head_gate else 0), dtype, device)
        self.up_q = Linear(q_rank, heads * head_dim, dtype, device)
        self.up_k = Linear(kv_rank, heads * head_dim, dtype, device)       # used transposed, head by head
        self.up_v = Linear(kv_rank, heads * v_head_dim, dtype, device)
        self.out = Linear(heads * v_head_dim, width, dtype, device)
        self.q_norm_w = torch.empty((q_rank,), dtype=torch.float32, device=device)
        self.kv_norm_w = torch.empty((kv_rank,), dtype=torch.float32, device=device)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(1, self.kv_rank, self.window, 0, self.kv_rank, values_are_keys=True)

    def weight_slots(self) -> List[WeightSlot]:
        p, (dq, uq, dkv, uk, uv, g, o) = self.prefix, self.names
        w, r = self.down.weight, self.q_rank + self.kv_rank
        slots = [WeightSlot(p + dq, w[:self.q_rank]), WeightSlot(p + dkv, w[self.q_rank:r]),
                 WeightSlot(p + dq + ".norm", self.q_norm_w, "norm"), WeightSlot(p + dkv + ".norm", self.kv_norm_w, "norm"),
                 WeightSlot(p + uq, self.up_q.weight), WeightSlot(p + uk, self.up_k.weight), WeightSlot(p + uv, self.up_v.weight),
                 WeightSlot(p + o, self.out.weight)]
        if self.head_gate:
            slots.append(WeightSlot(p + g, w[r:]))
        return slots

    def forward(self, x: torch.Tensor, batch, cache, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        T, H, R = x.shape[0], self.heads, self.kv_rank
        fused = self.down.forward(x)
        cq = torch.empty((T, self.q_rank), dtype=self.dtype, device=x.device)
        gate = torch.empty((T, H), dtype=torch.float32, device=x.device) if self.head_gate else None
        table = batch.block_table(cache.group)
        ops.latent_prepare(fused, self.q_norm_w, self.kv_norm_w, self.norm_eps, batch.positions, batch.seq_of_token, table, cache.page_size,
                           cache.k, cq, gate)
        q = self.up_q.forward(cq).reduce(self.dtype)                           # [T, H d]
        q_lat = ops.head_gemm(q, self.up_k.weight, H, w_kn=True)               # [T, H kv_rank]: Uk_n^T q_n
        a = torch.empty((T, H * R), dtype=self.dtype, device=x.device)
        if self.dtype == torch.bfloat16 and not self.force_plain and ops.attention_window_supported(R, R, H, 1):
            ops.attention_window(q_lat, cache.k, cache.k, batch, table, cache.page_size, a, H, 1, R, R, self.window, 0, gate, self.scale)
        else:
            ops.attention_plain_ex(q_lat, cache.k, cache.k, batch.positions, batch.seq_of_token, table, cache.page_size, a, H, 1, R, R,
                                   self.window, 0, gate, self.scale)
        o = ops.head_gemm(a, self.up_v.weight, H, w_kn=False)                  # [T, H dv]: Uv_n (mixed latent)
        return self.out.forward(o, residual=residual)      # many tokens: the product adds itself to the stream
