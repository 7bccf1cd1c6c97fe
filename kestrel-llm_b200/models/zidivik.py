"""The Zidivik decoder assembled from parts.

Embedding plus a sinusoidal position vector; layers in the order the configuration lists them,
each a `ParallelBlock` (one RMSNorm, a mixer and a routed feed-forward that both read it, then a
per-layer token input); a final RMSNorm and the output head.  A layer's mixer is a
`GatedWindowAttention` (softmax attention without rotation over a window that keeps the first
tokens, with an output gate; optionally over another layer's keys and values) or a
`ChannelDeltaMixer` (gated delta rule with a decay per key channel).  Checkpoint tensors:
``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_architecture
from ..config.zidivik_config import NAME, AttentionSpec, DeltaSpec, ZidivikConfig
from ..parts import (ChannelDeltaMixer, GatedWindowAttention, LMHead, ParallelBlock, RMSNorm, RoutedExperts, SinusoidalPositions,
                     TokenEmbedding, TokenSideInput, TokenTable)
from .decoder import DecoderModel, LayerCall


def build_zidivik(config: ZidivikConfig, dtype: torch.dtype, device) -> DecoderModel:
    c = config
    W, L = c.hidden_size, len(c.layers)
    emb = TokenEmbedding(c.vocab_size, W, dtype, device, "embed")
    pos = SinusoidalPositions(W, device)
    table = TokenTable(c.vocab_size, L * c.side_dim, dtype, device, "side.embed") if c.side_dim else None
    # the pages a layer writes must hold what every layer that reads them can see
    need = {}
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if isinstance(m, AttentionSpec):
            j = i if m.kv_from is None else m.kv_from
            w, k = need.get(j, (m.window, m.keep_first))
            full = w == 0 or m.window == 0
            need[j] = (0 if full else max(w, m.window), max(k, m.keep_first))
    blocks, order, cache_of = [], [], {}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, AttentionSpec):
            own = m.kv_from is None
            cw, ck = need[i if own else m.kv_from]
            mixer = GatedWindowAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, dtype, device, p + "mix.", m.scale, c.norm_eps,
                                         window=m.window, keep_first=m.keep_first, own_kv=own, cache_window=cw, cache_keep_first=ck)
            if own:
                cache_of[i] = len(cache_of)
            order.append(LayerCall(block=i, cache=cache_of[i if own else m.kv_from], writes_cache=own))
        else:
            assert isinstance(m, DeltaSpec)
            if not (m.decay_rank and m.gate_rank):
                raise ValueError(f"layer {i}: the ranks of the low-rank projections are unknown (ZidivikConfig.with_tensor_shapes)")
            mixer = ChannelDeltaMixer(W, m.heads, m.kv_heads, m.dim, m.vdim, m.taps, m.decay_rank, m.gate_rank, c.norm_eps, dtype,
                                      device, p + "mix.")
            cache_of[i] = len(cache_of)
            order.append(LayerCall(block=i, cache=cache_of[i], writes_cache=True))
        f = layer.mlp
        ffn = RoutedExperts(W, f.ff, f.experts, f.top, f.limit, dtype, device, p + "mlp.") if f is not None else None
        side = TokenSideInput(W, c.side_dim, table, i * c.side_dim, c.norm_eps, dtype, device, p + "side.") if table is not None else None
        blocks.append(ParallelBlock(RMSNorm(W, c.norm_eps, device, p + "norm1"), mixer, ffn, side, dtype))
    return DecoderModel(c, dtype, device, emb, pos, blocks, order, RMSNorm(W, c.norm_eps, device, "final.norm"),
                        LMHead(c.vocab_size, W, dtype, device, "head"), shared_parts=[table] if table is not None else [])


register_architecture(NAME, ZidivikConfig, build_zidivik)
