"""The Tidavik decoder assembled from parts.

Embedding plus a sinusoidal position vector, then an RMSNorm of its own; layers in the order the
configuration lists them, each a `PreNormBlock` (norm, mixer, residual; norm, gated feed-forward,
residual - the second half absent where the layer has no feed-forward); a final RMSNorm and the
output head.  A layer's mixer is one of

* ``attention``: `GatedWindowAttention` without gate, with biased projections, q and k normed over
  their whole projections, capped scores less a distance term, sigmoid weights with a number per head;
* ``attention_2``: the same part with biased projections, values of unit root mean square, capped
  scores and a softmax with one more term in its denominator;
* ``latent_attention``: `LatentAttention` (queries through a latent, keys and values expanded from a
  cached latent, a gate per head),

all over a sliding window.  Checkpoint tensors: ``embed``, ``embed.norm``, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_architecture
from ..config.tidavik_config import NAME, SIGMOID_ATTENTION, GroupedSpec, LatentSpec, TidavikConfig
from ..parts import GatedMLP, GatedWindowAttention, LatentAttention, LMHead, PreNormBlock, RMSNorm, SinusoidalPositions, TokenEmbedding
from .decoder import DecoderModel, LayerCall


def build_tidavik(config: TidavikConfig, dtype: torch.dtype, device) -> DecoderModel:
    c = config
    W = c.hidden_size
    blocks, order, optional = [], [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, GroupedSpec):
            sigmoid = layer.kind == SIGMOID_ATTENTION
            mixer = GatedWindowAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, dtype, device, p + "mix.", m.scale, c.norm_eps,
                                         window=m.window, head_gate=False, bias=True, softcap=m.softcap,
                                         qk_norm="projection" if sigmoid else None, v_norm=not sigmoid, distance_bias=sigmoid,
                                         head_bias=sigmoid, weighting="sigmoid" if sigmoid else "softmax_sink")
        else:
            assert isinstance(m, LatentSpec)
            mixer = LatentAttention(W, m.heads, m.dim, m.vdim, m.q_rank, m.kv_rank, dtype, device, p + "mix.", m.scale, c.norm_eps,
                                    window=m.window)
        ffn = norm2 = None
        if layer.mlp is not None:
            ffn = GatedMLP(W, layer.mlp.ff, dtype, device, p + "mlp.", names=("gate", "up", "down"))
            norm2 = RMSNorm(W, c.norm_eps, device, p + "norm2")
        else:
            optional.append(p + "norm2")      # a layer without feed-forward has no use for its second norm
        blocks.append(PreNormBlock(RMSNorm(W, c.norm_eps, device, p + "norm1"), mixer, norm2, ffn, dtype))
        order.append(LayerCall(block=i, cache=i))
    return DecoderModel(c, dtype, device, TokenEmbedding(c.vocab_size, W, dtype, device, "embed"), SinusoidalPositions(W, device),
                        blocks, order, RMSNorm(W, c.norm_eps, device, "final.norm"), LMHead(c.vocab_size, W, dtype, device, "head"),
                        optional_tensors=optional, embedding_norm=RMSNorm(W, c.norm_eps, device, "embed.norm"))


register_architecture(NAME, TidavikConfig, build_tidavik)
