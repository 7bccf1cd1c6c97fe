"""Typed configuration of the Tidavik decoder, read from its own ``config.json`` keys.

Top level: ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list
with one entry per layer: ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp``
(``{"kind": "dense", "ff": n}``, or null for a layer without feed-forward).  Mixers:

* ``attention`` and ``attention_2``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
  ``softcap`` and ``mask.size`` (the sliding window).  The first norms q and k over their whole
  projections, takes a logarithmic distance term off the capped scores and weighs keys by a sigmoid;
  the second norms the values per head and uses a softmax with one more term in its denominator.
* ``latent_attention``: ``heads``, ``dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale`` and
  ``mask.size``: queries through a latent, keys and values from a cached latent, a gate per head.

Every size and constant comes from the file; nothing is assumed equal between layers.  A mixer
without ``mask`` sees every earlier token; one without ``softcap`` (or with 0) has no cap.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, ModelConfig
from .zidivik_config import _number, _pos_int

NAME = "Tidavik"

SIGMOID_ATTENTION, SINK_ATTENTION, LATENT_ATTENTION = "attention", "attention_2", "latent_attention"


@dataclass(frozen=True)
class GroupedSpec:
    """Mixers ``attention`` and ``attention_2``."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float            # 0: none
    window: int               # 0: every earlier token


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int


@dataclass(frozen=True)
class DenseSpec:
    ff: int


@dataclass(frozen=True)
class TidavikLayer:
    kind: str                 # one of the three mixer names
    mixer: Any                # GroupedSpec | LatentSpec
    mlp: Optional[DenseSpec]


def _window(m: Dict[str, Any], where: str) -> int:
    mask = m.get("mask")
    if mask is None:
        return 0
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object with 'size'")
    return _pos_int(mask, "size", where + ".mask") if mask.get("size") is not None else 0


@dataclass(frozen=True)
class TidavikConfig(ModelConfig):
    layers: Tuple[TidavikLayer, ...] = ()
    norm_eps: float = 1e-6

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "TidavikConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _number(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m, kind = L["mixer"], L.get("type")
            heads, dim, vdim = _pos_int(m, "heads", where), _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
            scale, window = _number(m, "scale", where), _window(m, where)
            if kind in (SIGMOID_ATTENTION, SINK_ATTENTION):
                kv_heads = _pos_int(m, "kv_heads", where)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
                cap = _number(m, "softcap", where) if m.get("softcap") is not None else 0.0
                if cap < 0:
                    raise ConfigError(f"config.json: {where}.softcap must be positive (or 0 or absent for none)")
                mixer: Any = GroupedSpec(heads, kv_heads, dim, vdim, scale, cap, window)
            elif kind == LATENT_ATTENTION:
                mixer = LatentSpec(heads, dim, vdim, _pos_int(m, "q_rank", where), _pos_int(m, "kv_rank", where), scale, window)
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is none of '{SIGMOID_ATTENTION}', '{SINK_ATTENTION}', "
                                  f"'{LATENT_ATTENTION}'")
            f = L.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'dense' with 'ff'")
                mlp = DenseSpec(_pos_int(f, "ff", where + ".mlp"))
            layers.append(TidavikLayer(kind, mixer, mlp))
        max_pos = raw.get("max_positions")
        return cls(architecture=NAME, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(max_pos) if max_pos else 1 << 17, bos_token_id=None,
                   eos_token_ids=tuple(int(e) for e in raw.get("eos", ())), layers=tuple(layers), norm_eps=eps)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": NAME, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                               "max_positions": self.max_position_embeddings, "layers": []}
        if self.eos_token_ids:
            out["eos"] = list(self.eos_token_ids)
        for L in self.layers:
            m = L.mixer
            if isinstance(m, GroupedSpec):
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.softcap:
                    mixer["softcap"] = m.softcap
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale}
            if m.window:
                mixer["mask"] = {"size": m.window}
            out["layers"].append({"type": L.kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": L.mlp.ff} if L.mlp is not None else None})
        return out
