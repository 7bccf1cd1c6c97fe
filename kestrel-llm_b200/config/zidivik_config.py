"""Typed configuration of the Zidivik decoder, read from its own ``config.json`` keys.

Top level: ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, ``token_side.dim``
(absent or null: no per-layer token input) and ``layers``, a list with one entry per layer:
``type`` ("attention" or "channel_delta"), ``mixer`` (the mixer's sizes) and ``mlp`` (null
for none).  Attention mixers: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``mask.size``, ``mask.keep_first`` and optionally ``kv_from`` (the layer whose keys and values
this one uses).  Delta-rule mixers: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps);
the ranks of their two low-rank projections are sizes of the checkpoint's tensors
(``decay_rank`` / ``gate_rank`` may name them in the file; `with_tensor_shapes` fills them in
otherwise).  Feed-forward: ``kind`` "moe", ``router.experts``, ``router.top``, ``expert.ff``,
``expert.limit``.  Every size and constant comes from the file; nothing is assumed equal
between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, ModelConfig

NAME = "Zidivik"


def _pos_int(d: Dict[str, Any], key: str, where: str, allow_zero: bool = False) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0 or (v == 0 and not allow_zero):
        raise ConfigError(f"config.json: {where}.{key} must be a {'non-negative' if allow_zero else 'positive'} integer, got {v!r}")
    return v


def _number(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int               # 0: every earlier token
    keep_first: int
    kv_from: Optional[int]    # layer whose keys and values are used; None: its own


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int           # 0 until known
    gate_rank: int


@dataclass(frozen=True)
class MoESpec:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class LayerSpec:
    kind: str                 # "attention" | "channel_delta"
    mixer: Any                # AttentionSpec | DeltaSpec
    mlp: Optional[MoESpec]


@dataclass(frozen=True)
class ZidivikConfig(ModelConfig):
    layers: Tuple[LayerSpec, ...] = ()
    norm_eps: float = 1e-6
    side_dim: int = 0         # 0: no per-layer token input

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ZidivikConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _number(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        side = raw.get("token_side")
        side_dim = _pos_int(side, "dim", "token_side") if isinstance(side, dict) else 0
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and 'mixer'")
            m, kind = L["mixer"], L.get("type")
            heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
            dim, vdim = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
            if kind == "attention":
                mask = m.get("mask") or {}
                window = _pos_int(mask, "size", where + ".mask") if mask.get("size") is not None else 0
                keep = _pos_int(mask, "keep_first", where + ".mask", allow_zero=True) if mask.get("keep_first") is not None else 0
                kv_from = m.get("kv_from")
                if kv_from is not None:
                    src = layers[kv_from].mixer if isinstance(kv_from, int) and not isinstance(kv_from, bool) and 0 <= kv_from < i else None
                    if not isinstance(src, AttentionSpec) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {where}.kv_from must name an earlier attention layer with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (kv_heads, dim, vdim):
                        raise ConfigError(f"config.json: {where} and layer {kv_from}, whose keys and values it uses, differ in head sizes")
                mixer: Any = AttentionSpec(heads, kv_heads, dim, vdim, _number(m, "scale", where), window, keep, kv_from)
            elif kind == "channel_delta":
                mixer = DeltaSpec(heads, kv_heads, dim, vdim, _pos_int(m, "conv", where),
                                  int(m.get("decay_rank") or 0), int(m.get("gate_rank") or 0))
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is neither 'attention' nor 'channel_delta'")
            f = L.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "moe" or not isinstance(f.get("router"), dict) or not isinstance(f.get("expert"), dict):
                    raise ConfigError(f"config.json: {where}.mlp must be null or a 'moe' with 'router' and 'expert'")
                experts, top = _pos_int(f["router"], "experts", where + ".mlp.router"), _pos_int(f["router"], "top", where + ".mlp.router")
                if top > experts:
                    raise ConfigError(f"config.json: {where}.mlp uses {top} of {experts} experts")
                mlp = MoESpec(experts, top, _pos_int(f["expert"], "ff", where + ".mlp.expert"), _number(f["expert"], "limit", where + ".mlp.expert"))
            layers.append(LayerSpec(kind, mixer, mlp))
        max_pos = raw.get("max_positions")
        return cls(architecture=NAME, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(max_pos) if max_pos else 1 << 17, bos_token_id=None,
                   eos_token_ids=tuple(int(e) for e in raw.get("eos", ())), layers=tuple(layers), norm_eps=eps, side_dim=side_dim)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "ZidivikConfig":
        """The sizes that only the checkpoint tells: the ranks of the delta-rule mixers' low-rank
        projections, from the shapes of their first matrices."""
        layers = list(self.layers)
        for i, L in enumerate(layers):
            if isinstance(L.mixer, DeltaSpec):
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                if a1 is None or g1 is None or len(a1) != 2 or len(g1) != 2:
                    raise ConfigError(f"layer {i}: the checkpoint has no l{i}.mix.a1 / l{i}.mix.g1 to size the low-rank projections by")
                layers[i] = replace(L, mixer=replace(L.mixer, decay_rank=int(a1[0]), gate_rank=int(g1[0])))
        return replace(self, layers=tuple(layers))

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": NAME, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                               "max_positions": self.max_position_embeddings, "layers": []}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos"] = list(self.eos_token_ids)
        for L in self.layers:
            m = L.mixer
            if isinstance(m, AttentionSpec):
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.window:
                    mixer["mask"] = {"size": m.window, "keep_first": m.keep_first}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.taps,
                         "decay_rank": m.decay_rank, "gate_rank": m.gate_rank}
            mlp = None
            if L.mlp is not None:
                mlp = {"kind": "moe", "router": {"experts": L.mlp.experts, "top": L.mlp.top}, "expert": {"ff": L.mlp.ff, "limit": L.mlp.limit}}
            out["layers"].append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        return out
