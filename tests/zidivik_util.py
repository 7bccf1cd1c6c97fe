"""Helpers of the Zidivik tests: small configurations of their own, a writer of random weights
whose scale lets every mechanism matter, and the comparison of the engine with the plain
implementation (`plain_zidivik`).  The writer is independent of the engine's random-weights mode:
it names every tensor itself, so a weight slot that the engine forgets or misnames shows as a
loading error."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_zidivik as P


def attn(heads, kv_heads, dim, vdim, scale, size=None, keep_first=0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# Z1: grouped heads, values wider than keys, a reader of another layer's pages with a mask of its own, a window shorter
# than a page, two delta layers that differ in every size, one expert of three, a layer without feed-forward.
Z1 = {"architecture": "Zidivik", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8}, "layers": [
    layer(attn(4, 2, 16, 24, 0.3, size=24, keep_first=5), moe(6, 2, 40, 1.0)),
    layer(delta(4, 2, 16, 8, 3), moe(3, 1, 24, 2.5)),
    layer(attn(4, 2, 16, 24, 0.45, size=40, keep_first=3, kv_from=0), None),
    layer(attn(2, 1, 32, 16, 0.2, size=9, keep_first=0), moe(6, 2, 40, 1.0)),
    layer(delta(2, 2, 40, 48, 4), moe(5, 5, 16, 0.75)),
]}
# Z2: a delta layer first, a width that is no multiple of 8, no token input, attention over all keys, kept tokens beyond
# the window's length, one tap, ranks of the low-rank projections that differ.
Z2 = {"architecture": "Zidivik", "vocab": 97, "width": 70, "norm": {"eps": 1e-6}, "layers": [
    layer(delta(3, 1, 24, 20, 1), moe(4, 2, 30, 1.25)),
    layer(attn(5, 5, 14, 14, 0.5), moe(4, 1, 30, 2.0)),
    layer(attn(6, 3, 8, 40, 0.7, size=16, keep_first=33), moe(7, 3, 18, 3.0)),
    layer(attn(6, 3, 8, 40, 0.9, size=50, keep_first=2, kv_from=2), moe(2, 2, 50, 1.0)),
    layer(delta(6, 2, 64, 32, 5), None),
]}
CONFIGS = {"Z1": (Z1, 3), "Z2": (Z2, 8)}
RANKS = {"Z1": (12, 9), "Z2": (7, 16)}          # (decay rank, gate rank) of the delta layers: sizes of tensors, not of config.json


def tensors_of(cfg: dict, seed: int, ranks=(12, 9)) -> Dict[str, np.ndarray]:
    """Random float32 tensors for ``cfg``, by name.  Matrices N(0, g / sqrt(in)) so that activations keep their size
    through the layers; norm weights around 1; convolution taps, decay parameters and router biases of order 1."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        W[name] = (rng.standard_normal((out, inn)) * gain / np.sqrt(inn)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        W[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    W["embed"] = rng.standard_normal((V, D)).astype(np.float32)
    side = cfg.get("token_side")
    if side:
        W["side.embed"] = rng.standard_normal((V, len(cfg["layers"]) * side["dim"])).astype(np.float32)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 1.0, 0.1)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            mat(p + "mix.q", H * d, D)
            if m.get("kv_from") is None:
                mat(p + "mix.k", G * d, D)
                mat(p + "mix.v", G * dv, D)
            mat(p + "mix.g", H, D, 2.0)
            mat(p + "mix.o", D, H * dv)
        else:
            taps, (ra, rg) = m["conv"], ranks
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                mat(p + "mix." + n, rows, D)
                W[p + f"mix.{n}.conv"] = (rng.standard_normal((rows, taps)) * 0.6).astype(np.float32)
            mat(p + "mix.b", H, D, 2.0)
            vec(p + "mix.A_log", H, -0.5, 0.7)
            vec(p + "mix.norm", dv, 1.0, 0.1)
            mat(p + "mix.a1", ra, D)
            mat(p + "mix.a2", H * d, ra, 2.0)
            vec(p + "mix.dt_bias", H * d, -1.0, 1.0)
            mat(p + "mix.g1", rg, D)
            mat(p + "mix.g2", H * dv, rg, 2.0)
            mat(p + "mix.o", D, H * dv)
        f = L.get("mlp")
        if f is not None:
            for e in range(f["router"]["experts"]):
                mat(f"{p}mlp.e{e}.gate", f["expert"]["ff"], D, 1.5)
                mat(f"{p}mlp.e{e}.up", f["expert"]["ff"], D, 1.5)
                mat(f"{p}mlp.e{e}.down", D, f["expert"]["ff"])
            mat(p + "mlp.router", f["router"]["experts"], D, 2.0)
            vec(p + "mlp.router.b", f["router"]["experts"], 0.0, 0.5)
        if side:
            mat(p + "side.gate", side["dim"], D)
            mat(p + "side.proj", D, side["dim"])
            vec(p + "side.norm", D, 0.5, 0.1)
    vec("final.norm", D, 1.0, 0.1)
    mat("head", V, D)
    return W


def write_model(cfg: dict, W: Dict[str, np.ndarray], base) -> Dict[str, str]:
    """Writes the model twice: tensors in bfloat16, and the same values widened to float32.  Returns {dtype: folder}."""
    import torch
    from kestrel_llm_b200.weights.safetensors_io import write_safetensors
    out = {}
    rounded = {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in W.items()}
    for dtype in ("bfloat16", "float32"):
        d = os.path.join(str(base), dtype)
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          ((n, t if dtype == "bfloat16" else t.to(torch.float32)) for n, t in rounded.items()))
        out[dtype] = d
    return out


@functools.lru_cache(maxsize=None)
def _model(model_dir: str):
    return P.read_model(model_dir)


@functools.lru_cache(maxsize=None)
def plain_logits(model_dir: str, tokens: Tuple[int, ...]) -> np.ndarray:
    cfg, W = _model(model_dir)
    return P.forward(cfg, W, list(tokens))


@functools.lru_cache(maxsize=None)
def first_close_call(model_dir: str, tokens: Tuple[int, ...], margin: float) -> int:
    """First position at which some layer's router separates its last chosen expert from the best one left out by
    less than ``margin``: from there on a run in reduced precision may route otherwise (len(tokens) if none)."""
    cfg, W = _model(model_dir)
    eps = cfg["norm"]["eps"]
    first = len(tokens)
    x = P.embed(W, tokens, cfg["width"])
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = P.rms_norm(x, W[p + "norm1"], eps)
        if L["type"] == "attention":
            kv = kept[m["kv_from"]] if m.get("kv_from") is not None else kept.setdefault(i, P.attention_keys_values(W, p + "mix.", m, h, eps))
            y = P.attention(W, p + "mix.", m, h, eps, kv)
        else:
            y = P.channel_delta(W, p + "mix.", m, h, eps)
        f = L.get("mlp")
        if f is not None:
            top = f["router"]["top"]
            if top < f["router"]["experts"]:
                z = np.sort(P.linear(h, W[p + "mlp.router"]) + W[p + "mlp.router.b"], axis=1)[:, ::-1]
                close = np.nonzero(z[:, top - 1] - z[:, top] < margin)[0]
                if close.size:
                    first = min(first, int(close[0]))
            y = y + P.moe(W, p + "mlp.", f, h)
        x = x + y
        if cfg.get("token_side"):
            x = x + P.token_side(W, p + "side.", i, cfg["token_side"]["dim"], x, tokens, eps)
    return first


# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the request.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def compare_with_plain(model_dir_f32: str, reqs: Dict[str, List[int]], got, dtype: str, label: str = "") -> float:
    """Every logits row of a trace against the plain implementation.  In bfloat16, positions from a request's first close
    router call on are left out (the float32 run covers them).  Names the first wrong (request, position)."""
    worst = 0.0
    for name, toks in reqs.items():
        ref = plain_logits(model_dir_f32, tuple(toks))
        scale = float(np.abs(ref).max())
        upto = len(toks) if dtype == "float32" else first_close_call(model_dir_f32, tuple(toks), 0.25)
        assert set(got[name]) == set(range(len(toks))), f"{label}: {name} misses positions"
        for p in range(upto):
            row = got[name][p]
            assert np.isfinite(row).all(), f"{label}: {name} position {p}: logits are not finite"
            err = float(np.abs(row - ref[p]).max()) / scale
            worst = max(worst, err)
            assert err <= TOL[dtype], (f"{label}: first wrong place: request {name} position {p} of {len(toks)}: "
                                       f"error {err:.3e} of the largest logit, allowed {TOL[dtype]:.1e}")
    return worst


# ---- one part alone ------------------------------------------------------------------------------

class PartHarness:
    """Runs one mixer through the engine's cache manager and step description, without a model around it: portions of
    rows [T, width] per request go in, the summed product comes out."""

    def __init__(self, mixer, dtype: str, max_tokens: int = 512, page_size: int = 16, slots: int = 4, extra_specs=()):
        import torch
        from kestrel_llm_b200.cache import CacheManager
        self.torch = torch
        self.mixer = mixer
        self.dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        self.cache = CacheManager([mixer.cache_spec()] + list(extra_specs), self.dtype, "cuda:0", page_size, (max_tokens + page_size - 1) // page_size,
                                  slots, 1 << 14)

    def step(self, portions: Sequence[Tuple[int, np.ndarray]], layer: int = 0, writable: bool = True, mixer=None,
             commit: bool = True) -> List[np.ndarray]:
        """portions: (request id, rows float [n, width]); returns each portion's output rows as float64.  A mixer that
        only reads the layer (``writable`` False) runs between the writer's step (``commit`` False) and `commit`."""
        torch = self.torch
        from kestrel_llm_b200.engine.batch import Entry, StepBatch
        entries = []
        for rid, rows in portions:
            if not self.cache.is_live(rid):
                self.cache.admit(rid)
            if writable:
                self.cache.reserve(rid, len(rows))
            entries.append(Entry(rid, [0] * len(rows), []))
        self.cache.clear_admitted()
        batch = StepBatch(entries, self.cache, "cuda:0")
        x = torch.from_numpy(np.concatenate([r for _, r in portions]).astype(np.float32)).to("cuda:0").to(self.dtype)
        y = (mixer or self.mixer).forward(x, batch, self.cache.layer(layer, writable)).reduce(torch.float32).cpu().numpy().astype(np.float64)
        self.last = [(rid, len(rows)) for rid, rows in portions]
        if writable and commit:
            self.commit()
        out, at = [], 0
        for _, rows in portions:
            out.append(y[at:at + len(rows)])
            at += len(rows)
        return out

    def commit(self):
        for rid, n in self.last:
            self.cache.commit(rid, n)


def load_part(part, W: Dict[str, np.ndarray]):
    """Fills a part's weight slots from ``W`` (rounded to bfloat16 first, as a checkpoint stores them)."""
    import torch
    names = set()
    for s in part.weight_slots():
        with torch.no_grad():
            s.dest.copy_(torch.from_numpy(W[s.name]).to(torch.bfloat16).to(s.dest.dtype))
        names.add(s.name)
    return names


def bf16_round(W: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    import torch
    return {n: torch.from_numpy(a).to(torch.bfloat16).to(torch.float64).numpy() for n, a in W.items()}
