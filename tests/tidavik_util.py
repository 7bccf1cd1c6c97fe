"""Helpers of the Tidavik tests: small configurations of their own, a writer of random weights whose scale lets
every mechanism matter, and the comparison of the engine with the plain implementation (`plain_tidavik`).  The
writer names every tensor itself, so a weight slot that the engine forgets or misnames shows as a loading error."""
from __future__ import annotations

import functools
from typing import Dict, List, Tuple

import numpy as np

import plain_tidavik as P
from zidivik_util import PartHarness, bf16_round, load_part, write_model  # noqa: F401  (helpers that know no architecture)


def grouped(kind, heads, kv_heads, dim, vdim, scale, size=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": kind, "mixer": m}


def sigmoid_attn(heads, kv_heads, dim, vdim, scale, size=None, softcap=None):
    return grouped("attention", heads, kv_heads, dim, vdim, scale, size, softcap)


def sink_attn(heads, kv_heads, dim, vdim, scale, size=None, softcap=None):
    return grouped("attention_2", heads, kv_heads, dim, vdim, scale, size, softcap)


def latent(heads, dim, vdim, q_rank, kv_rank, scale, size=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    return {"type": "latent_attention", "mixer": m}


def layer(mixer, ff=None):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


# T1: a latent layer first; grouped heads with values wider and narrower than keys; a window shorter than a page; a layer
# without feed-forward; as many kv heads as heads; one head; caps that differ; a query latent narrower than the cached one.
T1 = {"architecture": "Tidavik", "vocab": 173, "width": 72, "norm": {"eps": 1e-5}, "layers": [
    layer(latent(3, 24, 16, 40, 32, 0.2, size=19), 96),
    layer(sigmoid_attn(4, 2, 16, 24, 0.3, size=24, softcap=30.0), None),
    layer(sink_attn(6, 2, 8, 40, 0.5, size=9, softcap=12.0), 40),
    layer(sigmoid_attn(2, 2, 32, 8, 0.25, size=40, softcap=5.0), 56),
    layer(latent(1, 16, 48, 24, 56, 0.3, size=24), None),              # the window of layer 1: one cache group, planes of two shapes
    layer(sink_attn(2, 1, 24, 16, 0.2, size=70, softcap=40.0), 88),
]}
# T2: a width and head sizes that are no multiples of 8 (the plain kernels in bfloat16 too); a layer that sees every earlier
# token; layers without cap; a window longer than any request; five heads on one kv head.
T2 = {"architecture": "Tidavik", "vocab": 97, "width": 70, "norm": {"eps": 1e-6}, "layers": [
    layer(sink_attn(3, 3, 14, 10, 0.4), 30),
    layer(sigmoid_attn(5, 1, 12, 20, 0.35, size=16), 50),
    layer(latent(2, 12, 12, 36, 20, 0.3, size=500), 44),
    layer(sigmoid_attn(4, 4, 8, 8, 0.5, size=50, softcap=8.0), None),
    layer(latent(5, 8, 24, 16, 64, 0.45), 62),
]}
# T3: heads of 128 (prompt portions on the tcgen05 attention kernel), windows longer than a key tile of 128.
T3 = {"architecture": "Tidavik", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    layer(sigmoid_attn(2, 1, 128, 128, 0.09, size=150, softcap=20.0), 72),
    layer(sink_attn(4, 2, 128, 128, 0.1, size=70, softcap=25.0), None),
    layer(latent(2, 32, 32, 48, 40, 0.2, size=200), 48),
    layer(sink_attn(2, 2, 128, 128, 0.08, size=260), 72),
    layer(latent(3, 128, 128, 56, 72, 0.09, size=140), None),              # starting portions: keys and values expanded for the step
]}
CONFIGS = {"T1": (T1, 3), "T2": (T2, 8), "T3": (T3, 5)}


def tensors_of(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Random float32 tensors for ``cfg``, by name.  Matrices N(0, g / sqrt(in)) so that activations keep their size
    through the layers; norm weights around 1; biases, the heads' numbers and the distance terms of order 1."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        W[name] = (rng.standard_normal((out, inn)) * gain / np.sqrt(inn)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        W[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    W["embed"] = rng.standard_normal((V, D)).astype(np.float32)
    vec("embed.norm", D, 1.0, 0.1)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 1.0, 0.1)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "latent_attention":
            rq, rk = m["q_rank"], m["kv_rank"]
            mat(p + "mix.dq", rq, D)
            vec(p + "mix.dq.norm", rq, 1.0, 0.1)
            mat(p + "mix.uq", H * d, rq, 2.0)
            mat(p + "mix.dkv", rk, D)
            vec(p + "mix.dkv.norm", rk, 1.0, 0.1)
            mat(p + "mix.uk", H * d, rk, 2.0)
            mat(p + "mix.uv", H * dv, rk)
            mat(p + "mix.g", H, D, 2.0)
            mat(p + "mix.o", D, H * dv)
        else:
            G = m["kv_heads"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(p + "mix." + n, rows, D, 2.0 if n != "v" else 1.0)
                vec(p + f"mix.{n}.b", rows, 0.0, 0.3)
            mat(p + "mix.o", D, H * dv, 1.0 if L["type"] == "attention_2" else 0.3)
            vec(p + "mix.o.b", D, 0.0, 0.3)
            if L["type"] == "attention":
                vec(p + "mix.q.norm", H * d, 1.5, 0.2)
                vec(p + "mix.k.norm", G * d, 1.5, 0.2)
                W[p + "mix.r1"] = rng.uniform(0.2, 1.2, H).astype(np.float32)
                W[p + "mix.r2"] = rng.uniform(0.05, 0.8, H).astype(np.float32)
                vec(p + "mix.pb", H, -1.0, 1.0)
        f = L.get("mlp")
        if f is not None:
            vec(p + "norm2", D, 1.0, 0.1)
            mat(p + "mlp.gate", f["ff"], D, 1.5)
            mat(p + "mlp.up", f["ff"], D, 1.5)
            mat(p + "mlp.down", D, f["ff"])
    vec("final.norm", D, 1.0, 0.1)
    mat("head", V, D)
    return W


@functools.lru_cache(maxsize=None)
def _model(model_dir: str):
    return P.read_model(model_dir)


@functools.lru_cache(maxsize=None)
def plain_logits(model_dir: str, tokens: Tuple[int, ...]) -> np.ndarray:
    cfg, W = _model(model_dir)
    return P.forward(cfg, W, list(tokens))


# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the request.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def compare_with_plain(model_dir_f32: str, reqs: Dict[str, List[int]], got, dtype: str, label: str = "") -> float:
    """Every logits row of a trace against the plain implementation; names the first wrong (request, position)."""
    worst = 0.0
    for name, toks in reqs.items():
        ref = plain_logits(model_dir_f32, tuple(toks))
        scale = float(np.abs(ref).max())
        assert set(got[name]) == set(range(len(toks))), f"{label}: {name} misses positions"
        for p in range(len(toks)):
            row = got[name][p]
            assert np.isfinite(row).all(), f"{label}: {name} position {p}: logits are not finite"
            err = float(np.abs(row - ref[p]).max()) / scale
            worst = max(worst, err)
            assert err <= TOL[dtype], (f"{label}: first wrong place: request {name} position {p} of {len(toks)}: "
                                       f"error {err:.3e} of the largest logit, allowed {TOL[dtype]:.1e}")
    return worst
