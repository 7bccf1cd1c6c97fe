"""Plain restatement of the Tidavik decoder, for tests only.

Whole sequences, no cache, no batching, numpy float64 throughout, one function per mechanism.
Nothing here is imported by the engine and nothing of the engine is imported here: the file has
its own reader of config.json and of safetensors.

Notation.  T tokens at positions 0..T-1, width D.  The embedded tokens get a sinusoidal position
vector and a norm; a layer is

    x <- x + mixer(norm1(x));   x <- x + ff(norm2(x))          (the second line only if it has a feed-forward)

and the mixer is one of three kinds of attention over a sliding window: query i sees key j when
0 <= i - j < size.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F = np.float64


def read_safetensors(path: str) -> dict:
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[base + b: base + e]
        dt = info["dtype"]
        if dt == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(F)
        elif dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F)
        elif dt == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(tuple(info["shape"])).copy()
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---- small functions -------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def linear(x, w, b=None):
    """Rows of x times w^T, w stored [out, in]."""
    y = x @ w.T
    return y if b is None else y + b


def sinusoid(T: int, D: int, base: float = 10000.0):
    """[T, D]: entry 2i of position p is sin(p * base^(-2i / D)), entry 2i + 1 the cosine of that angle."""
    out = np.zeros((T, D), dtype=F)
    p = np.arange(T, dtype=F)[:, None]
    i = np.arange((D + 1) // 2, dtype=F)[None, :]
    ang = p * np.power(base, -2.0 * i / D)
    out[:, 0::2] = np.sin(ang)[:, :out[:, 0::2].shape[1]]
    out[:, 1::2] = np.cos(ang)[:, :out[:, 1::2].shape[1]]
    return out


def embed(W, tokens, D, eps):
    x = W["embed"][np.asarray(tokens)] + sinusoid(len(tokens), D)
    return rms_norm(x, W["embed.norm"], eps)


def window_mask(T: int, size):
    """[T, T] booleans: row i, column j is True when 0 <= i - j < size (no size: when 0 <= i - j)."""
    d = np.arange(T)[:, None] - np.arange(T)[None, :]
    return (d >= 0) & (d < (size if size else T))


def mask_of(m, T):
    return window_mask(T, (m.get("mask") or {}).get("size"))


def soft_cap(s, cap):
    """cap * tanh(s / cap); no cap (absent or 0): s."""
    return cap * np.tanh(s / cap) if cap else s


# ---- the three mixers ------------------------------------------------------------------------

def _heads(y, n, d):
    return y.reshape(y.shape[0], n, d).transpose(1, 0, 2)            # [n, T, d]


def sigmoid_attention(W, p, m, h, eps):
    """Grouped heads with biased projections; q and k each normed over the whole projection; capped
    scores less a logarithmic distance term; every visible key weighs sigmoid(score + head's number),
    with no normalisation over keys."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(linear(h, W[p + "q"], W[p + "q.b"]), W[p + "q.norm"], eps)
    k = rms_norm(linear(h, W[p + "k"], W[p + "k.b"]), W[p + "k.norm"], eps)
    v = linear(h, W[p + "v"], W[p + "v.b"])
    q, k, v = _heads(q, H, d), _heads(k, G, d), _heads(v, G, dv)
    vis = mask_of(m, T)
    dist = np.maximum(np.arange(T)[:, None] - np.arange(T)[None, :], 0).astype(F)
    out = np.zeros((T, H, dv), dtype=F)
    for n in range(H):
        g = n // (H // G)
        s = soft_cap((q[n] @ k[g].T) * m["scale"], m.get("softcap"))
        s = s - W[p + "r1"][n] * np.log(1.0 + W[p + "r2"][n] * dist)
        w = np.where(vis, sigmoid(s + W[p + "pb"][n]), 0.0)
        out[:, n] = w @ v[g]
    return linear(out.reshape(T, H * dv), W[p + "o"], W[p + "o.b"])


def sink_attention(W, p, m, h, eps):
    """Grouped heads with biased projections; values of unit root mean square per head; capped scores;
    softmax whose denominator has one more term, exp(0), that carries no value."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _heads(linear(h, W[p + "q"], W[p + "q.b"]), H, d)
    k = _heads(linear(h, W[p + "k"], W[p + "k.b"]), G, d)
    v = unit_rms(_heads(linear(h, W[p + "v"], W[p + "v.b"]), G, dv), eps)
    vis = mask_of(m, T)
    out = np.zeros((T, H, dv), dtype=F)
    for n in range(H):
        g = n // (H // G)
        s = soft_cap((q[n] @ k[g].T) * m["scale"], m.get("softcap"))
        e = np.where(vis, np.exp(s), 0.0)
        out[:, n] = (e / (1.0 + e.sum(axis=1, keepdims=True))) @ v[g]
    return linear(out.reshape(T, H * dv), W[p + "o"], W[p + "o.b"])


def latent_attention(W, p, m, h, eps):
    """Queries through a normed latent; keys and values of all heads expanded from one normed latent of
    ``kv_rank`` numbers a token; ordinary softmax over the window; a sigmoid gate per head."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(linear(h, W[p + "dq"]), W[p + "dq.norm"], eps)
    q = _heads(linear(cq, W[p + "uq"]), H, d)
    c = rms_norm(linear(h, W[p + "dkv"]), W[p + "dkv.norm"], eps)
    k = _heads(linear(c, W[p + "uk"]), H, d)
    v = _heads(linear(c, W[p + "uv"]), H, dv)
    gate = sigmoid(linear(h, W[p + "g"]))                             # [T, H]
    vis = mask_of(m, T)
    out = np.zeros((T, H, dv), dtype=F)
    for n in range(H):
        s = np.where(vis, (q[n] @ k[n].T) * m["scale"], -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, n] = (e / e.sum(axis=1, keepdims=True)) @ v[n] * gate[:, n:n + 1]
    return linear(out.reshape(T, H * dv), W[p + "o"])


MIXERS = {"attention": sigmoid_attention, "attention_2": sink_attention, "latent_attention": latent_attention}


def dense_ff(W, p, h):
    return linear(silu(linear(h, W[p + "gate"])) * linear(h, W[p + "up"]), W[p + "down"])


# ---- the model -------------------------------------------------------------------------------

def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; ``layers_out``, a list, receives the stream after every layer."""
    eps, D = cfg["norm"]["eps"], cfg["width"]
    x = embed(W, tokens, D, eps)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[L["type"]](W, p + "mix.", L["mixer"], rms_norm(x, W[p + "norm1"], eps), eps)
        if L.get("mlp") is not None:
            if L["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {L['mlp']['kind']}")
            x = x + dense_ff(W, p + "mlp.", rms_norm(x, W[p + "norm2"], eps))
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(rms_norm(x, W["final.norm"], eps), W["head"])
