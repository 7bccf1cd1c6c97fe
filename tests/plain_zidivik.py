"""Plain restatement of the Zidivik decoder, for tests only.

Whole sequences, no cache, no batching, numpy float64 throughout, one function per mechanism.
Nothing here is imported by the engine and nothing of the engine is imported here: the file has
its own reader of config.json and of safetensors.

Notation.  T tokens at positions 0..T-1, width D.  A layer is

    h = norm1(x);  x <- x + mixer(h) + ff(h);  x <- x + side(x, token)

with one norm whose output both sublayers read, and a per-layer token input after them.
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


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def linear(x, w):
    return x @ w.T


# ---- embedding -------------------------------------------------------------------------------

def sinusoid(positions, width: int):
    """Entry 2i is sin(p * 10000^(-2i/width)), entry 2i+1 the cosine of the same angle."""
    p = np.asarray(positions, dtype=F)[:, None]
    i = np.arange((width + 1) // 2, dtype=F)[None, :]
    ang = p * np.power(10000.0, -2.0 * i / width)
    out = np.zeros((p.shape[0], width), dtype=F)
    out[:, 0::2] = np.sin(ang)[:, : (width + 1) // 2]
    out[:, 1::2] = np.cos(ang)[:, : width // 2]
    return out


def embed(W, tokens, width):
    toks = np.asarray(tokens, dtype=np.int64)
    return W["embed"][toks] + sinusoid(np.arange(len(toks)), width)


# ---- attention -------------------------------------------------------------------------------

def visible(T: int, size: int, keep_first: int):
    """[T, T] mask: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention_keys_values(W, p, m, h, eps):
    """Keys as the cache holds them (unit root mean square per head) and values, [T, G, .]."""
    T = h.shape[0]
    G = m["kv_heads"]
    k = unit_rms(linear(h, W[p + "k"]).reshape(T, G, m["dim"]), eps)
    v = linear(h, W[p + "v"]).reshape(T, G, m["vdim"])
    return k, v


def attention(W, p, m, h, eps, kv):
    """Gated softmax attention without rotation over a window that keeps the first tokens.
    ``kv`` = (k, v) of the layer whose keys and values this one uses."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(linear(h, W[p + "q"]).reshape(T, H, d), eps)
    k, v = kv
    gate = sigmoid(linear(h, W[p + "g"]))                      # [T, H]
    mask = visible(T, m["mask"]["size"], m["mask"]["keep_first"]) if m.get("mask") else visible(T, T, 0)    # no mask: every earlier token
    out = np.zeros((T, H, dv), dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w = w / w.sum(axis=1, keepdims=True)
        out[:, hh] = (w @ v[:, g]) * gate[:, hh:hh + 1]
    return linear(out.reshape(T, H * dv), W[p + "o"])


# ---- gated delta rule with one decay per key channel -------------------------------------------

def causal_conv(x, w):
    """y[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C), dtype=F), x], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += xp[j:j + T] * w[:, j][None, :]
    return y


def unit_vector(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def channel_delta(W, p, m, h, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(linear(h, W[p + "q"]), W[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(linear(h, W[p + "k"]), W[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(linear(h, W[p + "v"]), W[p + "v.conv"])).reshape(T, H, dv)
    q = unit_vector(q) * d ** -0.5
    k = unit_vector(k)
    beta = sigmoid(linear(h, W[p + "b"]))                                              # [T, H]
    a = linear(linear(h, W[p + "a1"]), W[p + "a2"]) + W[p + "dt_bias"]
    decay = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, d))   # [T, H, d]
    out = np.zeros((T, H, dv), dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((d, dv), dtype=F)
        for t in range(T):
            S = decay[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = rms_norm(out, W[p + "norm"], eps)
    out = out * sigmoid(linear(linear(h, W[p + "g1"]), W[p + "g2"])).reshape(T, H, dv)
    return linear(out.reshape(T, H * dv), W[p + "o"])


# ---- feed-forward ----------------------------------------------------------------------------

def expert(W, p, h, limit):
    g = np.minimum(linear(h, W[p + "gate"]), limit)
    u = np.clip(linear(h, W[p + "up"]), -limit, limit)
    return linear(g * sigmoid(1.702 * g) * (u + 1.0), W[p + "down"])


def route(z, top):
    """The ``top`` largest logits of each row (ids [T, top]) and the softmax over them."""
    ids = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zz = np.take_along_axis(z, ids, axis=1)
    w = np.exp(zz - zz.max(axis=1, keepdims=True))
    return ids, w / w.sum(axis=1, keepdims=True)


def moe(W, p, f, h):
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    z = linear(h, W[p + "router"]) + W[p + "router.b"]
    ids, w = route(z, top)
    y = np.zeros((T, W[p + "e0.down"].shape[0]), dtype=F)
    for e in range(E):
        rows, slot = np.nonzero(ids == e)
        if rows.size:
            y[rows] += w[rows, slot][:, None] * expert(W, f"{p}e{e}.", h[rows], f["expert"]["limit"])
    return y


# ---- the per-layer token input -----------------------------------------------------------------

def token_side(W, p, layer, dim, x, tokens, eps):
    e = W["side.embed"][np.asarray(tokens, dtype=np.int64)][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(linear(x, W[p + "gate"])) * e
    return rms_norm(linear(g, W[p + "proj"]), W[p + "norm"], eps)


# ---- the model ---------------------------------------------------------------------------------

def forward(cfg, W, tokens, want_layers: bool = False):
    """Logits [T, vocab]; with ``want_layers`` also the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embed(W, tokens, cfg["width"])
    kept = {}
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = rms_norm(x, W[p + "norm1"], eps)
        if L["type"] == "attention":
            if "kv_from" in m and m["kv_from"] is not None:
                kv = kept[m["kv_from"]]
            else:
                kv = kept[i] = attention_keys_values(W, p + "mix.", m, h, eps)
            y = attention(W, p + "mix.", m, h, eps, kv)
        elif L["type"] == "channel_delta":
            y = channel_delta(W, p + "mix.", m, h, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            y = y + moe(W, p + "mlp.", L["mlp"], h)
        x = x + y
        if cfg.get("token_side"):
            x = x + token_side(W, p + "side.", i, cfg["token_side"]["dim"], x, tokens, eps)
        layers.append(x.copy())
    logits = linear(rms_norm(x, W["final.norm"], eps), W["head"])
    return (logits, np.stack(layers)) if want_layers else logits


def greedy(logits_row) -> int:
    return int(np.argmax(logits_row))
