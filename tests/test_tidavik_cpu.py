"""Tidavik without a GPU: its configuration class, the registry, the weight slots against the tensors a checkpoint
holds, what its layers ask of the cache, and the plain implementation against itself (masks, the extra term of the
softmax, the latent form of attention, prefixes)."""
import json
import os

import numpy as np
import pytest

import plain_tidavik as P
import tidavik_util as T


def test_config_round_trip_and_registry(tmp_path):
    from kestrel_llm_b200.config import ConfigError, TidavikConfig, load_config
    for name, (raw, _) in T.CONFIGS.items():
        d = tmp_path / name
        os.makedirs(d)
        with open(d / "config.json", "w") as f:
            json.dump(raw, f)
        cfg = load_config(str(d))                    # "architecture": a string names the class
        assert isinstance(cfg, TidavikConfig) and cfg.num_hidden_layers == len(raw["layers"])
        assert TidavikConfig.from_dict(cfg.to_json_dict()) == cfg
    c = TidavikConfig.from_dict(T.T1)
    assert (c.layers[0].mixer.q_rank, c.layers[0].mixer.kv_rank, c.layers[0].mixer.window, c.layers[0].mlp.ff) == (40, 32, 19, 96)
    assert c.layers[1].mlp is None and c.layers[1].mixer.softcap == 30.0 and c.layers[2].mixer.kv_heads == 2
    c2 = TidavikConfig.from_dict(T.T2)
    assert c2.layers[0].mixer.window == 0 and c2.layers[0].mixer.softcap == 0.0 and c2.layers[4].mixer.window == 0
    for breaker in (lambda r: r["layers"][1]["mixer"].update(kv_heads=3),         # 4 heads on 3 kv heads
                    lambda r: r["layers"][0]["mixer"].pop("kv_rank"),
                    lambda r: r["layers"][2]["mixer"].update(softcap=-1.0),
                    lambda r: r["layers"][0]["mlp"].update(kind="moe"),
                    lambda r: r["layers"][0].update(type="attention_3"),
                    lambda r: r["layers"][3]["mixer"].update(mask={"size": 0}),
                    lambda r: r.pop("norm")):
        bad = json.loads(json.dumps(T.T1))
        breaker(bad)
        with pytest.raises(ConfigError):
            TidavikConfig.from_dict(bad)


def test_weight_slots_are_the_checkpoints_tensors():
    import torch
    from kestrel_llm_b200.config import TidavikConfig, resolve_architecture
    from kestrel_llm_b200.parts import PagedKVSpec
    for name, (raw, seed) in T.CONFIGS.items():
        W = T.tensors_of(raw, seed)
        model = resolve_architecture("Tidavik").build(TidavikConfig.from_dict(raw), torch.bfloat16, "meta")
        slots = {s.name: tuple(s.dest.shape) for s in model.weight_slots()}
        assert slots == {n: a.shape for n, a in W.items()}
        assert model.graph_safe and model.step_program(None) is None     # decode steps are captured; other steps walk the parts
        for L, spec in zip(raw["layers"], model.cache_specs()):
            m = L["mixer"]
            window = (m.get("mask") or {}).get("size") or 0
            if L["type"] == "latent_attention":      # one vector of kv_rank numbers a token, whatever the number of heads
                assert spec == PagedKVSpec(1, m["kv_rank"], window, 0, m["kv_rank"], values_are_keys=True)
            else:
                assert spec == PagedKVSpec(m["kv_heads"], m["dim"], window, 0, m["vdim"])


def test_cache_of_a_layer_whose_values_are_its_keys():
    import torch
    from kestrel_llm_b200.cache import CacheManager
    from kestrel_llm_b200.parts import PagedKVSpec
    cm = CacheManager([PagedKVSpec(1, 24, 16, 0, 24, values_are_keys=True), PagedKVSpec(2, 8, 16, 0, 12)], torch.float32, "cpu", 8, 6, 2, 256)
    assert cm.v[0] is cm.k[0] and cm.v[1] is not cm.k[1] and tuple(cm.v[1].shape) == (7, 2, 8, 12)
    assert cm.bytes_per_token() == 4 * (24 + 2 * (8 + 12))
    assert cm.layer_group == [0, 0]                   # one window, one block table
    with pytest.raises(Exception):
        CacheManager([PagedKVSpec(1, 24, 0, 0, 16, values_are_keys=True)], torch.float32, "cpu", 8, 6, 2, 256)


def test_plain_mask_and_prefixes():
    m = P.window_mask(9, 3)
    assert m[8].tolist() == [False] * 6 + [True] * 3 and m[1].tolist() == [True, True] + [False] * 7
    assert P.window_mask(5, None).tolist() == np.tril(np.ones((5, 5), bool)).tolist()
    # a position's logits depend on the tokens before it only
    for name, (cfg, seed) in T.CONFIGS.items():
        W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, seed).items()}
        toks = np.random.default_rng(1).integers(0, cfg["vocab"], 45).tolist()
        whole = P.forward(cfg, W, toks)
        for k in (1, 2, 20, 44):
            assert np.allclose(P.forward(cfg, W, toks[:k])[-1], whole[k - 1], atol=1e-9)


def test_plain_mixers_by_their_definitions():
    rng = np.random.default_rng(0)
    # the extra term: one token, one head -> weight exp(s) / (1 + exp(s)) on its own value of unit root mean square
    m = T.sink_attn(1, 1, 4, 6, 0.7, size=5, softcap=3.0)["mixer"]
    cfg = {"width": 10, "vocab": 5, "norm": {"eps": 1e-6}, "layers": [{"type": "attention_2", "mixer": m, "mlp": None}]}
    W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, 1).items()}
    h = rng.standard_normal((1, 10))
    p = "l0.mix."
    q, k, v = (P.linear(h, W[p + n], W[p + n + ".b"]) for n in "qkv")
    s = 3.0 * np.tanh((q @ k.T).item() * 0.7 / 3.0)
    o = np.exp(s) / (1.0 + np.exp(s)) * v / np.sqrt(np.mean(v * v) + 1e-6)
    assert np.allclose(P.sink_attention(W, p, m, h, 1e-6), P.linear(o, W[p + "o"], W[p + "o.b"]), atol=1e-12)
    # sigmoid weights: two tokens, the second sees both; nothing is normalised, the distance term applies to the first key only
    m = T.sigmoid_attn(1, 1, 4, 3, 0.5, size=2, softcap=2.0)["mixer"]
    cfg = {"width": 10, "vocab": 5, "norm": {"eps": 1e-6}, "layers": [{"type": "attention", "mixer": m, "mlp": None}]}
    W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, 2).items()}
    h = rng.standard_normal((2, 10))
    q = P.rms_norm(P.linear(h, W[p + "q"], W[p + "q.b"]), W[p + "q.norm"], 1e-6)
    k = P.rms_norm(P.linear(h, W[p + "k"], W[p + "k.b"]), W[p + "k.norm"], 1e-6)
    v = P.linear(h, W[p + "v"], W[p + "v.b"])
    s0 = 2.0 * np.tanh(float(q[1] @ k[0]) * 0.5 / 2.0) - W[p + "r1"][0] * np.log(1.0 + W[p + "r2"][0])
    s1 = 2.0 * np.tanh(float(q[1] @ k[1]) * 0.5 / 2.0)
    o = P.sigmoid(s0 + W[p + "pb"][0]) * v[0] + P.sigmoid(s1 + W[p + "pb"][0]) * v[1]
    assert np.allclose(P.sigmoid_attention(W, p, m, h, 1e-6)[1], P.linear(o[None], W[p + "o"], W[p + "o.b"])[0], atol=1e-12)
    # a third token no longer sees the first (size 2)
    h3 = np.concatenate([h, rng.standard_normal((1, 10))])
    h3b = h3.copy()
    h3b[0] += 1.0
    assert np.allclose(P.sigmoid_attention(W, p, m, h3, 1e-6)[2], P.sigmoid_attention(W, p, m, h3b, 1e-6)[2], atol=1e-12)
    # the latent form: scores and mixtures taken over the cached latents themselves give the same output
    m = T.latent(3, 6, 5, 7, 9, 0.4, size=4)["mixer"]
    cfg = {"width": 10, "vocab": 5, "norm": {"eps": 1e-6}, "layers": [{"type": "latent_attention", "mixer": m, "mlp": None}]}
    W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, 3).items()}
    h = rng.standard_normal((8, 10))
    cq = P.rms_norm(P.linear(h, W[p + "dq"]), W[p + "dq.norm"], 1e-6)
    c = P.rms_norm(P.linear(h, W[p + "dkv"]), W[p + "dkv.norm"], 1e-6)
    qh = P.linear(cq, W[p + "uq"]).reshape(8, 3, 6)
    vis = P.window_mask(8, 4)
    out = np.zeros((8, 3, 5))
    for n in range(3):
        ql = qh[:, n] @ W[p + "uk"][n * 6:(n + 1) * 6]                       # queries in the latent space
        s = np.where(vis, ql @ c.T * 0.4, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, n] = ((e / e.sum(axis=1, keepdims=True)) @ c) @ W[p + "uv"][n * 5:(n + 1) * 5].T * P.sigmoid(P.linear(h, W[p + "g"]))[:, n:n + 1]
    assert np.allclose(P.latent_attention(W, p, m, h, 1e-6), P.linear(out.reshape(8, 15), W[p + "o"]), atol=1e-10)
