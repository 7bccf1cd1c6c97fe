"""Zidivik without a GPU: its configuration class, the registry, the cache manager's kept first pages, the weight
slots against the tensors a checkpoint holds, and the plain implementation against itself (token by token, masks)."""
import json
import os

import numpy as np
import pytest

import plain_zidivik as P
import zidivik_util as Z


def test_config_round_trip_and_registry(tmp_path):
    from kestrel_llm_b200.config import ConfigError, ZidivikConfig, load_config
    for name, (raw, _) in Z.CONFIGS.items():
        d = tmp_path / name
        os.makedirs(d)
        with open(d / "config.json", "w") as f:
            json.dump(raw, f)
        cfg = load_config(str(d))                    # "architecture": a string names the class
        assert isinstance(cfg, ZidivikConfig) and cfg.num_hidden_layers == len(raw["layers"])
        assert ZidivikConfig.from_dict(cfg.to_json_dict()) == cfg
    c = ZidivikConfig.from_dict(Z.Z1)
    assert c.layers[2].mixer.kv_from == 0 and c.layers[2].mixer.window == 40 and c.layers[2].mlp is None
    assert c.layers[1].mixer.taps == 3 and c.layers[1].mlp.top == 1 and c.side_dim == 8
    assert ZidivikConfig.from_dict(Z.Z2).side_dim == 0 and ZidivikConfig.from_dict(Z.Z2).layers[1].mixer.window == 0
    for breaker in (lambda r: r["layers"][2]["mixer"].update(kv_from=1),          # not an attention layer
                    lambda r: r["layers"][2]["mixer"].update(kv_from=2),          # itself
                    lambda r: r["layers"][2]["mixer"].update(dim=8),              # other head size than the layer it reads
                    lambda r: r["layers"][0]["mlp"]["router"].update(top=9),
                    lambda r: r["layers"][0].update(type="conv"),
                    lambda r: r.pop("norm")):
        bad = json.loads(json.dumps(Z.Z1))
        breaker(bad)
        with pytest.raises(ConfigError):
            ZidivikConfig.from_dict(bad)


def test_weight_slots_are_the_checkpoints_tensors():
    import torch
    from kestrel_llm_b200.config import ZidivikConfig, resolve_architecture
    for name, (raw, seed) in Z.CONFIGS.items():
        W = Z.tensors_of(raw, seed, Z.RANKS[name])
        cfg = ZidivikConfig.from_dict(raw).with_tensor_shapes({n: a.shape for n, a in W.items()})
        model = resolve_architecture("Zidivik").build(cfg, torch.bfloat16, "meta")
        slots = {s.name: tuple(s.dest.shape) for s in model.weight_slots()}
        assert slots == {n: a.shape for n, a in W.items()}
        ranks = [(L.mixer.decay_rank, L.mixer.gate_rank) for L in cfg.layers if L.kind == "channel_delta"]
        assert ranks and all(r == Z.RANKS[name] for r in ranks)
    # a reader's wider mask widens what the writer's pages keep
    specs = resolve_architecture("Zidivik").build(
        ZidivikConfig.from_dict(Z.Z1).with_tensor_shapes({n: a.shape for n, a in Z.tensors_of(Z.Z1, 0).items()}), torch.bfloat16, "meta").cache_specs()
    assert (specs[0].window, specs[0].keep_first, specs[0].head_dim, specs[0].value_dim) == (40, 5, 16, 24)


def test_cache_manager_keeps_the_first_pages():
    from kestrel_llm_b200.cache import PageTable
    page, window, keep = 8, 20, 11
    t = PageTable([window, window, 0], [64, 64, 64], page, 4, 64)
    assert t._lib.kcache_set_keep_first(t.handle, 1, keep) == 0
    t.admit(1)
    n = 0
    for k in (3, 30, 1, 1, 2, 50, 1, 1, 1, 70):
        t.reserve(1, k)
        t.commit(1, k)
        n += k
        t.check()
        first = max(0, n - window + 1) // page                # first block a later query can reach
        plain = set(range(first, (n + page - 1) // page))
        kept = set(range((keep + page - 1) // page)) & set(range((n + page - 1) // page))
        for g, want in ((0, plain), (1, plain | kept), (2, set(range((n + page - 1) // page)))):
            tab = t.block_table(1, g)
            assert {b for b, p in enumerate(tab) if p >= 0} == want, (g, n)
    t.release(1)
    assert [t.free_pages(g) for g in range(3)] == [64, 64, 64]
    t.check()


def test_plain_masks_and_token_by_token_delta():
    m = P.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8 and m[5, 1] and m[5, 2] and not m[6, 2]
    # the convolution with zeros before the start, by its definition
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = P.causal_conv(x, w)
    for t in range(9):
        for c in range(3):
            assert abs(y[t, c] - sum(w[c, j] * (x[t - 3 + j, c] if t - 3 + j >= 0 else 0.0) for j in range(4))) < 1e-12
    # the recurrence's read-out sees the token's own write: one token, S = k u^T, o = (k . q) beta v
    cfg = {"width": 16, "vocab": 5, "norm": {"eps": 1e-6}, "layers": [dict(Z.delta(1, 1, 4, 3, 1), mlp=None)]}
    W = {n: a.astype(np.float64) for n, a in Z.tensors_of(cfg, 1, (2, 2)).items()}
    h = rng.standard_normal((1, 16))
    q = P.unit_vector(P.silu(P.linear(h, W["l0.mix.q"]) * W["l0.mix.q.conv"][:, 0])) * 0.5
    k = P.unit_vector(P.silu(P.linear(h, W["l0.mix.k"]) * W["l0.mix.k.conv"][:, 0]))
    v = P.silu(P.linear(h, W["l0.mix.v"]) * W["l0.mix.v.conv"][:, 0])
    o = float(q @ k.T) * P.sigmoid(P.linear(h, W["l0.mix.b"])) * v
    o = P.rms_norm(o, W["l0.mix.norm"], 1e-6) * P.sigmoid(P.linear(P.linear(h, W["l0.mix.g1"]), W["l0.mix.g2"]))
    assert np.allclose(P.channel_delta(W, "l0.mix.", cfg["layers"][0]["mixer"], h, 1e-6), P.linear(o, W["l0.mix.o"]), atol=1e-12)


def test_plain_routing():
    z = np.array([[0.1, 2.0, 2.0, -1.0], [3.0, 0.0, 1.0, 2.0]])
    ids, w = P.route(z, 2)
    assert ids.tolist() == [[1, 2], [0, 3]]
    assert np.allclose(w[0], [0.5, 0.5]) and np.allclose(w[1], np.exp([3.0, 2.0]) / np.exp([3.0, 2.0]).sum())
