"""The Tidavik decoder in the engine against its plain statement (`plain_tidavik`): every mechanism alone, then whole
models under every way of cutting and batching the work, then generation through the scheduler (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_tidavik as P
import replay_util as R
import tidavik_util as T

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
PART_TOL = {"float32": 3e-5, "bfloat16": 4e-2}      # of the largest entry of the plain result
KINDS = ("attention", "attention_2", "latent_attention")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tdirs(tmp_path_factory):
    return {name: T.write_model(cfg, T.tensors_of(cfg, seed), tmp_path_factory.mktemp("tidavik_" + name)) for name, (cfg, seed) in T.CONFIGS.items()}


def _close(got, want, dtype, what, scale=None):
    scale = float(np.abs(want).max()) if scale is None else scale
    err = float(np.abs(got - want).max()) / scale
    assert err <= PART_TOL[dtype], f"{what}: error {err:.3e} of the largest entry, allowed {PART_TOL[dtype]:.1e}"
    return err


def _torch_dtype(dtype):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]


def _rows(rng, n, width):
    """Input rows that both number formats hold exactly, so that the parts' inputs are the same."""
    import torch
    x = rng.standard_normal((n, width)).astype(np.float32)
    return torch.from_numpy(x).to(torch.bfloat16).to(torch.float64).numpy()


def _mixer_of(kind, m, width, dtype, eps=1e-6, seed=0):
    """A one-layer model's mixer as the model builder makes it, with weights of `tidavik_util.tensors_of`."""
    from kestrel_llm_b200.config import TidavikConfig, resolve_architecture
    cfg = {"architecture": "Tidavik", "width": width, "vocab": 11, "norm": {"eps": eps}, "layers": [{"type": kind, "mixer": m, "mlp": None}]}
    W = T.tensors_of(cfg, seed)
    model = resolve_architecture("Tidavik").build(TidavikConfig.from_dict(cfg), _torch_dtype(dtype), "cuda:0")
    return model.blocks[0].mixer, W


def _spike(W, kind, m, h, i, j):
    """Inputs and weights such that query i scores key j far above every other key and key j's value stands out: whether
    j is visible decides the output at i."""
    h *= 0.05
    h[:, 0] = 0.0
    h[i, 0] = h[j, 0] = 6.0
    p = "l0.mix."
    if kind == "latent_attention":
        rq, rk = m["q_rank"], m["kv_rank"]
        h[:, 1] = 0.0
        h[j, 0], h[j, 1] = 0.0, 6.0             # token i spikes as a query only, token j as a key and value only
        W[p + "dq"][:, 0] = 1.0                 # their latents point along (1, 1, ..., 1),
        W[p + "dkv"][:, 0] = 0.0
        W[p + "dkv"][:, 1] = 1.0
        W[p + "uq"][:] = 1.0 / np.sqrt(rq)      # so their queries, keys and values are sqrt(rank) in every channel,
        W[p + "uk"][:] = 1.0 / np.sqrt(rk)      # against N(0, 1) for any other token
        W[p + "uv"][:] = 1.0 / np.sqrt(rk)
        W[p + "g"][:, 0] = 0.5
    else:
        h[j, 1] = 6.0
        W[p + "q"][:, 0] = 1.0
        W[p + "k"][:, 0] = 1.0
        W[p + "v"][:, 1] = 1.0
        W[p + "v.b"] *= 0.05
        if kind == "attention":
            W[p + "pb"][:] = -3.0               # an ordinary key weighs little; the spiking one about 1


def _mixer_case(kind, dtype, m, page, n_tokens, cuts, spike=None, seed=0, width=48, flip_size=None):
    """One mixer alone; ``cuts`` are the portion sizes the tokens arrive in.  Returns (engine, plain) and, with
    ``flip_size``, also the plain result under that other window size."""
    rng = np.random.default_rng(seed)
    mixer, W = _mixer_of(kind, m, width, dtype, seed=seed)
    h = _rows(rng, n_tokens, width)
    if spike is not None:
        _spike(W, kind, m, h, *spike)
        h = np.asarray(h, dtype=np.float32).astype(np.float64)
        import torch
        h = torch.from_numpy(h).to(torch.bfloat16).to(torch.float64).numpy()
    names = T.load_part(mixer, W)
    assert names == {k for k in W if k.startswith("l0.mix.")}
    Wr = T.bf16_round(W)
    want = P.MIXERS[kind](Wr, "l0.mix.", m, h, 1e-6)
    hs = T.PartHarness(mixer, dtype, max_tokens=((n_tokens + 63) // 64) * 64 + 64, page_size=page)
    got, at = [], 0
    for n in cuts:
        got.append(hs.step([(7, h[at:at + n])])[0])
        at += n
    assert at == n_tokens
    if flip_size is not None:
        return np.concatenate(got), want, P.MIXERS[kind](Wr, "l0.mix.", dict(m, mask={"size": flip_size}), h, 1e-6)
    return np.concatenate(got), want, hs


def _m(kind, sizes, scale, size, cap=None):
    if kind == "latent_attention":
        H, d, dv, rq, rk = sizes
        return T.latent(H, d, dv, rq, rk, scale, size)["mixer"]
    H, G, d, dv = sizes
    return T.grouped(kind, H, G, d, dv, scale, size, cap)["mixer"]


# ---- each mechanism alone --------------------------------------------------------------------------

def test_embedding_positions_and_norm():
    import torch
    from kestrel_llm_b200.config import TidavikConfig, resolve_architecture
    cfg = dict(T.T2, layers=T.T2["layers"][:1])
    W = T.tensors_of(cfg, 1)
    model = resolve_architecture("Tidavik").build(TidavikConfig.from_dict(cfg), torch.float32, "cuda:0")
    for part in (model.embedding, model.embedding_norm):
        T.load_part(part, W)
    positions, tokens = [0, 1, 2, 77, 4095, 30000], [5, 0, 96, 40, 41, 5]

    class B:
        pass
    b = B()
    b.positions = torch.tensor(positions, dtype=torch.int32, device="cuda:0")
    b.token_ids = torch.tensor(tokens, dtype=torch.int32, device="cuda:0")
    x, pending = model.forward_embed(b)
    assert pending is None and x.dtype == torch.float32
    Wr = T.bf16_round(W)
    want = P.rms_norm(Wr["embed"][tokens] + P.sinusoid(max(positions) + 1, cfg["width"])[positions], Wr["embed.norm"], cfg["norm"]["eps"])
    # a float32 angle of size p carries an error of p * 2^-24; the norm divides by a root mean square of about 1
    assert np.abs(x.cpu().numpy() - want).max() <= 2e-5 + max(positions) * 2.4e-7


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,sizes,page", [
    ("attention", (4, 2, 16, 24), 16), ("attention", (3, 1, 40, 8), 8), ("attention", (2, 2, 64, 64), 32), ("attention", (5, 1, 12, 20), 16),
    ("attention_2", (4, 2, 16, 24), 16), ("attention_2", (3, 3, 40, 8), 8), ("attention_2", (6, 2, 14, 10), 16),
    ("latent_attention", (3, 24, 16, 40, 32), 16), ("latent_attention", (1, 16, 48, 24, 56), 8), ("latent_attention", (5, 8, 24, 16, 20), 32)])
def test_mixer_alone_whole_and_cut(dtype, kind, sizes, page):
    n, size = 90, 20
    m = _m(kind, sizes, 0.4, size, 9.0)
    whole, want, _ = _mixer_case(kind, dtype, m, page, n, [n])
    _close(whole, want, dtype, f"{kind}, whole")
    cut, want, hs = _mixer_case(kind, dtype, m, page, n, [33, 2, 17, 2, 30] + [1] * 6)
    _close(cut, want, dtype, f"{kind}, portions and single tokens")
    # pages behind the window were given back
    held = hs.cache.num_pages(0) - hs.cache.free_pages(0)
    assert held <= (size + page - 1) // page + 1
    if kind == "latent_attention":          # one vector a token is cached: the value plane is the key plane
        spec = hs.mixer.cache_spec()
        assert spec.values_are_keys and hs.cache.v[0] is hs.cache.k[0] and hs.cache.bytes_per_token() == spec.head_dim * hs.cache.k[0].element_size()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("size", [1, 2, 17])
def test_shortest_windows_and_first_tokens(kind, dtype, size):
    """A window of one key (the token itself), of two, and one that ends inside the second page; requests of one and two
    tokens; the first positions, where the window is not yet full."""
    sizes = (3, 16, 24, 40, 32) if kind == "latent_attention" else (4, 2, 16, 24)
    m = _m(kind, sizes, 0.4, size, 6.0)
    for n, cuts in ((1, [1]), (2, [2]), (2, [1, 1]), (40, [3, 2, 30] + [1] * 5)):
        got, want, _ = _mixer_case(kind, dtype, m, 16, n, cuts, seed=n)
        _close(got, want, dtype, f"{kind}, window {size}, {n} tokens as {cuts[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("where", ["window_in", "window_out", "page_border", "first_token", "far_full"])
@pytest.mark.parametrize("kind", KINDS)
def test_mixer_sees_exactly_its_keys(kind, dtype, decode, where):
    """One key stands out by its score and its value; it lies just inside or just outside the window, at a page border,
    at the request's first position, or far back under a layer without mask.  The plain result with the key's
    visibility flipped differs widely from the true one: the engine must match the true one."""
    size, page, n, i = 24, 16, 100, 97
    j = {"window_in": i - size + 1, "window_out": i - size, "page_border": 80, "first_token": 0, "far_full": 3}[where]
    if where == "first_token":
        size, flip = 98, 97
    elif where == "far_full":
        size, flip = None, 50
    else:
        flip = {"window_in": size - 1, "window_out": size + 1, "page_border": 17}[where]
    cuts = [90] + [1] * 10 if decode else [40, 60]
    sizes = (2, 16, 8, 24, 32) if kind == "latent_attention" else (2, 1, 16, 8)
    got, want, other = _mixer_case(kind, dtype, _m(kind, sizes, 0.5, size, 30.0), page, n, cuts, spike=(i, j), flip_size=flip)
    scale = float(np.abs(want).max())
    assert np.abs(want[i] - other[i]).max() > 0.25 * scale, f"{kind}, {where}: the case does not tell a visible key from a hidden one"
    _close(got, want, dtype, f"{kind}, {where}, {'decoded' if decode else 'prompt'}")
    assert np.abs(got[i] - want[i]).max() < 0.1 * np.abs(want[i] - other[i]).max()


@pytest.mark.parametrize("kind,sizes,size,page,n,cuts", [
    ("attention", (8, 2, 64, 64), 100, 16, 300, [300]), ("attention", (8, 2, 64, 64), 100, 16, 300, [129, 2, 140] + [1] * 29),
    ("attention", (4, 4, 128, 128), 64, 32, 200, [200]), ("attention", (20, 1, 16, 16), 33, 16, 90, [80] + [1] * 10),
    ("attention_2", (4, 1, 128, 64), 70, 16, 260, [250] + [1] * 10), ("attention_2", (6, 3, 24, 40), None, 8, 150, [75, 75]),
    ("attention_2", (2, 2, 256, 256), 40, 16, 100, [90] + [1] * 10), ("attention_2", (8, 2, 64, 64), 100, 16, 300, [129, 2, 140] + [1] * 29),
    ("latent_attention", (8, 64, 64, 96, 128), 100, 16, 300, [300]), ("latent_attention", (4, 32, 48, 64, 256), 70, 16, 200, [190] + [1] * 10),
    ("latent_attention", (20, 16, 16, 24, 64), 33, 8, 90, [40, 40] + [1] * 10), ("latent_attention", (3, 128, 128, 72, 40), None, 32, 150, [75, 75])])
def test_mixers_on_tensor_cores_against_the_plain_kernels(kind, sizes, size, page, n, cuts):
    """bfloat16: the tensor-core attention kernel (row tiles for portions, key splits for single tokens) with each way of
    weighing keys, and the tensor-core head-wise products, against the same mixer on the plain kernels and against the
    plain statement: more rows than a tile, windows over several key tiles, twenty heads on one key head, head size 256."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import GatedWindowAttention, LatentAttention
    m = _m(kind, sizes, 0.35, size, 15.0)
    fast, want, _ = _mixer_case(kind, "bfloat16", m, page, n, cuts, seed=sizes[2], width=64)
    _close(fast, want, "bfloat16", f"{kind} on the tensor cores")
    GatedWindowAttention.force_plain = LatentAttention.force_plain = True
    ops.head_gemm_set_plain(True)
    try:
        slow, _, _ = _mixer_case(kind, "bfloat16", m, page, n, cuts, seed=sizes[2], width=64)
    finally:
        GatedWindowAttention.force_plain = LatentAttention.force_plain = False
        ops.head_gemm_set_plain(False)
    assert np.abs(fast - slow).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("kind,sizes,size,page,n,cuts", [
    ("attention", (8, 2, 128, 128), 300, 16, 700, [300, 400]), ("attention", (2, 2, 128, 128), 64, 32, 200, [200]),
    ("attention", (4, 1, 128, 128), 100, 16, 300, [129, 2, 140] + [1] * 29), ("attention_2", (8, 2, 128, 128), 100, 16, 300, [129, 2, 140] + [1] * 29),
    ("attention_2", (2, 1, 128, 128), None, 64, 400, [400]), ("attention_2", (6, 6, 128, 128), 130, 8, 520, [260, 100, 160]),
    ("attention", (16, 1, 128, 128), 20, 16, 90, [50, 40])])
def test_portions_of_head_size_128_on_tcgen05(kind, sizes, size, page, n, cuts):
    """Prompt portions of head size 128 take the tcgen05 kernel with the layer's options applied to the scores in the
    softmax threads' registers: against the plain statement and against the same mixer kept on the mma.sync kernel; several
    key tiles, more rows than a CTA's two row tiles, windows that start inside a key tile, pages of 8 to 64."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import GatedWindowAttention
    m = _m(kind, sizes, 0.3, size, 15.0)
    calls = {"n": 0}
    real = ops.attention_tc

    def counted(*a, **kw):
        calls["n"] += 1
        return real(*a, **kw)
    ops.attention_tc = counted
    try:
        fast, want, _ = _mixer_case(kind, "bfloat16", m, page, n, cuts, seed=5, width=64)
    finally:
        ops.attention_tc = real
    ops.raise_on_kernel_error()
    assert calls["n"] == sum(1 for c in cuts if c * (sizes[0] // sizes[1]) > GatedWindowAttention.TC_MIN_ROWS)
    _close(fast, want, "bfloat16", f"{kind} on tcgen05")
    GatedWindowAttention.tcgen05 = False
    try:
        slow, _, _ = _mixer_case(kind, "bfloat16", m, page, n, cuts, seed=5, width=64)
    finally:
        GatedWindowAttention.tcgen05 = True
    assert np.abs(fast - slow).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("kind,sizes,size,n", [("attention", (4, 2, 64, 64), 300, 420), ("attention_2", (8, 2, 32, 48), None, 500),
                                               ("latent_attention", (6, 16, 16, 24, 136), 260, 400), ("attention_2", (3, 3, 128, 128), 70, 200),
                                               ("latent_attention", (20, 16, 16, 24, 64), 200, 330), ("attention", (24, 1, 32, 32), 100, 300)])
def test_single_token_steps_share_their_keys_out_over_ctas(kind, sizes, size, n):
    """bfloat16: a step of single tokens cuts its key rounds into shares, a CTA each, merged by a second kernel - against
    the plain statement and against the same steps with one CTA a request and key head; shares without keys, requests
    of several row tiles of 16 (twenty heads on one key head, a portion of two tokens) included."""
    from kestrel_llm_b200.csrc import ops
    m = _m(kind, sizes, 0.3, size, 15.0)
    cuts = [n - 12, 2] + [1] * 10
    assert ops.library().kestrel_attention_window_splits(1, 1, sizes[0], 1 if kind == "latent_attention" else sizes[1], 128, 128, size or 0, n) >= 2
    shared, want, _ = _mixer_case(kind, "bfloat16", m, 16, n, cuts, seed=9, width=64)
    _close(shared, want, "bfloat16", f"{kind}, keys over several CTAs")
    ops.attention_window_set_splits(False)
    try:
        one, _, _ = _mixer_case(kind, "bfloat16", m, 16, n, cuts, seed=9, width=64)
    finally:
        ops.attention_window_set_splits(True)
    assert np.abs(shared - one).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("sizes,size,page,cuts", [((4, 128, 128, 64, 96), 100, 16, [300, 2, 30] + [1] * 8), ((2, 128, 128, 40, 256), None, 32, [200]),
                                                  ((5, 128, 128, 72, 40), 130, 8, [65, 70, 65]), ((3, 128, 128, 56, 72), 300, 64, [700])])
def test_starting_portions_of_the_latent_mixer_expand_their_keys(sizes, size, page, cuts):
    """bfloat16, d = dv = 128: a request's first portion (if long enough) runs the tcgen05 kernel over keys and values
    expanded for the step, everything after it over the cached latents - against the plain statement and against the
    same steps with the expanded form switched off; the latents the first portion left in the cache serve the later ones."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import LatentAttention
    m = _m("latent_attention", sizes, 0.09, size)
    n = sum(cuts)
    calls = {"n": 0}
    real = ops.attention_tc

    def counted(*a, **kw):
        calls["n"] += 1
        return real(*a, **kw)
    ops.attention_tc = counted
    try:
        fast, want, _ = _mixer_case("latent_attention", "bfloat16", m, page, n, cuts, seed=7, width=64)
    finally:
        ops.attention_tc = real
    ops.raise_on_kernel_error()
    assert calls["n"] == (1 if cuts[0] > LatentAttention.EXPAND_MIN_TOKENS else 0)
    _close(fast, want, "bfloat16", "latent attention, first portion expanded")
    LatentAttention.expand_prompts = False
    try:
        slow, _, _ = _mixer_case("latent_attention", "bfloat16", m, page, n, cuts, seed=7, width=64)
    finally:
        LatentAttention.expand_prompts = True
    assert np.abs(fast - slow).max() <= 2e-2 * np.abs(want).max()


def test_requests_that_start_together_expand_their_keys_side_by_side():
    """Three requests of unequal length start in one step (each from a page border of the scratch cache), then go on in
    unequal portions and single tokens beside each other over the cached latents."""
    rng = np.random.default_rng(12)
    m = _m("latent_attention", (3, 128, 128, 48, 64), 0.09, 90)
    mixer, W = _mixer_of("latent_attention", m, 64, "bfloat16", seed=3)
    T.load_part(mixer, W)
    Wr = T.bf16_round(W)
    hs_in = [_rows(rng, n, 64) for n in (150, 97, 201)]
    want = [P.MIXERS["latent_attention"](Wr, "l0.mix.", m, h, 1e-6) for h in hs_in]
    hs = T.PartHarness(mixer, "bfloat16", max_tokens=640, page_size=16)
    got = [[], [], []]
    at = [0, 0, 0]
    for cuts in [(100, 67, 131), (30, 2, 50), (1, 1, 1), (19, 27, 19)]:
        out = hs.step([(i + 1, hs_in[i][at[i]:at[i] + c]) for i, c in enumerate(cuts)])
        for i, c in enumerate(cuts):
            got[i].append(out[i])
            at[i] += c
    assert at == [150, 97, 201]
    for i in range(3):
        _close(np.concatenate(got[i]), want[i], "bfloat16", f"latent attention, request {i} of three that started together")


@pytest.mark.parametrize("dtype,plain", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("T_,H,N,K", [(1, 3, 16, 24), (70, 4, 96, 64), (200, 2, 40, 136), (5, 1, 7, 5), (129, 20, 64, 16), (33, 2, 264, 72)])
def test_head_wise_products(dtype, plain, T_, H, N, K):
    """Both orientations of the heads' matrices, on the CUDA cores and (bfloat16, sizes in multiples of 8) on the tensor
    cores: more tokens than a tile, more columns than a tile, an inner size that is no multiple of the k-block."""
    import torch
    from kestrel_llm_b200.csrc import ops
    rng = np.random.default_rng(T_ + N)
    td = _torch_dtype(dtype)
    x = torch.from_numpy(rng.standard_normal((T_, H * K)).astype(np.float32)).to(torch.bfloat16)
    ops.head_gemm_set_plain(plain)
    try:
        for w_kn in (False, True):
            w = torch.from_numpy((rng.standard_normal((H * K, N) if w_kn else (H * N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
            got = ops.head_gemm(x.to("cuda:0").to(td), w.to("cuda:0").to(td), H, w_kn).float().cpu().numpy()
            xs, ws = x.to(torch.float64).numpy().reshape(T_, H, K), w.to(torch.float64).numpy()
            want = np.stack([xs[:, h] @ (ws[h * K:(h + 1) * K] if w_kn else ws[h * N:(h + 1) * N].T) for h in range(H)], axis=1).reshape(T_, H * N)
            _close(got, want, dtype, f"head-wise product, w_kn={w_kn}")
            # a token's result does not depend on the batch it is in: bitwise
            alone = ops.head_gemm(x[T_ // 2:T_ // 2 + 1].to("cuda:0").to(td).contiguous(), w.to("cuda:0").to(td), H, w_kn).float().cpu().numpy()
            assert np.array_equal(alone[0], got[T_ // 2])
    finally:
        ops.head_gemm_set_plain(False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_requests_beside_each_other_and_pages_used_again(dtype):
    """Each mixer alone with two requests of unequal portions in one batch against each request alone; a third request
    then runs on the pages the first two gave back."""
    for kind, sizes in (("attention", (4, 2, 16, 24)), ("attention_2", (6, 2, 8, 40)), ("latent_attention", (3, 24, 16, 40, 32))):
        rng = np.random.default_rng(3)
        m = _m(kind, sizes, 0.4, 21, 10.0)
        mixer, W = _mixer_of(kind, m, 48, dtype, seed=2)
        T.load_part(mixer, W)
        Wr = T.bf16_round(W)
        ha, hb, hc = _rows(rng, 60, 48), _rows(rng, 37, 48), _rows(rng, 64, 48)
        wa, wb, wc = (P.MIXERS[kind](Wr, "l0.mix.", m, h, 1e-6) for h in (ha, hb, hc))
        hs = T.PartHarness(mixer, dtype, max_tokens=128, page_size=16)
        got_a, got_b, at_a, at_b = [], [], 0, 0
        for ka, kb in [(7, 2), (2, 13), (30, 2), (2, 5), (3, 1), (1, 1), (15, 13)]:
            out = hs.step([(2, ha[at_a:at_a + ka]), (3, hb[at_b:at_b + kb])])
            got_a.append(out[0])
            got_b.append(out[1])
            at_a, at_b = at_a + ka, at_b + kb
        assert (at_a, at_b) == (60, 37)
        _close(np.concatenate(got_a), wa, dtype, f"{kind}, request a in portions beside b")
        _close(np.concatenate(got_b), wb, dtype, f"{kind}, request b in portions beside a")
        hs.cache.release(2)
        hs.cache.release(3)
        _close(np.concatenate([hs.step([(4, hc[:50])])[0]] + [hs.step([(4, hc[t:t + 1])])[0] for t in range(50, 64)]), wc, dtype,
               f"{kind}, a new request on pages that were given back")


# ---- whole models ----------------------------------------------------------------------------------

LENGTHS = {"T1": (1, 2, 37, 70, 129, 64), "T2": (3, 50, 97, 130, 17)}
LENGTHS_MIXED = {"T1": (5, 33, 70, 129, 47, 90, 16, 65, 31), "T2": (3, 50, 97, 130, 64, 81, 17, 49)}


def _run(tdirs, name, dtype, family, lengths=None, page_size=16, batch_max=4, graphs=False, **kw):
    cfg = T.CONFIGS[name][0]
    reqs = R.random_requests(cfg["vocab"], lengths or LENGTHS[name], seed=11 + len(name))
    steps, max_tokens = family(reqs, **kw)
    engine = R.make_engine(tdirs[name][dtype], dtype, max_tokens, page_size=page_size, batch_max=batch_max, graphs=graphs)
    got = R.run_trace(engine, steps)
    assert engine.cache.live_requests() == 0
    engine.cache.check()
    worst = T.compare_with_plain(tdirs[name]["float32"], reqs, got, dtype, f"{name}/{dtype}/{family.__name__}")
    print(f"[tidavik] {name} {dtype} {family.__name__}: worst {worst:.3e}")
    return got


def test_residual_stream_after_every_layer(tdirs):
    """float32: the stream after each layer call against the plain implementation's, so that a fault names its layer."""
    import torch
    from kestrel_llm_b200.engine import Entry
    from kestrel_llm_b200.engine.batch import StepBatch
    for name in ("T1", "T2"):
        cfg = T.CONFIGS[name][0]
        toks = R.random_requests(cfg["vocab"], (75,), seed=4)["r0"]
        pcfg, W = P.read_model(tdirs[name]["float32"])
        want = []
        P.forward(pcfg, W, toks, want)
        engine = R.make_engine(tdirs[name]["float32"], "float32", 128)
        engine.cache.admit(0)
        engine.cache.reserve(0, len(toks))
        engine.cache.clear_admitted()
        batch = StepBatch([Entry(0, toks, [])], engine.cache, "cuda:0")
        model = engine.model
        x, pending = model.forward_embed(batch)
        for i in range(len(model.order)):
            x, pending = model.forward_calls(x, pending, batch, engine.cache, i, i + 1)
            now = x.clone() if pending is None else x + pending.reduce(torch.float32)
            err = np.abs(now.cpu().numpy() - want[i]).max() / np.abs(want[i]).max()
            assert err < 2e-5, f"{name}: layer {i} ({cfg['layers'][i]['type']}): error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["T1", "T2"])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions])
def test_model_alone_whole_decoded_and_in_portions(tdirs, name, dtype, family):
    _run(tdirs, name, dtype, family)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("T1", 16), ("T2", 16), ("T1", 8), ("T2", 64)])
def test_model_mixed_batches_pages_and_slots_used_again(tdirs, name, dtype, page):
    """Up to four live requests, portions beside single tokens; nine requests through four slots and a pool that holds
    four of them, so that pages and slots are used again."""
    _run(tdirs, name, dtype, R.trace_mixed, lengths=LENGTHS_MIXED[name], page_size=page, live_max=4)


def test_model_with_heads_of_128_mixed_batches(tdirs):
    """bfloat16: portions of several requests in one step through the tcgen05 kernel beside single tokens on the mma.sync
    kernel, windows longer than a key tile, pages used again."""
    _run(tdirs, "T3", "bfloat16", R.trace_mixed, lengths=(150, 33, 400, 129, 260, 90, 16), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))
    _run(tdirs, "T3", "bfloat16", R.trace_portions, lengths=(300, 131), sizes=(70, 2, 130, 2, 50, 3, 170, 2, 31, 4))
    _run(tdirs, "T3", "float32", R.trace_mixed, lengths=(150, 33, 129, 90), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_captured_steps(tdirs, dtype):
    """Five prompt tokens, then 215 tokens one by one through captured decode steps: every window passes over decoded
    tokens, pages behind the windows come back to the pool."""
    _run(tdirs, "T1", dtype, R.trace_tail_decode, lengths=(220,), graphs=True, tail=215)


@pytest.mark.parametrize("name", ["T1", "T2"])
def test_cuttings_agree_in_float32(tdirs, name):
    """The float32 logits of a position do not depend on how the work was cut or batched: every sum's order is fixed per
    output element."""
    a = _run(tdirs, name, "float32", R.trace_whole, lengths=LENGTHS_MIXED[name])
    b = _run(tdirs, name, "float32", R.trace_mixed, lengths=LENGTHS_MIXED[name], live_max=4)
    c = _run(tdirs, name, "float32", R.trace_portions, lengths=LENGTHS_MIXED[name])
    for r in a:
        for p in a[r]:
            assert np.array_equal(a[r][p], b[r][p]) and np.array_equal(a[r][p], c[r][p]), f"{name}: request {r} position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(tdirs, dtype):
    """`LLM.generate`: six requests through three slots, prompts in portions of at most 24 tokens."""
    from kestrel_llm_b200 import LLM, SamplingParams
    name = "T1"
    cfg = T.CONFIGS[name][0]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (1, 40, 70, 9, 33, 55)]
    llm = LLM(tdirs[name][dtype], dtype=dtype, page_size=16, batch_max=3, max_tokens=512, prefill_batch=24, max_step_tokens=64)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    pcfg, W = P.read_model(tdirs[name]["float32"])
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        assert len(o.token_ids) == 8
        for got in o.token_ids:
            logits = P.forward(pcfg, W, toks)[-1]
            want = int(np.argmax(logits))
            if got != want:          # a tie within rounding is not a fault; anything else is
                gap = float(logits[want] - logits[got])
                assert gap <= (2e-5 if dtype == "float32" else 4e-2) * float(np.abs(logits).max()), f"{dtype}: token {got} instead of {want}"
            toks.append(got)


# ---- the programs a user runs ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,graphs", [("float32", 1), ("bfloat16", 1), ("bfloat16", 0)])
def test_trace_replay_program(tdirs, dtype, graphs, tmp_path):
    """bin/trace_run in a process of its own on a mixed trace: four slots for seven requests, decode steps replayed from
    captured graphs (the default) and launched kernel by kernel."""
    name = "T2"
    reqs = R.random_requests(T.CONFIGS[name][0]["vocab"], (5, 33, 70, 47, 90, 16, 65), seed=21)
    steps, max_tokens = R.trace_mixed(reqs, live_max=4, seed=5)
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tdirs[name][dtype], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_tokens), "--cuda-graphs", str(graphs)], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = T.CONFIGS[name][0]["vocab"]
    pos = {n: 0 for n in reqs}
    got = {n: {} for n in reqs}
    for i, s in enumerate(steps):
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[e["id"]][pos[e["id"]] + w] = arr[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        assert r == arr.shape[0]
    T.compare_with_plain(tdirs[name]["float32"], reqs, got, dtype, f"trace_run/{dtype}")


def test_command_line_writes_random_weights_and_generates(tmp_path):
    """bin/kestrel: `--random-weights` writes a Tidavik folder from a config.json with the design's own keys, and the
    streaming harness prints the plain implementation's greedy tokens."""
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(T.T1))
    model_dir = tmp_path / "written"
    prompt = R.random_requests(T.T1["vocab"], (23,), seed=2)["r0"]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kestrel"), "--model", str(model_dir), "--config", str(cfg_file),
                        "--random-weights", "5", "--dtype", "float32", "--stream-test", "--stream-n", "8", "--prompt-ids",
                        ",".join(str(t) for t in prompt), "--ignore-eos", "--max-tokens", "256", "--batch-max", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    pcfg, W = P.read_model(str(model_dir))
    assert (W["l1.mix.r2"] >= 0).all() and "l1.norm2" not in W and "l0.norm2" in W
    toks, want = list(prompt), []
    for _ in range(8):
        want.append(int(np.argmax(P.forward(pcfg, W, toks)[-1])))
        toks.append(want[-1])
    assert [int(t) for t in line[0].split(":")[1].split()] == want
