"""The Zidivik decoder in the engine against its plain statement (`plain_zidivik`): every mechanism alone, then whole
models under every way of cutting and batching the work, then generation through the scheduler (GPU)."""
import numpy as np
import pytest

import plain_zidivik as P
import replay_util as R
import zidivik_util as Z

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
PART_TOL = {"float32": 3e-5, "bfloat16": 4e-2}      # of the largest entry of the plain result


@pytest.fixture(scope="module")
def zdirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in Z.CONFIGS.items():
        out[name] = Z.write_model(cfg, Z.tensors_of(cfg, seed, Z.RANKS[name]), tmp_path_factory.mktemp("zidivik_" + name))
    return out


def _close(got, want, dtype, what):
    scale = float(np.abs(want).max())
    err = float(np.abs(got - want).max()) / scale
    assert err <= PART_TOL[dtype], f"{what}: error {err:.3e} of the largest entry, allowed {PART_TOL[dtype]:.1e}"
    return err


def _torch_dtype(dtype):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]


def _rows(rng, n, width, dtype):
    """Input rows that both number formats hold exactly, so that the parts' inputs are the same."""
    import torch
    x = rng.standard_normal((n, width)).astype(np.float32)
    return torch.from_numpy(x).to(torch.bfloat16).to(torch.float64).numpy()


# ---- each mechanism alone --------------------------------------------------------------------------

@pytest.mark.parametrize("width,positions", [(64, [0, 1, 2, 77, 4095, 50000]), (37, [3, 1000])])
def test_sinusoidal_positions(width, positions):
    import torch
    from kestrel_llm_b200.parts import SinusoidalPositions

    class B:
        pass
    b = B()
    b.positions = torch.tensor(positions, dtype=torch.int32, device="cuda:0")
    x = torch.zeros((len(positions), width), dtype=torch.float32, device="cuda:0")
    SinusoidalPositions(width, "cuda:0").add_to_embedding(x, b)
    want = P.sinusoid(positions, width)
    # a float32 angle of size p carries an error of p * 2^-24
    assert np.abs(x.cpu().numpy() - want).max() <= 2e-6 + max(positions) * 1.2e-7


def _attention_case(dtype, H, G, d, dv, scale, size, keep, page, n_tokens, cuts, spike=None, seed=0):
    """One attention mixer alone; ``cuts`` are the portion sizes the tokens arrive in.  ``spike`` = (i, j): the inputs are
    made so that query i scores key j far above every other key, and value j is large: whether j is visible decides
    the output at i."""
    import torch
    from kestrel_llm_b200.parts import GatedWindowAttention
    rng = np.random.default_rng(seed)
    width = 48
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale, "mask": {"size": size, "keep_first": keep}}
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-6}, "layers": [{"type": "attention", "mixer": m, "mlp": None}]}
    W = Z.tensors_of(cfg, seed)
    h = _rows(rng, n_tokens, width, dtype)
    if spike is not None:
        i, j = spike
        h *= 0.05
        h[:, 0] = 0.0
        h[i, 0] = h[j, 0] = 6.0
        h[j, 1] = 6.0
        W["l0.mix.q"][:, 0] = 1.0            # every query and key head reads entry 0 into all its channels: q . k = d when both spike,
        W["l0.mix.k"][:, 0] = 1.0            # against about sqrt(d) between any other pair
        W["l0.mix.v"][:, 1] = 1.0
        W["l0.mix.g"][:, 0] = 0.5            # the spiking query's gates are open
    mixer = GatedWindowAttention(width, H, G, d, dv, _torch_dtype(dtype), "cuda:0", "l0.mix.", scale, 1e-6, window=size or 0, keep_first=keep)
    Z.load_part(mixer, W)
    Wr = Z.bf16_round(W)
    want = P.attention(Wr, "l0.mix.", dict(m, mask={"size": size or 1 << 30, "keep_first": keep}), h, 1e-6,
                       P.attention_keys_values(Wr, "l0.mix.", m, h, 1e-6))
    hs = Z.PartHarness(mixer, dtype, max_tokens=((n_tokens + 63) // 64) * 64 + 64, page_size=page)
    got, at = [], 0
    for n in cuts:
        got.append(hs.step([(7, h[at:at + n])])[0])
        at += n
    assert at == n_tokens
    return np.concatenate(got), want, hs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,page", [(4, 2, 16, 24, 16), (3, 1, 40, 8, 8), (2, 2, 64, 64, 32)])
def test_attention_alone_whole_and_cut(dtype, H, G, d, dv, page):
    n = 90
    whole, want, _ = _attention_case(dtype, H, G, d, dv, 0.4, 20, 6, page, n, [n])
    _close(whole, want, dtype, "attention, whole")
    cut, want, hs = _attention_case(dtype, H, G, d, dv, 0.4, 20, 6, page, n, [33, 2, 17, 2, 30] + [1] * 6)
    _close(cut, want, dtype, "attention, portions and single tokens")
    # pages behind the window were given back, those of the kept first tokens were not
    held = hs.cache.num_pages(0) - hs.cache.free_pages(0)
    assert held <= (6 + page - 1) // page + (20 + page - 1) // page + 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("where", ["window_in", "window_out", "kept_in", "kept_out", "page_border", "first_token", "far_full"])
def test_attention_sees_exactly_its_keys(dtype, decode, where):
    """One key stands out by its score and carries a large value; it lies just inside or just outside the window, among
    the kept first tokens or right after them, at a page border, or far back under a mask-free layer."""
    size, keep, page, n = 24, 5, 16, 100
    i = 97
    j = {"window_in": i - size + 1, "window_out": i - size, "kept_in": keep - 1, "kept_out": keep, "page_border": 80, "first_token": 0,
         "far_full": 3}[where]
    if where == "far_full":
        size = None
    cuts = [90] + [1] * 10 if decode else [40, 60]
    got, want, _ = _attention_case(dtype, 2, 1, 16, 8, 1.0, size, keep if size else 0, page, n, cuts, spike=(i, j))
    # the plain result itself must tell the two cases apart, or the case shows nothing
    seen = np.abs(want[i]).max()
    visible = where not in ("window_out", "kept_out")
    assert (seen > 1.0) == visible, f"{where}: the case is not built as meant ({seen})"
    _close(got, want, dtype, f"attention, {where}, {'decoded' if decode else 'prompt'}")


@pytest.mark.parametrize("H,G,d,dv,size,keep,page,n,cuts", [
    (8, 2, 64, 64, 100, 7, 16, 300, [300]), (8, 2, 64, 64, 100, 7, 16, 300, [129, 2, 140] + [1] * 29), (4, 4, 128, 128, 64, 0, 32, 200, [200]),
    (4, 1, 128, 64, 70, 130, 16, 260, [250] + [1] * 10), (6, 3, 24, 40, None, 0, 8, 150, [75, 75]), (20, 1, 16, 16, 33, 3, 16, 90, [80] + [1] * 10),
    (2, 2, 256, 256, 40, 2, 16, 100, [90] + [1] * 10)])
def test_attention_on_tensor_cores_against_the_plain_kernel(H, G, d, dv, size, keep, page, n, cuts):
    """bfloat16: the tensor-core kernel (row tiles for portions, key splits for single tokens) and the plain kernel, both
    against the plain statement; more rows than a tile, windows over several key tiles, kept tokens beyond the window,
    twenty heads on one kv head, head size 256."""
    from kestrel_llm_b200.parts import GatedWindowAttention
    fast, want, _ = _attention_case("bfloat16", H, G, d, dv, 0.35, size, keep, page, n, cuts, seed=d)
    _close(fast, want, "bfloat16", "tensor-core attention")
    GatedWindowAttention.force_plain = True
    try:
        slow, _, _ = _attention_case("bfloat16", H, G, d, dv, 0.35, size, keep, page, n, cuts, seed=d)
    finally:
        GatedWindowAttention.force_plain = False
    assert np.abs(fast - slow).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_over_another_layers_pages(dtype):
    """A mixer without key and value projections attends over the pages another wrote, with its own mask and scale."""
    import torch
    from kestrel_llm_b200.parts import GatedWindowAttention
    rng = np.random.default_rng(5)
    width, n = 48, 70
    m0 = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 12, "keep_first": 2}}
    m1 = dict(m0, scale=0.6, mask={"size": 30, "keep_first": 7}, kv_from=0)
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-6}, "layers": [{"type": "attention", "mixer": m0, "mlp": None},
                                                                         {"type": "attention", "mixer": m1, "mlp": None}]}
    W = Z.tensors_of(cfg, 2)
    td = _torch_dtype(dtype)
    a = GatedWindowAttention(width, 4, 2, 16, 24, td, "cuda:0", "l0.mix.", 0.3, 1e-6, window=12, keep_first=2, cache_window=30, cache_keep_first=7)
    b = GatedWindowAttention(width, 4, 2, 16, 24, td, "cuda:0", "l1.mix.", 0.6, 1e-6, window=30, keep_first=7, own_kv=False)
    Z.load_part(a, W)
    Z.load_part(b, W)
    Wr = Z.bf16_round(W)
    h0, h1 = _rows(rng, n, width, dtype), _rows(rng, n, width, dtype)
    kv = P.attention_keys_values(Wr, "l0.mix.", m0, h0, 1e-6)
    want0, want1 = P.attention(Wr, "l0.mix.", m0, h0, 1e-6, kv), P.attention(Wr, "l1.mix.", m1, h1, 1e-6, kv)
    hs = Z.PartHarness(a, dtype, max_tokens=128)
    got0, got1, at = [], [], 0
    for k in [31, 2, 30] + [1] * 7:
        got0.append(hs.step([(1, h0[at:at + k])], commit=False)[0])
        got1.append(hs.step([(1, h1[at:at + k])], writable=False, mixer=b)[0])
        hs.commit()
        at += k
    _close(np.concatenate(got0), want0, dtype, "the layer that writes the pages")
    _close(np.concatenate(got1), want1, dtype, "the layer that reads them")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,taps", [(4, 2, 16, 8, 3), (2, 2, 40, 48, 4), (3, 1, 24, 20, 1), (2, 1, 136, 32, 6)])
def test_delta_rule_alone(dtype, H, G, d, dv, taps):
    """Whole, token by token, and in portions down to two tokens; two requests beside each other against each alone;
    a state slot that a finished request leaves is used again by a new one."""
    from kestrel_llm_b200.parts import ChannelDeltaMixer
    rng = np.random.default_rng(d)
    width, n = 56, 60
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-5}, "layers": [{"type": "channel_delta", "mixer": m, "mlp": None}]}
    W = Z.tensors_of(cfg, 4, (10, 6))
    mixer = ChannelDeltaMixer(width, H, G, d, dv, taps, 10, 6, 1e-5, _torch_dtype(dtype), "cuda:0", "l0.mix.")
    assert Z.load_part(mixer, W) == {k for k in W if k.startswith("l0.mix.")}
    Wr = Z.bf16_round(W)
    ha, hb = _rows(rng, n, width, dtype), _rows(rng, 37, width, dtype)
    wa, wb = P.channel_delta(Wr, "l0.mix.", m, ha, 1e-5), P.channel_delta(Wr, "l0.mix.", m, hb, 1e-5)
    hs = Z.PartHarness(mixer, dtype, slots=2)
    _close(hs.step([(1, ha)])[0], wa, dtype, "delta rule, whole")
    hs.cache.release(1)
    # request 2 takes the slot request 1 left, beside request 3; portions of unequal sizes, then single tokens
    got_a, got_b, at_a, at_b = [], [], 0, 0
    for ka, kb in [(7, 2), (2, 13), (30, 2), (2, 5), (3, 1), (1, 1), (15, 13)]:
        out = hs.step([(2, ha[at_a:at_a + ka]), (3, hb[at_b:at_b + kb])])
        got_a.append(out[0])
        got_b.append(out[1])
        at_a, at_b = at_a + ka, at_b + kb
    assert (at_a, at_b) == (n, 37)
    _close(np.concatenate(got_a), wa, dtype, "delta rule, request a in portions beside b")
    _close(np.concatenate(got_b), wb, dtype, "delta rule, request b in portions beside a")


def test_delta_rule_long_decoding():
    """300 tokens one by one: the state and the convolutions' tail carried through every step."""
    from kestrel_llm_b200.parts import ChannelDeltaMixer
    rng = np.random.default_rng(9)
    width, n = 40, 300
    m = {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "conv": 4}
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-6}, "layers": [{"type": "channel_delta", "mixer": m, "mlp": None}]}
    W = Z.tensors_of(cfg, 6, (5, 5))
    mixer = ChannelDeltaMixer(width, 2, 1, 24, 16, 4, 5, 5, 1e-6, _torch_dtype("float32"), "cuda:0", "l0.mix.")
    Z.load_part(mixer, W)
    h = _rows(rng, n, width, "float32")
    want = P.channel_delta(Z.bf16_round(W), "l0.mix.", m, h, 1e-6)
    hs = Z.PartHarness(mixer, "float32")
    got = np.concatenate([hs.step([(1, h[t:t + 1])])[0] for t in range(n)])
    _close(got, want, "float32", "delta rule, 300 single tokens")
    _close(got[-20:], want[-20:], "float32", "delta rule, the last tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,limit,n", [(6, 2, 40, 1.0, 75), (3, 1, 24, 2.5, 9), (5, 5, 16, 0.75, 33), (40, 4, 72, 1.75, 300), (2, 1, 8, 100.0, 1)])
def test_routed_experts_alone(dtype, E, top, ff, limit, n):
    import torch
    from kestrel_llm_b200.parts import RoutedExperts
    rng = np.random.default_rng(E)
    width = 64
    f = Z.moe(E, top, ff, limit)
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-5}, "layers": [dict(Z.attn(1, 1, 8, 8, 1.0), mlp=f)]}
    W = Z.tensors_of(cfg, 1)
    part = RoutedExperts(width, ff, E, top, limit, _torch_dtype(dtype), "cuda:0", "l0.mlp.")
    Z.load_part(part, W)
    Wr = Z.bf16_round(W)
    h = _rows(rng, n, width, dtype)
    want = P.moe(Wr, "l0.mlp.", f, h)
    x = torch.from_numpy(h.astype(np.float32)).to("cuda:0").to(_torch_dtype(dtype))
    got = part.forward(x, None).reduce(torch.float32).cpu().numpy()
    # tokens whose router all but ties may go either way in reduced precision; the clamp is met by some token or the case is idle
    z = np.sort(P.linear(h, Wr["l0.mlp.router"]) + Wr["l0.mlp.router.b"], axis=1)[:, ::-1]
    sure = np.ones(n, bool) if top == E or dtype == "float32" else (z[:, top - 1] - z[:, top] > 0.01)
    assert n < 20 or sure.sum() >= 0.8 * n
    _close(got[sure], want[sure], dtype, "routed experts")
    # a token's result does not depend on the batch it is in: bitwise
    alone = part.forward(x[n // 2:n // 2 + 1].contiguous(), None).reduce(torch.float32).cpu().numpy()
    if dtype == "float32":
        assert np.array_equal(alone[0], got[n // 2])


@pytest.mark.parametrize("tcgen05", [True, False])
@pytest.mark.parametrize("E,top,ff,width,n", [(8, 2, 96, 64, 200), (5, 3, 72, 136, 77), (16, 4, 200, 256, 1000), (3, 1, 8, 8, 3), (6, 2, 136, 200, 700),
                                              (40, 8, 64, 72, 333)])
def test_grouped_products_on_tensor_cores_against_cuda_cores(E, top, ff, width, n, tcgen05):
    """The bfloat16 expert products on the tensor cores against the same products on the CUDA cores: feature counts
    that do not fill a tile, a K that is no multiple of the k-block, experts without a token, more rows than a tile."""
    import torch
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import RoutedExperts
    rng = np.random.default_rng(E + n)
    cfg = {"width": width, "vocab": 11, "norm": {"eps": 1e-5}, "layers": [dict(Z.attn(1, 1, 8, 8, 1.0), mlp=Z.moe(E, top, ff, 1.25))]}
    part = RoutedExperts(width, ff, E, top, 1.25, torch.bfloat16, "cuda:0", "l0.mlp.")
    Z.load_part(part, Z.tensors_of(cfg, 1))
    x = torch.from_numpy(rng.standard_normal((n, width)).astype(np.float32)).to("cuda:0").to(torch.bfloat16)
    ops.moe_set_tcgen05(tcgen05)         # many pairs: tcgen05 tiles of 128 rows; off, and for few pairs: mma.sync tiles of 64
    try:
        fast = part.forward(x, None).reduce(torch.float32).cpu().numpy()
        alone = part.forward(x[n // 2:n // 2 + 1].contiguous(), None).reduce(torch.float32).cpu().numpy()
        ops.moe_set_plain(True)
        ops.moe_set_tcgen05(False)
        slow = part.forward(x, None).reduce(torch.float32).cpu().numpy()
    finally:
        ops.moe_set_plain(False)
        ops.moe_set_tcgen05(True)
    ops.raise_on_kernel_error()
    # same products, sums in another order, one rounding of the activation to bfloat16 in between
    assert np.abs(fast - slow).max() <= 1.5e-2 * np.abs(slow).max()
    assert np.abs(fast - slow).mean() <= 1e-3 * np.abs(slow).max()
    if not tcgen05 or n * top < ops.MOE_TC_MIN_PAIRS:
        assert np.array_equal(alone[0], fast[n // 2])       # the same kernel: a token's result does not depend on its batch
    else:                                                   # the two tensor-core kernels differ in the order of their sums only
        assert np.abs(alone[0] - fast[n // 2]).max() <= 2e-2 * np.abs(slow).max()


def test_router_choice_and_weights():
    import torch
    from kestrel_llm_b200.csrc import ops
    rng = np.random.default_rng(0)
    z = rng.standard_normal((50, 13)).astype(np.float32) * 3
    z[7, 3] = z[7, 9] = z[7].max() + 1           # equal logits: the lower index goes first
    b = rng.standard_normal(13).astype(np.float32)
    b[9] = b[3]
    ids, w = ops.moe_route(ops.Partials(torch.from_numpy(z).to("cuda:0")), torch.from_numpy(b).to("cuda:0"), 4)
    want_ids, want_w = P.route(z.astype(np.float64) + b, 4)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(w.cpu().numpy() - want_w).max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_side_input_alone(dtype):
    import torch
    from kestrel_llm_b200.parts import TokenSideInput, TokenTable
    rng = np.random.default_rng(2)
    width, dim, vocab, layers, n = 72, 8, 31, 3, 40
    cfg = {"width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "token_side": {"dim": dim},
           "layers": [dict(Z.attn(1, 1, 8, 8, 1.0), mlp=None)] * layers}
    W = Z.tensors_of(cfg, 3)
    td = _torch_dtype(dtype)
    table = TokenTable(vocab, layers * dim, td, "cuda:0", "side.embed")
    part = TokenSideInput(width, dim, table, 2 * dim, 1e-5, td, "cuda:0", "l2.side.")
    Z.load_part(table, W)
    Z.load_part(part, W)
    x = _rows(rng, n, width, dtype)
    toks = rng.integers(0, vocab, n)
    want = P.token_side(Z.bf16_round(W), "l2.side.", 2, dim, x, toks, 1e-5)

    class B:
        pass
    b = B()
    b.token_ids = torch.from_numpy(toks.astype(np.int32)).to("cuda:0")
    res = torch.zeros((n, width), dtype=torch.float32, device="cuda:0")
    part.add_forward(res, torch.from_numpy(x.astype(np.float32)).to("cuda:0").to(td), b)
    _close(res.cpu().numpy(), want, dtype, "token side input")


# ---- whole models ----------------------------------------------------------------------------------

LENGTHS = {"Z1": (1, 2, 37, 70, 129, 64), "Z2": (3, 50, 97, 130, 17)}
LENGTHS_MIXED = {"Z1": (5, 33, 70, 129, 47, 90, 16, 65, 31), "Z2": (3, 50, 97, 130, 64, 81, 17, 49)}


def _run(zdirs, name, dtype, family, lengths=None, page_size=16, batch_max=4, **kw):
    cfg = Z.CONFIGS[name][0]
    reqs = R.random_requests(cfg["vocab"], lengths or LENGTHS[name], seed=11 + len(name))
    steps, max_tokens = family(reqs, **kw)
    engine = R.make_engine(zdirs[name][dtype], dtype, max_tokens, page_size=page_size, batch_max=batch_max)
    got = R.run_trace(engine, steps)
    assert engine.cache.live_requests() == 0
    engine.cache.check()
    worst = Z.compare_with_plain(zdirs[name]["float32"], reqs, got, dtype, f"{name}/{dtype}/{family.__name__}")
    print(f"[zidivik] {name} {dtype} {family.__name__}: worst {worst:.3e}")
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Z1", "Z2"])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions])
def test_model_alone_whole_decoded_and_in_portions(zdirs, name, dtype, family):
    _run(zdirs, name, dtype, family)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("Z1", 16), ("Z2", 16), ("Z1", 8), ("Z2", 64)])
def test_model_mixed_batches_pages_and_slots_used_again(zdirs, name, dtype, page):
    """Up to four live requests, portions beside single tokens; nine requests through four state slots and a pool that
    holds four of them, so that pages and slots are used again."""
    _run(zdirs, name, dtype, R.trace_mixed, lengths=LENGTHS_MIXED[name], page_size=page, live_max=4)


@pytest.mark.parametrize("name", ["Z1", "Z2"])
def test_cuttings_agree_in_float32(zdirs, name):
    """The float32 logits of a position do not depend on how the work was cut or batched, beyond rounding of sums whose
    order a cut changes (the split of a product over K): far below the tolerance against the plain implementation."""
    a = _run(zdirs, name, "float32", R.trace_whole, lengths=LENGTHS_MIXED[name])
    b = _run(zdirs, name, "float32", R.trace_mixed, lengths=LENGTHS_MIXED[name], live_max=4)
    for r in a:
        for p in a[r]:
            assert np.abs(a[r][p] - b[r][p]).max() <= 2e-5 * np.abs(a[r][p]).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(zdirs, dtype):
    """`LLM.generate`: six requests through three state slots, prompts in portions of at most 24 tokens."""
    from kestrel_llm_b200 import LLM, SamplingParams
    name = "Z1"
    cfg = Z.CONFIGS[name][0]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (1, 40, 70, 9, 33, 55)]
    llm = LLM(zdirs[name][dtype], dtype=dtype, page_size=16, batch_max=3, max_tokens=512, prefill_batch=24, max_step_tokens=64)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    pcfg, W = P.read_model(zdirs[name]["float32"])
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        assert len(o.token_ids) == 8
        for got in o.token_ids:
            if dtype != "float32" and Z.first_close_call(zdirs[name]["float32"], tuple(toks), 0.25) < len(toks):
                break                # a router's close call: reduced precision may route otherwise from here on
            logits = P.forward(pcfg, W, toks)[-1]
            want = P.greedy(logits)
            if got != want:          # a tie within rounding is not a fault; anything else is
                gap = float(logits[want] - logits[got])
                assert gap <= (2e-5 if dtype == "float32" else 4e-2) * float(np.abs(logits).max()), f"{dtype}: token {got} instead of {want}"
            toks.append(got)


# ---- the programs a user runs ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,graphs", [("float32", 1), ("bfloat16", 1), ("bfloat16", 0)])
def test_trace_replay_program(zdirs, dtype, graphs, tmp_path):
    """bin/trace_run in a process of its own on a mixed trace: four state slots for seven requests, decode steps replayed
    from captured graphs (the default) and launched kernel by kernel."""
    import json
    import os
    import subprocess
    import sys
    name = "Z1"
    reqs = R.random_requests(Z.CONFIGS[name][0]["vocab"], (5, 33, 70, 47, 90, 16, 65), seed=21)
    steps, max_tokens = R.trace_mixed(reqs, live_max=4, seed=5)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", zdirs[name][dtype], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_tokens), "--cuda-graphs", str(graphs)], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = Z.CONFIGS[name][0]["vocab"]
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
    Z.compare_with_plain(zdirs[name]["float32"], reqs, got, dtype, f"trace_run/{dtype}")


def test_command_line_writes_random_weights_and_generates(tmp_path):
    """bin/kestrel: `--random-weights` writes a Zidivik folder from a config.json with the design's own keys (the ranks of
    the low-rank projections named in it), and the streaming harness prints the plain implementation's greedy tokens."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    raw = json.loads(json.dumps(Z.Z1))
    for L in raw["layers"]:
        if L["type"] == "channel_delta":
            L["mixer"].update(decay_rank=6, gate_rank=10)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(raw))
    model_dir = tmp_path / "written"
    prompt = R.random_requests(raw["vocab"], (23,), seed=2)["r0"]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "kestrel"), "--model", str(model_dir), "--config", str(cfg_file),
                        "--random-weights", "5", "--dtype", "float32", "--stream-test", "--stream-n", "8", "--prompt-ids",
                        ",".join(str(t) for t in prompt), "--ignore-eos", "--max-tokens", "256", "--batch-max", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    pcfg, W = P.read_model(str(model_dir))
    assert W["l1.mix.a1"].shape[0] == 6 and W["l1.mix.g1"].shape[0] == 10
    toks, want = list(prompt), []
    for _ in range(8):
        want.append(P.greedy(P.forward(pcfg, W, toks)[-1]))
        toks.append(want[-1])
    assert [int(t) for t in line[0].split(":")[1].split()] == want
