"""Parity of the CUDA path, called through the C ABI, against the CPU oracle on identical
seeded inputs.  Reference-order mode must be bit-identical to the oracle's F32 results
(max_abs = RMSE = 0, inside the stated 2e-5 / 2e-6); pairwise mode is held to the relative
bound of assert_pairwise_close against the double-accumulated reference."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from colormlm_b200 import _lib as L
from colormlm_b200 import synth
from colormlm_b200.pages import ExpertPageLayout
from colormlm_b200.s14 import (ExpertKey, RouteDecision, S14Context, S14Error, S14MatvecShape,
                               S14MoePages, TokenRoute, VramPool)

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("cuda_lib")]

MAX_ABS, RMSE = 2e-5, 2e-6  # the stated tolerance per layer; met bit-exactly in reference order


def assert_pairwise_close(oracle, y, ref_acc64, ref32=None):
    """Pairwise order sums F32 products in another order than the reference, so it cannot
    be held to an absolute bound tighter than the reference's own summation noise (the two
    F32 orders differ by ~2e-4 at these magnitudes).  It is held to a relative bound against
    the double-accumulated reference: RMSE <= 1e-6 of the output RMS and max error <= 8e-6 of
    the largest output (a few F32 ulps), and it must be at least as close to that value as
    the reference's own F32 order is."""
    ref = np.asarray(ref_acc64, np.float32)
    e = oracle.error_stats(np.asarray(y, np.float32), ref)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert e["rmse"] <= 1e-6 * rms, (e, rms)
    assert e["max_abs"] <= 8e-6 * float(np.abs(ref).max()), e
    if ref32 is not None:
        noise = oracle.error_stats(np.asarray(ref32, np.float32), ref)
        assert e["rmse"] <= noise["rmse"] + 1e-7 * rms, (e, noise)
    return e


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = S14Context(0)
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def dev_page(tensor_page, hidden, inter, kind=L.PAGE_MXFP4):
    """The oracle reads the page of checkpoint tensors; the GPU reads the expert page made from it."""
    return dev(ExpertPageLayout(hidden, inter, kind).to_expert_page(tensor_page))


def run_mxfp4(ctx, x, w, s, n, k):
    dx, dw, ds = dev(x), dev(w), dev(s)
    dy = torch.empty(n, dtype=torch.float32, device="cuda")
    d = ctx.pipelines.bind_mxfp4(S14MatvecShape(n, k), dx, dw, ds, dy)
    ctx.pipelines.cmd_mxfp4_matvec(d)
    torch.cuda.synchronize()
    return dy.cpu().numpy()


def run_fp8(ctx, x, w, s, n, k):
    x = np.atleast_2d(x)
    # buffers hold whole 32-bit words, as the reference's storage_bytes() requires (s14_vulkan.rs:128-130)
    wpad = np.zeros((w.size + 3) // 4 * 4, np.uint8)
    wpad[:w.size] = w.ravel()
    spad = s
    if s.dtype == np.uint8:
        spad = np.zeros((s.size + 3) // 4 * 4, np.uint8)
        spad[:s.size] = s.ravel()
    dx, dw, ds = dev(x), dev(wpad), dev(spad)
    dy = torch.empty((x.shape[0], n), dtype=torch.float32, device="cuda")
    fmt = L.SCALE_UE8M0 if s.dtype == np.uint8 else L.SCALE_F32
    d = ctx.pipelines.bind_fp8(S14MatvecShape(n, k), dx, dw, ds, dy, scale_format=fmt, n_tokens=x.shape[0])
    ctx.pipelines.cmd_fp8_matvec(d)
    torch.cuda.synchronize()
    return dy.cpu().numpy()


def stats(oracle, a, b):
    return oracle.error_stats(np.asarray(a, np.float32), np.asarray(b, np.float32))


@pytest.mark.parametrize("n,k", [(1, 128), (3, 128), (96, 1024), (2048, 4096), (4096, 2048), (7, 8192)])
def test_mxfp4_matvec_both_orders(ctx, oracle, n, k):
    g = synth.rng(10 + n + k)
    w, s, x = synth.mxfp4_codes(g, n, k), synth.mxfp4_scales(g, n, k), synth.activations(g, 1, k)[0]
    ref32 = oracle.mxfp4_matvec(x, w, s, n, k)
    ref64 = oracle.mxfp4_matvec_f64(x, w, s, n, k)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    assert np.array_equal(run_mxfp4(ctx, x, w, s, n, k).view(np.uint32), ref32.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_mxfp4(ctx, x, w, s, n, k)
    # F32 only inside a 32-element scale block: within a few ulps of the F64 value
    assert np.abs(y - ref64).max() <= 4 * np.spacing(np.abs(ref64).max().astype(np.float32))
    if n >= 96:
        assert_pairwise_close(oracle, y, ref64, ref32)


def test_mxfp4_extreme_scales_and_all_codes(ctx, oracle):
    """Scale codes 0 (2^-127, subnormal) .. 254 (2^127) and every nibble value."""
    n, k = 16, 256
    w = np.tile(np.arange(256, dtype=np.uint8), (n, k // 2 // 256 + 1))[:, :k // 2].copy()
    s = np.array([[0, 1, 2, 60, 126, 127, 128, 200][(r + c) % 8] for r in range(n) for c in range(k // 32)],
                 np.uint8).reshape(n, k // 32)
    x = synth.activations(synth.rng(5), 1, k)[0]
    ref = oracle.mxfp4_matvec(x, w, s, n, k)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    assert np.array_equal(run_mxfp4(ctx, x, w, s, n, k).view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    ref64 = oracle.mxfp4_matvec_f64(x, w, s, n, k)
    y = run_mxfp4(ctx, x, w, s, n, k)
    assert np.abs(y - ref64).max() <= 4 * np.spacing(np.abs(ref64).max().astype(np.float32))
    s[:] = 200
    ref = oracle.mxfp4_matvec(x, w, s, n, k)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    assert np.array_equal(run_mxfp4(ctx, x, w, s, n, k).view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


def test_golden_mxfp4_fixture_on_gpu(ctx, golden):
    """The reference's own deterministic fixture (test_primitives.py:58-72), its tolerance."""
    w, s, x = golden["fx_packed"], golden["fx_scales"], golden["fx_x"]
    for mode in (L.ACCUM_REFERENCE, L.ACCUM_PAIRWISE):
        ctx.set_accumulation(mode)
        for t in range(2):
            np.testing.assert_allclose(run_mxfp4(ctx, x[t], w, s, 3, 128), golden["fx_y_f32"][t],
                                       rtol=2e-6, atol=2e-6)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


@pytest.mark.parametrize("n,k,tokens", [(129, 130, 2), (1024, 4096, 1), (1024, 4096, 4), (1024, 4096, 8),
                                        (5, 16, 3), (256, 512, 4)])
@pytest.mark.parametrize("f32_scale", [False, True])
def test_fp8_matvec_both_orders(ctx, oracle, n, k, tokens, f32_scale):
    g = synth.rng(77 + n + k + tokens)
    w = synth.e4m3_codes(g, n, k)
    s = synth.fp8_block_scales_f32(g, n, k) if f32_scale else synth.fp8_block_scales_ue8m0(g, n, k)
    x = synth.activations(g, tokens, k)
    ref32 = np.stack([oracle.fp8_matvec(x[t], w, s, n, k) for t in range(tokens)])
    ref64 = np.stack([oracle.fp8_matvec_f64(x[t], w, s, n, k) for t in range(tokens)])
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    assert np.array_equal(run_fp8(ctx, x, w, s, n, k).view(np.uint32), ref32.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_fp8(ctx, x, w, s, n, k)
    assert np.abs(y - ref64).max() <= 4 * np.spacing(np.abs(ref64).max().astype(np.float32))
    # the reference harness's own FP8 gate (examples/s14_vulkan_numeric.rs:1537) against its F32 order
    e = stats(oracle, y, ref32)
    assert e["max_abs"] <= 2.5e-5 * max(1.0, np.abs(ref32).max()) and e["rmse"] <= 3.5e-6 * max(1.0, np.abs(ref32).max())


def test_golden_fp8_fixture_on_gpu(ctx, golden):
    w, s, x = golden["f8_w"], golden["f8_s"], golden["f8_x"]
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_fp8(ctx, x, w, s, 129, 130)
    np.testing.assert_allclose(y, golden["f8_y_f64"], rtol=3e-7, atol=1e-6)


def test_elementwise_operators(ctx, oracle):
    g = synth.rng(3)
    n = 2048 + 37
    gate = (g.standard_normal(n) * 7).astype(np.float32)
    up = (g.standard_normal(n) * 7).astype(np.float32)
    gate[:4] = [-20.0, 20.0, 10.0, -10.0]
    dg, du = dev(gate), dev(up)
    dy = torch.empty(n, dtype=torch.float32, device="cuda")
    p = ctx.pipelines
    p.cmd_swiglu_limit(p.bind_swiglu_limit(n, dg, du, dy))
    torch.cuda.synchronize()
    ref = oracle.swiglu_limit(gate, up)
    assert np.array_equal(dy.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    routed = torch.empty(n, dtype=torch.float32, device="cuda")
    p.cmd_route_mix(p.bind_route_mix(n, 0.3, dy, routed))
    acc = torch.zeros(n, dtype=torch.float32, device="cuda")
    p.cmd_moe_accumulate(p.bind_moe_accumulate(n, 0.3, dy, acc))
    p.cmd_moe_accumulate(p.bind_moe_accumulate(n, 1.0, du, acc))
    torch.cuda.synchronize()
    assert np.array_equal(routed.cpu().numpy(), np.float32(0.3) * ref)
    assert np.array_equal(acc.cpu().numpy(), (np.float32(0.0) + np.float32(0.3) * ref) + np.float32(1.0) * up)
    for bad in (float("nan"), -0.1, float("inf")):
        with pytest.raises(S14Error):
            p.bind_route_mix(n, bad, dy, routed)
        with pytest.raises(S14Error):
            p.bind_moe_accumulate(n, bad, dy, acc)
    with pytest.raises(S14Error):
        p.bind_swiglu_limit(0, dg, du, dy)


def test_bind_rejects_short_buffers(ctx):
    x = torch.zeros(4096, device="cuda")
    w = torch.zeros(2048 * 2048, dtype=torch.uint8, device="cuda")
    s = torch.zeros(2048 * 128, dtype=torch.uint8, device="cuda")
    y = torch.zeros(2048, device="cuda")
    shape = S14MatvecShape(2048, 4096)
    ctx.pipelines.bind_mxfp4(shape, x, w, s, y)
    for bufs in ((x[:4095], w, s, y), (x, w[:-1], s, y), (x, w, s[:-4], y), (x, w, s, y[:2047])):
        with pytest.raises(S14Error) as e:
            ctx.pipelines.bind_mxfp4(shape, *bufs)
        assert e.value.code == L.ERR_CONTRACT
    with pytest.raises(S14Error):
        ctx.pipelines.bind_mxfp4(S14MatvecShape(2048, 4000), x, w, s, y)


def make_layer(seed, hidden, inter, n_experts, shared_kind):
    g = synth.rng(seed)
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(n_experts)]
    shared = (synth.mxfp4_expert_page(g, hidden, inter) if shared_kind == L.PAGE_MXFP4
              else synth.fp8_expert_page(g, hidden, inter))
    return g, pages, shared


def run_layer(ctx, x, pages_dev, shared_dev, routes, shared_kind, hidden, inter):
    dx = dev(x)
    dy = torch.empty_like(dx)
    tr = [TokenRoute(ids, w, [pages_dev[i].data_ptr() for i in ids]) for ids, w in routes]
    ctx.cmd_moe_layer(dx, dy, tr, shared_dev.data_ptr() if shared_dev is not None else None, shared_kind,
                      hidden, inter)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0  # no bounded wait of a fused kernel ran out
    return dy.cpu().numpy()


@pytest.mark.parametrize("hidden,inter", [(1024, 1024), (2048, 1024), (4096, 2048)])
@pytest.mark.parametrize("shared_kind", [L.PAGE_MXFP4, L.PAGE_FP8])
def test_moe_layer_decode(ctx, oracle, hidden, inter, shared_kind):
    """One token, six routed experts and the shared expert (examples/s14_vulkan_numeric.rs:929-947)."""
    g, pages, shared = make_layer(200 + hidden + inter + shared_kind, hidden, inter, 9, shared_kind)
    x = synth.activations(g, 1, hidden)
    ids = [7, 2, 5, 0, 8, 3]
    w = np.asarray([0.31, 0.22, 0.17, 0.13, 0.1, 0.07], np.float32)
    pages_dev = [dev_page(p, hidden, inter) for p in pages]
    shared_dev = dev_page(shared, hidden, inter, shared_kind)
    ref32 = oracle.moe_layer(x[0], [pages[i] for i in ids], w, shared, shared_kind, hidden, inter)
    ref64 = oracle.moe_layer_acc64(x[0], [pages[i] for i in ids], w, shared, shared_kind, hidden, inter)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    y = run_layer(ctx, x, pages_dev, shared_dev, [(ids, w)], shared_kind, hidden, inter)[0]
    assert np.array_equal(y.view(np.uint32), ref32.view(np.uint32)), stats(oracle, y, ref32)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_layer(ctx, x, pages_dev, shared_dev, [(ids, w)], shared_kind, hidden, inter)[0]
    assert_pairwise_close(oracle, y, ref64, ref32)
    # against the F32-order oracle the difference is that oracle's own summation noise
    e32, noise = stats(oracle, y, ref32), stats(oracle, ref32, ref64)
    assert e32["rmse"] <= 1.5 * noise["rmse"] + RMSE


def test_moe_layer_decode_wide_range_and_zero_blocks(ctx, oracle):
    """The tensor-core layer kernel writes activations as digit rows per scale block: blocks of
    zeros, magnitudes from 1e-6 to 1e3 side by side, exact powers of two and a lone large value
    in a block of small ones.  Gate and up sums reach 2e4 here while only values inside the +-10
    clamp pass on, so the input is ill-conditioned: the reference's own F32 order is 3.7e-6 of
    the output RMS away from the double-accumulated result.  The pairwise result is held to
    twice that noise instead of the 1e-6 bound of well-conditioned inputs."""
    hidden, inter = 2048, 1024
    g, pages, shared = make_layer(4321, hidden, inter, 8, L.PAGE_MXFP4)
    x = synth.activations(g, 1, hidden)
    x[0] *= 10.0 ** g.uniform(-6.0, 3.0, hidden).astype(np.float32)
    x[0, 64:160] = 0.0                      # three scale blocks of zeros
    x[0, 256:288] = 2.0 ** np.arange(-16, 16, dtype=np.float32)  # powers of two, 2^-16 .. 2^15 in one block
    x[0, 320:352] = 1e-4
    x[0, 333] = -7.0e3                      # a lone large value among small ones
    ids = [1, 6, 3, 0, 7, 4]
    w = np.asarray([0.4, 0.2, 0.15, 0.1, 0.1, 0.05], np.float32)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    ref64 = oracle.moe_layer_acc64(x[0], [pages[i] for i in ids], w, shared, 0, hidden, inter)
    ref32 = oracle.moe_layer(x[0], [pages[i] for i in ids], w, shared, 0, hidden, inter)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_layer(ctx, x, pages_dev, shared_dev, [(ids, w)], L.PAGE_MXFP4, hidden, inter)[0]
    assert np.isfinite(y).all()
    ref = np.asarray(ref64, np.float32)
    e, noise = oracle.error_stats(y, ref), oracle.error_stats(ref32, ref)
    assert e["rmse"] <= 2.0 * noise["rmse"] and e["max_abs"] <= 2.0 * noise["max_abs"], (e, noise)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    y = run_layer(ctx, x, pages_dev, shared_dev, [(ids, w)], L.PAGE_MXFP4, hidden, inter)[0]
    assert np.array_equal(y.view(np.uint32), ref32.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


def test_single_expert_chain_route_weight(ctx, oracle):
    """w1, w3 -> limited SwiGLU -> w2 -> x 0.3 (examples/s14_vulkan_numeric.rs:1296-1300)."""
    hidden, inter = 4096, 2048
    g = synth.rng(126)
    page = synth.mxfp4_expert_page(g, hidden, inter)
    x = synth.activations(g, 1, hidden)
    ref, _ = oracle.expert_chain_mxfp4(x[0], page, hidden, inter, 0.3)
    pd = dev_page(page, hidden, inter)
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    y = run_layer(ctx, x, [pd], None, [([0], [0.3])], L.PAGE_MXFP4, hidden, inter)[0]
    # the layer starts from acc = 0 and adds w * down; 0 + v == v exactly
    assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


@pytest.mark.parametrize("n_tokens", [2, 4, 8])
def test_moe_layer_verify_block(ctx, oracle, n_tokens):
    """K tokens through one layer; tokens share experts; every token equals its own decode."""
    hidden, inter, n_experts = 2048, 1024, 16
    g, pages, shared = make_layer(900 + n_tokens, hidden, inter, n_experts, L.PAGE_MXFP4)
    x = synth.activations(g, n_tokens, hidden)
    routes = []
    for t in range(n_tokens):
        ids = g.permutation(n_experts)[:6].tolist()
        w = g.uniform(0.05, 0.4, 6).astype(np.float32)
        routes.append((ids, w))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    for mode in (L.ACCUM_REFERENCE, L.ACCUM_PAIRWISE):
        ctx.set_accumulation(mode)
        y = run_layer(ctx, x, pages_dev, shared_dev, routes, L.PAGE_MXFP4, hidden, inter)
        assert ctx.last_layer_path == (L.LAYER_PATH_REFERENCE if mode == L.ACCUM_REFERENCE else L.LAYER_PATH_TENSOR_PER_TOKEN)
        for t in range(n_tokens):
            ids, w = routes[t]
            if mode == L.ACCUM_REFERENCE:
                ref = oracle.moe_layer(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
                bad = np.nonzero(y[t].view(np.uint32) != ref.view(np.uint32))[0]
                assert bad.size == 0, (t, bad.size, bad[:8], y[t][bad[:4]], ref[bad[:4]])
            else:
                ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
                assert_pairwise_close(oracle, y[t], ref)
            # a token of a block against its own one-token call: bit-identical in both orders (in
            # pairwise order a block of MXFP4 experts is one launch of the tcgen05 kernel per token, and
            # the result is the double-accumulated oracle's, bit for bit)
            single = run_layer(ctx, x[t:t + 1], pages_dev, shared_dev, [routes[t]], L.PAGE_MXFP4, hidden, inter)[0]
            assert ctx.last_layer_path == (L.LAYER_PATH_REFERENCE if mode == L.ACCUM_REFERENCE else L.LAYER_PATH_TENSOR)
            assert np.array_equal(single.view(np.uint32), y[t].view(np.uint32))
            if mode == L.ACCUM_PAIRWISE:
                assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


def test_moe_layer_verify_block_at_the_benchmark_shape(ctx, oracle):
    """Eight tokens, 4096 x 2048, 48 experts of which the block uses 25 or more distinct ones: in
    pairwise order every token is its own one-token call and the double-accumulated oracle, bit for
    bit; in reference order the F32 oracle."""
    hidden, inter, n_experts, n_tokens = 4096, 2048, 48, 8
    g, pages, shared = make_layer(977, hidden, inter, n_experts, L.PAGE_MXFP4)
    x = synth.activations(g, n_tokens, hidden)
    routes = []
    for t in range(n_tokens):
        routes.append((g.permutation(n_experts)[:6].tolist(), g.uniform(0.05, 0.4, 6).astype(np.float32)))
    assert len({e for ids, _ in routes for e in ids}) >= 25
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    y = run_layer(ctx, x, pages_dev, shared_dev, routes, L.PAGE_MXFP4, hidden, inter)
    assert ctx.last_layer_path == L.LAYER_PATH_TENSOR_PER_TOKEN
    for t in range(n_tokens):
        ids, w = routes[t]
        ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
        assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32)), (t, stats(oracle, y[t], ref))
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    y = run_layer(ctx, x[:2], pages_dev, shared_dev, routes[:2], L.PAGE_MXFP4, hidden, inter)
    for t in range(2):
        ids, w = routes[t]
        ref = oracle.moe_layer(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
        assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


def test_moe_layer_rejects_bad_routes(ctx):
    hidden, inter = 1024, 1024
    page = torch.zeros(ExpertPageLayout(hidden, inter).page_bytes, dtype=torch.uint8, device="cuda")
    x = torch.zeros((1, hidden), device="cuda")
    y = torch.empty_like(x)
    ok = TokenRoute([0, 1], [0.5, 0.5], [page.data_ptr()] * 2)
    ctx.cmd_moe_layer(x, y, [ok], None, L.PAGE_MXFP4, hidden, inter)
    bad = [TokenRoute([0, 0], [0.5, 0.5], [page.data_ptr()] * 2),
           TokenRoute([0, 1], [0.5, float("nan")], [page.data_ptr()] * 2),
           TokenRoute([0, 1], [0.5, -1.0], [page.data_ptr()] * 2),
           TokenRoute([0, 1], [0.5, 0.5], [page.data_ptr(), 0])]
    for r in bad:
        with pytest.raises(S14Error):
            ctx.cmd_moe_layer(x, y, [r], None, L.PAGE_MXFP4, hidden, inter)
    with pytest.raises(S14Error):
        ctx.cmd_moe_layer(x, y, [ok], None, L.PAGE_MXFP4, 1000, inter)
    with pytest.raises(S14Error):
        ctx.cmd_moe_layer(x, y, [], None, L.PAGE_MXFP4, hidden, inter)
    torch.cuda.synchronize()


@pytest.mark.parametrize("score_fn", [L.SCORE_SIGMOID, L.SCORE_SQRT_SOFTPLUS])
def test_router_indices_bit_exact(ctx, oracle, score_fn):
    g = synth.rng(4242 + score_fn)
    n_experts, hidden, tokens = 256, 4096, 8
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    min_gap = np.inf
    for rep in range(4):
        x = synth.activations(g, tokens, hidden)
        ids = torch.empty((tokens, 6), dtype=torch.int32, device="cuda")
        wts = torch.empty((tokens, 6), dtype=torch.float32, device="cuda")
        ctx.cmd_router(dev(x), dev(wr), dev(bias), ids, wts, score_fn=score_fn, top_k=6, route_scale=1.5)
        torch.cuda.synchronize()
        for t in range(tokens):
            rid, rw, _, select = oracle.router(x[t], wr, bias, score_fn=score_fn, top_k=6, route_scale=1.5)
            srt = np.sort(select)[::-1]
            min_gap = min(min_gap, float(srt[5] - srt[6]))
            assert np.array_equal(ids[t].cpu().numpy(), rid)
            assert np.array_equal(wts[t].cpu().numpy().view(np.uint32), rw.view(np.uint32))
    assert min_gap > 0


def test_golden_router_fixture_on_gpu(ctx, golden):
    g = synth.rng(1004)
    wr, bias, x = synth.router_weight_bf16(g, 256, 1024), synth.router_bias(g, 256), synth.activations(g, 4, 1024)
    for fn, name in ((L.SCORE_SIGMOID, "sig"), (L.SCORE_SQRT_SOFTPLUS, "ssp")):
        ids = torch.empty((4, 6), dtype=torch.int32, device="cuda")
        wts = torch.empty((4, 6), dtype=torch.float32, device="cuda")
        ctx.cmd_router(dev(x), dev(wr), dev(bias), ids, wts, score_fn=fn, top_k=6, route_scale=1.5)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy(), golden[f"rt_{name}_ids"])
        np.testing.assert_allclose(wts.cpu().numpy(), golden[f"rt_{name}_w"], rtol=2e-6)


def test_routed_layer_without_host_round_trip(ctx, oracle):
    """Router and layer chained on the device: same route and same output as the two-step path."""
    hidden, inter, n_experts = 2048, 1024, 32
    g, pages, shared = make_layer(31337, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    x = synth.activations(g, 1, hidden)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    dx = dev(x)
    y = torch.empty_like(dx)
    ids = torch.empty(6, dtype=torch.int32, device="cuda")
    wts = torch.empty(6, dtype=torch.float32, device="cuda")
    for mode in (L.ACCUM_REFERENCE, L.ACCUM_PAIRWISE):
        ctx.set_accumulation(mode)
        ctx.cmd_routed_moe_layer(dx[0], dev(wr), dev(bias), table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, y,
                                 ids, wts)
        torch.cuda.synchronize()
        rid, rw, _, _ = oracle.router(x[0], wr, bias, 0, 6, 1.0)
        assert np.array_equal(ids.cpu().numpy(), rid)
        assert np.array_equal(wts.cpu().numpy().view(np.uint32), rw.view(np.uint32))
        if mode == L.ACCUM_REFERENCE:
            ref = oracle.moe_layer(x[0], [pages[i] for i in rid], rw, shared, 0, hidden, inter)
            assert np.array_equal(y.cpu().numpy()[0].view(np.uint32), ref.view(np.uint32))
        else:
            ref = oracle.moe_layer_acc64(x[0], [pages[i] for i in rid], rw, shared, 0, hidden, inter)
            assert_pairwise_close(oracle, y.cpu().numpy()[0], ref)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


def near_tie_bias(oracle, x, wr, bias, score_fn):
    """A copy of `bias` in which the seventh-best expert's selection value is moved to within 1e-5
    below the sixth-best one (the seventh expert has the lower id when possible, so that a kernel
    that confused the two would pick it)."""
    _, _, scores, select = oracle.router(x, wr, bias, score_fn, 6, 1.0)
    order = np.lexsort((np.arange(select.size), -select.astype(np.float64)))
    sixth, seventh = int(order[5]), int(order[6])
    b = bias.copy()
    want = np.float32(select[sixth]) - np.float32(3e-6)
    b[seventh] = np.float32(np.float64(want) - np.float64(scores[seventh]))
    return b, sixth, seventh


@pytest.mark.parametrize("score_fn", [L.SCORE_SIGMOID, L.SCORE_SQRT_SOFTPLUS])
def test_routed_layer_at_the_benchmark_shape(ctx, oracle, score_fn):
    """The configuration the benchmark times: 256 routed experts, hidden 4096, intermediate 2048,
    MXFP4 shared expert, the router inside the layer kernel (every CTA scores two experts).  Eight
    tokens over two layers; ids and weights bit-exact against the oracle's router, y bit-exact in
    reference order and, in pairwise order, inside the stated tolerance (max-abs 2e-5, RMSE 2e-6)
    against the double-accumulated oracle.  One token per layer has a sixth / seventh selection gap
    below 1e-5.  Only the pages a token selects are generated; every other table entry points at a
    page of other bytes, so a wrong pick cannot go unnoticed."""
    hidden, inter, n_experts, tokens_per_layer = 4096, 2048, 256, 4
    worst = {"max_abs": 0.0, "rmse": 0.0, "bit_equal": 1.0}
    for layer in range(2):
        g = synth.rng(7100 + 10 * layer + score_fn)
        wr, bias0 = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
        xs = synth.activations(g, tokens_per_layer, hidden)
        biases, gaps = [], []
        for t in range(tokens_per_layer):
            b = bias0
            if t == 1:
                b, sixth, seventh = near_tie_bias(oracle, xs[t], wr, bias0, score_fn)
            _, _, _, select = oracle.router(xs[t], wr, b, score_fn, 6, 1.0)
            srt = np.sort(select)[::-1]
            gaps.append(float(srt[5] - srt[6]))
            biases.append(b)
        assert 0.0 < gaps[1] < 1e-5, gaps
        routes = [oracle.router(xs[t], wr, biases[t], score_fn, 6, 1.0) for t in range(tokens_per_layer)]
        needed = sorted({int(e) for r in routes for e in r[0]})
        pages = {e: synth.mxfp4_expert_page(synth.rng(90_000 + 1000 * layer + e), hidden, inter) for e in needed}
        shared = synth.mxfp4_expert_page(synth.rng(95_000 + layer), hidden, inter)
        other = dev_page(synth.mxfp4_expert_page(synth.rng(96_000 + layer), hidden, inter), hidden, inter)
        pages_dev = {e: dev_page(p, hidden, inter) for e, p in pages.items()}
        shared_dev = dev_page(shared, hidden, inter)
        table = torch.tensor([pages_dev[e].data_ptr() if e in pages_dev else other.data_ptr() for e in range(n_experts)],
                             dtype=torch.int64, device="cuda")
        dwr = dev(wr.view(np.int16))
        ids = torch.empty(6, dtype=torch.int32, device="cuda")
        wts = torch.empty(6, dtype=torch.float32, device="cuda")
        for t in range(tokens_per_layer):
            rid, rw, _, _ = routes[t]
            dx, dbias = dev(xs[t:t + 1]), dev(biases[t])
            y = torch.empty_like(dx)
            sel = [pages[int(e)] for e in rid]
            for mode in ((L.ACCUM_PAIRWISE, L.ACCUM_REFERENCE) if t < 2 else (L.ACCUM_PAIRWISE,)):
                ctx.set_accumulation(mode)
                before = ctx.launch_count
                ctx.cmd_routed_moe_layer(dx[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, y,
                                         ids, wts, score_fn=score_fn)
                torch.cuda.synchronize()
                assert ctx.device_status() == 0
                assert np.array_equal(ids.cpu().numpy(), rid), (layer, t, mode)
                assert np.array_equal(wts.cpu().numpy().view(np.uint32), rw.view(np.uint32)), (layer, t, mode)
                got = y.cpu().numpy()[0]
                if mode == L.ACCUM_REFERENCE:
                    ref = oracle.moe_layer(xs[t], sel, rw, shared, 0, hidden, inter)
                    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), stats(oracle, got, ref)
                else:
                    assert ctx.launch_count - before == 1  # scores, routes and the layer in one launch
                    ref = oracle.moe_layer_acc64(xs[t], sel, rw, shared, 0, hidden, inter)
                    e = stats(oracle, got, ref)
                    assert e["max_abs"] <= MAX_ABS and e["rmse"] <= RMSE, (layer, t, e)
                    worst["max_abs"] = max(worst["max_abs"], e["max_abs"])
                    worst["rmse"] = max(worst["rmse"], e["rmse"])
                    worst["bit_equal"] = min(worst["bit_equal"], float((got.view(np.uint32) == ref.view(np.uint32)).mean()))
        del pages_dev, shared_dev, other
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    print("benchmark-shape parity, pairwise vs double-accumulated oracle:", worst)


def assert_chain_close(oracle, got, ref, what):
    """A chain of layers without normalisation grows (outputs reach the hundreds after a few layers),
    so the stated absolute tolerance (max-abs 2e-5, RMSE 2e-6, written for outputs of magnitude ~100
    and RMS ~27, i.e. about three F32 ulps of the largest value and one ulp of the RMS) is kept in
    those units: max error <= max(2e-5, 3 ulps of the largest reference value), RMSE <= max(2e-6,
    one ulp of the reference RMS)."""
    ref = np.asarray(ref, np.float32)
    e = stats(oracle, got, ref)
    rms = np.float32(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert e["max_abs"] <= max(MAX_ABS, 3.0 * float(np.spacing(np.abs(ref).max()))), (what, e)
    assert e["rmse"] <= max(RMSE, float(np.spacing(rms))), (what, e)
    return e


def oracle_stack(oracle, x, layers, hidden, inter, residual, acc64, score_fn=0):
    """The chain h <- h + moe_l(h) on the CPU: every layer routed by the oracle's router on the
    layer's own input; returns the final h, the per-layer outputs and routes."""
    h = np.asarray(x, np.float32).copy()
    ys, routes = [], []
    for ly in layers:
        rid, rw, _, _ = oracle.router(h, ly["wr"], ly["bias"], score_fn, 6, 1.0)
        sel = [ly["page"](int(e)) for e in rid]
        fn = oracle.moe_layer_acc64 if acc64 else oracle.moe_layer
        yl = fn(h, sel, rw, ly["shared"], 0, hidden, inter)
        ys.append(yl)
        routes.append((rid, rw))
        h = (h + yl).astype(np.float32) if residual else yl
    return h, ys, routes


@pytest.mark.parametrize("residual", [True, False])
def test_decode_stack_small(ctx, oracle, residual):
    """Four chained layers (hidden 2048, intermediate 1024, 32 experts) in one launch: routes of every
    layer bit-exact, every layer's output and the final token equal to the same layers run one by one
    and inside the stated tolerance against the double-accumulated oracle chain; reference order
    (layers launched one by one) bit-identical to the F32 oracle chain."""
    from colormlm_b200.s14 import DecodeStack

    hidden, inter, n_experts, n_layers = 2048, 1024, 32, 4
    host_layers, dev_layers, keep = [], [], []
    for l in range(n_layers):
        g, pages, shared = make_layer(8800 + l, hidden, inter, n_experts, L.PAGE_MXFP4)
        wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
        host_layers.append({"wr": wr, "bias": bias, "shared": shared, "page": (lambda e, p=pages: p[e])})
        pd, sd = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
        keep.append((pd, sd))
        dev_layers.append({"wr": dev(wr.view(np.int16)), "bias": dev(bias),
                           "table": torch.tensor([p.data_ptr() for p in pd], dtype=torch.int64, device="cuda"),
                           "shared": sd.data_ptr(),
                           "ids": torch.empty(6, dtype=torch.int32, device="cuda"),
                           "weights": torch.empty(6, dtype=torch.float32, device="cuda"),
                           "y": torch.empty(hidden, dtype=torch.float32, device="cuda")})
    x = synth.activations(synth.rng(8899), 1, hidden)[0] * np.float32(0.25)
    dx = dev(x)
    stack = DecodeStack(ctx, dev_layers, inter=inter, residual=residual)
    try:
        for mode, acc64 in ((L.ACCUM_PAIRWISE, True), (L.ACCUM_REFERENCE, False)):
            ctx.set_accumulation(mode)
            want_h, want_y, want_routes = oracle_stack(oracle, x, host_layers, hidden, inter, residual, acc64)
            h = torch.full((hidden,), float("nan"), device="cuda")
            before = ctx.launch_count
            stack.cmd_decode(dx, h)
            torch.cuda.synchronize()
            assert ctx.device_status() == 0
            if mode == L.ACCUM_PAIRWISE:
                assert ctx.launch_count - before == 1  # the whole stack is one launch
            for l in range(n_layers):
                rid, rw = want_routes[l]
                assert np.array_equal(dev_layers[l]["ids"].cpu().numpy(), rid), (mode, l)
                assert np.array_equal(dev_layers[l]["weights"].cpu().numpy().view(np.uint32), rw.view(np.uint32)), (mode, l)
                got = dev_layers[l]["y"].cpu().numpy()
                if mode == L.ACCUM_REFERENCE:
                    assert np.array_equal(got.view(np.uint32), want_y[l].view(np.uint32)), (l, stats(oracle, got, want_y[l]))
                else:
                    assert_chain_close(oracle, got, want_y[l], ("layer", l))
            got_h = h.cpu().numpy()
            if mode == L.ACCUM_REFERENCE:
                assert np.array_equal(got_h.view(np.uint32), want_h.view(np.uint32))
            else:
                assert_chain_close(oracle, got_h, want_h, "final token")
                # the same layers one by one, the step between them on the host side of the call
                cur = dx.clone()
                for l in range(n_layers):
                    yl = torch.empty(1, hidden, device="cuda")
                    ly = dev_layers[l]
                    ctx.cmd_routed_moe_layer(cur, ly["wr"], ly["bias"], ly["table"], ly["shared"], L.PAGE_MXFP4, inter, yl)
                    cur = cur + yl[0] if residual else yl[0].clone()
                torch.cuda.synchronize()
                assert torch.equal(cur, h)
        # a second token through the same stack (the counters are back at zero, the barriers start again)
        ctx.set_accumulation(L.ACCUM_PAIRWISE)
        x2 = synth.activations(synth.rng(8900), 1, hidden)[0] * np.float32(0.25)
        want_h, _, _ = oracle_stack(oracle, x2, host_layers, hidden, inter, residual, True)
        h = torch.empty(hidden, device="cuda")
        stack.cmd_decode(dev(x2), h)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        assert_chain_close(oracle, h.cpu().numpy(), want_h, "second token")
    finally:
        stack.close()
        ctx.set_accumulation(L.ACCUM_PAIRWISE)


def test_decode_stack_at_the_benchmark_shape(ctx, oracle):
    """Three chained layers of 256 experts, hidden 4096, intermediate 2048 with the residual, one
    launch: routes bit-exact, outputs inside the stated tolerance against the double-accumulated
    oracle chain.  Only the pages the chain selects are generated (the oracle chain is run first)."""
    from colormlm_b200.s14 import DecodeStack

    hidden, inter, n_experts, n_layers = 4096, 2048, 256, 3
    cache = {}

    def page(layer, e):
        if (layer, e) not in cache:
            cache[(layer, e)] = synth.mxfp4_expert_page(synth.rng(70_000 + 1000 * layer + e), hidden, inter)
        return cache[(layer, e)]

    host_layers = []
    for l in range(n_layers):
        g = synth.rng(7700 + l)
        host_layers.append({"wr": synth.router_weight_bf16(g, n_experts, hidden), "bias": synth.router_bias(g, n_experts),
                            "shared": synth.mxfp4_expert_page(synth.rng(79_000 + l), hidden, inter),
                            "page": (lambda e, l=l: page(l, e))})
    x = synth.activations(synth.rng(7799), 1, hidden)[0]
    want_h, want_y, want_routes = oracle_stack(oracle, x, host_layers, hidden, inter, True, True)
    dev_layers, keep = [], []
    for l in range(n_layers):
        other = dev_page(synth.mxfp4_expert_page(synth.rng(78_000 + l), hidden, inter), hidden, inter)
        pd = {int(e): dev_page(page(l, int(e)), hidden, inter) for e in want_routes[l][0]}
        sd = dev_page(host_layers[l]["shared"], hidden, inter)
        keep.append((other, pd, sd))
        dev_layers.append({"wr": dev(host_layers[l]["wr"].view(np.int16)), "bias": dev(host_layers[l]["bias"]),
                           "table": torch.tensor([pd[e].data_ptr() if e in pd else other.data_ptr() for e in range(n_experts)],
                                                 dtype=torch.int64, device="cuda"),
                           "shared": sd.data_ptr(),
                           "ids": torch.empty(6, dtype=torch.int32, device="cuda"),
                           "weights": torch.empty(6, dtype=torch.float32, device="cuda"),
                           "y": torch.empty(hidden, dtype=torch.float32, device="cuda")})
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    stack = DecodeStack(ctx, dev_layers, inter=inter, residual=True)
    try:
        h = torch.empty(hidden, device="cuda")
        for rep in range(2):
            before = ctx.launch_count
            stack.cmd_decode(dev(x), h)
            torch.cuda.synchronize()
            assert ctx.device_status() == 0 and ctx.launch_count - before == 1
            for l in range(n_layers):
                rid, rw = want_routes[l]
                assert np.array_equal(dev_layers[l]["ids"].cpu().numpy(), rid), l
                assert np.array_equal(dev_layers[l]["weights"].cpu().numpy().view(np.uint32), rw.view(np.uint32)), l
                assert_chain_close(oracle, dev_layers[l]["y"].cpu().numpy(), want_y[l], ("layer", l))
            assert_chain_close(oracle, h.cpu().numpy(), want_h, "final token")
    finally:
        stack.close()


def test_routed_layer_on_host_buffers_and_the_bound_call(ctx, oracle):
    """The call a host program makes per token: x from host memory, y and the route back.  The bound
    call (descriptor recorded once) and the one-shot call give the device path's bits."""
    hidden, inter, n_experts = 2048, 1024, 32
    g, pages, shared = make_layer(4711, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    dwr, dbias = dev(wr.view(np.int16)), dev(bias)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    bound = ctx.bind_routed_moe_layer_host(dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter)
    for step in range(3):
        x = synth.activations(g, 1, hidden)
        want = torch.empty((1, hidden), dtype=torch.float32, device="cuda")
        ctx.cmd_routed_moe_layer(dev(x)[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, want)
        torch.cuda.synchronize()
        rid, rw, _, _ = oracle.router(x[0], wr, bias, 0, 6, 1.0)
        for call in ("bound", "one-shot"):
            y = np.full(hidden, np.nan, np.float32)
            ids, wts = np.full(6, -1, np.int32), np.zeros(6, np.float32)
            if call == "bound":
                bound(x[0], y, ids, wts)
            else:
                ctx.routed_moe_layer_host(x[0], y, dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, ids, wts)
            assert np.array_equal(ids, rid) and np.array_equal(wts.view(np.uint32), rw.view(np.uint32))
            assert np.array_equal(y.view(np.uint32), want.cpu().numpy()[0].view(np.uint32)), (step, call)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_expert_parallel_slots_add_up_to_the_single_gpu_layer(ctx, world):
    """Every rank's share is run in turn on one GPU; the slot buffers are summed as the all-reduce
    would and mixed in route order: bit-identical to the undivided layer for any world size."""
    from colormlm_b200 import ep

    hidden, inter, n_experts = 2048, 1024, 32
    g, pages, shared = make_layer(4040, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    x = dev(synth.activations(g, 1, hidden))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    dwr, dbias = dev(wr.view(np.int16)), dev(bias)
    for mode in (L.ACCUM_REFERENCE, L.ACCUM_PAIRWISE):
        ctx.set_accumulation(mode)
        want = torch.empty_like(x)
        ctx.cmd_routed_moe_layer(x[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, want)
        total = torch.zeros((7, hidden), device="cuda")
        ids = torch.empty(6, dtype=torch.int32, device="cuda")
        wts = torch.empty(6, dtype=torch.float32, device="cuda")
        owned = 0
        for rank in range(world):
            slots = torch.full((7, hidden), float("nan"), device="cuda")
            ctx.cmd_routed_moe_experts_ep(x[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, slots,
                                          ids, wts, ep_rank=rank, ep_world=world,
                                          shared_owner=ep.shared_owner(5, world))
            torch.cuda.synchronize()
            mine = [j for j, e in enumerate(ids.tolist()) if ep.expert_owner(e, world) == rank]
            if ep.shared_owner(5, world) == rank:
                mine.append(6)
            owned += len(mine)
            others = [j for j in range(7) if j not in mine]
            assert float(slots[others].abs().sum()) == 0.0
            total += slots
        assert owned == 7
        got = torch.empty_like(x)
        ctx.cmd_moe_mix_slots(total, wts, 6, True, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_exchange_in_the_layer_kernel(ctx, world):
    """The exchange over mapped slot buffers, every rank a context of this process on one GPU.  Ranks
    1 .. world-1 publish their down vectors and flags without waiting (no launch waits for a later
    launch of the same GPU); rank 0 runs last, finds every flag, and mixes: bit-identical to the
    undivided layer, over several steps (the slot buffers alternate, the step count advances)."""
    from colormlm_b200 import ep
    from colormlm_b200.s14 import S14Context

    hidden, inter, n_experts = 2048, 1024, 32
    g, pages, shared = make_layer(5050, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    dwr, dbias = dev(wr.view(np.int16)), dev(bias)
    ranks = [S14Context(0) for _ in range(world)]
    try:
        for r, c in enumerate(ranks):
            c.set_accumulation(L.ACCUM_PAIRWISE)
            c.ep_exchange_create(r, world, hidden)
        for c in ranks:
            c.ep_exchange_connect_local(ranks)
        ctx.set_accumulation(L.ACCUM_PAIRWISE)
        for step in range(5):
            x = dev(synth.activations(g, 1, hidden))
            want = torch.empty_like(x)
            ctx.cmd_routed_moe_layer(x[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, want)
            got = torch.full_like(x, float("nan"))
            ids = torch.empty(6, dtype=torch.int32, device="cuda")
            wts = torch.empty(6, dtype=torch.float32, device="cuda")
            owner = ep.shared_owner(step, world)
            for r in range(world - 1, -1, -1):
                ranks[r].cmd_routed_moe_layer_ep(x[0], got if r == 0 else None, dwr, dbias, table, shared_dev.data_ptr(),
                                                 inter, shared_owner=owner, wait_and_mix=(r == 0),
                                                 ids_out=ids if r == 0 else None, weights_out=wts if r == 0 else None)
                torch.cuda.synchronize()
                assert ranks[r].device_status() == 0
            assert torch.equal(got, want), step
    finally:
        for c in ranks:
            c.close()


def test_expert_loader_ring_on_the_device(ctx):
    """Five pages through a ring of two pinned staging buffers into a device pool
    (expert_loader.rs:299-442): hidden until published, every page intact in its slot afterwards."""
    from cuda import cudart

    slot_bytes = 1 << 20
    pool, ld = C.c_void_p(), C.c_void_p()
    L.check(L.lib().s14_pool_create(ctx._h, 6, slot_bytes, C.byref(pool)))
    try:
        L.check(L.lib().s14_loader_create(pool, 2, C.byref(ld)))
        g = synth.rng(55)
        ids = [3, 8, 3, 1, 9, 4]
        pages = {i: g.integers(0, 256, slot_bytes, dtype=np.uint8) for i in set(ids)}
        keys = (L.ExpertKey * len(ids))(*[L.ExpertKey(2, 0, i) for i in ids])
        datas = (C.c_void_p * len(ids))(*[pages[i].ctypes.data for i in ids])
        sizes = (C.c_uint64 * len(ids))(*[slot_bytes] * len(ids))
        slots = (C.c_uint32 * len(ids))()
        L.check(L.lib().s14_loader_batch_enqueue_from_bufs(ld, keys, datas, sizes, len(ids), slots))
        assert L.lib().s14_loader_stat_loads(ld) == 5 and slots[0] == slots[2]
        found, slot = C.c_int32(), C.c_uint32()
        L.check(L.lib().s14_pool_lookup(pool, L.ExpertKey(2, 0, 4), C.byref(found), C.byref(slot)))
        assert found.value == 0  # the last wave is in flight: not visible yet
        L.check(L.lib().s14_loader_wait_all(ld))
        assert L.lib().s14_loader_in_flight(ld) == 0
        for pos, i in enumerate(ids):
            back = np.empty(slot_bytes, np.uint8)
            (err,) = cudart.cudaMemcpy(back.ctypes.data, L.lib().s14_pool_slot_ptr(pool, slots[pos]), slot_bytes,
                                       cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost)
            assert err == cudart.cudaError_t.cudaSuccess
            assert np.array_equal(back, pages[i]), i
    finally:
        L.lib().s14_loader_destroy(ld)
        L.lib().s14_pool_destroy(pool)


def test_exchange_teardown_order_is_enforced():
    """A context whose exchange is connected is not destroyed, and its buffer is not freed: both calls
    return the contract error until the rank has disconnected (which waits for its device's work and
    closes its mappings).  Two ranks of this process on one GPU."""
    from colormlm_b200.s14 import S14Context

    ranks = [S14Context(0) for _ in range(2)]
    for r, c in enumerate(ranks):
        c.ep_exchange_create(r, 2, 1024)
    for c in ranks:
        c.ep_exchange_connect_local(ranks)
    lib = L.lib()
    assert lib.s14_ep_exchange_destroy(ranks[0]._h) == L.ERR_CONTRACT
    assert lib.s14_ctx_destroy(ranks[0]._h) == L.ERR_CONTRACT
    for c in ranks:  # step 1 on every rank; no host barrier is needed inside one process
        c.ep_exchange_disconnect()
    for c in ranks:  # step 3
        c.ep_exchange_destroy()
        c.close()
    assert all(c._h is None for c in ranks)


def test_expert_parallel_wait_runs_out_when_a_rank_never_publishes(ctx):
    """Failure detection without a fault: rank 1 never runs its step, rank 0's bounded wait (set to
    a few milliseconds here) runs out, the kernel reports status 0x5503 and returns, and the GPU
    and the context go on working."""
    from colormlm_b200.s14 import S14Context

    hidden, inter, n_experts = 2048, 1024, 32
    g, pages, shared = make_layer(6060, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    dwr, dbias = dev(wr.view(np.int16)), dev(bias)
    x = dev(synth.activations(g, 1, hidden))
    ranks = [S14Context(0) for _ in range(2)]
    try:
        for r, c in enumerate(ranks):
            c.set_accumulation(L.ACCUM_PAIRWISE)
            c.ep_exchange_create(r, 2, hidden)
        for c in ranks:
            c.ep_exchange_connect_local(ranks)
        ranks[0].ep_exchange_set_wait_limit(3000)
        got = torch.full_like(x, float("nan"))
        ranks[0].cmd_routed_moe_layer_ep(x[0], got, dwr, dbias, table, shared_dev.data_ptr(), inter, shared_owner=1)
        torch.cuda.synchronize()
        assert ranks[0].device_status() == 0x5503
        assert ranks[0].device_status() == 0  # reading clears it
        # the same context computes an undivided layer afterwards, equal to another context's
        want, again = torch.empty_like(x), torch.empty_like(x)
        ctx.set_accumulation(L.ACCUM_PAIRWISE)
        ctx.cmd_routed_moe_layer(x[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, want)
        ranks[0].cmd_routed_moe_layer(x[0], dwr, dbias, table, shared_dev.data_ptr(), L.PAGE_MXFP4, inter, again)
        torch.cuda.synchronize()
        assert torch.equal(again, want) and ranks[0].device_status() == 0
    finally:
        for c in ranks:
            c.close()


def test_sharded_head_on_one_rank_and_by_row_shards(ctx, oracle):
    """ep.sharded_head with one rank, and the row shards of two ranks computed in turn: the pieces are
    the full logits bit for bit, the combined greedy token is the oracle's."""
    from colormlm_b200 import ep

    g = synth.rng(732)
    vocab, hidden = 3001, 2048
    w = synth.head_weight_bf16(g, vocab, hidden)
    x = synth.activations(g, 1, hidden)
    dw, dx = dev(w.view(np.int16)), dev(x)
    logits, token = ep.sharded_head(ctx, dx[0], dw, vocab, 0, 1)
    full = logits.cpu().numpy()
    ref = oracle.head_logits(x[0], w)
    assert np.allclose(full, ref, rtol=2e-7, atol=3e-7)  # tolerance of tests/test_final_head.py:68-70
    assert token == oracle.greedy_argmax(full)
    pieces = []
    best = []
    for rank in range(2):
        r0, r1 = ep.head_rows(rank, 2, vocab)
        local = torch.empty(r1 - r0, dtype=torch.float32, device="cuda")
        ctx.cmd_head_logits(dx[0], dw[r0:r1], local)
        torch.cuda.synchronize()
        pieces.append(local.cpu().numpy())
        a = int(np.argmax(pieces[-1]))
        best.append((float(pieces[-1][a]), r0 + a))
    assert np.array_equal(np.concatenate(pieces).view(np.uint32), full.view(np.uint32))
    assert max(best, key=lambda p: (p[0], -p[1]))[1] == token


def test_head_logits_and_argmax(ctx, oracle, golden):
    g = synth.rng(99)
    vocab, hidden = 5003, 4096
    w = synth.head_weight_bf16(g, vocab, hidden)
    x = synth.activations(g, 3, hidden)
    dw, dx = dev(w.view(np.int16)), dev(x)
    logits = torch.empty((3, vocab), dtype=torch.float32, device="cuda")
    ctx.cmd_head_logits(dx, dw, logits)
    res = torch.empty(1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    for t in range(3):
        ref = oracle.head_logits(x[t], w)
        # local_s14_primitives/tests/test_final_head.py:68-70 accepts rtol 2e-7 / atol 3e-7
        np.testing.assert_allclose(logits[t].cpu().numpy(), ref, rtol=2e-7, atol=3e-7)
        ctx.cmd_greedy_argmax(logits[t], res)
        torch.cuda.synchronize()
        assert int(res.item()) == oracle.greedy_argmax(ref)
    # a vocabulary shard: rows [1000, 3000) written at their place in the full logits
    part = torch.zeros(vocab, dtype=torch.float32, device="cuda")
    ctx.cmd_head_logits(dx[0], dw[1000:3000], part[1000:3000], n_rows=2000)
    torch.cuda.synchronize()
    assert torch.equal(part[1000:3000], logits[0, 1000:3000]) and float(part[:1000].abs().sum()) == 0.0
    # ties -> lowest id, NaN -> -1
    tie = torch.tensor([1.0, 5.0, 5.0, 2.0], device="cuda")
    ctx.cmd_greedy_argmax(tie, res)
    torch.cuda.synchronize()
    assert int(res.item()) == 1
    tie[3] = float("nan")
    ctx.cmd_greedy_argmax(tie, res)
    torch.cuda.synchronize()
    assert int(res.item()) == -1
    # the reference's seed-731 head fixture
    hx, hw = golden["hd_x"], golden["hd_w"]
    out = torch.empty((1, 13), dtype=torch.float32, device="cuda")
    for b in range(2):
        for s in range(3):
            ctx.cmd_head_logits(dev(hx[b, s]), dev(hw.view(np.int16)), out)
            torch.cuda.synchronize()
            np.testing.assert_allclose(out.cpu().numpy()[0], golden["hd_logits"][b, s], rtol=2e-7, atol=3e-7)


def test_pool_upload_publish_compute_release(ctx, oracle):
    """The page transaction end to end: route -> reserve -> pinned async upload on the copy
    stream -> transfer fence -> publish -> layer on the slot addresses -> release."""
    hidden, inter = 1024, 1024
    lay = ExpertPageLayout(hidden, inter)
    slot_bytes = lay.page_bytes
    g, pages, shared = make_layer(555, hidden, inter, 256, L.PAGE_MXFP4)
    routed_pool, shared_pool = VramPool(ctx, 8, slot_bytes), VramPool(ctx, 1, slot_bytes)
    mp = S14MoePages(routed_pool, shared_pool, min_routed_bytes=slot_bytes, min_shared_bytes=slot_bytes)
    staging = torch.empty((7, slot_bytes), dtype=torch.uint8).pin_memory()
    x = synth.activations(g, 1, hidden)
    dx = dev(x)
    y = torch.empty_like(dx)

    def step(ids, weights):
        rd = RouteDecision(layer=42, kind=1, expert_ids=ids, weights=weights)
        batch = mp.begin_after_official_route(rd)
        missing = batch.missing()
        for i, (res, is_shared) in enumerate(missing):
            src = shared if is_shared else pages[res.key.slot]
            staging[i].copy_(torch.from_numpy(lay.to_expert_page(src)))  # reordered once, at load time
            (shared_pool if is_shared else routed_pool).upload_page_async(res, staging[i].data_ptr(), slot_bytes)
        routed_pool.transfer_fence()
        routed_pool.wait_transfer_fence()
        lease = mp.publish_after_transfer_fence(batch)
        tr = TokenRoute(lease.expert_ids(), lease.route_weights(),
                        [routed_pool.slot_ptr(b.slot) for b in lease.routed_bindings()])
        ctx.cmd_moe_layer(dx, y, [tr], shared_pool.slot_ptr(lease.shared_binding().slot), L.PAGE_MXFP4, hidden, inter)
        torch.cuda.synchronize()
        mp.release_after_compute_fence(lease)
        return len(missing), y.cpu().numpy()[0].copy()

    ctx.set_accumulation(L.ACCUM_REFERENCE)
    w = [0.25] * 6
    n_up, out = step([126, 12, 205, 149, 227, 174], w)
    assert n_up == 7
    ref = oracle.moe_layer(x[0], [pages[i] for i in [126, 12, 205, 149, 227, 174]], np.asarray(w, np.float32),
                           shared, 0, hidden, inter)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    n_up, out2 = step([126, 12, 205, 149, 227, 174], w)  # all cached now
    assert n_up == 0 and np.array_equal(out2, out)
    n_up, out3 = step([1, 12, 3, 149, 5, 174], w)  # three misses evict the least recently used
    assert n_up == 3
    ref = oracle.moe_layer(x[0], [pages[i] for i in [1, 12, 3, 149, 5, 174]], np.asarray(w, np.float32), shared, 0,
                           hidden, inter)
    assert np.array_equal(out3.view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    # a NaN scale code in a payload is refused before upload
    from colormlm_b200.s14 import validate_ue8m0_codes
    bad = pages[9].copy()
    bad[lay.offsets["s1"] + 5] = 0xFF
    with pytest.raises(S14Error):
        validate_ue8m0_codes(bad[lay.offsets["s1"]:])


def test_moe_layer_host_buffers(ctx, oracle):
    hidden, inter = 1024, 1024
    g, pages, shared = make_layer(808, hidden, inter, 7, L.PAGE_MXFP4)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    x = synth.activations(g, 2, hidden)
    y = np.empty_like(x)
    w = np.asarray([0.3, 0.2, 0.2, 0.1, 0.1, 0.1], np.float32)
    routes = [TokenRoute([0, 1, 2, 3, 4, 5], w, [p.data_ptr() for p in pages_dev[:6]]),
              TokenRoute([5, 4, 3, 2, 1, 6], w, [pages_dev[i].data_ptr() for i in [5, 4, 3, 2, 1, 6]])]
    torch.cuda.synchronize()
    ctx.set_accumulation(L.ACCUM_REFERENCE)
    before = ctx.launch_count
    ctx.moe_layer_host(x, y, routes, shared_dev.data_ptr(), L.PAGE_MXFP4, hidden, inter)
    assert ctx.launch_count - before == 3  # reference order: up, down, mix
    for t, ids in enumerate(([0, 1, 2, 3, 4, 5], [5, 4, 3, 2, 1, 6])):
        ref = oracle.moe_layer(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
        assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32))
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    assert ctx.device_status() == 0
