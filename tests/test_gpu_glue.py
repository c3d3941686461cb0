"""The steps on either side of the MoE inside one layer on the GPU (hyper-connection reduce / expand,
RMSNorm, the head's reduce, the hash route) against the CPU oracle on the same seeded inputs, and
against the vectors the reference's Python code produced (tests/golden/make_golden.py).

GPU and oracle use the same arithmetic - long sums in double rounded to F32 once, exp in double, F32
operations in the Python code's order - and differ only where a double sum, taken in another order,
rounds to the neighbouring F32 value: coefficients are compared within 2 ulps, streams must be
bit-equal on 99.9 % of the elements and within 2 ulps (F32) / one BF16 ulp on the rest."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from colormlm_b200 import _lib as L
from colormlm_b200 import synth
from colormlm_b200.s14 import S14Context, S14Error

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("cuda_lib")]


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = S14Context(0)
    yield c
    c.close()


def dev(a, bf16=False):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(torch.bfloat16) if bf16 else t


def bits16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def f32_of_bits(a):
    return (np.asarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def close_streams(got, want, bf16):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert (got == want).mean() >= 0.999, (got == want).mean()
    tol = 2.0 ** -7 if bf16 else 2.0 ** -22
    assert np.abs(got - want).max() <= tol * np.abs(want).max()


def close_coeff(got, want):
    np.testing.assert_allclose(np.asarray(got), np.asarray(want), rtol=3e-7, atol=3e-7)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("n_tokens,hidden", [(1, 4096), (5, 4096), (3, 1024)])
def test_hc_pre_post_and_norm_against_the_oracle(ctx, oracle, bf16, n_tokens, hidden):
    g = synth.rng(3100 + n_tokens + hidden)
    fn, scale, base = synth.hc_params(g, hidden)
    xs, branch = synth.hc_streams(g, n_tokens, hidden), synth.activations(g, n_tokens, hidden)
    nw = g.uniform(0.5, 1.5, size=hidden).astype(np.float32)
    dx, db = dev(xs, bf16), dev(branch, bf16)
    xin = bits16(dx) if bf16 else xs
    bin_ = bits16(db) if bf16 else branch
    red = torch.empty((n_tokens, hidden), dtype=dx.dtype, device="cuda")
    post = torch.empty((n_tokens, 4), dtype=torch.float32, device="cuda")
    comb = torch.empty((n_tokens, 4, 4), dtype=torch.float32, device="cuda")
    ctx.cmd_hc_pre(dx, dev(fn), dev(scale), dev(base), red, post, comb)
    merged = torch.empty_like(dx)
    ctx.cmd_hc_post(db, dx, post, comb, merged)
    normed = torch.empty_like(red)
    ctx.cmd_rms_norm(red, dev(nw), normed)
    torch.cuda.synchronize()
    r_ref, p_ref, c_ref = oracle.hc_pre(xin, fn, scale, base, dtype=int(bf16))
    close_coeff(post.cpu().numpy(), p_ref)
    close_coeff(comb.cpu().numpy(), c_ref)
    as_f32 = (lambda t: f32_of_bits(bits16(t))) if bf16 else (lambda t: t.cpu().numpy())
    ref_f32 = (lambda a: f32_of_bits(a)) if bf16 else (lambda a: a)
    close_streams(as_f32(red), ref_f32(r_ref), bf16)
    # expand and norm from the GPU's own coefficients and reduce: the same inputs on both sides, so the same bits
    m_ref = oracle.hc_post(bin_, xin, post.cpu().numpy(), comb.cpu().numpy(), dtype=int(bf16))
    assert np.array_equal(as_f32(merged), ref_f32(m_ref))
    n_ref = oracle.rms_norm(bits16(red) if bf16 else red.cpu().numpy(), nw, dtype=int(bf16))
    close_streams(as_f32(normed), ref_f32(n_ref), bf16)


def test_golden_vectors_of_the_reference_on_gpu(ctx, golden):
    """The seeded streams of the model's size, against what the reference's Python code produced."""
    g = synth.rng(1005)
    fn, scale, base = synth.hc_params(g, 4096)
    xs, branch = synth.hc_streams(g, 3, 4096), synth.activations(g, 3, 4096)
    nw = g.uniform(0.5, 1.5, size=4096).astype(np.float32)
    for name, bf16 in (("f32", False), ("bf16", True)):
        dx, db = dev(xs, bf16), dev(branch, bf16)
        red = torch.empty((3, 4096), dtype=dx.dtype, device="cuda")
        post = torch.empty((3, 4), dtype=torch.float32, device="cuda")
        comb = torch.empty((3, 4, 4), dtype=torch.float32, device="cuda")
        merged, normed = torch.empty_like(dx), torch.empty_like(red)
        ctx.cmd_hc_pre(dx, dev(fn), dev(scale), dev(base), red, post, comb)
        ctx.cmd_hc_post(db, dx, post, comb, merged)
        ctx.cmd_rms_norm(red, dev(nw), normed)
        torch.cuda.synchronize()
        # the reference's 16 384-term F32 dot products carry their own summation noise (tests/test_oracle_hc.py)
        np.testing.assert_allclose(post.cpu().numpy(), golden[f"hc_{name}_post"], rtol=0, atol=5e-6)
        np.testing.assert_allclose(comb.cpu().numpy(), golden[f"hc_{name}_comb"], rtol=0, atol=5e-6)
        for got, want in ((red, golden[f"hc_{name}_reduced"]), (merged, golden[f"hc_{name}_merged"]),
                          (normed, golden[f"hc_{name}_normed"])):
            got = got.float().cpu().numpy()
            tol = 2.0 ** -7 if bf16 else 1e-5
            assert np.abs(got - want).max() <= tol * np.abs(want).max()
            if bf16:
                assert (got == want).mean() >= 0.995


def test_head_reduce_on_the_references_fixture(ctx, oracle, golden):
    # tests/test_final_head.py:22-46: BF16 streams [6, 4, 8] -> not a multiple of 256: the oracle covers that size;
    # the GPU takes the model's size
    g = synth.rng(3200)
    fn, scale, base = synth.hc_params(g, 4096, head=True)
    xs = synth.hc_streams(g, 4, 4096)
    for bf16 in (False, True):
        dx = dev(xs, bf16)
        red = torch.empty((4, 4096), dtype=dx.dtype, device="cuda")
        pre = torch.empty((4, 4), dtype=torch.float32, device="cuda")
        ctx.cmd_hc_head_reduce(dx, dev(fn), dev(scale), dev(base), red, pre)
        torch.cuda.synchronize()
        r_ref, p_ref = oracle.hc_head_reduce(bits16(dx) if bf16 else xs, fn, scale, base, dtype=int(bf16))
        close_coeff(pre.cpu().numpy(), p_ref)
        close_streams(red.float().cpu().numpy(), f32_of_bits(r_ref) if bf16 else r_ref, bf16)


def test_hash_route(ctx, oracle, golden):
    g = synth.rng(1006)
    wr = synth.router_weight_bf16(g, 256, 1024)
    x = synth.activations(g, 3, 1024)
    tid2eid = np.stack([g.permutation(256)[:6] for _ in range(3)]).astype(np.int64)
    ids = torch.empty((3, 6), dtype=torch.int32, device="cuda")
    wts = torch.empty((3, 6), dtype=torch.float32, device="cuda")
    ctx.cmd_router_hash(dev(x), dev(wr.view(np.int16)), dev(tid2eid), ids, wts, score_fn=L.SCORE_SQRT_SOFTPLUS, route_scale=1.5)
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy(), tid2eid.astype(np.int32))
    np.testing.assert_allclose(wts.cpu().numpy(), golden["rh_w"], rtol=2e-6, atol=0)
    for t in range(3):
        _, w = oracle.router_hash(x[t], wr, tid2eid[t], score_fn=1, route_scale=1.5)
        assert np.array_equal(wts[t].cpu().numpy().view(np.uint32), w.view(np.uint32))


def test_glue_rejects_what_it_cannot_run(ctx):
    x = torch.zeros((2, 4, 1024), device="cuda")
    fn, sc, ba = torch.zeros((24, 4096), device="cuda"), torch.ones(3, device="cuda"), torch.zeros(24, device="cuda")
    red, post, comb = torch.empty((2, 1024), device="cuda"), torch.empty((2, 4), device="cuda"), torch.empty((2, 4, 4), device="cuda")
    ctx.cmd_hc_pre(x, fn, sc, ba, red, post, comb)
    with pytest.raises(S14Error):
        ctx.cmd_hc_pre(x, fn, sc, ba, red, post, comb, iters=0)
    with pytest.raises(S14Error):
        ctx.cmd_hc_pre(torch.zeros((2, 3, 1024), device="cuda"), fn, sc, ba, red, post, comb)
    with pytest.raises(S14Error):
        ctx.cmd_hc_pre(torch.zeros((2, 4, 1000), device="cuda"), fn, sc, ba, red, post, comb)
    with pytest.raises(S14Error):
        ctx.cmd_hc_pre(x.to(torch.float16), fn, sc, ba, red, post, comb)
    with pytest.raises(S14Error):
        ctx.cmd_rms_norm(red, torch.ones(1024, device="cuda"), red, eps=0.0)
    torch.cuda.synchronize()


def test_exec_hc_head_norm_full_logits(ctx, oracle, golden):
    """The executor's final step (runner.rs:86-118, final_head.py:152-191) as one call, against the oracle's
    composition and against native_final_logits' own output."""
    g = synth.rng(1007)
    fn, sc, ba = synth.hc_params(g, 1024, head=True)
    x = synth.hc_streams(g, 2, 1024)
    nw = g.uniform(0.5, 1.5, size=1024).astype(np.float32)
    hw = synth.head_weight_bf16(g, 768, 1024)
    d_hw = dev(hw.view(np.int16))
    for t in range(2):
        state = dev(x[t:t + 1], bf16=True)
        logits = torch.empty(768, dtype=torch.float32, device="cuda")
        ctx.exec_hc_head_norm_full_logits(state, dev(fn), dev(sc), dev(ba), dev(nw), d_hw, logits)
        torch.cuda.synchronize()
        red, _ = oracle.hc_head_reduce(bits16(state), fn, sc, ba, dtype=1)
        normed = oracle.rms_norm(red, nw, dtype=1)
        want = oracle.head_logits(f32_of_bits(normed[0]), hw)
        got = logits.cpu().numpy()
        # the head kernel carries 8 products in F32 before its double sum: a few ulps against the double-accumulated oracle
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()
        assert np.abs(got - golden["nf_logits"][t]).max() <= 2e-3 * np.abs(golden["nf_logits"][t]).max()


def test_exec_routed_and_shared_moe_then_hc_post(ctx, oracle):
    """The executor's MoE step as one call: BF16 FFN input -> experts -> BF16 branch -> hc_post over the
    post-attention state, against the oracle's composition, bit for bit."""
    from colormlm_b200.s14 import TokenRoute
    from .test_gpu_parity import dev_page, make_layer

    hidden, inter = 2048, 1024
    g, pages, shared = make_layer(3300, hidden, inter, 8, L.PAGE_MXFP4)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    ffn_in = dev(synth.activations(g, 1, hidden)[0], bf16=True)
    residual = dev(synth.hc_streams(g, 1, hidden)[0], bf16=True)
    post_np = g.uniform(0.2, 1.8, size=4).astype(np.float32)
    comb_np = g.uniform(0.05, 0.6, size=(4, 4)).astype(np.float32)
    ids = [5, 1, 7, 0, 3, 6]
    w = np.asarray([0.4, 0.3, 0.25, 0.2, 0.2, 0.15], np.float32)
    route = TokenRoute(ids, w, [pages_dev[i].data_ptr() for i in ids])
    state_out = torch.empty((4, hidden), dtype=torch.bfloat16, device="cuda")
    branch_out = torch.empty(hidden, dtype=torch.bfloat16, device="cuda")
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    ctx.exec_routed_and_shared_moe_then_hc_post(ffn_in, residual, dev(post_np), dev(comb_np), route, shared_dev.data_ptr(),
                                                L.PAGE_MXFP4, inter, state_out, branch_out)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    y = oracle.moe_layer_acc64(f32_of_bits(bits16(ffn_in)), [pages[i] for i in ids], w, shared, 0, hidden, inter)
    branch_ref = synth.f32_to_bf16_bits(y)
    assert np.array_equal(bits16(branch_out), branch_ref)
    merged = oracle.hc_post(branch_ref[None], bits16(residual)[None], post_np[None], comb_np[None], dtype=1)
    assert np.array_equal(bits16(state_out), merged[0])
