"""Pins the CPU oracle's hyper-connection reduce / expand, RMSNorm, head reduce and hash route
against outputs of the reference's Python code (local_s14_primitives/hc.py:19-148,
final_head.py:43-110, s14_first_real_token/executor.py:638-668) on the reference's own fixtures and
on seeded streams of the model's size (tests/golden/make_golden.py).  No GPU.

Tolerance: the Python code leaves the F32 summation order of F.linear / mean and the exp to torch's
CPU kernels; the oracle accumulates the long sums in double.  With 16 384-term F32 dot products on
the reference's side, the mixing coefficients (pre, post, comb; O(1)) agree within 5e-6 absolute at
the model's size (1e-6 on the small fixtures), F32 streams within 1e-5 of the largest output, BF16
streams within one BF16 ulp on at most 0.2 % of the elements (a rounding that falls the other way)."""
import hashlib

import numpy as np

from colormlm_b200 import synth


def _digest(*arrays) -> bytes:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.digest()


def _bf16(a):
    return (np.asarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def test_split_sinkhorn_on_the_references_fixture(oracle, golden):
    # tests/test_primitives.py:126-132: logits from -1000 to 1000, 20 Sinkhorn rounds
    # (the fixture's linspace inputs are torch's, stored with the outputs)
    scale = np.asarray([0.5, -0.25, 0.01], np.float32)
    pre, post, comb = oracle.hc_split_sinkhorn(golden["hcf_mixes"], scale, golden["hcf_base"])
    np.testing.assert_allclose(pre, golden["hcf_pre"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(post, golden["hcf_post"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(comb, golden["hcf_comb"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(comb.sum(axis=0), np.ones(4), rtol=2e-5, atol=2e-5)   # the reference's own check


def test_pre_and_post_on_the_references_fixture(oracle, golden):
    # tests/test_primitives.py:134-141
    x, fn = golden["hcf_x"], golden["hcf_fn"]
    scale, base = np.asarray([0.5, -0.25, 0.01], np.float32), golden["hcf_base"]
    red, post, comb = oracle.hc_pre(x, fn, scale, base)
    np.testing.assert_allclose(post[0], golden["hcf_post2"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(comb[0], golden["hcf_comb2"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(red[0], golden["hcf_reduced"], rtol=0, atol=2e-6)
    merged = oracle.hc_post(golden["hcf_branch"], x, golden["hcf_post2"][None], golden["hcf_comb2"][None])
    np.testing.assert_allclose(merged[0], golden["hcf_merged"], rtol=0, atol=5e-7)


def test_head_reduce_and_rms_norm_on_the_seed_731_fixture(oracle, golden):
    # tests/test_final_head.py:22-58: BF16 streams [2, 3, 4, 8]
    x = golden["hh_x"]
    red, pre = oracle.hc_head_reduce(x, golden["hh_fn"], np.asarray([0.7], np.float32), golden["hh_base"], dtype=1)
    np.testing.assert_allclose(pre, golden["hh_pre"], rtol=0, atol=2e-7)
    assert np.abs(_bf16(red) - _bf16(golden["hh_reduced"])).max() <= 2.0 ** -7 * np.abs(_bf16(golden["hh_reduced"])).max()
    assert (red == golden["hh_reduced"]).mean() >= 0.95
    normed = oracle.rms_norm(x[:, 0], golden["hh_nw"], dtype=1)
    assert (normed == golden["hh_norm"]).mean() >= 0.95
    assert np.abs(_bf16(normed) - _bf16(golden["hh_norm"])).max() <= 2.0 ** -7 * np.abs(_bf16(golden["hh_norm"])).max()


def _model_size_inputs(golden):
    g = synth.rng(1005)
    fn, scale, base = synth.hc_params(g, 4096)
    xs = synth.hc_streams(g, 3, 4096)
    branch = synth.activations(g, 3, 4096)
    nw = g.uniform(0.5, 1.5, size=4096).astype(np.float32)
    assert _digest(fn, scale, base, xs, branch, nw) == golden["hc_inputs_sha256"].tobytes()
    return fn, scale, base, xs, branch, nw


def test_model_size_streams_f32(oracle, golden):
    fn, scale, base, xs, branch, nw = _model_size_inputs(golden)
    red, post, comb = oracle.hc_pre(xs, fn, scale, base)
    np.testing.assert_allclose(post, golden["hc_f32_post"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(comb, golden["hc_f32_comb"], rtol=0, atol=5e-6)
    assert np.abs(red - golden["hc_f32_reduced"]).max() <= 1e-5 * np.abs(golden["hc_f32_reduced"]).max()
    merged = oracle.hc_post(branch, xs, golden["hc_f32_post"], golden["hc_f32_comb"])
    assert np.array_equal(merged.view(np.uint32), golden["hc_f32_merged"].view(np.uint32))   # same coefficients: same bits
    normed = oracle.rms_norm(golden["hc_f32_reduced"], nw)
    assert np.abs(normed - golden["hc_f32_normed"]).max() <= 1e-5 * np.abs(golden["hc_f32_normed"]).max()


def test_model_size_streams_bf16(oracle, golden):
    fn, scale, base, xs, branch, nw = _model_size_inputs(golden)
    xb, bb = synth.f32_to_bf16_bits(xs), synth.f32_to_bf16_bits(branch)
    red, post, comb = oracle.hc_pre(xb, fn, scale, base, dtype=1)
    np.testing.assert_allclose(post, golden["hc_bf16_post"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(comb, golden["hc_bf16_comb"], rtol=0, atol=5e-6)
    want = golden["hc_bf16_reduced"]
    assert (_bf16(red) == want).mean() >= 0.998
    assert np.abs(_bf16(red) - want).max() <= 2.0 ** -7 * np.abs(want).max()
    merged = oracle.hc_post(bb, xb, golden["hc_bf16_post"], golden["hc_bf16_comb"], dtype=1)
    assert np.array_equal(_bf16(merged), golden["hc_bf16_merged"])
    normed = oracle.rms_norm(synth.f32_to_bf16_bits(want), nw, dtype=1)
    assert (_bf16(normed) == golden["hc_bf16_normed"]).mean() >= 0.998


def test_hash_route_weights(oracle, golden):
    g = synth.rng(1006)
    wr = synth.router_weight_bf16(g, 256, 1024)
    x = synth.activations(g, 3, 1024)
    tid2eid = np.stack([g.permutation(256)[:6] for _ in range(3)]).astype(np.int64)
    assert _digest(wr, x, tid2eid) == golden["rh_inputs_sha256"].tobytes()
    for t in range(3):
        ids, w = oracle.router_hash(x[t], wr, tid2eid[t], score_fn=1, route_scale=1.5)
        assert np.array_equal(ids, tid2eid[t].astype(np.int32))
        np.testing.assert_allclose(w, golden["rh_w"][t], rtol=2e-6, atol=0)
        assert abs(float(w.sum()) - 1.5) <= 2e-7 * 6   # executor.py:665-667 checks the sum


def test_final_path_composition(oracle, golden):
    """final_head.py:152-191 (head reduce -> RMSNorm -> BF16 head) composed from the oracle's pieces, against
    native_final_logits itself."""
    g = synth.rng(1007)
    fn, sc, ba = synth.hc_params(g, 1024, head=True)
    x = synth.hc_streams(g, 2, 1024)
    nw = g.uniform(0.5, 1.5, size=1024).astype(np.float32)
    hw = synth.head_weight_bf16(g, 768, 1024)
    assert _digest(fn, sc, ba, x, nw, hw) == golden["nf_inputs_sha256"].tobytes()
    red, pre = oracle.hc_head_reduce(synth.f32_to_bf16_bits(x), fn, sc, ba, dtype=1)
    np.testing.assert_allclose(pre, golden["nf_pre"], rtol=0, atol=2e-6)
    normed = oracle.rms_norm(red, nw, dtype=1)
    assert (_bf16(normed) == golden["nf_normalized"]).mean() >= 0.995
    for t in range(2):
        logits = oracle.head_logits(_bf16(normed[t]), hw)
        # a BF16 ulp of one normalized element moves a logit by up to 2^-8 * |x_k w_k|
        assert np.abs(logits - golden["nf_logits"][t]).max() <= 2e-3 * np.abs(golden["nf_logits"][t]).max()
        exact = oracle.head_logits(golden["nf_normalized"][t], hw)   # from the reference's own normalized vector
        np.testing.assert_allclose(exact, golden["nf_logits"][t], rtol=2e-6, atol=2e-6)
