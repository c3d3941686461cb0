"""Pins the CPU oracle against the reference's own known-answer vectors and against
outputs of the reference's Python code (tests/golden/s14_golden.npz).  No GPU."""
import hashlib

import numpy as np
import pytest

from colormlm_b200 import synth
from colormlm_b200.pages import ExpertPageLayout


def _digest(*arrays) -> bytes:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.digest()


def test_e2m1_all_codes_and_nibble_order(oracle, golden):
    # local_s14_primitives/tests/test_primitives.py:37-46
    table = np.array([oracle.e2m1(c) for c in range(16)], np.float32)
    assert np.array_equal(table, golden["e2m1_table"])
    assert np.signbit(table[8]) and table[8] == 0.0
    # bytes 0x21, 0xF7 hold (.5, 1, 6, -6): low nibble is the even k
    packed = np.zeros((1, 64), np.uint8)
    packed[0, :2] = [0x21, 0xF7]
    scale = np.full((1, 4), 127, np.uint8)
    got = []
    for k in range(4):
        x = np.zeros(128, np.float32)
        x[k] = 1.0
        got.append(oracle.mxfp4_matvec(x, packed, scale, 1, 128)[0])
    assert got == [0.5, 1.0, 6.0, -6.0]


def test_ue8m0_edges(oracle, golden):
    # test_primitives.py:49-55 (0xFF is rejected on the host before any decode)
    table = np.array([oracle.ue8m0(c) for c in range(255)], np.float32)
    assert np.array_equal(table, golden["ue8m0_table"])
    for code in (0, 1, 120, 121, 126, 127, 128, 254):
        assert oracle.ue8m0(code) == np.float32(2.0) ** (code - 127)


def test_e4m3_all_codes(oracle, golden):
    # test_primitives.py:86-94
    table = np.array([oracle.e4m3fn(int(c)) for c in golden["e4m3_codes"]], np.float32)
    assert np.array_equal(table, golden["e4m3_table"])
    known = {0x00: 0.0, 0x01: 2.0 ** -9, 0x07: 7 * 2.0 ** -9, 0x08: 2.0 ** -6, 0x38: 1.0,
             0x7E: 448.0, 0xB8: -1.0, 0xFE: -448.0}
    for code, value in known.items():
        assert oracle.e4m3fn(code) == value
    assert np.signbit(np.float32(oracle.e4m3fn(0x80)))


def test_reference_mxfp4_fixture(oracle, golden):
    # test_primitives.py:58-72; the reference accepts rtol = atol = 2e-6 there
    w, s, x = golden["fx_packed"], golden["fx_scales"], golden["fx_x"]
    for t in range(2):
        y = oracle.mxfp4_matvec(x[t], w, s, 3, 128)
        np.testing.assert_allclose(y, golden["fx_y_f32"][t], rtol=2e-6, atol=2e-6)
        y64 = oracle.mxfp4_matvec_f64(x[t], w, s, 3, 128)
        np.testing.assert_allclose(y64, golden["fx_y_f64"][t], rtol=1e-13, atol=1e-13)


def test_seeded_mxfp4_matvec(oracle, golden):
    g = synth.rng(1001)
    n, k = 96, 1024
    w, s, x = synth.mxfp4_codes(g, n, k), synth.mxfp4_scales(g, n, k), synth.activations(g, 2, k)
    assert _digest(w, s, x) == golden["mx_inputs_sha256"].tobytes()
    for t in range(2):
        y64 = oracle.mxfp4_matvec_f64(x[t], w, s, n, k)
        np.testing.assert_allclose(y64, golden["mx_y_f64"][t], rtol=1e-12, atol=1e-12)
        # F32, two different summation orders: both within F32 noise of the F64 value
        y = oracle.mxfp4_matvec(x[t], w, s, n, k)
        scale = np.abs(golden["mx_y_f64"][t]).max()
        assert np.abs(y - golden["mx_y_f64"][t]).max() < 2e-6 * scale
        assert np.abs(golden["mx_y_f32"][t] - golden["mx_y_f64"][t]).max() < 2e-6 * scale


def test_reference_fp8_fixture_ragged(oracle, golden):
    # test_primitives.py:97-112: 129 x 130, partial blocks on both axes.  Terms reach
    # 448 * 2 while results are O(1..1000), so F32 results of different summation orders
    # are compared with a bound scaled by the row's sum of |terms| (F32 eps = 6e-8 per add).
    w, s, x = golden["f8_w"], golden["f8_s"], golden["f8_x"]
    for t in range(2):
        y64 = oracle.fp8_matvec_f64(x[t], w, s, 129, 130)
        np.testing.assert_allclose(y64, golden["f8_y_f64"][t], rtol=1e-12, atol=1e-12)
        abs_terms = oracle.fp8_matvec_f64(np.abs(x[t]), w & 0x7F, s, 129, 130)
        bound = 1e-6 * abs_terms
        assert (np.abs(oracle.fp8_matvec(x[t], w, s, 129, 130) - y64) <= bound).all()
        assert (np.abs(golden["f8_y"][t] - y64) <= bound).all()
        ysf = oracle.fp8_matvec(x[t], w, golden["f8_sf"], 129, 130)
        ysf64 = oracle.fp8_matvec_f64(x[t], w, golden["f8_sf"], 129, 130)
        abs_sf = oracle.fp8_matvec_f64(np.abs(x[t]), w & 0x7F, golden["f8_sf"], 129, 130)
        assert (np.abs(ysf - ysf64) <= 1e-6 * abs_sf).all()
        assert (np.abs(golden["f8_y_sf"][t] - ysf64) <= 1e-6 * abs_sf).all()


def test_seeded_fp8_projection(oracle, golden):
    g = synth.rng(1002)
    n, k = 256, 512
    w = synth.e4m3_codes(g, n, k)
    s = synth.fp8_block_scales_ue8m0(g, n, k)
    sf = synth.fp8_block_scales_f32(g, n, k)
    x = synth.activations(g, 4, k)
    assert _digest(w, s, sf, x) == golden["p8_inputs_sha256"].tobytes()
    assert not np.isin(w, (0x7F, 0xFF)).any()
    for t in range(4):
        for scale, key in ((s, "p8_y"), (sf, "p8_y_sf")):
            ref = golden[key][t]
            tol = 4e-6 * np.abs(ref).max()
            assert np.abs(oracle.fp8_matvec(x[t], w, scale, n, k) - ref).max() < tol
            assert np.abs(oracle.fp8_matvec_f64(x[t], w, scale, n, k) - ref).max() < tol


def _layer_inputs(golden):
    hidden, inter = 1024, 1024
    g = synth.rng(1003)
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(7)]
    page8 = synth.fp8_expert_page(g, hidden, inter)
    x = synth.activations(g, 1, hidden)[0]
    assert _digest(*pages, page8, x) == golden["ly_inputs_sha256"].tobytes()
    return hidden, inter, pages, page8, x, golden["ly_w"]


def test_expert_chain_and_layer_against_python_reference(oracle, golden):
    hidden, inter, pages, page8, x, w = _layer_inputs(golden)
    assert ExpertPageLayout(hidden, inter, 0).page_bytes == pages[0].size
    # chain: down output of expert 0 (F64-accumulated Python reference)
    y, down = oracle.expert_chain_mxfp4(x, pages[0], hidden, inter, 0.3)
    ref = golden["ly_chain0_down"]
    scale = np.abs(ref).max()
    assert np.abs(down - ref).max() < 4e-6 * scale
    assert np.array_equal(y, np.float32(0.3) * down)
    # layer, MXFP4 shared and FP8 shared; F64-carried oracle is tight, F32 oracle within F32 noise
    for kind, page, key in ((0, pages[6], "ly_y_mxfp4_shared"), (1, page8, "ly_y_fp8_shared")):
        ref = golden[key]
        scale = np.abs(ref).max()
        y64 = oracle.moe_layer_acc64(x, pages[:6], w, page, kind, hidden, inter)
        assert np.abs(y64 - ref).max() < 2e-6 * scale
        y32 = oracle.moe_layer(x, pages[:6], w, page, kind, hidden, inter)
        assert np.abs(y32 - ref).max() < 1e-5 * scale


def test_swiglu_limit_is_one_sided_on_the_gate(oracle):
    # examples/s14_vulkan_numeric.rs:1543-1556: gate min(g, 10) only, up clamp(-10, 10)
    gate = np.array([-20.0, 20.0, 10.0, 0.5, -0.5], np.float32)
    up = np.array([3.0, 30.0, -30.0, 2.0, 2.0], np.float32)
    y = oracle.swiglu_limit(gate, up)
    silu = lambda v: np.float32(v) / (np.float32(1.0) + np.exp(np.float32(-v), dtype=np.float32))
    expect = np.array([silu(-20.0) * 3.0, silu(10.0) * 10.0, silu(10.0) * -10.0, silu(0.5) * 2.0,
                       silu(-0.5) * 2.0], np.float32)
    np.testing.assert_allclose(y, expect, rtol=3e-7)
    assert y[0] != 0.0 and abs(y[0] - silu(-10.0) * 3.0) > 1e-4  # -20 is NOT clamped to -10


def test_swiglu_exp_definition_vs_libm(oracle):
    """The oracle rounds a double exp once; libm's expf may differ in the last bit for a few
    arguments per 10^5, which moves the SwiGLU value by at most one ulp."""
    g = synth.rng(8)
    gate = (g.standard_normal(400_000) * 6.2).astype(np.float32)
    up = (g.standard_normal(400_000) * 6.2).astype(np.float32)
    a, b = oracle.swiglu_limit(gate, up), oracle.swiglu_limit_libm(gate, up)
    differ = np.nonzero(a != b)[0]
    assert differ.size < 400  # < 1e-3 of the arguments
    if differ.size:
        ulp = np.spacing(np.abs(a[differ]))
        assert (np.abs(a[differ] - b[differ]) <= 2 * ulp).all()


def test_router_against_torch_reference(oracle, golden):
    g = synth.rng(1004)
    wr, bias, x = synth.router_weight_bf16(g, 256, 1024), synth.router_bias(g, 256), synth.activations(g, 4, 1024)
    assert _digest(wr, bias, x) == golden["rt_inputs_sha256"].tobytes()
    for fn, name in ((0, "sig"), (1, "ssp")):
        for t in range(4):
            ids, w, scores, select = oracle.router(x[t], wr, bias, score_fn=fn, top_k=6, route_scale=1.5)
            assert golden[f"rt_{name}_gap"][t] > 1e-6  # the fixture has no near tie
            assert np.array_equal(ids, golden[f"rt_{name}_ids"][t])
            np.testing.assert_allclose(w, golden[f"rt_{name}_w"][t], rtol=2e-6, atol=0)
            assert abs(float(w.sum()) - 1.5) < 1e-6
            assert len(set(ids.tolist())) == 6


def test_router_tie_break_lowest_index(oracle):
    wr = np.zeros((8, 256), np.uint16)  # all logits 0 -> all scores equal
    ids, w, _, _ = oracle.router(np.ones(256, np.float32), wr, None, score_fn=0, top_k=6)
    assert ids.tolist() == [0, 1, 2, 3, 4, 5]
    np.testing.assert_allclose(w, np.full(6, 1 / 6, np.float32), rtol=1e-6)


def test_head_logits_and_argmax(oracle, golden):
    # local_s14_primitives/tests/test_final_head.py:57-72 (rtol 2e-7, atol 3e-7 there)
    x, w = golden["hd_x"], golden["hd_w"]
    for b in range(2):
        for s in range(3):
            np.testing.assert_allclose(oracle.head_logits(x[b, s], w), golden["hd_logits"][b, s],
                                       rtol=2e-7, atol=3e-7)
    assert oracle.greedy_argmax(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1
    assert oracle.greedy_argmax(np.array([1.0, np.nan, 3.0], np.float32)) == -1


def test_error_stats(oracle):
    # examples/s14_vulkan_numeric.rs:1745-1771
    s = oracle.error_stats(np.array([1.0, 2.0, 3.5], np.float32), np.array([1.0, 2.5, 3.0], np.float32))
    assert s["max_abs"] == 0.5 and abs(s["mean_abs"] - 1 / 3) < 1e-12
    assert abs(s["rmse"] - np.sqrt(0.5 / 3)) < 1e-12 and abs(s["max_rel"] - 0.2) < 1e-7
    with pytest.raises(ValueError):
        oracle.error_stats(np.array([np.inf], np.float32), np.array([1.0], np.float32))
