"""The oracle's official expert arithmetic (oracle/s14_oracle.c: s14o_act_quant,
s14o_official_moe_layer) against vectors made by the reference's own Python code
(tests/golden/make_golden.py): ``_activation_quant`` (l42_real_reference/l42_reference.py:389-403) and
``finish_layer`` (s14_first_real_token/executor.py:712-743) run on synthetic pages."""
import hashlib

import numpy as np

from colormlm_b200 import synth


def _digest(*arrays) -> bytes:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.digest()


def official_fixture(golden):
    """The pages and tokens of the golden file's official layer, rebuilt from their seed."""
    hidden, inter = 4096, 512
    g = synth.rng(1012)
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(7)]
    page8 = synth.fp8_expert_page(g, hidden, inter)
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(synth.activations(g, 2, hidden)))
    assert _digest(*pages, page8, x) == golden["of_inputs_sha256"].tobytes()
    return hidden, inter, pages, page8, x


def test_act_quant_equals_the_references(golden, oracle):
    """Rows with amax below the 1e-4 floor, a large row, an all-zero group, amax / 448 an exact power of two,
    a BF16-valued row: bit for bit."""
    x, want = golden["aq_x"], golden["aq_y"]
    got = oracle.act_quant(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # every value is an E4M3FN value times a power of two: four significant bits
    m, _ = np.frexp(got[got != 0])
    assert np.all(m * 16 == np.round(m * 16))
    # and a value that is representable stays what it is
    assert np.array_equal(oracle.act_quant(np.full(128, 0.4375, np.float32)), np.full(128, 0.4375, np.float32))


def test_official_layer_equals_the_references_finish_layer(golden, oracle):
    """moe_branch of two tokens, six routed MXFP4 experts and an MXFP4 or FP8 shared expert, 4096 x 512:
    the reference's float32 BLAS products and the oracle's exact sums give the same BF16 values
    throughout."""
    hidden, inter, pages, page8, x = official_fixture(golden)
    for name, shared, kind in (("mxfp4_shared", pages[6], 0), ("fp8_shared", page8, 1)):
        for t in range(2):
            got = oracle.official_moe_layer(x[t], pages[:6], golden["of_w"][t], shared, kind, hidden, inter)
            want = golden["of_branch_" + name][t]
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (name, t)
            assert np.array_equal(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(got)), got)  # BF16 values


def test_official_layer_differs_from_the_f32_semantics(golden, oracle):
    """The two arithmetics are different functions (a guard against a switch that does nothing)."""
    hidden, inter, pages, _, x = official_fixture(golden)
    off = oracle.official_moe_layer(x[0], pages[:6], golden["of_w"][0], pages[6], 0, hidden, inter)
    f32 = oracle.moe_layer_acc64(x[0], pages[:6], golden["of_w"][0], pages[6], 0, hidden, inter)
    rel = np.abs(off - f32).max() / np.abs(f32).max()
    assert 1e-4 < rel < 0.2, rel
