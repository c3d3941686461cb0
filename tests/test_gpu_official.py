"""The official expert arithmetic on the grouped block path (s14_block_set_semantics): every token's y has
the bits of the oracle's official layer (oracle/s14_oracle.c s14o_official_moe_layer, pinned to the
reference's finish_layer by tests/test_oracle_official.py) and of the reference's own finish_layer output
stored in the golden file."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from colormlm_b200 import _lib as L
from colormlm_b200 import synth
from colormlm_b200.s14 import MoeBlock, S14Context, S14Error

from .test_gpu_block import random_routes, run_block
from .test_gpu_parity import dev, dev_page, make_layer
from .test_oracle_official import official_fixture

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("cuda_lib")]


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = S14Context(0)
    yield c
    c.close()


def test_official_block_equals_the_references_finish_layer(ctx, golden, oracle):
    """The golden file's two tokens (4096 x 512, routes 0..5, MXFP4 shared expert) as one block: moe_branch as
    the reference's own code computed it, bit for bit; then back to this library's arithmetic."""
    hidden, inter, pages, _, x = official_fixture(golden)
    pages_dev = [dev_page(p, hidden, inter) for p in pages]
    routes = [(list(range(6)), golden["of_w"][t]) for t in range(2)]
    blk = MoeBlock(ctx, hidden, inter, 8)
    try:
        blk.set_semantics(True)
        y = run_block(ctx, blk, x, pages_dev[:6], pages_dev[6], routes)
        want = golden["of_branch_mxfp4_shared"]
        bad = np.nonzero(y.view(np.uint32) != want.view(np.uint32))
        assert bad[0].size == 0, (bad[0].size, y[bad][:4], want[bad][:4])
        blk.set_semantics(False)
        y32 = run_block(ctx, blk, x, pages_dev[:6], pages_dev[6], routes)
        for t in range(2):
            ref = oracle.moe_layer_acc64(x[t], pages[:6], golden["of_w"][t], pages[6], 0, hidden, inter)
            assert np.array_equal(y32[t].view(np.uint32), ref.view(np.uint32))
    finally:
        blk.close()


@pytest.mark.parametrize("n_tokens", [1, 5, 13, 29])
def test_official_block_equals_the_oracle_per_token(ctx, oracle, n_tokens):
    """2048 x 1024, 12 experts, ragged routes from the host, F32 inputs that are not BF16 values: small blocks
    (chunks of two, one row tile per item) and larger ones (chunks of six, several chunks per expert), with
    and without shared expert, and y = x + moe_branch with the residual switch."""
    hidden, inter, n_experts = 2048, 1024, 12
    g, pages, shared = make_layer(2100 + n_tokens, hidden, inter, n_experts, L.PAGE_MXFP4)
    x = synth.activations(g, n_tokens, hidden)
    x[0, :128] *= np.float32(1e-6)   # a group under the floor of amax
    routes = random_routes(g, n_tokens, n_experts, ragged=True)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 32)
    try:
        blk.set_semantics(True)
        y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        y_ns = run_block(ctx, blk, x, pages_dev, None, routes)
        blk.set_residual(True)
        y_res = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        for t in range(n_tokens):
            ids, w = routes[t]
            ref = oracle.official_moe_layer(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
            bad = np.nonzero(y[t].view(np.uint32) != ref.view(np.uint32))[0]
            assert bad.size == 0, (t, bad.size, bad[:8], y[t][bad[:4]], ref[bad[:4]])
            assert np.array_equal(y_res[t].view(np.uint32), (x[t] + ref).view(np.uint32))
            ref_ns = oracle.official_moe_layer(x[t], [pages[i] for i in ids], w, None, 2, hidden, inter)
            assert np.array_equal(y_ns[t].view(np.uint32), ref_ns.view(np.uint32)), t
    finally:
        blk.close()


def test_official_routed_block_with_wide_chunks(ctx, oracle):
    """Router on the device, 44 BF16-valued tokens over 16 experts at 2048 x 1024: chunks
    of twelve tokens; ids and weights are the oracle's, y the oracle's official layer for them."""
    hidden, inter, n_experts, n_tokens = 2048, 1024, 16, 44
    g, pages, shared = make_layer(2200, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(synth.activations(g, n_tokens, hidden)))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    ids = torch.empty((n_tokens, 6), dtype=torch.int32, device="cuda")
    wts = torch.empty((n_tokens, 6), dtype=torch.float32, device="cuda")
    dx = dev(x)
    dy = torch.full_like(dx, float("nan"))
    blk = MoeBlock(ctx, hidden, inter, 48)
    try:
        blk.set_semantics(True)
        blk.cmd_routed_moe_block(dx, dev(wr), dev(bias), table, shared_dev.data_ptr(), dy, ids, wts,
                                 score_fn=L.SCORE_SQRT_SOFTPLUS, top_k=6, route_scale=1.5)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        chunks = blk.last_counts()[0]
        assert chunks < (7 * n_tokens) // 6   # wide chunks: fewer than chunks of six would give
        y = dy.cpu().numpy()
        for t in range(n_tokens):
            rid, rw, _, _ = oracle.router(x[t], wr, bias, score_fn=L.SCORE_SQRT_SOFTPLUS, top_k=6, route_scale=1.5)
            assert np.array_equal(ids[t].cpu().numpy(), rid)
            assert np.array_equal(wts[t].cpu().numpy().view(np.uint32), rw.view(np.uint32))
            ref = oracle.official_moe_layer(x[t], [pages[i] for i in rid], rw, shared, 0, hidden, inter)
            assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32)), t
    finally:
        blk.close()


def test_official_block_runs_on_one_gpu_only(ctx):
    """The expert-parallel calls refuse an official block, and a block with an exchange refuses the switch."""
    blk = MoeBlock(ctx, 1024, 1024, 8)
    try:
        blk.set_semantics(True)
        with pytest.raises(S14Error):
            blk.ep_create(0, 2)
        blk.set_semantics(False)
        blk.ep_create(0, 2)
        with pytest.raises(S14Error):
            blk.set_semantics(True)
    finally:
        blk.close()
