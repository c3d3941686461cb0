"""Parity of the grouped block path (s14_cmd_moe_block / s14_cmd_routed_moe_block): a block of
tokens through one MoE layer with the tokens grouped by expert must give, for EVERY token, the bits
of the double-accumulated CPU oracle for that token alone -- the reference's per-token layer loop
(examples/s14_vulkan_numeric.rs:929-947) applied to each token of the block -- and the bits of the
one-token tensor-core call."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from colormlm_b200 import _lib as L
from colormlm_b200 import synth
from colormlm_b200.s14 import MoeBlock, S14Context, S14Error, TokenRoute

from .test_gpu_parity import dev, dev_page, make_layer, run_layer

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("cuda_lib")]


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = S14Context(0)
    yield c
    c.close()


def run_block(ctx, blk, x, pages_dev, shared_dev, routes):
    dx = dev(x)
    dy = torch.full_like(dx, float("nan"))
    tr = [TokenRoute(ids, w, [pages_dev[i].data_ptr() for i in ids]) for ids, w in routes]
    blk.cmd_moe_block(dx, dy, tr, shared_dev.data_ptr() if shared_dev is not None else None)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0  # no bounded wait ran out
    assert ctx.last_layer_path == L.LAYER_PATH_TENSOR_BLOCK
    return dy.cpu().numpy()


def random_routes(g, n_tokens, n_experts, ragged=False):
    routes = []
    for t in range(n_tokens):
        k = 6 if not ragged else int(g.integers(1, 7))
        routes.append((g.permutation(n_experts)[:k].tolist(), g.uniform(0.05, 0.4, k).astype(np.float32)))
    return routes


@pytest.mark.parametrize("n_tokens", [1, 5, 8, 13])
def test_block_equals_every_tokens_own_layer(ctx, oracle, n_tokens):
    """2048 x 1024, 16 experts: with 13 tokens every expert has several tokens, some more than one
    chunk of six; the shared expert has three chunks.  Ragged routes (1..6 experts per token)."""
    hidden, inter, n_experts = 2048, 1024, 16
    g, pages, shared = make_layer(1200 + n_tokens, hidden, inter, n_experts, L.PAGE_MXFP4)
    x = synth.activations(g, n_tokens, hidden)
    routes = random_routes(g, n_tokens, n_experts, ragged=n_tokens == 5)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 16)
    try:
        y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        chunks, n_up, n_down, bad = blk.last_counts()
        per_item = 1 if n_tokens <= 12 else 2   # slices / row tiles per item: a large block takes two
        assert bad == 0 and n_up == chunks * (inter // 64) // per_item and n_down == chunks * (hidden // 128) // per_item
        members = {}
        for ids, _ in routes:
            for e in ids:
                members[e] = members.get(e, 0) + 1
        cap = 2 if n_tokens <= 12 else 6   # tokens per chunk: a small block takes short chunks (routes from the host: never wide chunks)
        assert chunks == sum(-(-m // cap) for m in members.values()) + -(-n_tokens // cap)
        ctx.set_accumulation(L.ACCUM_PAIRWISE)
        for t in range(n_tokens):
            ids, w = routes[t]
            ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
            bad_at = np.nonzero(y[t].view(np.uint32) != ref.view(np.uint32))[0]
            assert bad_at.size == 0, (t, bad_at.size, bad_at[:8], y[t][bad_at[:4]], ref[bad_at[:4]])
            single = run_layer(ctx, x[t:t + 1], pages_dev, shared_dev, [routes[t]], L.PAGE_MXFP4, hidden, inter)[0]
            assert np.array_equal(single.view(np.uint32), y[t].view(np.uint32))
        # the same block again on the same object, and without a shared expert
        y2 = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        assert np.array_equal(y2.view(np.uint32), y.view(np.uint32))
        full = [r for r in routes if len(r[0]) > 0]
        y3 = run_block(ctx, blk, x, pages_dev, None, full)
        for t in (0, n_tokens - 1):
            single = run_layer(ctx, x[t:t + 1], pages_dev, None, [routes[t]], L.PAGE_MXFP4, hidden, inter)[0]
            assert np.array_equal(single.view(np.uint32), y3[t].view(np.uint32))
    finally:
        blk.close()


@pytest.mark.parametrize("hidden,inter", [(1024, 1024), (1024, 4096), (4096, 4096)])
def test_block_at_the_other_sizes(ctx, oracle, hidden, inter):
    """The smallest and the largest sizes the kernels take, a small block (chunks of two, one row tile per
    item) and a large one (chunks of six, two row tiles per item)."""
    n_experts = 8
    g, pages, shared = make_layer(1600 + hidden + inter, hidden, inter, n_experts, L.PAGE_MXFP4)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 32)
    try:
        for n_tokens in (3, 17):
            x = synth.activations(g, n_tokens, hidden)
            routes = random_routes(g, n_tokens, n_experts, ragged=True)
            y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
            for t in range(n_tokens):
                ids, w = routes[t]
                ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
                assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32)), (n_tokens, t)
    finally:
        blk.close()


def test_block_sweep_of_block_sizes_against_the_one_token_kernel(ctx):
    """Block sizes around every boundary of the chunking (1, 2, 6, 7, 12, 13 tokens; 33 and 64 with experts of
    many chunks), ragged routes, few experts so that groups are large: every token equals its own one-token call
    (which the other tests pin to the oracle)."""
    hidden, inter, n_experts = 2048, 1024, 10
    g, pages, shared = make_layer(1800, hidden, inter, n_experts, L.PAGE_MXFP4)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 64)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    try:
        for n_tokens in (1, 2, 6, 7, 12, 13, 33, 64):
            x = synth.activations(g, n_tokens, hidden)
            routes = random_routes(g, n_tokens, n_experts, ragged=True)
            y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
            for t in range(n_tokens):
                single = run_layer(ctx, x[t:t + 1], pages_dev, shared_dev, [routes[t]], L.PAGE_MXFP4, hidden, inter)[0]
                assert np.array_equal(single.view(np.uint32), y[t].view(np.uint32)), (n_tokens, t)
    finally:
        blk.close()


def test_block_of_the_largest_size(ctx):
    """1024 tokens (the most a block object takes) over 16 experts: every expert has hundreds of tokens, and with
    64 slices per chunk a CTA of the up kernel holds some 260 items, i.e. walks three batches of item records;
    sampled tokens against their own one-token call."""
    hidden, inter, n_experts, n_tokens = 1024, 4096, 16, 1024
    g, pages, shared = make_layer(1900, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = dev(synth.router_weight_bf16(g, n_experts, hidden)), dev(synth.router_bias(g, n_experts))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    x = synth.activations(g, n_tokens, hidden)
    dx = dev(x)
    dy = torch.full_like(dx, float("nan"))
    ids = torch.empty((n_tokens, 6), dtype=torch.int32, device="cuda")
    wts = torch.empty((n_tokens, 6), dtype=torch.float32, device="cuda")
    blk = MoeBlock(ctx, hidden, inter, n_tokens)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    try:
        blk.cmd_routed_moe_block(dx, wr, bias, table, shared_dev.data_ptr(), dy, ids, wts)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        chunks, n_up, n_down, bad = blk.last_counts()
        assert bad == 0 and chunks >= (7 * n_tokens) // 12 and n_up == chunks * (inter // 64) // 2
        assert not torch.isnan(dy).any()
        y = dy.cpu().numpy()
        ids_np, w_np = ids.cpu().numpy(), wts.cpu().numpy()
        for t in (0, 1, 511, 777, 1023):
            single = run_layer(ctx, x[t:t + 1], pages_dev, shared_dev, [(ids_np[t].tolist(), w_np[t])], L.PAGE_MXFP4, hidden, inter)[0]
            assert np.array_equal(single.view(np.uint32), y[t].view(np.uint32)), t
    finally:
        blk.close()


def test_block_at_the_benchmark_shape(ctx, oracle):
    """4096 x 2048, 48 experts.  A verify block of 8 tokens against the oracle, bit for bit; 40 tokens
    (every expert several tokens, the shared expert seven chunks) against every token's own one-token
    call, which the other tests pin to the oracle."""
    hidden, inter, n_experts = 4096, 2048, 48
    g, pages, shared = make_layer(1977, hidden, inter, n_experts, L.PAGE_MXFP4)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 64)
    try:
        x = synth.activations(g, 8, hidden)
        routes = random_routes(g, 8, n_experts)
        y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        for t in range(8):
            ids, w = routes[t]
            ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in ids], w, shared, 0, hidden, inter)
            assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32)), t
        x = synth.activations(g, 40, hidden)
        routes = random_routes(g, 40, n_experts)
        y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        ctx.set_accumulation(L.ACCUM_PAIRWISE)
        for t in range(40):
            single = run_layer(ctx, x[t:t + 1], pages_dev, shared_dev, [routes[t]], L.PAGE_MXFP4, hidden, inter)[0]
            assert np.array_equal(single.view(np.uint32), y[t].view(np.uint32)), t
    finally:
        blk.close()


@pytest.mark.parametrize("n_tokens,n_experts", [(24, 32), (41, 24)])
@pytest.mark.parametrize("score_fn", [L.SCORE_SIGMOID, L.SCORE_SQRT_SOFTPLUS])
def test_routed_block_picks_the_oracles_routes(ctx, oracle, score_fn, n_tokens, n_experts):
    """Router on the device: ids and weights are the oracle's, every token's y is the oracle's layer for
    those routes, bit for bit.  24 tokens take the vector-pipe scores, 41 the FP64 tensor path (a ragged
    last tile of tokens, a ragged last tile of experts)."""
    hidden, inter = 2048, 1024
    g, pages, shared = make_layer(1300 + score_fn, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    x = synth.activations(g, n_tokens, hidden)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    ids = torch.empty((n_tokens, 6), dtype=torch.int32, device="cuda")
    wts = torch.empty((n_tokens, 6), dtype=torch.float32, device="cuda")
    dx = dev(x)
    dy = torch.full_like(dx, float("nan"))
    blk = MoeBlock(ctx, hidden, inter, 48)
    try:
        blk.cmd_routed_moe_block(dx, dev(wr), dev(bias), table, shared_dev.data_ptr(), dy, ids, wts,
                                 score_fn=score_fn, top_k=6, route_scale=1.5)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        y = dy.cpu().numpy()
        for t in range(n_tokens):
            rid, rw, _, _ = oracle.router(x[t], wr, bias, score_fn=score_fn, top_k=6, route_scale=1.5)
            assert np.array_equal(ids[t].cpu().numpy(), rid)
            assert np.array_equal(wts[t].cpu().numpy().view(np.uint32), rw.view(np.uint32))
            ref = oracle.moe_layer_acc64(x[t], [pages[i] for i in rid], rw, shared, 0, hidden, inter)
            assert np.array_equal(y[t].view(np.uint32), ref.view(np.uint32)), t
        # without the optional outputs the object's own buffers hold the routes
        dy2 = torch.full_like(dx, float("nan"))
        blk.cmd_routed_moe_block(dx, dev(wr), dev(bias), table, shared_dev.data_ptr(), dy2,
                                 score_fn=score_fn, top_k=6, route_scale=1.5)
        torch.cuda.synchronize()
        assert np.array_equal(dy2.cpu().numpy().view(np.uint32), y.view(np.uint32))
    finally:
        blk.close()


@pytest.mark.parametrize("world", [2, 4])
def test_block_expert_parallel_ranks_add_up_to_the_single_gpu_block(ctx, world):
    """The ranks of an expert-parallel block, run one after the other on this GPU: the sum of their pair
    buffers (every row has one owner) mixed is the single-GPU block, bit for bit; with and without residual."""
    from colormlm_b200 import ep

    hidden, inter, n_experts, n_tokens = 2048, 1024, 32, 20
    g, pages, shared = make_layer(1500 + world, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = dev(synth.router_weight_bf16(g, n_experts, hidden)), dev(synth.router_bias(g, n_experts))
    dx = dev(synth.activations(g, n_tokens, hidden))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    blk = MoeBlock(ctx, hidden, inter, 32)
    try:
        want = torch.full_like(dx, float("nan"))
        blk.cmd_routed_moe_block(dx, wr, bias, table, shared_dev.data_ptr(), want)
        torch.cuda.synchronize()
        ids = torch.empty((n_tokens, 6), dtype=torch.int32, device="cuda")
        wts = torch.empty((n_tokens, 6), dtype=torch.float32, device="cuda")
        total = torch.zeros((n_tokens * 7, hidden), dtype=torch.float32, device="cuda")
        owners = torch.zeros(n_tokens * 7, dtype=torch.int32, device="cuda")
        for rank in range(world):
            part = torch.full_like(total, float("nan"))
            blk.cmd_routed_moe_block_experts_ep(dx, wr, bias, table, shared_dev.data_ptr(), part, ids, wts, ep_rank=rank,
                                                ep_world=world, shared_owner=ep.shared_owner(3, world))
            torch.cuda.synchronize()
            assert ctx.device_status() == 0
            assert not torch.isnan(part).any()
            owners += (part != 0).any(dim=1).int()
            total += part
        assert int(owners.max().item()) == 1   # no row has two contributors
        got = torch.full_like(dx, float("nan"))
        blk.cmd_mix(total, ids, wts, got, has_shared=True)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
        blk.cmd_mix(total, ids, wts, got, has_shared=True, x_residual=dx)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint32), (dx + want).cpu().numpy().view(np.uint32))
    finally:
        blk.close()


@pytest.mark.parametrize("by_token", [False, True])
@pytest.mark.parametrize("world", [2, 4])
def test_block_exchange_inside_the_kernels(ctx, world, by_token):
    """The ranks as block objects on this GPU, connected to one another: ranks 0 .. G-2 publish their rows into every
    rank's pair buffer and return, the last rank waits for all of them and mixes; several calls in a row (the
    two buffers alternate) with different tokens; the result is the single-GPU block's, bit for bit."""
    from colormlm_b200 import ep

    hidden, inter, n_experts, n_tokens = 2048, 1024, 32, 20
    g, pages, shared = make_layer(1700 + world, hidden, inter, n_experts, L.PAGE_MXFP4)
    wr, bias = dev(synth.router_weight_bf16(g, n_experts, hidden)), dev(synth.router_bias(g, n_experts))
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    table = torch.tensor([p.data_ptr() for p in pages_dev], dtype=torch.int64, device="cuda")
    single = MoeBlock(ctx, hidden, inter, 32)
    ranks = [MoeBlock(ctx, hidden, inter, 32) for _ in range(world)]
    try:
        for r, b in enumerate(ranks):
            b.ep_create(r, world)
        for b in ranks:
            b.ep_connect_local(ranks)
            b.ep_set_wait_limit(1 << 12)
        for call in range(3):
            dx = dev(synth.activations(g, n_tokens, hidden))
            want = torch.full_like(dx, float("nan"))
            single.cmd_routed_moe_block(dx, wr, bias, table, shared_dev.data_ptr(), want)
            got = torch.full_like(dx, float("nan"))
            for r, b in enumerate(ranks):
                last = r == world - 1
                # (by_token: the shared expert's tokens are dealt to the ranks, t mod world)
                b.cmd_routed_moe_block_ep(dx, wr, bias, table, shared_dev.data_ptr(), got if last else None,
                                          shared_owner=L.EP_SHARED_BY_TOKEN if by_token else ep.shared_owner(call, world),
                                          wait_and_mix=last)
            torch.cuda.synchronize()
            assert ctx.device_status() == 0
            assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32)), call
        # a rank whose peers never publish does not hang: the wait runs out, the status says so, the context goes on
        lonely = ranks[world - 1]
        dx = dev(synth.activations(g, n_tokens, hidden))
        got = torch.full_like(dx, float("nan"))
        lonely.ep_set_wait_limit(200)
        lonely.cmd_routed_moe_block_ep(dx, wr, bias, table, shared_dev.data_ptr(), got, shared_owner=0, wait_and_mix=True)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0x5508
        assert torch.isnan(got).all()
        single.cmd_routed_moe_block(dx, wr, bias, table, shared_dev.data_ptr(), got)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0 and not torch.isnan(got).any()
    finally:
        for b in ranks:
            b.ep_disconnect()
        for b in ranks + [single]:
            b.close()


def test_block_with_residual_in_place(ctx):
    """y = x + moe(x), written over x: the step of a stack of layers."""
    hidden, inter, n_experts, n_tokens = 2048, 1024, 16, 9
    g, pages, shared = make_layer(1400, hidden, inter, n_experts, L.PAGE_MXFP4)
    x = synth.activations(g, n_tokens, hidden)
    routes = random_routes(g, n_tokens, n_experts)
    pages_dev, shared_dev = [dev_page(p, hidden, inter) for p in pages], dev_page(shared, hidden, inter)
    blk = MoeBlock(ctx, hidden, inter, 16)
    try:
        y = run_block(ctx, blk, x, pages_dev, shared_dev, routes)
        blk.set_residual(True)
        buf = dev(x)
        tr = [TokenRoute(ids, w, [pages_dev[i].data_ptr() for i in ids]) for ids, w in routes]
        blk.cmd_moe_block(buf, buf, tr, shared_dev.data_ptr())
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        assert np.array_equal(buf.cpu().numpy().view(np.uint32), (x + y).astype(np.float32).view(np.uint32))
        blk.set_residual(False)
        assert np.array_equal(run_block(ctx, blk, x, pages_dev, shared_dev, routes).view(np.uint32), y.view(np.uint32))
    finally:
        blk.close()


def test_block_rejects_what_it_cannot_run(ctx):
    hidden, inter = 1024, 1024
    with pytest.raises(S14Error):
        MoeBlock(ctx, 1000, inter, 8)
    with pytest.raises(S14Error):
        MoeBlock(ctx, hidden, inter, 0)
    with pytest.raises(S14Error):
        MoeBlock(ctx, hidden, inter, 5000)
    blk = MoeBlock(ctx, hidden, inter, 4)
    try:
        from colormlm_b200.pages import ExpertPageLayout
        page = torch.zeros(ExpertPageLayout(hidden, inter).page_bytes, dtype=torch.uint8, device="cuda")
        x = torch.zeros((5, hidden), device="cuda")
        y = torch.empty_like(x)
        ok = TokenRoute([0, 1], [0.5, 0.5], [page.data_ptr()] * 2)
        with pytest.raises(S14Error):   # more tokens than the object holds
            blk.cmd_moe_block(x, y, [ok] * 5, None)
        for r in (TokenRoute([0, 0], [0.5, 0.5], [page.data_ptr()] * 2),
                  TokenRoute([0, 300], [0.5, 0.5], [page.data_ptr()] * 2),
                  TokenRoute([0, 1], [0.5, float("nan")], [page.data_ptr()] * 2),
                  TokenRoute([0, 1], [0.5, 0.5], [page.data_ptr(), 0]),
                  TokenRoute([], [], [])):
            with pytest.raises(S14Error):
                blk.cmd_moe_block(x[:1], y[:1], [r], None)
        blk.cmd_moe_block(x[:2], y[:2], [ok, ok], None)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        assert torch.count_nonzero(y[:2]).item() == 0   # zero pages: every output is +0
    finally:
        blk.close()
