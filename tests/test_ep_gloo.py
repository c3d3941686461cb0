"""The expert-parallel exchange with two CPU ranks over gloo: ownership, slot buffers, all-reduce
and the ordered mix reproduce the single-rank layer bit for bit.  The per-expert arithmetic comes
from the CPU oracle here (no GPU); on GPUs the same exchange runs over NCCL."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from colormlm_b200 import ep, synth
    from oracle import s14_oracle as oracle

    hidden, inter, n_experts, layer = 1024, 1024, 16, 3
    g = synth.rng(2468)  # every rank draws the same tensors; a rank only uses the pages it owns
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(n_experts)]
    shared = synth.mxfp4_expert_page(g, hidden, inter)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    x = synth.activations(g, 1, hidden)[0]
    ids, w, _, _ = oracle.router(x, wr, bias, 0, 6, 1.0)  # replicated router
    slots = torch.zeros((7, hidden), dtype=torch.float32)
    for j, e in enumerate(ids.tolist()):
        if ep.expert_owner(e, world) == rank:
            slots[j] = torch.from_numpy(oracle.expert_chain_mxfp4(x, pages[e], hidden, inter, 1.0)[1])
    if ep.shared_owner(layer, world) == rank:
        slots[6] = torch.from_numpy(oracle.expert_chain_mxfp4(x, shared, hidden, inter, 1.0)[1])
    ep.all_reduce_slots(slots)
    acc = np.zeros(hidden, np.float32)
    for j in range(6):
        acc = acc + w[j] * slots[j].numpy()
    acc = acc + slots[6].numpy()
    want = oracle.moe_layer(x, [pages[e] for e in ids], w, shared, 0, hidden, inter)
    ok = np.array_equal(acc.view(np.uint32), want.view(np.uint32))
    owned = sorted(set(ep.owned_experts(rank, world, n_experts)))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok)} {len(owned)}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_exchange_matches_single_rank(tmp_path, world):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    total_owned = 0
    for r in range(world):
        ok, owned = open(tmp_path / f"rank{r}.txt").read().split()
        assert ok == "1"
        total_owned += int(owned)
    assert total_owned == 16


def _head_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from colormlm_b200 import ep, synth
    from oracle import s14_oracle as oracle

    vocab, hidden = 1003, 512  # rows do not divide evenly
    g = synth.rng(731)
    w = synth.head_weight_bf16(g, vocab, hidden)
    x = synth.activations(g, 1, hidden)[0]
    full = oracle.head_logits(x, w)
    r0, r1 = ep.head_rows(rank, world, vocab)
    local = oracle.head_logits(x, w[r0:r1])
    got = ep.gather_head_logits(torch.from_numpy(local), vocab, world).numpy()
    ok = np.array_equal(got.view(np.uint32), full.view(np.uint32))
    cases = []
    for name, logits in (("plain", full), ("tie", np.where(np.arange(vocab) % 97 == 5, np.float32(99.0), full)),
                         ("nan", np.where(np.arange(vocab) == vocab - 2, np.float32(np.nan), full))):
        mine = logits[r0:r1]
        a = oracle.greedy_argmax(mine)
        token = ep.combine_greedy(float(mine[a]) if a >= 0 else 0.0, r0 + a if a >= 0 else -1, world)
        cases.append(token == oracle.greedy_argmax(logits))
    with open(os.path.join(out_dir, f"head{rank}.txt"), "w") as f:
        f.write(f"{int(ok)} {int(all(cases))}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_sharded_head_gathers_the_full_logits_and_the_greedy_token(tmp_path, world):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_head_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"head{r}.txt").read().split() == ["1", "1"]


def test_ownership_is_a_partition():
    sys.path.insert(0, ROOT)
    from colormlm_b200 import ep

    for world in (1, 2, 4, 8):
        seen = sorted(e for r in range(world) for e in ep.owned_experts(r, world))
        assert seen == list(range(256))
        assert all(0 <= ep.shared_owner(layer, world) < world for layer in range(43))


class _RecordingContext:
    """Stands in for an S14Context in the teardown: counts, in the ranks' shared store, how many ranks
    have disconnected, and on destroy reads how many had when this rank freed its buffer."""

    def __init__(self, store, rank):
        self.store, self.rank, self.seen_at_destroy = store, rank, None

    def ep_exchange_disconnect(self):
        import time

        time.sleep(0.05 * self.rank)  # the ranks reach the teardown at different times
        self.store.add("disconnected", 1)

    def ep_exchange_destroy(self):
        self.seen_at_destroy = self.store.add("disconnected", 0)


def _teardown_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from colormlm_b200 import ep

    store = dist.distributed_c10d._get_default_store()
    ctx = _RecordingContext(store, rank)
    ep.disconnect_exchange(ctx)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{ctx.seen_at_destroy}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_no_rank_frees_its_exchange_buffer_before_every_rank_has_disconnected(tmp_path, world):
    """ep.disconnect_exchange: disconnect, host barrier, destroy.  Every rank, at the moment it frees
    its buffer, finds that all ranks have closed their mappings of it."""
    port = 29500 + ((os.getpid() + 7) % 2000)
    mp.spawn(_teardown_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert int(open(tmp_path / f"rank{r}.txt").read()) == world


def test_verify_block_is_one_expert_parallel_step_per_token():
    """ep.verify_block_fused: K tokens are K steps of the fused exchange, in token order, each with the
    token's own rows of the outputs and the layer's shared-expert owner (tokens are replicated, experts
    are sharded, so nothing is dispatched)."""
    sys.path.insert(0, ROOT)
    from colormlm_b200 import ep

    calls = []

    class Ctx:
        def cmd_routed_moe_layer_ep(self, x, y, wr, bias, table, shared, inter, **kw):
            calls.append((x, y, wr, bias, table, shared, inter, kw))

    xs, ys = torch.arange(12.0).reshape(3, 4), torch.zeros(3, 4)
    ids, wts = torch.zeros((3, 6), dtype=torch.int32), torch.zeros((3, 6))
    state = {"wr": "WR", "bias": "B", "table": "T", "shared": 77}
    ep.verify_block_fused(Ctx(), xs, state, ys, layer=5, world=4, inter=2048, ids=ids, weights=wts, stream=9)
    assert len(calls) == 3
    for t, (x, y, wr, bias, table, shared, inter, kw) in enumerate(calls):
        assert torch.equal(x, xs[t]) and y.data_ptr() == ys[t].data_ptr()
        assert (wr, bias, table, shared, inter) == ("WR", "B", "T", 77, 2048)
        assert kw["shared_owner"] == ep.shared_owner(5, 4) and kw["stream"] == 9
        assert kw["ids_out"].data_ptr() == ids[t].data_ptr() and kw["weights_out"].data_ptr() == wts[t].data_ptr()


def _block_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    """ep.block_layer's host side with a stand-in for the block object: the rank fills the pair rows of the experts
    it owns from the CPU oracle (zeros elsewhere), the all-reduce adds the ranks' buffers up, every rank mixes."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from colormlm_b200 import ep, synth
    from oracle import s14_oracle as oracle

    hidden, inter, n_experts, layer, n_tok = 1024, 1024, 16, 3, 5
    g = synth.rng(2469)
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(n_experts)]
    shared = synth.mxfp4_expert_page(g, hidden, inter)
    wr, bias = synth.router_weight_bf16(g, n_experts, hidden), synth.router_bias(g, n_experts)
    xs_np = synth.activations(g, n_tok, hidden)

    class Block:
        """What MoeBlock does for ep.block_layer, on the CPU oracle."""

        def cmd_routed_moe_block_experts_ep(self, xs, wr_, bias_, table, shared_page, pairs, ids, weights, *, ep_rank, ep_world,
                                            shared_owner, stream=None):
            pairs.zero_()
            for t in range(n_tok):
                rid, rw, _, _ = oracle.router(xs[t].numpy(), wr, bias, 0, 6, 1.0)
                ids[t] = torch.from_numpy(rid)
                weights[t] = torch.from_numpy(rw)
                for m, e in enumerate(rid.tolist()):
                    if ep.expert_owner(e, ep_world) == ep_rank:
                        pairs[t * 7 + m] = torch.from_numpy(oracle.expert_chain_mxfp4(xs[t].numpy(), pages[e], hidden, inter, 1.0)[1])
                if shared_owner == ep_rank:
                    pairs[t * 7 + 6] = torch.from_numpy(oracle.expert_chain_mxfp4(xs[t].numpy(), shared, hidden, inter, 1.0)[1])

        def cmd_mix(self, pairs, ids, weights, ys, *, has_shared=True, x_residual=None, stream=None):
            for t in range(n_tok):
                acc = np.zeros(hidden, np.float32)
                for m in range(6):
                    acc = acc + weights[t, m].numpy() * pairs[t * 7 + m].numpy()
                acc = acc + pairs[t * 7 + 6].numpy()
                ys[t] = torch.from_numpy(acc if x_residual is None else (x_residual[t].numpy() + acc).astype(np.float32))

    xs = torch.from_numpy(xs_np)
    pairs = torch.full((n_tok * 7, hidden), float("nan"))
    ids, wts = torch.zeros((n_tok, 6), dtype=torch.int32), torch.zeros((n_tok, 6))
    ys = torch.zeros((n_tok, hidden))
    ep.block_layer(Block(), xs, {"wr": None, "bias": None, "table": None, "shared": 1}, pairs, ids, wts, ys, layer=layer,
                   rank=rank, world=world)
    ok = True
    for t in range(n_tok):
        rid, rw, _, _ = oracle.router(xs_np[t], wr, bias, 0, 6, 1.0)
        want = oracle.moe_layer(xs_np[t], [pages[e] for e in rid], rw, shared, 0, hidden, inter)
        ok = ok and np.array_equal(ys[t].numpy().view(np.uint32), want.view(np.uint32))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok)}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_block_combine_matches_the_single_rank_layer(tmp_path, world):
    port = 29500 + ((os.getpid() + 13) % 2000)
    mp.spawn(_block_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read().strip() == "1"


def test_block_exchange_calls_and_teardown_order():
    """ep.block_layer_fused is one call per rank with the layer's shared-expert owner; ep.disconnect_block disconnects
    before the barrier (the object is destroyed only afterwards, by its owner)."""
    sys.path.insert(0, ROOT)
    from colormlm_b200 import ep

    log = []

    class Block:
        def cmd_routed_moe_block_ep(self, xs, wr, bias, table, shared, ys, ids, weights, **kw):
            log.append(("call", xs, ys, wr, bias, table, shared, ids, weights, kw))

        def ep_disconnect(self):
            log.append(("disconnect",))

    state = {"wr": "WR", "bias": "B", "table": "T", "shared": 5}
    ep.block_layer_fused(Block(), "X", state, "Y", layer=6, world=4, ids="I", weights="W", stream=3)
    assert log[0][:9] == ("call", "X", "Y", "WR", "B", "T", 5, "I", "W")
    assert log[0][9] == {"shared_owner": ep.shared_owner(6, 4), "stream": 3}
    ep.block_layer_fused(Block(), "X", state, "Y", layer=6, world=4, shared_by_token=True)
    assert log.pop()[9]["shared_owner"] == 0xFFFFFFFF
    ep.disconnect_block(Block(), barrier=lambda: log.append(("barrier",)))
    assert [e[0] for e in log[1:]] == ["disconnect", "barrier"]
