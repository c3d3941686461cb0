"""Expert-parallel decode across the GPUs of one node (one process per GPU, torch.distributed).

Partition: routed expert ``e`` of every layer lives on rank ``e mod world``; router weights are
replicated; the shared expert of layer ``l`` is computed by rank ``l mod world`` (its page is
resident there).  Exchange: every rank writes the unmixed down vectors of the experts it owns
into a ``[top_k + 1, hidden]`` slot buffer (zeros elsewhere); one all-reduce (sum) gives every
rank all slots exactly, because each slot has a single non-zero contributor; the reference's
ordered mix then runs on every rank, so the result is bit-identical for any world size.  The
reference has no multi-GPU code; the partition is built on the
reference's per-expert semantics (examples/s14_vulkan_numeric.rs:929-947).

Two exchanges exist.  ``decode_step`` is the baseline: owned experts, one NCCL all-reduce of the
slot buffer, a mix kernel.  ``decode_step_fused`` is one launch per rank: the layer kernel stores
the down vectors of the experts it owns into every rank's mapped slot buffer over NVLink (each
value with the step's number in one 8-byte store), waits (bounded) for the other ranks' values and
mixes; ``connect_exchange`` maps the ranks'
buffers once (CUDA IPC handles passed through torch.distributed)."""
from __future__ import annotations

from typing import Optional


def expert_owner(expert_id: int, world: int) -> int:
    return expert_id % world


def shared_owner(layer: int, world: int) -> int:
    return layer % world


def owned_experts(rank: int, world: int, n_experts: int = 256):
    return [e for e in range(n_experts) if expert_owner(e, world) == rank]


def all_reduce_slots(slots, group=None) -> None:
    """Sum of the ranks' slot buffers in place (NCCL on GPUs, gloo in the CPU tests)."""
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(slots, op=dist.ReduceOp.SUM, group=group)


def decode_step(ctx, x, layer_state: dict, slots, ids, weights, y, *, layer: int, rank: int, world: int,
                inter: int, shared_kind: int = 0, stream: Optional[int] = None, group=None) -> None:
    """One expert-parallel layer-token on this rank: owned experts, all-reduce, ordered mix.

    ``layer_state``: ``wr`` (BF16 router weight), ``bias``, ``table`` (device page addresses, only the
    owned entries need to be valid), ``shared`` (device address of the shared page on its owner)."""
    ctx.cmd_routed_moe_experts_ep(x, layer_state["wr"], layer_state["bias"], layer_state["table"],
                                  layer_state["shared"], shared_kind, inter, slots, ids, weights,
                                  ep_rank=rank, ep_world=world, shared_owner=shared_owner(layer, world),
                                  stream=stream)
    all_reduce_slots(slots, group)
    ctx.cmd_moe_mix_slots(slots, weights, ids.numel(), True, y, stream=stream)


def connect_exchange(ctx, rank: int, world: int, hidden: int, group=None) -> None:
    """Creates this rank's exchange buffer and maps every other rank's (one process per GPU)."""
    import torch.distributed as dist

    handle = ctx.ep_exchange_create(rank, world, hidden)
    handles = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    ctx.ep_exchange_connect(handles)
    dist.barrier(group=group)  # every rank has mapped every buffer before the first step


def disconnect_exchange(ctx, group=None, barrier=None) -> None:
    """The teardown of the exchange, on every rank: wait for this rank's work and close its mappings
    of the other ranks' buffers, pass a host barrier (after it no rank writes into or maps another
    rank's buffer), then free this rank's buffer.  `barrier` replaces `dist.barrier` (tests)."""
    ctx.ep_exchange_disconnect()
    if barrier is not None:
        barrier()
    else:
        import torch.distributed as dist

        dist.barrier(group=group)
    ctx.ep_exchange_destroy()


def decode_step_fused(ctx, x, layer_state: dict, y, *, layer: int, world: int, inter: int, ids=None, weights=None,
                      stream: Optional[int] = None) -> None:
    """One expert-parallel layer-token on this rank in one launch (exchange inside the kernel).
    Every rank must call it for the same sequence of steps."""
    ctx.cmd_routed_moe_layer_ep(x, y, layer_state["wr"], layer_state["bias"], layer_state["table"],
                                layer_state["shared"], inter, shared_owner=shared_owner(layer, world),
                                ids_out=ids, weights_out=weights, stream=stream)


def verify_block_fused(ctx, xs, layer_state: dict, ys, *, layer: int, world: int, inter: int, ids=None, weights=None,
                       stream: Optional[int] = None) -> None:
    """A block of K tokens (a verify block, K <= 8) through one expert-parallel layer: xs, ys are
    [K, hidden]; ids, weights [K, top_k] or None.  Tokens are replicated, experts are sharded: every rank
    holds all K tokens (16 KB each), routes each of them itself and computes the experts it owns, so no
    token has to be dispatched; the experts' outputs of a token are combined inside its step's kernel.
    K steps, one launch each, on every rank; a token's result is that of its own decode step."""
    for t in range(xs.shape[0]):
        ctx.cmd_routed_moe_layer_ep(xs[t], ys[t], layer_state["wr"], layer_state["bias"], layer_state["table"],
                                    layer_state["shared"], inter, shared_owner=shared_owner(layer, world),
                                    ids_out=None if ids is None else ids[t],
                                    weights_out=None if weights is None else weights[t], stream=stream)


def block_layer(blk, xs, layer_state: dict, pairs, ids, weights, ys, *, layer: int, rank: int, world: int,
                residual: bool = False, stream: Optional[int] = None, group=None) -> None:
    """A block of tokens (a verify block, a prefill) through one expert-parallel layer on the grouped block
    path: xs, ys [T, hidden]; pairs [T * 7, hidden], ids, weights [T, top_k] device buffers.  Tokens are
    replicated, experts sharded: every rank routes all tokens, runs the grouped contractions of the experts
    it owns (each of their pages streamed once for all its tokens), one all-reduce adds the ranks' pair
    buffers up (every row has one non-zero contributor, so the sum is exact), and the ordered mix runs on
    every rank: ys is bit-identical to the single-GPU block for any world size."""
    blk.cmd_routed_moe_block_experts_ep(xs, layer_state["wr"], layer_state["bias"], layer_state["table"],
                                        layer_state["shared"], pairs, ids, weights, ep_rank=rank, ep_world=world,
                                        shared_owner=shared_owner(layer, world), stream=stream)
    all_reduce_slots(pairs, group)
    blk.cmd_mix(pairs, ids, weights, ys, has_shared=True, x_residual=xs if residual else None, stream=stream)


def connect_block(blk, rank: int, world: int, group=None) -> None:
    """Creates this rank's pair buffers of the block exchange and maps every other rank's (one process per GPU)."""
    import torch.distributed as dist

    handle = blk.ep_create(rank, world)
    handles = [None] * world
    dist.all_gather_object(handles, handle, group=group)
    blk.ep_connect(handles)
    dist.barrier(group=group)


def disconnect_block(blk, group=None, barrier=None) -> None:
    """The block exchange's teardown: disconnect on every rank, a host barrier, then the object may be destroyed."""
    blk.ep_disconnect()
    if barrier is not None:
        barrier()
    else:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.barrier(group=group)


def block_layer_fused(blk, xs, layer_state: dict, ys, *, layer: int, world: int, ids=None, weights=None,
                      shared_by_token: bool = False, stream: Optional[int] = None) -> None:
    """``block_layer`` with the exchange inside the kernels: one call per rank, no collective; the w2 kernel stores the
    rows of the experts this rank owns into every rank's pair buffer over NVLink, the mix waits (bounded) for every
    rank's rows.  ys is bit-identical to the single-GPU block on every rank."""
    # shared_by_token: the shared page is resident on every rank and rank r takes the tokens t with t mod world == r
    owner = 0xFFFFFFFF if shared_by_token else shared_owner(layer, world)
    blk.cmd_routed_moe_block_ep(xs, layer_state["wr"], layer_state["bias"], layer_state["table"], layer_state["shared"], ys,
                                ids, weights, shared_owner=owner, stream=stream)


# ---- vocabulary-sharded LM head ---------------------------------------------------------------
# The head weight [vocab, hidden] BF16 is split by rows: rank r holds rows [vocab r / G, vocab (r+1) / G)
# (final_head.py:113-149 computes all rows on one device; the runner's contract wants the full logits,
# s14_runner/src/runner.rs:111-117, and picks the greedy token with the lowest id on ties and rejects
# NaN, runner.rs:485-508).  Every row's logit is the same sum whichever rank computes it, so the
# gathered logits and the token are identical for every G.


def head_rows(rank: int, world: int, vocab: int):
    return vocab * rank // world, vocab * (rank + 1) // world


def gather_head_logits(local_logits, vocab: int, world: int, group=None):
    """All-gather of the ranks' row shards ([rows of this rank] F32) into the full [vocab] logits."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return local_logits
    sizes = [head_rows(r, world, vocab)[1] - head_rows(r, world, vocab)[0] for r in range(world)]
    widest = max(sizes)
    mine = torch.zeros(widest, dtype=local_logits.dtype, device=local_logits.device)
    mine[: local_logits.numel()] = local_logits
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)])


def combine_greedy(local_best: float, local_token: int, world: int, group=None, device="cpu") -> int:
    """The greedy token over all shards from every rank's (largest logit, its global id): largest
    value, lowest id on ties; a rank that met a NaN reports token -1 and the result is -1."""
    import torch
    import torch.distributed as dist

    pair = torch.tensor([float(local_best), float(local_token)], dtype=torch.float64, device=device)
    pairs = [pair]
    if world > 1:
        pairs = [torch.empty_like(pair) for _ in range(world)]
        dist.all_gather(pairs, pair, group=group)
    best, token = None, -1
    for p in pairs:
        v, t = float(p[0]), int(p[1])
        if t < 0:
            return -1
        if best is None or v > best or (v == best and t < token):
            best, token = v, t
    return token


def sharded_head(ctx, x, w_shard_bf16, vocab: int, rank: int, world: int, group=None, stream: Optional[int] = None):
    """Full logits [vocab] and the greedy token from this rank's row shard of the head weight (GPU)."""
    import torch

    row0, row1 = head_rows(rank, world, vocab)
    local = torch.empty(row1 - row0, dtype=torch.float32, device=x.device)
    ctx.cmd_head_logits(x, w_shard_bf16, local, stream=stream)
    arg = torch.empty(1, dtype=torch.int64, device=x.device)
    ctx.cmd_greedy_argmax(local, arg, stream=stream)
    # Without `stream` the head kernels ran on torch's current stream, like the gather below.  With
    # one, the gather (which reads `local` on torch's current stream) is ordered after them by an event.
    if stream is not None:
        done = torch.cuda.Event()
        done.record(torch.cuda.ExternalStream(stream))
        torch.cuda.current_stream().wait_event(done)
    logits = gather_head_logits(local, vocab, world, group)
    torch.cuda.synchronize()
    a = int(arg.item())
    token = combine_greedy(float(local[a]) if a >= 0 else 0.0, row0 + a if a >= 0 else -1, world, group,
                           device=x.device)
    return logits, token
