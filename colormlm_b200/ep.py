"""Expert-parallel decode across the GPUs of one node (one process per GPU, torch.distributed).

Partition: routed expert ``e`` of every layer lives on rank ``e mod world``; router weights are
replicated; the shared expert of layer ``l`` is computed by rank ``l mod world`` (its page is
resident there).  Exchange: every rank writes the unmixed down vectors of the experts it owns
into a ``[top_k + 1, hidden]`` slot buffer (zeros elsewhere); one all-reduce (sum) gives every
rank all slots exactly, because each slot has a single non-zero contributor; the reference's
ordered mix then runs on every rank, so the result is bit-identical for any world size.  The
reference has no multi-GPU code; this is the design SURVEY-level analysis asked for, built on the
reference's per-expert semantics (examples/s14_vulkan_numeric.rs:929-947).

Two exchanges exist.  ``decode_step`` is the baseline: owned experts, one NCCL all-reduce of the
slot buffer, a mix kernel.  ``decode_step_fused`` is one launch per rank: the layer kernel stores
the down vectors of the experts it owns into every rank's mapped slot buffer over NVLink, publishes
a flag, waits (bounded) for the other ranks' flags and mixes; ``connect_exchange`` maps the ranks'
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


def decode_step_fused(ctx, x, layer_state: dict, y, *, layer: int, world: int, inter: int, ids=None, weights=None,
                      stream: Optional[int] = None) -> None:
    """One expert-parallel layer-token on this rank in one launch (exchange inside the kernel).
    Every rank must call it for the same sequence of steps."""
    ctx.cmd_routed_moe_layer_ep(x, y, layer_state["wr"], layer_state["bias"], layer_state["table"],
                                layer_state["shared"], inter, shared_owner=shared_owner(layer, world),
                                ids_out=ids, weights_out=weights, stream=stream)
