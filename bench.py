#!/usr/bin/env python
"""Benchmark of the S14 MoE expert path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload stack|layer|expert_chain|wq_a|verify8|prefill|glue|decode] [--accum pairwise|reference]

A step is one layer-token: one token through one MoE layer (router top-6 of 256, six routed MXFP4
experts and the shared MXFP4 expert, hidden 4096, intermediate 2048).  14 layers of 257 expert pages
are resident (48 GB), so the 96 MB a step touches never come from L2.

  stack   (default on one GPU) the 14 layers chained as the decode of one token does it,
          h <- h + moe_l(h), in ONE launch of the layer kernel per 14 steps (s14_cmd_stack_decode);
  layer   one launch per step with independent tokens (s14_cmd_routed_moe_layer); with several GPUs
          the experts are partitioned and the down vectors exchanged inside the kernel;
  expert_chain, wq_a   the single-expert chain and the FP8 projection matvec of the other
          configurations, each with its own roofline entry;
  verify8, prefill   a block of tokens (8; 370, or --tokens N) through one layer with the tokens
          grouped by expert, every distinct expert page streamed once (s14_cmd_routed_moe_block);
  glue    the steps on either side of the MoE at one site of a layer (hc_pre -> RMSNorm -> hc_post,
          --tokens N tokens, BF16 streams).

The timed region is exactly K steps, taken with CUDA events on the launching stream; it is repeated
(--repeats, default 50) and the median repeat is reported with the spread.  Pages are a function of
(layer, expert, byte position) that the GPU and the host evaluate alike, so the CPU arm and the
parity check run the very bytes the GPU holds (a SHA-256 of one page from both sides is in the line).

One JSON line is printed by rank 0: `value` is layer-tokens/s with inputs resident in HBM, `e2e` the
same through the host-buffer C-ABI call (H2D of the token, D2H of the result inside the timed region),
`roofline` the layer kernel against the measured copy bandwidth, `parity` the error of the timed path
on its own steps against the CPU oracle, `cpu_baseline` the CPU oracle on this box's host cores on a
bounded sample.  `--impl reference` times that CPU implementation alone.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, N_EXPERTS, TOP_K, N_LAYERS = 4096, 2048, 256, 6, 14
PREFILL_TOKENS = 370   # the reference's prefill length (README.md:139)
PAGE_BYTES = 13_369_344
# algorithmic bytes of one layer-token: 7 expert pages + router weights + bias + x + y
ROUTER_BYTES = N_EXPERTS * HIDDEN * 2 + N_EXPERTS * 4
STEP_BYTES = 7 * PAGE_BYTES + ROUTER_BYTES + HIDDEN * 4 + HIDDEN * 4
# layer kernel with the routes given: 7 expert pages, x in, y out
LAYER_BYTES = 7 * PAGE_BYTES + HIDDEN * 4 + HIDDEN * 4
# DRAM bytes of one layer of a launch of the layer kernel at this workload: dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of a 14-layer launch (1 312.389 MB read + 3.994 MB written)
# divided by 14 = 94 027 346 B per layer.  The capture ran on a reduced pool (14 layers of 16 routed experts,
# 3.2 GB resident: the full workload holds 48 GB, more than a capture may); a layer's traffic differs from
# the full workload's only by the router rows it reads (16 instead of 256), which are added here.  The
# summary of the capture is kept under profiles/.
NCU_TRAFFIC_BYTES = 94_027_346 - (16 * HIDDEN * 2 + 16 * 4) + (256 * HIDDEN * 2 + 256 * 4)
WORKLOAD = ("moe_layer_decode: 1 token, router top-6 of 256 + 6 routed + 1 shared MXFP4 expert, "
            "hidden 4096, intermediate 2048")
TOKEN_SEED = 99


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.rows = []
        self.proc = None
        self.device = device

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def samples(self) -> int:
        return len(self.rows)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 4), ("hw_thermal_slowdown", 5),
                              ("sw_thermal_slowdown", 6), ("sw_power_cap", 7)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------- inputs both arms share

def tokens(n: int) -> np.ndarray:
    from colormlm_b200 import synth

    return synth.activations(synth.rng(TOKEN_SEED), n, HIDDEN)


def router_of_layer(layer: int):
    from colormlm_b200 import synth

    gl = synth.rng(500 + layer)
    return synth.router_weight_bf16(gl, N_EXPERTS, HIDDEN), synth.router_bias(gl, N_EXPERTS)


class HostPages:
    """Tensor pages (what the CPU oracle reads) of the very bytes the GPU holds, made on demand."""

    def __init__(self, limit: int = 96):
        self.cache, self.limit = {}, limit

    def get(self, layer: int, expert: int) -> np.ndarray:
        from colormlm_b200 import synth

        key = (layer, int(expert))
        if key not in self.cache:
            if len(self.cache) >= self.limit:
                self.cache.clear()
            self.cache[key] = synth.hashed_tensor_page(layer, int(expert), HIDDEN, INTER)
        return self.cache[key]


def cpu_layer(oracle, pages: HostPages, layer: int, x: np.ndarray, acc64: bool = False, official: bool = False):
    """Router + layer of one token on the CPU oracle; returns (y, ids, weights)."""
    wr, bias = router_of_layer(layer)
    ids, w, _, _ = oracle.router(x, wr, bias, 0, TOP_K, 1.0)
    sel = [pages.get(layer, e) for e in ids]
    fn = oracle.official_moe_layer if official else (oracle.moe_layer_acc64 if acc64 else oracle.moe_layer)
    return fn(x, sel, w, pages.get(layer, N_EXPERTS), 0, HIDDEN, INTER), ids, w


# ------------------------------------------------------------------ CPU reference arm

def cpu_steps(oracle, n_steps: int, first_token: int = 0):
    """(x, wr, bias, routed tensor pages, shared page) of n layer-token steps (untimed set-up)."""
    pages = HostPages(limit=10 ** 6)
    xs = tokens(first_token + n_steps)
    out = []
    for i in range(n_steps):
        layer = i % N_LAYERS
        wr, bias = router_of_layer(layer)
        x = xs[first_token + i]
        ids, _, _, _ = oracle.router(x, wr, bias, 0, TOP_K, 1.0)
        out.append((x, wr, bias, [pages.get(layer, e) for e in ids], pages.get(layer, N_EXPERTS)))
    return out


def cpu_run(oracle, steps) -> float:
    t0 = time.perf_counter()
    for x, wr, bias, sel, shared in steps:
        _, w, _, _ = oracle.router(x, wr, bias, 0, TOP_K, 1.0)
        oracle.moe_layer(x, sel, w, shared, 0, HIDDEN, INTER)
    return time.perf_counter() - t0


def cpu_threads(oracle) -> int:
    """All host cores, whatever OMP_NUM_THREADS a launcher set."""
    n = os.cpu_count() or 1
    oracle.set_threads(n)
    return n


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import s14_oracle as oracle

    oracle.build()
    cores = cpu_threads(oracle)
    steps = cpu_steps(oracle, args.warmup + args.steps)
    cpu_run(oracle, steps[:args.warmup])
    sec = cpu_run(oracle, steps[args.warmup:])
    value = args.steps / sec
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "layer-tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sec / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers_resident": N_LAYERS, "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": "layer-tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} layer-tokens (router + 7 experts each), OpenMP over rows"},
        "e2e": {"value": value, "unit": "layer-tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "hbm_gbs_equivalent": value * STEP_BYTES / 1e9,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm

def _note(msg: str) -> None:
    """Progress lines on stderr when S14_BENCH_VERBOSE is set."""
    if os.environ.get("S14_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def resident_layers(torch, n_layers: int, rank: int, world: int, shared_everywhere: bool = False):
    """The pages this rank owns (expert e on rank e mod world, the shared expert of layer l on rank
    l mod world, or on every rank), router weights and page tables, all on the device."""
    from colormlm_b200 import ep, synth

    writer = synth.HashedPageWriter(torch, HIDDEN, INTER)
    layers = []
    for layer in range(n_layers):
        owned = ep.owned_experts(rank, world, N_EXPERTS)
        has_shared = shared_everywhere or ep.shared_owner(layer, world) == rank
        pages = torch.empty((len(owned) + (1 if has_shared else 0), PAGE_BYTES), dtype=torch.uint8, device="cuda")
        for slot, e in enumerate(owned):
            writer.fill(pages[slot], layer, e)
        if has_shared:
            writer.fill(pages[len(owned)], layer, N_EXPERTS)
        wr_np, bias_np = router_of_layer(layer)
        base = pages.data_ptr()
        addr = [0] * N_EXPERTS
        for slot, e in enumerate(owned):
            addr[e] = base + slot * PAGE_BYTES
        layers.append({"pages": pages, "wr": torch.from_numpy(wr_np.view(np.int16)).cuda(),
                       "bias": torch.from_numpy(bias_np).cuda(),
                       "table": torch.tensor(addr, dtype=torch.int64, device="cuda"),
                       "shared": base + len(owned) * PAGE_BYTES if has_shared else None,
                       "owned": owned})
    return layers


def timed_repeats(torch, stream, enqueue, repeats: int, barrier=None):
    """enqueue() launches exactly one region; every repeat is bracketed by CUDA events."""
    ms = []
    for _ in range(repeats):
        if barrier:
            barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            enqueue()
            e1.record(stream)
        stream.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms


def error_block(oracle, got, ref) -> dict:
    e = oracle.error_stats(np.asarray(got, np.float32), np.asarray(ref, np.float32))
    ref64 = np.asarray(ref, np.float64)
    rms = float(np.sqrt(np.mean(ref64 ** 2)))
    peak = float(np.abs(ref64).max())
    return {"max_abs": e["max_abs"], "rmse": e["rmse"], "max_abs_over_rms": e["max_abs"] / rms if rms else None,
            "max_abs_in_ulps_of_largest": e["max_abs"] / float(np.spacing(np.float32(peak))) if peak else None,
            "bit_equal_fraction": float((np.asarray(got, np.float32).view(np.uint32) ==
                                         np.asarray(ref, np.float32).view(np.uint32)).mean())}


def worst(blocks) -> dict:
    out = {}
    for k in blocks[0]:
        vals = [b[k] for b in blocks if b[k] is not None]
        out[k] = (min(vals) if k == "bit_equal_fraction" else max(vals)) if vals else None
    return out


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from colormlm_b200 import _lib as L
    from colormlm_b200 import build as cuda_build
    from colormlm_b200 import ep, synth
    from colormlm_b200.s14 import DecodeStack, S14Context, TokenRoute

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    if rank == 0:
        cuda_build.build()
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    workload = args.workload or ("stack" if world == 1 else "layer")
    if world > 1 and workload in ("prefill", "verify8"):
        return run_prefill_ep(args, torch, dist, L, ep, S14Context, rank, world, local_rank, 8 if workload == "verify8" else None)
    if world > 1 and workload != "layer":
        raise SystemExit("several GPUs: the expert-parallel workloads are `layer`, `prefill` and `verify8`")
    if workload in ("expert_chain", "wq_a", "verify8", "prefill", "glue"):
        return run_small_workload(args, workload, torch, L, synth, S14Context, TokenRoute)
    if workload == "decode":
        return run_decode_workload(args, torch, L, synth, S14Context)

    ctx = S14Context(local_rank)
    mode = L.ACCUM_REFERENCE if args.accum == "reference" else L.ACCUM_PAIRWISE
    ctx.set_accumulation(mode)
    n_layers = max(1, min(args.layers, N_LAYERS))
    layers = resident_layers(torch, n_layers, rank, world)
    _note("layers resident")
    n_tok = 64
    xs_np = tokens(n_tok)
    xs = torch.from_numpy(xs_np).cuda()
    ys = torch.empty((max(n_layers, 2), HIDDEN), dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    barrier = (lambda: (dist.barrier(), torch.cuda.synchronize())) if world > 1 else None
    peer_exchange = world > 1 and args.exchange == "peer" and args.accum == "pairwise"
    if peer_exchange:
        ep.connect_exchange(ctx, rank, world, HIDDEN)
        # a rank that waits longer than about 20 ms for a peer gives the step up (status 0x5503,
        # reported below for every rank) instead of stalling the run
        ctx.ep_exchange_set_wait_limit(1 << 14)
    slots = torch.zeros((TOP_K + 1, HIDDEN), dtype=torch.float32, device="cuda")
    ep_ids = torch.empty(TOP_K, dtype=torch.int32, device="cuda")
    ep_w = torch.empty(TOP_K, dtype=torch.float32, device="cuda")
    ep_states = []
    for ly in layers:
        st_ = dict(ly)
        if st_["shared"] is None:
            st_["shared"] = ly["pages"].data_ptr()  # never read: this rank is not the owner
        ep_states.append(st_)

    # ---- what a region of K steps launches -------------------------------------------------
    stacks = {}

    def stack_of(first: int, count: int):
        key = (first, count)
        if key not in stacks:
            stacks[key] = DecodeStack(ctx, [layers[(first + i) % n_layers] for i in range(count)], inter=INTER, residual=True)
        return stacks[key]

    h_out = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")

    def enqueue_steps(k_steps: int, first_step: int, handle):
        """k_steps layer-tokens starting at step `first_step`; returns the launches of the layer kernel."""
        if workload == "stack":
            done, launches = 0, 0
            while done < k_steps:
                # a launch walks N_LAYERS layers; with fewer resident layers (profiler captures) it cycles through them
                count = min(N_LAYERS, k_steps - done)
                stack_of(0, count).cmd_decode(xs[((first_step + done) // N_LAYERS) % n_tok], h_out, stream=handle)
                done += count
                launches += 1
            return launches
        for i in range(first_step, first_step + k_steps):
            ly = layers[i % n_layers]
            if world == 1:
                ctx.cmd_routed_moe_layer(xs[i % n_tok], ly["wr"], ly["bias"], ly["table"], ly["shared"], L.PAGE_MXFP4,
                                         INTER, ys[i % n_layers], stream=handle)
            elif peer_exchange:
                ep.decode_step_fused(ctx, xs[i % n_tok], ep_states[i % n_layers], ys[i % n_layers], layer=i % n_layers,
                                     world=world, inter=INTER, stream=handle)
            else:
                ep.decode_step(ctx, xs[i % n_tok], ep_states[i % n_layers], slots, ep_ids, ep_w, ys[i % n_layers],
                               layer=i % n_layers, rank=rank, world=world, inter=INTER, stream=handle)
        return k_steps

    if world > 1:
        dist.barrier()
    if world == 1:
        # the stacks a region needs are bound before anything is captured (binding allocates)
        stack_of(0, N_LAYERS)
        if args.steps % N_LAYERS:
            stack_of(0, args.steps % N_LAYERS)
    with torch.cuda.stream(stream):
        enqueue_steps(min(n_layers, 3) if workload == "layer" else N_LAYERS, 0, stream.cuda_stream)  # module load
    stream.synchronize()
    _note("eager warm-up launches done")
    use_graph = world == 1 or peer_exchange
    graph = None
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                enqueue_steps(args.steps, 0, stream.cuda_stream)
        launch_mode = f"cuda graph of the {args.steps} steps of a region"
    else:
        # NCCL all-reduces replayed from a CUDA graph ran ~10x slower than eager ones here
        launch_mode = "eager launches (layer kernel with its router, NCCL all-reduce, mix per step)"
    launches_per_region = None

    def region():
        nonlocal launches_per_region
        if graph is not None:
            graph.replay()
        else:
            enqueue_steps(args.steps, 0, stream.cuda_stream)

    # launches of our kernels per region, counted by the context on an eager pass
    with torch.cuda.stream(stream):
        c0 = ctx.launch_count
        enqueue_steps(args.steps, 0, stream.cuda_stream)
        launches_per_region = ctx.launch_count - c0
    stream.synchronize()
    warm_regions = max(1, -(-args.warmup // args.steps))
    with torch.cuda.stream(stream):
        for _ in range(warm_regions):
            region()
    stream.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ctx.device_status()  # read and clear: what is reported covers the timed regions and the host leg
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    # keep the regions running until the sampler has seen the GPU under load a few times
    ms_all = timed_repeats(torch, stream, region, args.repeats, barrier)
    extra = 0
    while rank == 0 and world == 1 and sampler.samples() < 6 and extra < 2000:
        ms_all += timed_repeats(torch, stream, region, 10)
        extra += 10
    if world > 1:
        t = torch.tensor(ms_all[:args.repeats], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every repeat: the slowest rank
        ms_all = [float(v) for v in t.tolist()]
    clocks = sampler.stop() if rank == 0 else None
    ms = float(np.median(ms_all))
    value = args.steps / (ms / 1e3)
    _note(f"timed regions done: median {ms:.4f} ms")
    # the status word of every rank after the timed regions alone (reading clears it)
    status_timed = ctx.device_status()
    if world > 1:
        t = torch.tensor([status_timed], dtype=torch.int64, device="cuda")
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        status_timed = [int(g.item()) for g in gathered]

    # ---- optional: one launch of the profiling build, time marks of its second layer
    layer_trace = None
    if args.trace and world == 1 and workload == "stack":
        layer_trace = trace_of_a_launch(torch, ctx, stack_of(0, N_LAYERS), xs[0], h_out, stream,
                                        (clocks or {}).get("sm_mhz") or 1965.0)

    # ---- the layer kernel with the routes given (no expert scoring), for the roofline entry's breakdown
    layer_ms = None
    if world == 1 and not args.kernel_only_skip_fixed:
        rr = np.random.default_rng(7)
        fixed = []
        for k in range(n_layers):
            ly = layers[k]
            ids = rr.permutation(N_EXPERTS)[:TOP_K].tolist()
            fixed.append(([TokenRoute(ids, [1.0 / TOP_K] * TOP_K, [ly["pages"].data_ptr() + e * PAGE_BYTES for e in ids])],
                          ly["shared"]))

        def enqueue_fixed():
            for k in range(n_layers):
                route, shared = fixed[k]
                ctx.cmd_moe_layer(xs[k:k + 1], ys[k:k + 1], route, shared, L.PAGE_MXFP4, HIDDEN, INTER,
                                  stream=stream.cuda_stream)

        with torch.cuda.stream(stream):
            enqueue_fixed()
        stream.synchronize()
        g_fixed = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g_fixed, stream=stream):
                enqueue_fixed()
        layer_ms = float(np.median(timed_repeats(torch, stream, g_fixed.replay, 30))) / n_layers

    # ---- the other way of launching the same steps, and the bit-identical order, for comparison
    other = {}
    if world == 1 and not args.kernel_only:
        def time_variant(name, accum, wl):
            nonlocal workload
            saved_mode, saved_wl = ctx.accumulation, workload
            ctx.set_accumulation(accum)
            workload = wl
            try:
                with torch.cuda.stream(stream):
                    enqueue_steps(n_layers, 0, stream.cuda_stream)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    with torch.cuda.graph(g, stream=stream):
                        enqueue_steps(n_layers, 0, stream.cuda_stream)
                other[name] = float(np.median(timed_repeats(torch, stream, g.replay, 20))) / n_layers
            finally:
                ctx.set_accumulation(saved_mode)
                workload = saved_wl

        if args.accum == "pairwise":
            time_variant("single_layer_launch_ms_per_step" if workload == "stack" else "stack_launch_ms_per_step",
                         L.ACCUM_PAIRWISE, "layer" if workload == "stack" else "stack")
            time_variant("reference_order_ms_per_step", L.ACCUM_REFERENCE, "layer")

    # ---- parity of the timed path on its own steps, against the CPU oracle on the same bytes
    parity = None
    sha = None
    if not args.kernel_only and (rank == 0 or world > 1):
        from oracle import s14_oracle as oracle

        oracle.build()
        cpu_threads(oracle)
        hp = HostPages()
        if rank == 0:
            page0 = layers[0]["pages"][0].cpu().numpy()
            host0 = synth.hashed_expert_page(0, layers[0]["owned"][0], HIDDEN, INTER)
            sha = {"gpu": hashlib.sha256(page0.tobytes()).hexdigest(), "host": hashlib.sha256(host0.tobytes()).hexdigest()}
            sha["match"] = sha["gpu"] == sha["host"]
        if workload == "stack" and rank == 0:
            # one token through the whole chain: every layer's output and the final token
            outs = []
            per_layer = [dict(ly) for ly in layers]
            for ly in per_layer:
                ly["y"] = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
                ly["ids"] = torch.empty(TOP_K, dtype=torch.int32, device="cuda")
            st = DecodeStack(ctx, per_layer, inter=INTER, residual=True)
            hh = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
            st.cmd_decode(xs[0], hh)
            torch.cuda.synchronize()
            b32, b64, routes_ok = [], [], True
            h64 = xs_np[0].copy()
            for l in range(n_layers):
                # the CPU chain runs on its own (double-accumulated layers); the F32-order layer is given
                # the same layer input, so that its figure is the summation-order noise of one layer and
                # not the divergence of two chains
                y64, ids64, _ = cpu_layer(oracle, hp, l, h64, acc64=True)
                y32, _, _ = cpu_layer(oracle, hp, l, h64, acc64=False)
                got = per_layer[l]["y"].cpu().numpy()
                routes_ok = routes_ok and bool(np.array_equal(per_layer[l]["ids"].cpu().numpy(), ids64))
                b64.append(error_block(oracle, got, y64))
                b32.append(error_block(oracle, got, y32))
                h64 = (h64 + y64).astype(np.float32)
            st.close()
            parity = {"steps": n_layers, "what": "one token through the chain, every layer's output, independent CPU chain "
                                                 "(double-accumulated); outputs grow with depth, see max_abs_in_ulps_of_largest",
                      "routes_bit_exact": routes_ok,
                      "vs_double_accumulated_oracle": worst(b64), "vs_f32_order_oracle": worst(b32),
                      "final_token_vs_double_accumulated": error_block(oracle, hh.cpu().numpy(), h64)}
        elif workload == "layer":
            n_check = 8
            b32, b64, routes_ok = [], [], True
            idsd = torch.empty(TOP_K, dtype=torch.int32, device="cuda")
            yd = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
            digest = hashlib.sha256()
            # the GPU steps first, all ranks in step (a rank that waited for rank 0's CPU check between the
            # steps would run out of its wait limit); the CPU oracle afterwards
            gots, got_ids = [], []
            if world > 1:
                dist.barrier()
            for i in range(n_check):
                ly = layers[i % n_layers]
                if world == 1:
                    ctx.cmd_routed_moe_layer(xs[i], ly["wr"], ly["bias"], ly["table"], ly["shared"], L.PAGE_MXFP4, INTER, yd, idsd)
                elif peer_exchange:
                    ep.decode_step_fused(ctx, xs[i], ep_states[i % n_layers], yd, layer=i % n_layers, world=world, inter=INTER,
                                         ids=idsd)
                else:
                    ep.decode_step(ctx, xs[i], ep_states[i % n_layers], slots, idsd, ep_w, yd, layer=i % n_layers, rank=rank,
                                   world=world, inter=INTER)
                torch.cuda.synchronize()
                gots.append(yd.cpu().numpy().copy())
                got_ids.append(idsd.cpu().numpy().copy())
                digest.update(gots[-1].tobytes())
            for i in range(n_check if rank == 0 else 0):
                y64, ids64, _ = cpu_layer(oracle, hp, i % n_layers, xs_np[i], acc64=True)
                y32, _, _ = cpu_layer(oracle, hp, i % n_layers, xs_np[i], acc64=False)
                routes_ok = routes_ok and bool(np.array_equal(got_ids[i], ids64))
                b64.append(error_block(oracle, gots[i], y64))
                b32.append(error_block(oracle, gots[i], y32))
            y_digest = digest.hexdigest()
            equal = True
            if world > 1:
                all_d = [None] * world
                dist.all_gather_object(all_d, y_digest)
                equal = all(d == all_d[0] for d in all_d)
            if rank == 0:
                parity = {"steps": n_check, "what": "the first layer-tokens of the timed sequence", "routes_bit_exact": routes_ok,
                          "vs_double_accumulated_oracle": worst(b64), "vs_f32_order_oracle": worst(b32),
                          "y_digest": y_digest, "y_equal_across_ranks": equal}

    # ---- end to end through the host-buffer call: pinned x in, result out, every call
    hx = torch.from_numpy(xs_np.copy()).pin_memory()
    hy = torch.empty((HIDDEN,), dtype=torch.float32).pin_memory()
    ids_np, w_np = np.empty(TOP_K, np.int32), np.empty(TOP_K, np.float32)
    hx_addr, hy_addr = hx.data_ptr(), hy.data_ptr()
    e2e_steps = 0 if args.kernel_only else min(max(args.steps, 280), 2800)
    h2d = d2h = 0.0
    if e2e_steps:
        if workload == "stack":
            full = stack_of(0, n_layers)
            e2e_steps = (e2e_steps // n_layers) * n_layers
            calls = e2e_steps // n_layers
            h2d, d2h = HIDDEN * 4 / n_layers, HIDDEN * 4 / n_layers  # one token in and out per n_layers steps

            def e2e_call(i):
                full.decode_host_addresses(hx_addr + (i % n_tok) * HIDDEN * 4, hy_addr)
        elif world == 1:
            bound = [ctx.bind_routed_moe_layer_host(ly["wr"], ly["bias"], ly["table"], ly["shared"], L.PAGE_MXFP4, INTER)
                     for ly in layers]
            calls = e2e_steps
            h2d, d2h = HIDDEN * 4, HIDDEN * 4 + TOP_K * 8

            def e2e_call(i):
                bound[i % n_layers].run_addresses(hx_addr + (i % n_tok) * HIDDEN * 4, hy_addr, ids_np.ctypes.data, w_np.ctypes.data)
        else:
            xd = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
            calls = e2e_steps
            h2d, d2h = HIDDEN * 4, HIDDEN * 4

            def e2e_call(i):
                with torch.cuda.stream(stream):
                    xd.copy_(hx[i % n_tok], non_blocking=True)
                    if peer_exchange:
                        ep.decode_step_fused(ctx, xd, ep_states[i % n_layers], ys[0], layer=i % n_layers, world=world,
                                             inter=INTER, stream=stream.cuda_stream)
                    else:
                        ep.decode_step(ctx, xd, ep_states[i % n_layers], slots, ep_ids, ep_w, ys[0], layer=i % n_layers,
                                       rank=rank, world=world, inter=INTER, stream=stream.cuda_stream)
                    hy.copy_(ys[0], non_blocking=True)
                stream.synchronize()

        if world > 1:
            dist.barrier()
        for i in range(min(calls, 20)):
            e2e_call(i)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(calls):
            e2e_call(i)
        e2e_sec = max(time.perf_counter() - t0, 1e-9)
        if world > 1:
            t = torch.tensor([e2e_sec], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_sec = float(t.item())
        e2e_value = e2e_steps / e2e_sec
    else:
        e2e_value = None
    _note("end-to-end leg done")

    # ---- several GPUs: what every rank streams in a region (the pages of the experts it owns among the
    # steps' routes, its router weights, the token), from the routes of one eager pass over the region
    rank_bytes = None
    if world > 1 and peer_exchange:
        ids_all = torch.zeros((args.steps, TOP_K), dtype=torch.int32, device="cuda")
        dist.barrier()
        with torch.cuda.stream(stream):
            for i in range(args.steps):
                ep.decode_step_fused(ctx, xs[i % n_tok], ep_states[i % n_layers], ys[i % n_layers], layer=i % n_layers,
                                     world=world, inter=INTER, ids=ids_all[i], stream=stream.cuda_stream)
        stream.synchronize()
        ids_np = ids_all.cpu().numpy()
        owned = int(np.sum(ids_np % world == rank)) + sum(1 for i in range(args.steps) if ep.shared_owner(i % n_layers, world) == rank)
        mine = owned * PAGE_BYTES + args.steps * (ROUTER_BYTES + 2 * HIDDEN * 4)
        t = torch.tensor([mine], dtype=torch.int64, device="cuda")
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        rank_bytes = [int(g.item()) for g in gathered]

    # ---- several GPUs: the vocabulary-sharded head (full logits and the greedy token on every rank)
    head_leg = None
    if world > 1 and not args.kernel_only:
        r0, r1 = ep.head_rows(rank, world, VOCAB)
        shard = synth.hashed_head_rows_torch(torch, r0, r1 - r0, HIDDEN)
        n_head = 8
        ep.sharded_head(ctx, xs[0], shard, VOCAB, rank, world)  # warm-up (NCCL all-gather buffers)
        dist.barrier()
        t0 = time.perf_counter()
        toks, lg = [], None
        for i in range(n_head):
            lg, t = ep.sharded_head(ctx, xs[i], shard, VOCAB, rank, world)
            toks.append(int(t))
        head_sec = time.perf_counter() - t0
        mine = (hashlib.sha256(lg.cpu().numpy().tobytes()).hexdigest(), toks)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        if rank == 0:
            from oracle import s14_oracle as oracle

            oracle.build()
            cpu_threads(oracle)
            ref = oracle.head_logits(xs_np[n_head - 1], synth.hashed_head_rows(0, VOCAB, HIDDEN))
            got = lg.cpu().numpy()
            head_leg = {"what": f"BF16 head {VOCAB} x {HIDDEN} in row shards over the ranks, all-gather of the logits, "
                                "greedy token from the ranks' (largest logit, id) pairs",
                        "calls": n_head, "ms_per_call": head_sec / n_head * 1e3,
                        "logits_equal_across_ranks": all(e[0] == everyone[0][0] for e in everyone),
                        "tokens_equal_across_ranks": all(e[1] == everyone[0][1] for e in everyone),
                        "logits_max_abs_vs_oracle": float(np.max(np.abs(got - ref))),
                        "token_equals_oracle": toks[-1] == oracle.greedy_argmax(ref)}
        del shard

    status = ctx.device_status()  # 0 unless a bounded wait of a kernel ran out
    status_all = status
    if world > 1:
        t = torch.tensor([status], dtype=torch.int64, device="cuda")
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        status_all = [int(g.item()) for g in gathered]
    if rank == 0:
        peak, peak_kind = measured_peaks()
        cpu = None
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            from oracle import s14_oracle as oracle

            oracle.build()
            cores = cpu_threads(oracle)
            sample = cpu_steps(oracle, 2 + args.cpu_steps)
            cpu_run(oracle, sample[:2])
            sec = cpu_run(oracle, sample[2:])
            cpu = {"value": args.cpu_steps / sec, "unit": "layer-tokens/s", "cores": cores, "kind": "port",
                   "sample": f"{args.cpu_steps} layer-tokens of the same workload and the same bytes (router + 7 experts), "
                             f"{sec:.1f} s of CPU work"}
        kernels_per_step = launches_per_region / args.steps
        achieved = STEP_BYTES * args.steps / (ms * 1e-3) / 1e9
        if world > 1:  # one rank's memory system: the busiest rank's bytes over the same time
            achieved = (max(rank_bytes) if rank_bytes else STEP_BYTES * args.steps / world) / (ms * 1e-3) / 1e9
        # several GPUs: a rank streams the pages it owns; the busiest rank bounds the step
        per_rank = None
        if world > 1:
            hp2 = None
            per_rank = "see parity.y_equal_across_ranks; per-rank bytes depend on the routes"
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "layer-tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "warmup_effective": warm_regions * args.steps,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "launch": ("14 chained layers (h <- h + moe(h)) per launch of the layer kernel, " if workload == "stack"
                                  else "one launch per layer-token, independent tokens, ") + launch_mode,
                       "bench_workload": workload, "layers_resident": n_layers, "accumulation": args.accum,
                       "l2": "inputs larger than L2: 14 x 3.4 GB of pages walked layer by layer, 96 MB per step",
                       "parallelism": (f"ep{world}: expert e on rank e mod {world}, "
                                       + ("down vectors stored into every rank's slot buffer over peer memory by the "
                                          "layer kernel, bounded wait, ordered mix in the same launch" if peer_exchange
                                          else "NCCL all-reduce of the slot buffer + ordered mix"))
                       if world > 1 else "single"},
            "repeats": {"count": len(ms_all), "region_ms_median": ms, "region_ms_min": float(np.min(ms_all)),
                        "region_ms_max": float(np.max(ms_all)), "region_ms_p10": float(np.percentile(ms_all, 10)),
                        "region_ms_p90": float(np.percentile(ms_all, 90))},
            "hbm_gbs": achieved, "hbm_frac_of_measured_peak": achieved / (peak * world),
            "algorithmic_bytes_per_step": STEP_BYTES,
            "roofline": {"bound": "hbm",
                         "kernel": ("k_moe_layer_umma: expert scores + routes, 7 MXFP4 experts (up projections, SwiGLU, "
                                    "down projection), ordered mix" + (", 14 layers per launch" if workload == "stack" else "")
                                    if args.accum == "pairwise" else "reference-order layer kernels (router, up, down, mix)"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         **({} if world == 1 else {
                             "what": "the busiest rank: the bytes it streams in a region (pages of the experts it owns "
                                     "among the routes, its router weights, the tokens) over the region's time",
                             "per_rank_bytes_per_step": None if rank_bytes is None else [b / args.steps for b in rank_bytes]}),
                         "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_BYTES,
                         "bytes_per_launch": STEP_BYTES * (N_LAYERS if workload == "stack" else 1),
                         "ms_per_launch": ms / args.steps * (N_LAYERS if workload == "stack" else 1),
                         "timed": "the timed regions (median repeat): every step is part of a launch of this kernel, "
                                  "CUDA events on the launching stream",
                         "fixed_routes_ms_per_launch": layer_ms, **other},
            "parity": parity, "pages_sha256_sample": sha,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "layer-tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps,
                    "call": ("s14_stack_decode_host: one token per call through the 14 layers" if workload == "stack" else
                             "s14_routed_moe_layer_host per layer-token" if world == 1 else
                             "pinned token in, expert-parallel step, result out per layer-token")},
            "layer_trace": layer_trace, "sharded_head": head_leg,
            "gpu_launches": launches_per_region, "kernels_per_step": kernels_per_step,
            "device_status": status, "device_status_all": status_all, "device_status_timed_regions": status_timed,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        if peer_exchange:
            # teardown of the exchange in its order: every rank disconnects, host barrier, buffers freed
            ep.disconnect_exchange(ctx)
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)  # skip NCCL teardown, which did not return here after the run
    for st in stacks.values():
        st.close()
    ctx.close()


VOCAB = 129_280  # scheduler/s14_runner/src/memory.rs:7


def run_decode_workload(args, torch, L, synth, S14Context) -> None:
    """Sequential greedy decode steps through the stack (runner.rs:312-358, 485-508): per step ONE
    launch of the layer kernel over the 14 chained layers, the BF16 head (129 280 x 4096) and the
    greedy argmax; the next step's input is looked up by the token just produced, so no step can
    start before the one before it has finished.  `--steps` decode steps (default 128) replay from
    a CUDA graph; a metric unit is one decode step (token)."""
    from colormlm_b200.s14 import DecodeStack
    from oracle import s14_oracle as oracle

    steps = args.steps if args.steps_given else 128
    ctx = S14Context(0)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    layers = resident_layers(torch, N_LAYERS, 0, 1)
    head = synth.hashed_head_rows_torch(torch, 0, VOCAB, HIDDEN)
    n_tok = 64
    xs_np = tokens(n_tok)
    xs = torch.from_numpy(xs_np).cuda()
    stack = DecodeStack(ctx, layers, inter=INTER, residual=True)
    stream = torch.cuda.Stream()

    # ---- the prefill that precedes the decode steps: PREFILL_TOKENS tokens through the 14 chained layers,
    # h <- h + moe_l(h) for every token, each layer one call of the grouped block path ----
    from colormlm_b200.s14 import MoeBlock

    n_pre = PREFILL_TOKENS
    blk = MoeBlock(ctx, HIDDEN, INTER, n_pre)
    blk.set_residual(True)
    xp_np = tokens(n_pre)
    xp = torch.from_numpy(xp_np).cuda()
    hp_buf = torch.empty_like(xp)

    def run_prefill(handle):
        hp_buf.copy_(xp)
        for lay in layers:
            blk.cmd_routed_moe_block(hp_buf, lay["wr"], lay["bias"], lay["table"], lay["shared"], hp_buf,
                                     score_fn=L.SCORE_SIGMOID, top_k=TOP_K, route_scale=1.0, stream=handle)

    with torch.cuda.stream(stream):
        run_prefill(stream.cuda_stream)
    stream.synchronize()
    prefill_h = hp_buf.cpu().numpy().copy()
    prefill_status = ctx.device_status()
    c0 = ctx.launch_count
    gpre = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(gpre, stream=stream):
            run_prefill(stream.cuda_stream)
    prefill_launches = ctx.launch_count - c0
    with torch.cuda.stream(stream):
        for _ in range(3):
            gpre.replay()
    stream.synchronize()
    pre_ms = timed_repeats(torch, stream, gpre.replay, 10)
    prefill_graph_equal = bool(np.array_equal(hp_buf.cpu().numpy().view(np.uint32), prefill_h.view(np.uint32)))
    prefill = {"tokens": n_pre, "layers": N_LAYERS, "ms_median": float(np.median(pre_ms)), "ms_min": float(np.min(pre_ms)),
               "tokens_per_s": n_pre / (float(np.median(pre_ms)) / 1e3), "layer_tokens_per_s": n_pre * N_LAYERS / (float(np.median(pre_ms)) / 1e3),
               "gpu_launches": prefill_launches, "device_status": prefill_status, "graph_equals_eager": prefill_graph_equal,
               "path": "s14_cmd_routed_moe_block with residual, one call per layer (router, digit rows, grouping, two tcgen05 "
                       "contractions, mix)"}
    h = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
    logits = torch.empty(VOCAB, dtype=torch.float32, device="cuda")
    tok = torch.zeros(1, dtype=torch.int64, device="cuda")
    x_cur = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
    toks_out = torch.zeros(steps, dtype=torch.int64, device="cuda")

    def one_step(i, handle):
        stack.cmd_decode(x_cur, h, stream=handle)
        ctx.cmd_head_logits(h, head, logits, stream=handle)
        ctx.cmd_greedy_argmax(logits, tok, stream=handle)
        toks_out[i:i + 1].copy_(tok)
        x_cur.copy_(xs.index_select(0, torch.remainder(tok, n_tok))[0])  # the next token's input

    def run_steps(handle):
        x_cur.copy_(xs[0])
        for i in range(steps):
            one_step(i, handle)

    with torch.cuda.stream(stream):
        run_steps(stream.cuda_stream)
    stream.synchronize()
    eager_tokens = toks_out.cpu().numpy().copy()
    c0 = ctx.launch_count
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            run_steps(stream.cuda_stream)
    launches = ctx.launch_count - c0
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.2)
    warm = max(3, -(-args.warmup // steps))
    with torch.cuda.stream(stream):
        for _ in range(warm):
            graph.replay()
    stream.synchronize()
    ms_all = timed_repeats(torch, stream, graph.replay, max(5, min(args.repeats, 20)))
    clocks = sampler.stop()
    ms = float(np.median(ms_all))
    graph_tokens = toks_out.cpu().numpy().copy()
    status = ctx.device_status()

    # parity: the first decode steps on the CPU oracle (double-accumulated layers, head, greedy argmax)
    parity = None
    cpu = None
    if not args.kernel_only:
        oracle.build()
        cores = cpu_threads(oracle)
        hp = HostPages()
        head_np = synth.hashed_head_rows(0, VOCAB, HIDDEN)
        n_check = 2
        x = xs_np[0].copy()
        cpu_tokens, worst_logit = [], 0.0
        t0 = time.perf_counter()
        for i in range(n_check):
            hh = x.copy()
            for l in range(N_LAYERS):
                y64, _, _ = cpu_layer(oracle, hp, l, hh, acc64=True)
                hh = (hh + y64).astype(np.float32)
            lg = oracle.head_logits(hh, head_np)
            t = oracle.greedy_argmax(lg)
            cpu_tokens.append(int(t))
            x = xs_np[t % n_tok].copy()
        cpu_sec = time.perf_counter() - t0
        # the GPU's logits of the last step of a one-step run, against the oracle's for the same token
        with torch.cuda.stream(stream):
            x_cur.copy_(xs[0])
            one_step(0, stream.cuda_stream)
        stream.synchronize()
        hh = xs_np[0].copy()
        for l in range(N_LAYERS):
            y64, _, _ = cpu_layer(oracle, hp, l, hh, acc64=True)
            hh = (hh + y64).astype(np.float32)
        lg = oracle.head_logits(hh, head_np)
        worst_logit = float(np.max(np.abs(logits.cpu().numpy() - lg)))
        # the prefill: the last token's (and the first's) state after the 14 layers against the CPU oracle chain
        pre_blocks = []
        for t in (0, n_pre - 1):
            hh = xp_np[t].copy()
            for l in range(N_LAYERS):
                y64, _, _ = cpu_layer(oracle, hp, l, hh, acc64=True)
                hh = (hh + y64).astype(np.float32)
            pre_blocks.append(error_block(oracle, prefill_h[t], hh))
        prefill["parity"] = {"what": "tokens 0 and 369 after the 14 chained layers against the CPU oracle chain (double-accumulated layers)",
                             "vs_double_accumulated_oracle": worst(pre_blocks)}
        parity = {"steps": n_check, "what": "greedy tokens of the first decode steps against the CPU oracle chain "
                                            "(14 double-accumulated layers, head, argmax); logits of the first step",
                  "tokens_gpu": [int(v) for v in graph_tokens[:n_check]], "tokens_cpu": cpu_tokens,
                  "tokens_equal": [int(v) for v in graph_tokens[:n_check]] == cpu_tokens,
                  "graph_equals_eager": bool(np.array_equal(graph_tokens, eager_tokens)),
                  "first_step_logits_max_abs": worst_logit,
                  "logits_tolerance": "rtol 2e-7 / atol 3e-7 of tests/test_final_head.py:68-70 scaled by the logits' size"}
        cpu = {"value": n_check / cpu_sec, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{n_check} decode steps (14 layers + head + argmax each) on the CPU oracle, {cpu_sec:.1f} s"}
    peak, peak_kind = measured_peaks()
    step_bytes = N_LAYERS * STEP_BYTES + VOCAB * HIDDEN * 2 + VOCAB * 4 * 2
    achieved = step_bytes * steps / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "S14 stack decode: 14 chained MoE layers (1 token, top-6 of 256 + shared, 4096 x 2048, MXFP4) "
                               "+ BF16 head 129 280 x 4096 + greedy argmax per step, every step fed by the token before",
                   "bench_workload": "decode", "launch": f"cuda graph of {steps} sequential steps",
                   "l2": "inputs larger than L2: 2.4 GB per step"},
        "repeats": {"count": len(ms_all), "region_ms_median": ms, "region_ms_min": float(np.min(ms_all)),
                    "region_ms_max": float(np.max(ms_all))},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": None, "bytes_per_step": step_bytes,
                     "kernel": "k_moe_layer_umma (14 layers) + k_head_logits + k_greedy_argmax per step"},
        "parity": parity, "cpu_baseline": cpu, "e2e": None, "gpu_launches": launches,
        "device_status": status, "clocks": clocks, "prefill": prefill,
    }
    print(json.dumps(line), flush=True)
    blk.close()
    stack.close()
    ctx.close()


TRACE_MARKS = [(64, "router dot products"), (5, "scores written"), (7, "all scores seen"), (9, "token digits written"),
               (6, "token digit scales in tensor memory"), (69, "selection, first level"), (71, "selection, second level"),
               (72, "routes written"), (16, "item 0: first unit in shared memory"), (17, "item 0: accumulators complete"),
               (18, "item 0: epilogue done"), (20, "item 1: first unit"), (21, "item 1: accumulators complete"),
               (22, "item 1: epilogue done"), (47, "item 1: digit tile in shared memory"),
               (24, "item 2: first unit"), (25, "item 2: accumulators complete"), (26, "item 2: epilogue done"),
               (48, "item 2: digit tile in shared memory")]


def trace_of_a_launch(torch, ctx, stack, x, h_out, stream, sm_mhz: float):
    """Medians over the CTAs (and min, max) of the kernel's time marks in the second layer of one
    14-layer launch, in microseconds after the CTA read that layer's token; CTA classes by their place
    in the deal (0-31 hold a shared-expert up item first, 32-75 two routed up items, the others one)."""
    ctx.set_layer_trace(True)
    with torch.cuda.stream(stream):
        stack.cmd_decode(x, h_out, stream=stream.cuda_stream)
    stream.synchronize()
    tr = ctx.read_layer_trace().astype(np.int64)
    ctx.set_layer_trace(False)
    t0 = tr[:, 4]
    out = {"unit": "us after the token of the launch's second layer was read; min/median/max over the CTAs of a class",
           "sm_mhz": sm_mhz, "classes": {}}
    classes = {"ctas 0-31": range(0, 32), "ctas 32-75": range(32, 76), "ctas 76-147": range(76, tr.shape[0])}
    for cname, rng_ in classes.items():
        rows = np.array([c for c in rng_ if c < tr.shape[0]])
        marks = {}
        for col, name in TRACE_MARKS:
            ok = (tr[rows, col] > 0) & (t0[rows] > 0)
            if ok.any():
                v = (tr[rows, col] - t0[rows])[ok] / sm_mhz
                marks[name] = [round(float(v.min()), 2), round(float(np.median(v)), 2), round(float(v.max()), 2)]
        out["classes"][cname] = marks
    return out


def run_prefill_ep(args, torch, dist, L, ep, S14Context, rank: int, world: int, local_rank: int, block_tokens=None) -> None:
    """The prefill block (PREFILL_TOKENS tokens through one layer) expert-parallel over `world` GPUs: tokens
    on every rank, experts sharded (expert e on rank e mod world), every rank runs the grouped block path on
    the experts it owns, one NCCL all-reduce adds the pair buffers up, every rank mixes.  Timed with CUDA
    events between barriers, max over ranks; y must be the same bits on every rank and equal the CPU
    oracle's for the sampled tokens."""
    from colormlm_b200.s14 import MoeBlock

    steps = args.steps if args.steps_given else (10 if block_tokens is None else 100)
    n_tok = block_tokens or max(1, min(1024, args.tokens if args.tokens > 8 else PREFILL_TOKENS))
    ctx = S14Context(local_rank)
    ctx.set_accumulation(L.ACCUM_PAIRWISE)
    by_token = args.exchange == "peer" and not args.shared_on_owner
    layers = resident_layers(torch, 2, rank, world, shared_everywhere=by_token)
    states = []
    for ly in layers:
        st_ = dict(ly)
        if st_["shared"] is None:
            st_["shared"] = ly["pages"].data_ptr()  # never read: this rank is not the owner
        states.append(st_)
    x_np = tokens(n_tok)
    x = torch.from_numpy(x_np).cuda()
    y = torch.empty_like(x)
    pairs = torch.empty((n_tok * (TOP_K + 1), HIDDEN), dtype=torch.float32, device="cuda")
    ids = torch.empty((n_tok, TOP_K), dtype=torch.int32, device="cuda")
    wts = torch.empty((n_tok, TOP_K), dtype=torch.float32, device="cuda")
    blk = MoeBlock(ctx, HIDDEN, INTER, n_tok)
    peer = args.exchange == "peer"
    if peer:
        ep.connect_block(blk, rank, world)
        blk.ep_set_wait_limit(1 << 16)   # a rank that waits longer than about 0.1 s for a peer gives the call up (status 0x5508)

    def step(i):
        if peer:
            ep.block_layer_fused(blk, x, states[i % 2], y, layer=i % 2, world=world, ids=ids, weights=wts, shared_by_token=by_token)
        else:
            ep.block_layer(blk, x, states[i % 2], pairs, ids, wts, y, layer=i % 2, rank=rank, world=world)

    for i in range(max(3, args.warmup // 4)):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_all = []
    for _ in range(max(5, min(args.repeats, 20))):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_all.append(float(t.item()))
    clocks = sampler.stop() if sampler else None
    # the checked call: the ranks enter it together (rank 0 has just spent a while stopping its clock sampler, and
    # a rank that waits longer than its limit for a peer gives the call up)
    dist.barrier()
    torch.cuda.synchronize()
    step(0)
    torch.cuda.synchronize()
    y_np = y.cpu().numpy()
    digest = hashlib.sha256(y_np.tobytes()).hexdigest()
    digests = [None] * world
    dist.all_gather_object(digests, digest)
    statuses = [None] * world
    dist.all_gather_object(statuses, ctx.device_status())
    chunks = [None] * world   # the ranks' load of the checked call: chunks (expert page, <= 2 or 6 tokens) each runs
    dist.all_gather_object(chunks, blk.last_counts()[0])
    if rank == 0:
        from oracle import s14_oracle as oracle

        oracle.build()
        cores = cpu_threads(oracle)
        hp = HostPages()
        sample = sorted({0, n_tok // 2, n_tok - 1})
        b64 = []
        t0 = time.perf_counter()
        for t_ in sample:
            y64, ids64, _ = cpu_layer(oracle, hp, 0, x_np[t_], acc64=True)
            assert np.array_equal(ids[t_].cpu().numpy(), ids64), "the device's routes differ from the oracle's"
            b64.append(error_block(oracle, y_np[t_], y64))
        cpu_sec = (time.perf_counter() - t0) / len(sample)
        ms = float(np.median(ms_all))
        peak, peak_kind = measured_peaks()
        line = {"metric": "prefill_tokens_per_s" if block_tokens is None else "verify_block_tokens_per_s",
                "value": n_tok * steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
                "steps": steps, "warmup": args.warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"{n_tok}-token prefill through one layer, expert parallel over {world} GPUs: tokens on every "
                                       "rank, experts sharded, grouped block path per rank, " +
                                       ("the w2 kernel stores the owned rows into every rank's pair buffer over NVLink, the mix "
                                        "waits for every rank's rows (no collective call)" if peer else
                                        "one NCCL all-reduce of the pair buffers, mix on every rank"),
                           "exchange": args.exchange,
                           "shared_expert": ("its page on every rank, rank r takes the tokens t with t mod world == r" if by_token
                                             else "on the rank layer mod world"),
                           "bench_workload": "prefill" if block_tokens is None else "verify8",
                           "l2": "inputs larger than L2: two layers of pages alternate",
                           "launch": "eager launches; CUDA events between barriers, max over ranks"},
                "repeats": {"count": len(ms_all), "region_ms_median": ms, "region_ms_min": float(np.min(ms_all)),
                            "region_ms_max": float(np.max(ms_all))},
                "roofline": None,
                "parity": {"vs_double_accumulated_oracle": worst(b64), "tokens_checked": list(sample),
                           "y_sha256_per_rank_equal": len(set(digests)) == 1, "y_sha256": digest},
                "cpu_baseline": {"value": 1.0 / cpu_sec, "unit": "tokens/s", "cores": cores, "kind": "port",
                                 "sample": f"{len(sample)} tokens of the block on the CPU oracle"},
                "e2e": None, "gpu_launches": None, "device_status_per_rank": statuses, "clocks": clocks,
                "exchange_bytes_per_step": int(pairs.numel() * 4), "chunks_per_rank": chunks}
        print(json.dumps(line), flush=True)
    dist.barrier()
    if peer:
        ep.disconnect_block(blk)
    blk.close()
    ctx.close()
    sys.stdout.flush()
    os._exit(0)   # as the layer workload: NCCL's communicator teardown took minutes on this pool


def run_small_workload(args, workload, torch, L, synth, S14Context, TokenRoute) -> None:
    """The single-expert chain (hidden 4096, intermediate 2048, route weight 0.3), the FP8 projection
    matvec (1024 x 4096, 1 / 4 / 8 tokens) and the 8-token verify block: L2-cold by rotating over
    more than 126 MB of distinct weights, timed like the main workload, each with its own roofline
    entry and the CPU oracle timed beside it."""
    from colormlm_b200.pages import ExpertPageLayout
    from oracle import s14_oracle as oracle

    oracle.build()
    cores = cpu_threads(oracle)
    if workload == "prefill" and not args.steps_given:
        args.steps = 10   # a region of ten prefills (some 15 ms)
    ctx = S14Context(0)
    ctx.set_accumulation(L.ACCUM_REFERENCE if args.accum == "reference" else L.ACCUM_PAIRWISE)
    stream = torch.cuda.Stream()
    peak, peak_kind = measured_peaks()
    g = synth.rng(126)
    n_tok = 1
    if workload == "expert_chain":
        n_pages = 16  # 214 MB of distinct pages
        writer = synth.HashedPageWriter(torch, HIDDEN, INTER)
        pages = torch.empty((n_pages, PAGE_BYTES), dtype=torch.uint8, device="cuda")
        for e in range(n_pages):
            writer.fill(pages[e], 100, e)
        x_np = synth.activations(g, 1, HIDDEN)
        x = torch.from_numpy(x_np).cuda()
        y = torch.empty_like(x)
        routes = [[TokenRoute([e], [0.3], [pages[e].data_ptr()])] for e in range(n_pages)]
        unit_bytes, what = PAGE_BYTES + 2 * HIDDEN * 4, "single routed expert: w1, w3 -> limited SwiGLU -> w2 -> x 0.3"

        def enqueue():
            for k in range(args.steps):
                ctx.cmd_moe_layer(x, y, routes[k % n_pages], None, L.PAGE_MXFP4, HIDDEN, INTER, stream=stream.cuda_stream)

        def check():
            ctx.cmd_moe_layer(x, y, routes[3], None, L.PAGE_MXFP4, HIDDEN, INTER)
            torch.cuda.synchronize()
            tp = synth.hashed_tensor_page(100, 3, HIDDEN, INTER)
            ref32, _ = oracle.expert_chain_mxfp4(x_np[0], tp, HIDDEN, INTER, 0.3)
            ref64 = oracle.moe_layer_acc64(x_np[0], [tp], np.asarray([0.3], np.float32), None, 2, HIDDEN, INTER)
            return {"vs_double_accumulated_oracle": error_block(oracle, y.cpu().numpy()[0], ref64),
                    "vs_f32_order_oracle": error_block(oracle, y.cpu().numpy()[0], ref32)}

        def cpu_once():
            tp = synth.hashed_tensor_page(100, 3, HIDDEN, INTER)
            t0 = time.perf_counter()
            for _ in range(20):
                oracle.expert_chain_mxfp4(x_np[0], tp, HIDDEN, INTER, 0.3)
            return (time.perf_counter() - t0) / 20
    elif workload == "wq_a":
        n, k, t = 1024, 4096, max(1, min(8, args.tokens))
        n_w = 40  # 168 MB of distinct matrices
        ws = torch.stack([torch.from_numpy(synth.e4m3_codes(synth.rng(900 + i), n, k)) for i in range(n_w)]).cuda()
        s_np = synth.fp8_block_scales_f32(g, n, k)
        sc = torch.from_numpy(s_np).cuda()
        x_np = synth.activations(g, t, k)
        x = torch.from_numpy(x_np).cuda()
        y = torch.empty((t, n), dtype=torch.float32, device="cuda")
        from colormlm_b200.s14 import S14MatvecShape
        disp = [ctx.pipelines.bind_fp8(S14MatvecShape(n, k), x, ws[i].reshape(-1), sc.reshape(-1), y, scale_format=L.SCALE_F32,
                                       n_tokens=t) for i in range(n_w)]
        unit_bytes = n * k + s_np.size * 4 + t * k * 4 + t * n * 4
        what = f"FP8 e4m3 projection matvec 1024 x 4096, one F32 scale per 128 x 128 block, {t} token(s)"

        def enqueue():
            for i in range(args.steps):
                ctx.pipelines.cmd_fp8_matvec(disp[i % n_w], stream=stream.cuda_stream)

        def check():
            ctx.pipelines.cmd_fp8_matvec(disp[2])
            torch.cuda.synchronize()
            w2 = ws[2].cpu().numpy()
            ref32 = np.stack([oracle.fp8_matvec(x_np[i], w2, s_np, n, k) for i in range(t)])
            ref64 = np.stack([oracle.fp8_matvec_f64(x_np[i], w2, s_np, n, k) for i in range(t)])
            return {"vs_double_accumulated_oracle": error_block(oracle, y.cpu().numpy(), ref64),
                    "vs_f32_order_oracle": error_block(oracle, y.cpu().numpy(), ref32)}

        def cpu_once():
            w2 = ws[2].cpu().numpy()
            t0 = time.perf_counter()
            for _ in range(20):
                for i in range(t):
                    oracle.fp8_matvec(x_np[i], w2, s_np, n, k)
            return (time.perf_counter() - t0) / 20
    elif workload == "glue":
        # the steps on either side of the MoE at one site of a layer: hc_pre -> RMSNorm -> (branch) -> hc_post,
        # BF16 streams [T, 4, 4096] as the reference's state; L2-cold by walking 96 distinct hc_fn (151 MB)
        n_tok = max(1, min(1024, args.tokens))
        n_fn = 96
        fn_np, sc_np, ba_np = synth.hc_params(g, HIDDEN)
        fns = torch.from_numpy(fn_np).cuda().unsqueeze(0).repeat(n_fn, 1, 1)
        fns += torch.arange(n_fn, device="cuda", dtype=torch.float32).view(-1, 1, 1) * 1e-4   # distinct matrices
        sc, ba = torch.from_numpy(sc_np).cuda(), torch.from_numpy(ba_np).cuda()
        xs_np = synth.hc_streams(g, n_tok, HIDDEN)
        xs = torch.from_numpy(xs_np).cuda().to(torch.bfloat16)
        nw_np = g.uniform(0.5, 1.5, size=HIDDEN).astype(np.float32)
        nw = torch.from_numpy(nw_np).cuda()
        red = torch.empty((n_tok, HIDDEN), dtype=torch.bfloat16, device="cuda")
        normed, merged = torch.empty_like(red), torch.empty_like(xs)
        post = torch.empty((n_tok, 4), dtype=torch.float32, device="cuda")
        comb = torch.empty((n_tok, 4, 4), dtype=torch.float32, device="cuda")
        unit_bytes = fn_np.nbytes + n_tok * (4 * HIDDEN * 2 * 3 + HIDDEN * 2 * 4) + HIDDEN * 4
        what = (f"layer glue at one site, {n_tok} token(s): hc_pre (24 x 16 384 F32 mixing matrix, Sinkhorn 20) -> RMSNorm -> "
                "hc_post, BF16 streams [T, 4, 4096]")

        def glue_call(i, st):
            ctx.cmd_hc_pre(xs, fns[i % n_fn], sc, ba, red, post, comb, stream=st)
            ctx.cmd_rms_norm(red, nw, normed, stream=st)
            ctx.cmd_hc_post(normed, xs, post, comb, merged, stream=st)

        def enqueue():
            for i in range(args.steps):
                glue_call(i, stream.cuda_stream)

        def _bits(t):
            return t.view(torch.int16).cpu().numpy().view(np.uint16)

        def _f(a):
            return (np.asarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)

        def check():
            glue_call(2, None)
            torch.cuda.synchronize()
            fn2 = fns[2].cpu().numpy()
            r_ref, p_ref, c_ref = oracle.hc_pre(_bits(xs), fn2, sc_np, ba_np, dtype=1)
            n_ref = oracle.rms_norm(r_ref, nw_np, dtype=1)
            m_ref = oracle.hc_post(n_ref, _bits(xs), p_ref, c_ref, dtype=1)
            blk_ = error_block(oracle, merged.float().cpu().numpy().ravel(), _f(m_ref).ravel())
            blk_["coefficients_max_abs"] = float(max(np.abs(post.cpu().numpy() - p_ref).max(), np.abs(comb.cpu().numpy() - c_ref).max()))
            return {"vs_oracle": blk_, "vs_double_accumulated_oracle": blk_}

        def cpu_once():
            fn2 = fns[2].cpu().numpy()
            xb = _bits(xs)
            t0 = time.perf_counter()
            r_ref, p_ref, c_ref = oracle.hc_pre(xb, fn2, sc_np, ba_np, dtype=1)
            n_ref = oracle.rms_norm(r_ref, nw_np, dtype=1)
            oracle.hc_post(n_ref, xb, p_ref, c_ref, dtype=1)
            return time.perf_counter() - t0
    else:  # verify8, prefill: a block of tokens through one layer, grouped by expert
        from colormlm_b200.s14 import MoeBlock

        n_tok = 8 if workload == "verify8" else max(1, min(1024, args.tokens if args.tokens > 8 else PREFILL_TOKENS))
        layers = resident_layers(torch, 2, 0, 1)
        x_np = tokens(n_tok)
        x = torch.from_numpy(x_np).cuda()
        y = torch.empty_like(x)
        ids_dev = torch.empty((n_tok, TOP_K), dtype=torch.int32, device="cuda")
        w_dev = torch.empty((n_tok, TOP_K), dtype=torch.float32, device="cuda")
        blk = MoeBlock(ctx, HIDDEN, INTER, n_tok)
        blk.set_semantics(args.official)
        distinct = []
        for l in range(2):
            wr, bias = router_of_layer(l)
            seen = set()
            for t in range(n_tok):
                ids, _, _, _ = oracle.router(x_np[t], wr, bias, 0, TOP_K, 1.0)
                seen.update(int(e) for e in ids)
            distinct.append(len(seen))
        d_avg = float(np.mean(distinct))
        unit_bytes = int((d_avg + 1) * PAGE_BYTES + ROUTER_BYTES + n_tok * 2 * HIDDEN * 4)
        what = (f"{n_tok}-token {'verify block' if workload == 'verify8' else 'prefill'} through one layer, routes picked on the "
                f"device, tokens grouped by expert: {d_avg:.0f} distinct routed experts + the shared one (every distinct page "
                "counted once), router weights, x and y"
                + ("; the official expert arithmetic (E4M3FN activation quantisation per 128 elements, BF16 results, "
                   "route weight before w2)" if args.official else ""))

        def block_call(l, st):
            lay = layers[l]
            blk.cmd_routed_moe_block(x, lay["wr"], lay["bias"], lay["table"], lay["shared"], y, ids_dev, w_dev,
                                     score_fn=L.SCORE_SIGMOID, top_k=TOP_K, route_scale=1.0, stream=st)

        def enqueue():
            for i in range(args.steps):
                block_call(i % 2, stream.cuda_stream)

        sample = (0, 5) if workload == "verify8" else (0, n_tok // 2, n_tok - 1)

        def check():
            block_call(0, None)
            torch.cuda.synchronize()
            assert ctx.last_layer_path == L.LAYER_PATH_TENSOR_BLOCK
            hp = HostPages()
            b64, b32 = [], []
            if args.official:
                for t in sample:
                    yo, ido, _ = cpu_layer(oracle, hp, 0, x_np[t], official=True)
                    assert np.array_equal(ids_dev[t].cpu().numpy(), ido), "the device's routes differ from the oracle's"
                    b64.append(error_block(oracle, y.cpu().numpy()[t], yo))
                return {"vs_official_oracle": worst(b64), "tokens_checked": list(sample)}
            for t in sample:
                y64, ids64, _ = cpu_layer(oracle, hp, 0, x_np[t], acc64=True)
                y32, _, _ = cpu_layer(oracle, hp, 0, x_np[t], acc64=False)
                assert np.array_equal(ids_dev[t].cpu().numpy(), ids64), "the device's routes differ from the oracle's"
                b64.append(error_block(oracle, y.cpu().numpy()[t], y64))
                b32.append(error_block(oracle, y.cpu().numpy()[t], y32))
            return {"vs_double_accumulated_oracle": worst(b64), "vs_f32_order_oracle": worst(b32), "tokens_checked": list(sample)}

        n_cpu = 8

        def cpu_once():
            # the reference's way through a block: token after token (forward.rs:544-549); a bounded sample of
            # n_cpu tokens, scaled to the block
            hp = HostPages()
            cpu_layer(oracle, hp, 0, x_np[0], official=args.official)
            t0 = time.perf_counter()
            for t in range(n_cpu):
                cpu_layer(oracle, hp, 0, x_np[t % n_tok], official=args.official)
            return (time.perf_counter() - t0) * n_tok / n_cpu

    with torch.cuda.stream(stream):
        enqueue()
    stream.synchronize()
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(gph, stream=stream):
            enqueue()
    c0 = ctx.launch_count
    with torch.cuda.stream(stream):
        enqueue()
    stream.synchronize()
    launches = ctx.launch_count - c0
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.2)
    ms_all = timed_repeats(torch, stream, gph.replay, args.repeats)
    while sampler.samples() < 6 and len(ms_all) < 4000:
        ms_all += timed_repeats(torch, stream, gph.replay, 20)
    clocks = sampler.stop()
    ms = float(np.median(ms_all))
    per_call = n_tok if workload == "prefill" else 1   # a prefill is counted in tokens
    e2e = None
    if workload in ("verify8", "prefill"):
        # the same calls with the block's tokens in pinned host memory and its result read back, inside the timed region
        x_host = torch.from_numpy(x_np).pin_memory()
        y_host = torch.empty_like(x_host).pin_memory()
        n_e2e = min(args.steps, 20)

        def e2e_region():
            for i in range(n_e2e):
                x.copy_(x_host, non_blocking=True)
                block_call(i % 2, stream.cuda_stream)
                y_host.copy_(y, non_blocking=True)

        timed_repeats(torch, stream, e2e_region, 2)
        e2e_ms = float(np.median(timed_repeats(torch, stream, e2e_region, 10)))
        e2e = {"value": per_call * n_e2e / (e2e_ms / 1e3), "unit": "tokens/s" if workload == "prefill" else "calls/s",
               "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": int(y_host.numel() * 4),
               "calls_per_region": n_e2e, "launch": "eager calls, pinned host buffers, copies on the calls' stream"}
    parity = check()
    cpu_sec = cpu_once()
    achieved = unit_bytes * args.steps / (ms * 1e-3) / 1e9
    line = {"metric": {"expert_chain": "expert_chains_per_s", "wq_a": "matvecs_per_s", "verify8": "verify_blocks_per_s",
                       "prefill": "prefill_tokens_per_s", "glue": "layer_glue_calls_per_s"}[workload],
            "value": per_call * args.steps / (ms / 1e3), "unit": "tokens/s" if workload == "prefill" else "calls/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": what, "bench_workload": workload, "accumulation": args.accum,
                       "semantics": "official" if args.official else "f32",
                       "l2": "inputs larger than L2: distinct weights of more than 126 MB walked round-robin",
                       "launch": f"cuda graph of the {args.steps} calls of a region"},
            "repeats": {"count": len(ms_all), "region_ms_median": ms, "region_ms_min": float(np.min(ms_all)),
                        "region_ms_max": float(np.max(ms_all))},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8000": achieved / 8000.0, "peak_kind": peak_kind, "traffic": None,
                         "bytes_per_call": unit_bytes,
                         "note": ("every distinct expert page counted once; the contraction kernels take in 2-3 x these bytes per SM "
                                  "(later chunks of an expert and the token tiles come from the L2), which is what bounds them"
                                  if workload in ("verify8", "prefill") else
                                  "a call of a few MB is bound by launch and memory latency, not by bandwidth")},
            "parity": parity,
            "cpu_baseline": {"value": per_call / cpu_sec, "unit": "tokens/s" if workload == "prefill" else "calls/s", "cores": cores,
                             "kind": "port",
                             "sample": ("8 tokens of the block, token after token, scaled to the block" if workload in ("verify8", "prefill")
                                        else "the same call on the CPU oracle, same bytes"),
                             "ms_per_call": cpu_sec * 1e3},
            "e2e": e2e, "gpu_launches": launches, "device_status": ctx.device_status(), "clocks": clocks}
    print(json.dumps(line), flush=True)
    ctx.close()


def main() -> None:
    global N_EXPERTS, ROUTER_BYTES, STEP_BYTES, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["stack", "layer", "expert_chain", "wq_a", "verify8", "prefill", "glue", "decode"])
    ap.add_argument("--tokens", type=int, default=1, help="tokens of the wq_a workload (1, 4 or 8); of the prefill workload (default 370)")
    ap.add_argument("--official", action="store_true",
                    help="verify8 / prefill on one GPU: the official expert arithmetic instead of the F32 one")
    ap.add_argument("--accum", default="pairwise", choices=["pairwise", "reference"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="several GPUs: down vectors exchanged inside the layer kernel over peer memory, or by NCCL all-reduce")
    ap.add_argument("--shared-on-owner", action="store_true",
                    help="prefill on several GPUs: the shared expert on one rank (layer mod world) instead of dealt by token")
    ap.add_argument("--repeats", type=int, default=50, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--cpu-steps", type=int, default=40)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=N_LAYERS,
                    help="resident layers (3.4 GB each); fewer than 14 is for profiler captures only")
    ap.add_argument("--experts", type=int, default=N_EXPERTS,
                    help="routed experts per layer; fewer than 256 is for profiler captures only (13.4 MB each)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the parity, end-to-end and CPU legs (profiler captures)")
    ap.add_argument("--kernel-only-skip-fixed", action="store_true", help="also skip the fixed-route launches")
    ap.add_argument("--trace", action="store_true",
                    help="stack workload, one GPU: one more launch with the kernel's time marks; their medians go into the line")
    args = ap.parse_args()
    args.steps_given = args.steps is not None
    if args.experts != N_EXPERTS:
        if not 8 <= args.experts <= 256:
            raise SystemExit("--experts: 8..256")
        N_EXPERTS = args.experts
        ROUTER_BYTES = N_EXPERTS * HIDDEN * 2 + N_EXPERTS * 4
        STEP_BYTES = 7 * PAGE_BYTES + ROUTER_BYTES + HIDDEN * 4 + HIDDEN * 4
        WORKLOAD = WORKLOAD.replace("top-6 of 256", f"top-6 of {N_EXPERTS} (reduced pool, not the benchmark)")
    if args.official and (args.gpus != 1 or args.impl != "ours" or args.workload not in ("verify8", "prefill")):
        raise SystemExit("--official: the verify8 and prefill workloads on one GPU")
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 40
        args.warmup = args.warmup if args.warmup is not None else 3
        run_reference(args)
    else:
        args.steps = args.steps if args.steps is not None else 280
        args.warmup = args.warmup if args.warmup is not None else 28
        run_gpu(args)


if __name__ == "__main__":
    main()
