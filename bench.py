#!/usr/bin/env python
"""Benchmark of the S14 MoE layer at 1-token decode: router top-6 + six routed MXFP4
experts + the shared MXFP4 expert, 256 routed experts per layer resident in the page pool.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--accum pairwise|reference]

A step is one layer-token: one token through one MoE layer, a single launch in pairwise order
(expert scores and routes, up projections, SwiGLU, down projection, sums over slices, ordered mix).  14 layers of 257 expert pages each are resident (the S14 stack, 48 GB); the
steps walk the layers round-robin with a fresh token each, so consecutive steps read
disjoint pages and the 96 MB a step touches never comes from L2.  Steps are replayed from
a CUDA graph of 14 layer-steps; time is taken with CUDA events on the launching stream.

One JSON line is printed by rank 0.  `value` is layer-tokens/s with inputs resident in HBM,
`e2e` the same through the host-buffer C-ABI call (H2D of the token and D2H of the result
inside the timed region), `roofline` the layer kernel (a step is one launch of it) against the measured copy bandwidth, `cpu_baseline` the CPU oracle on this box's host cores on a bounded sample.
`--impl reference` times that CPU implementation alone.
"""
from __future__ import annotations

import argparse
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
PAGE_BYTES = 13_369_344
# algorithmic bytes of one layer-token: 7 expert pages + router weights + bias + x + y
ROUTER_BYTES = N_EXPERTS * HIDDEN * 2 + N_EXPERTS * 4
STEP_BYTES = 7 * PAGE_BYTES + ROUTER_BYTES + HIDDEN * 4 + HIDDEN * 4
# layer kernel: 7 expert pages, x in, y out
LAYER_BYTES = 7 * PAGE_BYTES + HIDDEN * 4 + HIDDEN * 4
# DRAM bytes of one launch of the layer kernel at this workload (dram__bytes_read.sum + dram__bytes_write.sum
# of one ncu capture; the summary of that capture is kept under profiles/)
NCU_TRAFFIC_BYTES = 99_866_368
WORKLOAD = ("moe_layer_decode: 1 token, router top-6 of 256 + 6 routed + 1 shared MXFP4 expert, "
            "hidden 4096, intermediate 2048")


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
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
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


# ------------------------------------------------------------------ CPU reference arm

def cpu_pages(layer: int, ids, cache: dict):
    """Host copies of the pages a CPU step needs, generated on demand from per-page seeds."""
    from colormlm_b200 import synth

    out = []
    for e in list(ids) + [N_EXPERTS]:
        key = (layer, int(e))
        if key not in cache:
            cache[key] = synth.mxfp4_expert_page(synth.rng(10_000 + layer * 1000 + int(e)), HIDDEN, INTER)
        out.append(cache[key])
    return out


def cpu_step_setup(n_steps: int):
    """Router weights per layer, tokens, routes and pages for n_steps CPU steps (untimed)."""
    from colormlm_b200 import synth
    from oracle import s14_oracle as oracle

    g = synth.rng(77)
    layers = {}
    steps = []
    cache = {}
    for i in range(n_steps):
        layer = i % N_LAYERS
        if layer not in layers:
            gl = synth.rng(500 + layer)
            layers[layer] = (synth.router_weight_bf16(gl, N_EXPERTS, HIDDEN), synth.router_bias(gl, N_EXPERTS))
        x = synth.activations(g, 1, HIDDEN)[0]
        wr, bias = layers[layer]
        ids, _, _, _ = oracle.router(x, wr, bias, 0, TOP_K, 1.0)
        steps.append((x, wr, bias, cpu_pages(layer, ids, cache)))
        if len(cache) > 64:
            cache.clear()
    return steps


def cpu_run(steps) -> float:
    """Seconds for the CPU oracle to run the given layer-token steps (router + layer)."""
    from oracle import s14_oracle as oracle

    t0 = time.perf_counter()
    for x, wr, bias, pages in steps:
        ids, w, _, _ = oracle.router(x, wr, bias, 0, TOP_K, 1.0)
        oracle.moe_layer(x, pages[:TOP_K], w, pages[TOP_K], 0, HIDDEN, INTER)
    return time.perf_counter() - t0


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import s14_oracle as oracle

    oracle.build()
    cores = oracle.max_threads()
    steps = cpu_step_setup(args.warmup + args.steps)
    cpu_run(steps[:args.warmup])
    sec = cpu_run(steps[args.warmup:])
    value = args.steps / sec
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "layer-tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sec / args.steps, "higher_is_better": True, "scaling": "weak",
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

def make_layer_pages(torch, n_pages: int, gen) -> "torch.Tensor":
    """[n_pages, PAGE_BYTES] uint8 on the device: uniform E2M1 codes, scale codes in [119, 123]."""
    wb = 3 * (HIDDEN * INTER // 2)
    pages = torch.empty((n_pages, PAGE_BYTES), dtype=torch.uint8, device="cuda")
    pages[:, :wb] = torch.randint(0, 256, (n_pages, wb), dtype=torch.uint8, device="cuda", generator=gen)
    pages[:, wb:] = torch.randint(119, 124, (n_pages, PAGE_BYTES - wb), dtype=torch.uint8, device="cuda",
                                  generator=gen)
    return pages


def _note(msg: str) -> None:
    """Progress lines on stderr when S14_BENCH_VERBOSE is set."""
    if os.environ.get("S14_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from colormlm_b200 import _lib as L
    from colormlm_b200 import build as cuda_build
    from colormlm_b200 import synth
    from colormlm_b200.s14 import S14Context

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

    _note("process group ready")
    ctx = S14Context(local_rank)
    mode = L.ACCUM_REFERENCE if args.accum == "reference" else L.ACCUM_PAIRWISE
    ctx.set_accumulation(mode)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)

    # resident state: N_LAYERS x (256 routed + 1 shared) pages, router weights, page tables.
    # With several GPUs the experts are partitioned (expert e on rank e mod N, the shared expert of
    # layer l on rank l mod N) and every rank keeps only the pages it owns.
    from colormlm_b200 import ep

    layers = []
    n_layers = max(1, args.layers)
    for layer in range(n_layers):
        owned = ep.owned_experts(rank, world, N_EXPERTS)
        has_shared = ep.shared_owner(layer, world) == rank
        pages = make_layer_pages(torch, len(owned) + (1 if has_shared else 0), gen)
        gl = synth.rng(500 + layer)
        wr = torch.from_numpy(synth.router_weight_bf16(gl, N_EXPERTS, HIDDEN).view(np.int16)).cuda()
        bias = torch.from_numpy(synth.router_bias(gl, N_EXPERTS)).cuda()
        base = pages.data_ptr()
        addr = [0] * N_EXPERTS
        for slot, e in enumerate(owned):
            addr[e] = base + slot * PAGE_BYTES
        table = torch.tensor(addr, dtype=torch.int64, device="cuda")
        layers.append({"pages": pages, "wr": wr, "bias": bias, "table": table,
                       "shared": base + len(owned) * PAGE_BYTES if has_shared else None})
    n_tok = 64
    xgen = torch.Generator(device="cuda")
    xgen.manual_seed(99)  # the same tokens on every rank
    xs = torch.randn((n_tok, HIDDEN), dtype=torch.float32, device="cuda", generator=xgen)
    ys = torch.empty((N_LAYERS, HIDDEN), dtype=torch.float32, device="cuda")
    slots = torch.zeros((N_LAYERS, TOP_K + 1, HIDDEN), dtype=torch.float32, device="cuda")
    ep_ids = torch.empty((N_LAYERS, TOP_K), dtype=torch.int32, device="cuda")
    ep_w = torch.empty((N_LAYERS, TOP_K), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    # several GPUs, pairwise order: the exchange of the down vectors runs inside the layer kernel over
    # the ranks' mapped slot buffers (one launch per rank and step); --exchange nccl keeps the baseline
    # (owned experts, NCCL all-reduce of the slot buffer, mix kernel)
    peer_exchange = world > 1 and args.exchange == "peer" and args.accum == "pairwise"
    if peer_exchange:
        ep.connect_exchange(ctx, rank, world, HIDDEN)
        # the ranks start together (barrier before the timed region); a rank that waits longer than
        # about 20 ms for a peer gives the step up (status 0x5503, reported below) instead of stalling
        # the run
        ctx.ep_exchange_set_wait_limit(1 << 14)

    def enqueue_step(i: int, stream_handle=None):
        ly = layers[i % n_layers]
        if world == 1:
            ctx.cmd_routed_moe_layer(xs[i % n_tok], ly["wr"], ly["bias"], ly["table"], ly["shared"],
                                     L.PAGE_MXFP4, INTER, ys[i % N_LAYERS], stream=stream_handle)
        else:
            k = i % N_LAYERS
            ly_state = dict(ly)
            if ly_state["shared"] is None:
                ly_state["shared"] = ly["pages"].data_ptr()  # never read: this rank is not the owner
            if peer_exchange:
                ep.decode_step_fused(ctx, xs[i % n_tok], ly_state, ys[k], layer=i % n_layers, world=world,
                                     inter=INTER, stream=stream_handle)
            else:
                ep.decode_step(ctx, xs[i % n_tok], ly_state, slots[k], ep_ids[k], ep_w[k], ys[k],
                               layer=i % n_layers, rank=rank, world=world, inter=INTER, stream=stream_handle)

    _note("layers resident")
    stream = torch.cuda.Stream()
    # Kernels of ours per step, counted by the context: pairwise order one (the layer kernel scores the
    # experts and picks the routes itself); reference order router, up, down, mix.  Expert parallel adds
    # the mix of the exchanged slots (the slot memset is not a kernel of ours, the all-reduce is NCCL's).

    def capture(n_steps: int, first: int):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream):
                for i in range(n_steps):
                    enqueue_step(first + i, stream.cuda_stream)
        return g

    if world > 1:
        dist.barrier()  # first launches load the kernels; the ranks enter them together
    launched_before = ctx.launch_count
    with torch.cuda.stream(stream):
        for i in range(3):  # first launches outside capture (module load)
            enqueue_step(i, stream.cuda_stream)
    stream.synchronize()
    kernels_per_step = (ctx.launch_count - launched_before) // 3
    _note("eager warm-up steps done")
    rem = args.steps % N_LAYERS
    full = args.steps // N_LAYERS
    if world == 1 or peer_exchange:
        launch_mode = "cuda graph of 14 layer-steps"
        graph = capture(N_LAYERS, 0)
        graph_rem = capture(rem, 0) if rem else None
    else:
        # NCCL all-reduces replayed from a CUDA graph ran ~10x slower than eager ones here
        # (0.95 ms against 0.1 ms per step at 2 GPUs), so the expert-parallel steps are launched eagerly
        launch_mode = "eager launches (layer kernel with its router, NCCL all-reduce, mix per step)"
        graph = graph_rem = None

    def replay(n_full: int, with_rem: bool):
        with torch.cuda.stream(stream):
            if graph is None:
                for i in range(n_full * N_LAYERS + (rem if with_rem else 0)):
                    enqueue_step(i, stream.cuda_stream)
                return
            for _ in range(n_full):
                graph.replay()
            if with_rem and graph_rem is not None:
                graph_rem.replay()

    _note(f"launch mode: {launch_mode}")
    warm_full = max(1, (args.warmup + N_LAYERS - 1) // N_LAYERS)
    replay(warm_full, False)
    stream.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    time.sleep(0.25)
    if world > 1:
        dist.barrier()  # the ranks start the timed region together: a rank's kernels wait for the others'
        torch.cuda.synchronize()
    ctx.device_status()  # read and clear: what is reported covers the timed region and the host leg
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
    replay(full, True)
    with torch.cuda.stream(stream):
        e1.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    _note(f"timed region done: {ms:.3f} ms")
    # one token stream: with several GPUs the experts of the same tokens are spread over the ranks
    value = args.steps / (ms / 1e3)

    # The layer kernel with the routes given (no expert scoring): a CUDA graph of one launch per resident
    # layer with fixed routes (six routed experts + the shared one, other pages every launch), replayed back
    # to back and timed with CUDA events on the launching stream.  Not part of the headline number; it shows
    # what the routing costs inside the kernel.
    from colormlm_b200.s14 import TokenRoute

    layer_ms = None
    if world == 1:
        rr = np.random.default_rng(7)
        fixed = []
        for k in range(N_LAYERS):
            ly = layers[k % n_layers]
            ids = rr.permutation(N_EXPERTS)[:TOP_K].tolist()
            fixed.append(([TokenRoute(ids, [1.0 / TOP_K] * TOP_K, [ly["pages"].data_ptr() + e * PAGE_BYTES for e in ids])],
                          ly["shared"]))

        def enqueue_layer_only(k):
            route, shared = fixed[k]
            ctx.cmd_moe_layer(xs[k:k + 1], ys[k:k + 1], route, shared, L.PAGE_MXFP4, HIDDEN, INTER,
                              stream=stream.cuda_stream)

        with torch.cuda.stream(stream):
            for k in range(2):
                enqueue_layer_only(k)
        stream.synchronize()
        g_layer = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g_layer, stream=stream):
                for k in range(N_LAYERS):
                    enqueue_layer_only(k)
        reps = 60
        with torch.cuda.stream(stream):
            for _ in range(5):
                g_layer.replay()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for _ in range(reps):
                g_layer.replay()
            k1.record(stream)
        stream.synchronize()
        layer_ms = k0.elapsed_time(k1) / (reps * N_LAYERS)
    peak, peak_kind = measured_peaks()
    # pairwise order on one GPU: a step is one launch of the layer kernel (routing included), so the timed
    # region itself gives the kernel's duration; otherwise the fixed-route launches stand for it
    one_kernel_step = world == 1 and kernels_per_step == 1
    roof_ms, roof_bytes = (ms / args.steps, STEP_BYTES) if one_kernel_step else (layer_ms, LAYER_BYTES)
    achieved = roof_bytes / (roof_ms * 1e-3) / 1e9 if roof_ms else None

    # end to end through the host-buffer call: pinned x in, y (+ route) out, every step
    hgen = torch.Generator()
    hgen.manual_seed(4242)  # the same host tokens on every rank: the ranks must agree on the routes
    hx = torch.randn((n_tok, HIDDEN), dtype=torch.float32, generator=hgen).pin_memory()
    hy = torch.empty((HIDDEN,), dtype=torch.float32).pin_memory()
    hx_np, hy_np = hx.numpy(), hy.numpy()
    ids_np, w_np = np.empty(TOP_K, np.int32), np.empty(TOP_K, np.float32)
    xd = torch.empty(HIDDEN, dtype=torch.float32, device="cuda")
    e2e_steps = 0 if args.kernel_only else min(args.steps, 2000)
    # one GPU: every layer's call is bound once (descriptor validated and recorded), a step is the
    # foreign call alone: pinned x in, y and the route out
    bound = [ctx.bind_routed_moe_layer_host(ly["wr"], ly["bias"], ly["table"], ly["shared"], L.PAGE_MXFP4, INTER)
             for ly in layers] if world == 1 else None
    hx_addr, hy_addr, ids_addr, w_addr = hx.data_ptr(), hy.data_ptr(), ids_np.ctypes.data, w_np.ctypes.data
    ep_states = []
    for ly in layers:
        st_ = dict(ly)
        if st_["shared"] is None:
            st_["shared"] = ly["pages"].data_ptr()  # never read: this rank is not the owner
        ep_states.append(st_)

    def e2e_step(i):
        if world == 1:
            bound[i % n_layers].run_addresses(hx_addr + (i % n_tok) * HIDDEN * 4, hy_addr, ids_addr, w_addr)
        else:
            with torch.cuda.stream(stream):
                xd.copy_(hx[i % n_tok], non_blocking=True)
                # the per-token host round trip on several GPUs goes through the NCCL exchange (the exchange
                # inside the kernel was measured from CUDA graphs only)
                ep.decode_step(ctx, xd, ep_states[i % n_layers], slots[0], ep_ids[0], ep_w[0], ys[0],
                               layer=i % n_layers, rank=rank, world=world, inter=INTER, stream=stream.cuda_stream)
                hy.copy_(ys[0], non_blocking=True)
            stream.synchronize()

    if world > 1:
        dist.barrier()  # rank 0 has just stopped its clock sampler, which can take two seconds
    for i in range(0 if args.kernel_only else max(3, min(args.warmup, 100))):
        e2e_step(i)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_sec = max(time.perf_counter() - t0, 1e-9)
    if world > 1:
        t = torch.tensor([e2e_sec], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    e2e_value = e2e_steps / e2e_sec
    _note("end-to-end leg done")

    device_status = ctx.device_status()  # 0 unless a bounded wait of a kernel ran out
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            from oracle import s14_oracle as oracle

            oracle.build()
            sample = cpu_step_setup(2 + args.cpu_steps)
            cpu_run(sample[:2])
            sec = cpu_run(sample[2:])
            cpu = {"value": args.cpu_steps / sec, "unit": "layer-tokens/s", "cores": oracle.max_threads(),
                   "kind": "port",
                   "sample": f"{args.cpu_steps} layer-tokens of the same workload (router + 7 experts), "
                             f"{sec:.1f} s of CPU work"}
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "layer-tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm_full * N_LAYERS, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_resident": n_layers, "accumulation": args.accum,
                       "launch": launch_mode,
                       "l2": "inputs larger than L2: 14 x 3.4 GB of pages walked round-robin, 96 MB per step",
                       "parallelism": (f"ep{world}: expert e on rank e mod {world}, "
                                       + ("down vectors stored into every rank's slot buffer over peer memory by the "
                                          "layer kernel, flag wait, ordered mix in the same launch" if peer_exchange
                                          else "NCCL all-reduce of the slot buffer + ordered mix"))
                       if world > 1 else "single"},
            "hbm_gbs": value * STEP_BYTES / 1e9, "hbm_frac_of_measured_peak": value * STEP_BYTES / 1e9 / (peak * world),
            "algorithmic_bytes_per_step": STEP_BYTES,
            "roofline": {"bound": "hbm",
                         "kernel": ("k_moe_layer_umma: expert scores + routes, 7 MXFP4 experts (up projections, SwiGLU, "
                                    "down projection), sums over slices, ordered mix"
                                    if args.accum == "pairwise" else "reference-order layer kernels (up, down, mix)"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak if achieved else None,
                         "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_BYTES if one_kernel_step else None,
                         "bytes_per_launch": roof_bytes, "ms_per_launch": roof_ms,
                         "timed": ("the timed region: one launch per step, CUDA events on the launching stream"
                                   if one_kernel_step else
                                   "CUDA graph of 14 layer launches with fixed routes, 60 replays, CUDA events"),
                         "fixed_routes_ms_per_launch": layer_ms},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "layer-tokens/s", "h2d_bytes_per_step": HIDDEN * 4,
                    "d2h_bytes_per_step": HIDDEN * 4 + TOP_K * 8, "steps": e2e_steps},
            "gpu_launches": kernels_per_step * args.steps,
            "device_status": device_status,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)  # skip NCCL teardown, which did not return here after the run
    ctx.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--accum", default="pairwise", choices=["pairwise", "reference"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="several GPUs: down vectors exchanged inside the layer kernel over peer memory, or by NCCL all-reduce")
    ap.add_argument("--cpu-steps", type=int, default=60)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=N_LAYERS,
                    help="resident layers (3.4 GB each); fewer than 14 is for profiler captures only")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 60
        args.warmup = args.warmup if args.warmup is not None else 3
        run_reference(args)
    else:
        args.steps = args.steps if args.steps is not None else 28000
        args.warmup = args.warmup if args.warmup is not None else 140
        run_gpu(args)


if __name__ == "__main__":
    main()
