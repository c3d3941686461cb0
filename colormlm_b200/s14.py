"""Python mirror of the reference's S14 operator / page-pool interface over the C ABI.

Class and method names follow the Rust types of the reference
(``scheduler/ssd_inference/src/s14_vulkan.rs``, ``vram_pool.rs`` and
``scheduler/s14_runner/src/runner.rs``): ``S14MatvecShape``,
``S14NumericPipelines.bind_* / cmd_*``, ``VramPool``, ``S14MoePages``,
``RouteDecision``.  Device memory is held in torch tensors (torch is only the
allocator and the stream owner here); every operator runs in
``libpolaris_s14_cuda.so`` and raises :class:`S14Error` on any contract or CUDA
failure.  Nothing in this module computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L
from ._lib import S14Error, check

__all__ = [
    "S14Error", "S14MatvecShape", "validate_ue8m0_codes", "validate_e4m3fn_codes", "S14Context",
    "S14NumericPipelines", "VramPool", "S14MoePages", "RouteDecision", "TokenRoute", "DecodeStack",
]


def _u64_out(fn, shape) -> int:
    out = C.c_uint64()
    check(fn(shape, C.byref(out)))
    return out.value


class S14MatvecShape:
    """Byte contracts of one matvec (s14_vulkan.rs:40-114)."""

    def __init__(self, n: int, k: int):
        c = L.MatvecShape()
        check(L.lib().s14_shape_new(n, k, C.byref(c)))
        self.n, self.k = n, k
        self._c = c

    def validate_mxfp4(self) -> "S14MatvecShape":
        check(L.lib().s14_shape_validate_mxfp4(self._c))
        return self

    def validate_fp8(self) -> "S14MatvecShape":
        check(L.lib().s14_shape_validate_fp8(self._c))
        return self

    def fp32_input_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_fp32_input_bytes, self._c)

    def fp32_output_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_fp32_output_bytes, self._c)

    def mxfp4_weight_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_mxfp4_weight_bytes, self._c)

    def mxfp4_scale_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_mxfp4_scale_bytes, self._c)

    def fp8_weight_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_fp8_weight_bytes, self._c)

    def fp8_scale_bytes(self) -> int:
        return _u64_out(L.lib().s14_shape_fp8_scale_bytes, self._c)


def _host_bytes(codes) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(codes, dtype=np.uint8) if isinstance(codes, (bytes, bytearray))
                                else np.asarray(codes, dtype=np.uint8))


def validate_ue8m0_codes(codes) -> None:
    """Rejects the UE8M0 NaN code 0xFF before upload (s14_vulkan.rs:143-148)."""
    a = _host_bytes(codes)
    check(L.lib().s14_validate_ue8m0_codes(a.ctypes.data, a.size, None))


def validate_e4m3fn_codes(codes) -> None:
    """Rejects the E4M3FN NaN codes 0x7F / 0xFF before upload (s14_vulkan.rs:151-156)."""
    a = _host_bytes(codes)
    check(L.lib().s14_validate_e4m3fn_codes(a.ctypes.data, a.size, None))


def _buf(t) -> L.Buffer:
    """{pointer, size} of a torch CUDA tensor, the stand-in for the reference's GpuBuffer."""
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("operator buffers must be contiguous CUDA tensors")
    return L.Buffer(t.data_ptr(), t.numel() * t.element_size())


def _torch_stream() -> int:
    """The handle of torch's current stream.  torch reports its default stream as 0, which the C ABI
    reads as "the context's own stream"; the legacy default stream is passed by its own handle
    (cudaStreamLegacy) instead, so that a call without an explicit stream is ordered with the
    torch work around it."""
    import torch

    h = torch.cuda.current_stream().cuda_stream
    return h if h else 1


class S14Context:
    """One device context: streams, scratch and the accumulation mode (see the header)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(L.lib().s14_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device
        self.pipelines = S14NumericPipelines(self)

    def close(self) -> None:
        """Destroys the context.  A context whose expert-parallel exchange is connected is disconnected
        first (device synchronise, peer mappings closed); the ranks' host barrier between that and the
        freeing of the buffers is the caller's: use `ep.disconnect_exchange` on every rank before
        `close`, which includes it."""
        if self._h:
            L.lib().s14_ep_exchange_disconnect(self._h)
            check(L.lib().s14_ctx_destroy(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def set_accumulation(self, mode: int) -> None:
        check(L.lib().s14_ctx_set_accumulation(self._h, mode))

    @property
    def accumulation(self) -> int:
        return L.lib().s14_ctx_accumulation(self._h)

    @property
    def sm_count(self) -> int:
        return L.lib().s14_ctx_sm_count(self._h)

    @property
    def launch_count(self) -> int:
        return L.lib().s14_ctx_launch_count(self._h)

    @property
    def last_layer_path(self) -> int:
        """Which implementation the last layer or stack call ran (L.LAYER_PATH_*)."""
        return L.lib().s14_ctx_last_layer_path(self._h)

    def synchronize(self) -> None:
        check(L.lib().s14_ctx_synchronize(self._h))

    def device_status(self) -> int:
        s = C.c_uint32()
        check(L.lib().s14_ctx_device_status(self._h, C.byref(s)))
        return s.value

    # ---- fused layer / router / head -------------------------------------------------
    def cmd_moe_layer(self, x, y, routes: Sequence["TokenRoute"], shared_page: Optional[int],
                      shared_kind: int, hidden: int, inter: int, stream: Optional[int] = None) -> None:
        desc, keep = _layer_desc(routes, shared_page, shared_kind, hidden, inter)
        desc.x, desc.y = x.data_ptr(), y.data_ptr()
        check(L.lib().s14_cmd_moe_layer(self._h, stream if stream is not None else _torch_stream(),
                                        C.byref(desc)))
        del keep

    def moe_layer_host(self, host_x: np.ndarray, host_y: np.ndarray, routes: Sequence["TokenRoute"],
                       shared_page: Optional[int], shared_kind: int, hidden: int, inter: int) -> None:
        """Host buffers in, host buffers out (copies inside the call); pages stay resident."""
        desc, keep = _layer_desc(routes, shared_page, shared_kind, hidden, inter)
        assert host_x.dtype == np.float32 and host_y.dtype == np.float32
        check(L.lib().s14_moe_layer_host(self._h, C.byref(desc), host_x.ctypes.data, host_y.ctypes.data))
        del keep

    def cmd_router(self, x, wr_bf16, bias, ids_out, weights_out, *, score_fn: int = L.SCORE_SIGMOID,
                   top_k: int = 6, route_scale: float = 1.0, stream: Optional[int] = None) -> None:
        d = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        check(L.lib().s14_cmd_router(self._h, stream if stream is not None else _torch_stream(),
                                     C.byref(d)))

    def cmd_routed_moe_layer(self, x, wr_bf16, bias, page_table, shared_page: Optional[int],
                             shared_kind: int, inter: int, y, ids_out=None, weights_out=None, *,
                             score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0,
                             stream: Optional[int] = None) -> None:
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter = inter
        d.shared_kind = shared_kind
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        d.y = y.data_ptr()
        check(L.lib().s14_cmd_routed_moe_layer(
            self._h, stream if stream is not None else _torch_stream(), C.byref(d)))

    def cmd_routed_moe_experts_ep(self, x, wr_bf16, bias, page_table, shared_page: Optional[int],
                                  shared_kind: int, inter: int, slots_out, ids_out, weights_out, *,
                                  ep_rank: int, ep_world: int, shared_owner: int,
                                  score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0,
                                  stream: Optional[int] = None) -> None:
        """This rank's share of an expert-parallel decode step: route on every rank, own experts
        only, unmixed outputs by route slot (all-reduce them, then cmd_moe_mix_slots)."""
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter, d.shared_kind = inter, shared_kind
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        check(L.lib().s14_cmd_routed_moe_experts_ep(
            self._h, stream if stream is not None else _torch_stream(), C.byref(d), ep_rank, ep_world,
            shared_owner, slots_out.data_ptr()))

    EP_HANDLE_BYTES = 64

    def ep_exchange_create(self, rank: int, world: int, hidden: int) -> bytes:
        """Allocates this rank's exchange buffer of the expert-parallel layer; returns its CUDA IPC
        handle (64 bytes) for the other ranks' processes."""
        h = (C.c_uint8 * self.EP_HANDLE_BYTES)()
        check(L.lib().s14_ep_exchange_create(self._h, rank, world, hidden, C.cast(h, C.c_void_p)))
        return bytes(h)

    def ep_exchange_connect(self, handles) -> None:
        """``handles``: every rank's handle in rank order (this rank's own entry is not opened)."""
        blob = b"".join(bytes(h) for h in handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(L.lib().s14_ep_exchange_connect(self._h, C.cast(buf, C.c_void_p)))

    def ep_exchange_connect_local(self, ranks) -> None:
        """The ranks are contexts of this process on the same GPU (tests)."""
        arr = (C.c_void_p * len(ranks))(*[r._h for r in ranks])
        check(L.lib().s14_ep_exchange_connect_local(self._h, arr))

    def ep_exchange_set_wait_limit(self, polls: int) -> None:
        check(L.lib().s14_ep_exchange_set_wait_limit(self._h, polls))

    def ep_exchange_disconnect(self) -> None:
        check(L.lib().s14_ep_exchange_disconnect(self._h))

    def ep_exchange_destroy(self) -> None:
        check(L.lib().s14_ep_exchange_destroy(self._h))

    def cmd_routed_moe_layer_ep(self, x, y, wr_bf16, bias, page_table, shared_page: Optional[int], inter: int, *,
                                shared_owner: int, wait_and_mix: bool = True, ids_out=None, weights_out=None,
                                score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0,
                                stream: Optional[int] = None) -> None:
        """One expert-parallel decode step in one launch: routes, owned experts, exchange of the
        down vectors through the ranks' mapped slot buffers, ordered mix into y on every rank."""
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter, d.shared_kind = inter, L.PAGE_MXFP4
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        d.y = y.data_ptr() if y is not None else None
        check(L.lib().s14_cmd_routed_moe_layer_ep(
            self._h, stream if stream is not None else _torch_stream(), C.byref(d), shared_owner,
            1 if wait_and_mix else 0))

    def cmd_moe_mix_slots(self, slots, weights_dev, n_routed: int, has_shared: bool, y,
                          stream: Optional[int] = None) -> None:
        check(L.lib().s14_cmd_moe_mix_slots(self._h, stream if stream is not None else _torch_stream(),
                                            slots.data_ptr(), weights_dev.data_ptr(), n_routed,
                                            1 if has_shared else 0, y.data_ptr(), y.shape[-1]))

    def bind_routed_moe_layer_host(self, wr_bf16, bias, page_table, shared_page: Optional[int], shared_kind: int,
                                   inter: int, *, score_fn: int = L.SCORE_SIGMOID, top_k: int = 6,
                                   route_scale: float = 1.0) -> "RoutedLayerHostCall":
        """Validates and records a layer's routed host-buffer call once (the bind step of the
        reference's bind / cmd split, s14_vulkan.rs:207-415); the returned object runs it per token
        with nothing but the foreign call on the way."""
        d = L.RoutedLayerDesc()
        r = L.RouterDesc()
        r.n_experts, r.hidden, r.n_tokens = wr_bf16.shape[0], wr_bf16.shape[1], 1
        r.top_k, r.score_fn, r.route_scale = top_k, score_fn, route_scale
        r.router_weight_bf16 = wr_bf16.data_ptr()
        r.bias = bias.data_ptr() if bias is not None else None
        d.router = r
        d.inter, d.shared_kind = inter, shared_kind
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        return RoutedLayerHostCall(self, d, (wr_bf16, bias, page_table))

    def routed_moe_layer_host(self, host_x: np.ndarray, host_y: np.ndarray, wr_bf16, bias, page_table,
                              shared_page: Optional[int], shared_kind: int, inter: int,
                              host_ids: Optional[np.ndarray] = None,
                              host_weights: Optional[np.ndarray] = None, *,
                              score_fn: int = L.SCORE_SIGMOID, top_k: int = 6,
                              route_scale: float = 1.0) -> None:
        """One decode token held in host memory: H2D copy, router + layer, D2H copy, wait."""
        d = L.RoutedLayerDesc()
        r = L.RouterDesc()
        r.n_experts, r.hidden, r.n_tokens = wr_bf16.shape[0], wr_bf16.shape[1], 1
        r.top_k, r.score_fn, r.route_scale = top_k, score_fn, route_scale
        r.router_weight_bf16 = wr_bf16.data_ptr()
        r.bias = bias.data_ptr() if bias is not None else None
        d.router = r
        d.inter, d.shared_kind = inter, shared_kind
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        check(L.lib().s14_routed_moe_layer_host(
            self._h, C.byref(d), host_x.ctypes.data, host_y.ctypes.data,
            host_ids.ctypes.data if host_ids is not None else None,
            host_weights.ctypes.data if host_weights is not None else None))

    def set_layer_trace(self, enable: bool) -> None:
        """Time marks inside the tensor-core layer kernel (profiling runs)."""
        check(L.lib().s14_ctx_set_layer_trace(self._h, 1 if enable else 0))

    def read_layer_trace(self):
        """[n_ctas, words] uint64 marks of the last launch of the layer kernel (see the header)."""
        import numpy as np

        cap = 1024 * 128
        out = np.zeros(cap, np.uint64)
        n, w = C.c_uint32(), C.c_uint32()
        check(L.lib().s14_ctx_read_layer_trace(self._h, out.ctypes.data, cap, C.byref(n), C.byref(w)))
        return out[: n.value * w.value].reshape(n.value, w.value)

    def set_kernel_timing(self, enable: bool) -> None:
        check(L.lib().s14_ctx_set_kernel_timing(self._h, 1 if enable else 0))

    def kernel_times(self):
        """({'router','up','down','mix'} total ms, number of timed calls)."""
        ms = (C.c_double * 4)()
        calls = C.c_uint64()
        check(L.lib().s14_ctx_kernel_times(self._h, ms, C.byref(calls)))
        return dict(zip(("router", "up", "down", "mix"), [float(v) for v in ms])), calls.value

    # ---- the steps on either side of the MoE inside one layer (see the header) ---------
    def cmd_hc_pre(self, x, hc_fn, hc_scale, hc_base, reduced, post, comb, *, iters: int = 20, norm_eps: float = 1e-6,
                   hc_eps: float = 1e-6, stream: Optional[int] = None) -> None:
        """x [T, 4, hidden] (float32 or bfloat16) -> reduced [T, hidden], post [T, 4], comb [T, 4, 4]."""
        p = _hc_params(x, hc_fn, hc_scale, hc_base, iters, norm_eps, hc_eps)
        check(L.lib().s14_cmd_hc_pre(self._h, stream if stream is not None else _torch_stream(), C.byref(p), x.data_ptr(),
                                     reduced.data_ptr(), post.data_ptr(), comb.data_ptr()))

    def cmd_hc_post(self, branch, residual, post, comb, merged, stream: Optional[int] = None) -> None:
        """merged [T, 4, hidden] = post * branch + sum_h comb[h] * residual[h]."""
        check(L.lib().s14_cmd_hc_post(self._h, stream if stream is not None else _torch_stream(), residual.shape[0],
                                      residual.shape[1], residual.shape[2], _stream_type(residual), branch.data_ptr(),
                                      residual.data_ptr(), post.data_ptr(), comb.data_ptr(), merged.data_ptr()))

    def cmd_rms_norm(self, x, weight, out, *, eps: float = 1e-6, stream: Optional[int] = None) -> None:
        check(L.lib().s14_cmd_rms_norm(self._h, stream if stream is not None else _torch_stream(), x.shape[0], x.shape[1],
                                       _stream_type(x), x.data_ptr(), weight.data_ptr(), eps, out.data_ptr()))

    def cmd_hc_head_reduce(self, x, hc_fn, hc_scale, hc_base, reduced, pre, *, norm_eps: float = 1e-6, hc_eps: float = 1e-6,
                           stream: Optional[int] = None) -> None:
        p = _hc_params(x, hc_fn, hc_scale, hc_base, 1, norm_eps, hc_eps)
        check(L.lib().s14_cmd_hc_head_reduce(self._h, stream if stream is not None else _torch_stream(), C.byref(p),
                                             x.data_ptr(), reduced.data_ptr(), pre.data_ptr()))

    def cmd_router_hash(self, x, wr_bf16, tid2eid_rows, ids_out, weights_out, *, score_fn: int = L.SCORE_SQRT_SOFTPLUS,
                        route_scale: float = 1.5, stream: Optional[int] = None) -> None:
        """The hash-routed layers: ids from the tokens' tid2eid rows (int64 [T, top_k]), weights from the scores."""
        d = _router_desc(x, wr_bf16, None, ids_out, weights_out, score_fn, tid2eid_rows.shape[-1], route_scale)
        check(L.lib().s14_cmd_router_hash(self._h, stream if stream is not None else _torch_stream(), C.byref(d),
                                          tid2eid_rows.data_ptr()))

    # ---- the executor's two device steps as single calls (see the header) -------------
    def exec_routed_and_shared_moe_then_hc_post(self, ffn_input, residual, post, comb, route: "TokenRoute",
                                                shared_page: Optional[int], shared_kind: int, inter: int, state_out,
                                                moe_branch_out=None, stream: Optional[int] = None) -> None:
        """ffn_input bfloat16 [hidden], residual bfloat16 [4, hidden] -> state_out bfloat16 [4, hidden]."""
        ld, keep = _layer_desc([route], shared_page, shared_kind, ffn_input.shape[-1], inter)
        d = L.ExecMoeDesc()
        d.hidden, d.inter, d.shared_kind = ffn_input.shape[-1], inter, shared_kind
        d.route = C.cast(ld.routes, C.c_void_p)
        d.shared_page = shared_page
        d.ffn_input_bf16, d.residual_bf16 = ffn_input.data_ptr(), residual.data_ptr()
        d.post, d.comb = post.data_ptr(), comb.data_ptr()
        d.state_out_bf16 = state_out.data_ptr()
        d.moe_branch_out_bf16 = moe_branch_out.data_ptr() if moe_branch_out is not None else None
        check(L.lib().s14_exec_routed_and_shared_moe_then_hc_post(
            self._h, stream if stream is not None else _torch_stream(), C.byref(d)))
        del keep

    def exec_hc_head_norm_full_logits(self, state, hc_fn, hc_scale, hc_base, norm_weight, head_weight_bf16, logits_out, *,
                                      norm_eps: float = 1e-6, hc_eps: float = 1e-6, stream: Optional[int] = None) -> None:
        """state bfloat16 [1, 4, hidden] -> logits_out float32 [rows of head_weight_bf16]."""
        p = _hc_params(state, hc_fn, hc_scale, hc_base, 1, norm_eps, hc_eps)
        check(L.lib().s14_exec_hc_head_norm_full_logits(
            self._h, stream if stream is not None else _torch_stream(), C.byref(p), norm_weight.data_ptr(),
            head_weight_bf16.data_ptr(), head_weight_bf16.shape[0], state.data_ptr(), logits_out.data_ptr()))

    def cmd_head_logits(self, x, weight_bf16, logits_out, *, n_rows: Optional[int] = None,
                        stream: Optional[int] = None) -> None:
        n_tokens = 1 if x.dim() == 1 else x.shape[0]
        rows = n_rows if n_rows is not None else weight_bf16.shape[0]
        stride = logits_out.shape[-1]
        check(L.lib().s14_cmd_head_logits(self._h, stream if stream is not None else _torch_stream(),
                                          x.data_ptr(), n_tokens, weight_bf16.data_ptr(), rows,
                                          weight_bf16.shape[1], logits_out.data_ptr(), stride))

    def cmd_greedy_argmax(self, logits, result, stream: Optional[int] = None) -> None:
        check(L.lib().s14_cmd_greedy_argmax(self._h, stream if stream is not None else _torch_stream(),
                                            logits.data_ptr(), logits.numel(), result.data_ptr()))


def _stream_type(t) -> int:
    import torch

    if t.dtype == torch.float32:
        return L.STREAM_F32
    if t.dtype == torch.bfloat16:
        return L.STREAM_BF16
    raise S14Error(L.ERR_CONTRACT, "a token's streams are float32 or bfloat16 tensors")


def _hc_params(x, hc_fn, hc_scale, hc_base, iters, norm_eps, hc_eps) -> "L.HcParams":
    p = L.HcParams()
    p.n_tokens, p.hc, p.hidden = x.shape[0], x.shape[1], x.shape[2]
    p.dtype = _stream_type(x)
    p.sinkhorn_iters, p.norm_eps, p.hc_eps = iters, norm_eps, hc_eps
    p.hc_fn, p.hc_scale, p.hc_base = hc_fn.data_ptr(), hc_scale.data_ptr(), hc_base.data_ptr()
    return p


@dataclass
class TokenRoute:
    """One token's route with its pages resolved to device addresses of pinned slots."""

    expert_ids: Sequence[int]
    weights: Sequence[float]
    pages: Sequence[int]


def _layer_desc(routes, shared_page, shared_kind, hidden, inter):
    arr = (L.TokenRoute * len(routes))()
    for t, r in enumerate(routes):
        n = len(r.expert_ids)
        if n > L.EXPERTS_PER_TOKEN or len(r.weights) != n or len(r.pages) != n:
            raise S14Error(L.ERR_CONTRACT, "a token route holds at most 6 matching ids/weights/pages")
        arr[t].n_routed = n
        for j in range(n):
            arr[t].expert_ids[j] = int(r.expert_ids[j])
            arr[t].weights[j] = float(r.weights[j])
            arr[t].pages[j] = int(r.pages[j])
    d = L.MoeLayerDesc()
    d.hidden, d.inter, d.n_tokens = hidden, inter, len(routes)
    d.shared_kind = shared_kind
    d.shared_page = shared_page
    d.routes = C.cast(arr, C.POINTER(L.TokenRoute))
    return d, arr


class DecodeStack:
    """The MoE layers of a token step, bound once (see the header: s14_stack_create).  ``layers`` is a
    list of dicts with the device tensors ``wr`` (BF16 router weight as int16 / uint16), ``bias``,
    ``table`` (int64 page addresses), the device address ``shared`` (or None) and, optionally,
    ``ids``, ``weights`` ([top_k]) and ``y`` ([hidden]) outputs."""

    def __init__(self, ctx: "S14Context", layers, *, inter: int, shared_kind: int = L.PAGE_MXFP4,
                 score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0, residual: bool = True):
        self._ctx = ctx
        self._keep = layers
        cfg = L.StackConfig()
        cfg.n_layers = len(layers)
        cfg.n_experts, cfg.hidden = layers[0]["wr"].shape[0], layers[0]["wr"].shape[1]
        cfg.inter, cfg.top_k, cfg.score_fn, cfg.route_scale = inter, top_k, score_fn, route_scale
        cfg.shared_kind, cfg.residual = shared_kind, 1 if residual else 0
        arr = (L.StackLayer * len(layers))()
        for i, ly in enumerate(layers):
            arr[i].router_weight_bf16 = ly["wr"].data_ptr()
            arr[i].bias = ly["bias"].data_ptr() if ly.get("bias") is not None else None
            arr[i].page_table = ly["table"].data_ptr()
            arr[i].shared_page = ly.get("shared")
            for field, key in (("ids_out", "ids"), ("weights_out", "weights"), ("y_out", "y")):
                t = ly.get(key)
                setattr(arr[i], field, t.data_ptr() if t is not None else None)
        h = C.c_void_p()
        check(L.lib().s14_stack_create(ctx._h, C.byref(cfg), arr, C.byref(h)))
        self._h = h
        self.hidden, self.n_layers = cfg.hidden, cfg.n_layers

    def cmd_decode(self, x, h_out, stream: Optional[int] = None) -> None:
        check(L.lib().s14_cmd_stack_decode(self._ctx._h, stream if stream is not None else _torch_stream(), self._h,
                                           x.data_ptr(), h_out.data_ptr()))

    def decode_host(self, host_x: np.ndarray, host_h: np.ndarray) -> None:
        check(L.lib().s14_stack_decode_host(self._ctx._h, self._h, host_x.ctypes.data, host_h.ctypes.data))

    def decode_host_addresses(self, host_x: int, host_h: int) -> None:
        rc = L.lib().s14_stack_decode_host(self._ctx._h, self._h, host_x, host_h)
        if rc:
            check(rc)

    def close(self) -> None:
        if self._h:
            L.lib().s14_stack_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoeBlock:
    """A block of tokens (a verify block, a prefill) through one MoE layer with the tokens grouped by
    expert: every distinct expert's page is streamed once (see the header: s14_block_create)."""

    def __init__(self, ctx: "S14Context", hidden: int, inter: int, max_tokens: int):
        self._ctx = ctx
        self.hidden, self.inter, self.max_tokens = hidden, inter, max_tokens
        h = C.c_void_p()
        check(L.lib().s14_block_create(ctx.handle, hidden, inter, max_tokens, C.byref(h)))
        self._h = h

    def cmd_moe_block(self, x, y, routes: Sequence["TokenRoute"], shared_page: Optional[int],
                      stream: Optional[int] = None) -> None:
        """Routes from the host: x, y device [n_tokens, hidden]."""
        desc, keep = _layer_desc(routes, shared_page, L.PAGE_MXFP4, self.hidden, self.inter)
        desc.x, desc.y = x.data_ptr(), y.data_ptr()
        check(L.lib().s14_cmd_moe_block(self._ctx.handle, stream if stream is not None else _torch_stream(),
                                        self._h, C.byref(desc)))
        del keep

    def cmd_routed_moe_block(self, x, wr_bf16, bias, page_table, shared_page: Optional[int], y, ids_out=None,
                             weights_out=None, *, score_fn: int = L.SCORE_SIGMOID, top_k: int = 6,
                             route_scale: float = 1.0, stream: Optional[int] = None) -> None:
        """Router on the device: x, y device [n_tokens, hidden]; ids_out / weights_out [n_tokens, top_k]."""
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter = self.inter
        d.shared_kind = L.PAGE_MXFP4
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        d.y = y.data_ptr()
        check(L.lib().s14_cmd_routed_moe_block(self._ctx.handle, stream if stream is not None else _torch_stream(),
                                               self._h, C.byref(d)))

    def cmd_routed_moe_block_experts_ep(self, x, wr_bf16, bias, page_table, shared_page: Optional[int], pairs_out, ids_out,
                                        weights_out, *, ep_rank: int, ep_world: int, shared_owner: int,
                                        score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0,
                                        stream: Optional[int] = None) -> None:
        """Expert parallel: the pairs of the experts this rank owns into pairs_out [n_tokens * 7, hidden]."""
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter = self.inter
        d.shared_kind = L.PAGE_MXFP4
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        d.y = None
        check(L.lib().s14_cmd_routed_moe_block_experts_ep(
            self._ctx.handle, stream if stream is not None else _torch_stream(), self._h, C.byref(d), ep_rank, ep_world,
            shared_owner, pairs_out.data_ptr()))

    # ---- expert parallel with the exchange inside the block kernels ----
    def ep_create(self, rank: int, world: int) -> bytes:
        handle = (C.c_uint8 * S14Context.EP_HANDLE_BYTES)()
        check(L.lib().s14_block_ep_create(self._h, rank, world, C.cast(handle, C.c_void_p)))
        return bytes(handle)

    def ep_connect(self, handles) -> None:
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(L.lib().s14_block_ep_connect(self._h, C.cast(buf, C.c_void_p)))

    def ep_connect_local(self, ranks) -> None:
        arr = (C.c_void_p * len(ranks))(*[r._h for r in ranks])
        check(L.lib().s14_block_ep_connect_local(self._h, arr))

    def ep_set_wait_limit(self, polls: int) -> None:
        check(L.lib().s14_block_ep_set_wait_limit(self._h, polls))

    def ep_disconnect(self) -> None:
        check(L.lib().s14_block_ep_disconnect(self._h))

    def cmd_routed_moe_block_ep(self, x, wr_bf16, bias, page_table, shared_page: Optional[int], y, ids_out=None,
                                weights_out=None, *, shared_owner: int, wait_and_mix: bool = True,
                                score_fn: int = L.SCORE_SIGMOID, top_k: int = 6, route_scale: float = 1.0,
                                stream: Optional[int] = None) -> None:
        """One call per rank: the owned experts' rows go into every rank's pair buffer inside the w2 kernel, the mix waits
        for every rank's rows (see the header)."""
        d = L.RoutedLayerDesc()
        d.router = _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale)
        d.inter = self.inter
        d.shared_kind = L.PAGE_MXFP4
        d.page_table = page_table.data_ptr()
        d.shared_page = shared_page
        d.y = y.data_ptr() if y is not None else None
        check(L.lib().s14_cmd_routed_moe_block_ep(self._ctx.handle, stream if stream is not None else _torch_stream(), self._h,
                                                  C.byref(d), shared_owner, 1 if wait_and_mix else 0))

    def cmd_mix(self, pairs, ids, weights, y, *, has_shared: bool = True, x_residual=None,
                stream: Optional[int] = None) -> None:
        """The ordered mix of every token from a pairs buffer (after the ranks' buffers were added up)."""
        check(L.lib().s14_cmd_moe_block_mix(
            self._ctx.handle, stream if stream is not None else _torch_stream(), self._h, pairs.data_ptr(), ids.data_ptr(),
            weights.data_ptr(), ids.shape[0], ids.shape[1], 1 if has_shared else 0,
            x_residual.data_ptr() if x_residual is not None else None, y.data_ptr()))

    def set_residual(self, residual: bool) -> None:
        """The calls that follow write y = x + moe(x); y may then be x."""
        check(L.lib().s14_block_set_residual(self._h, 1 if residual else 0))

    def set_semantics(self, official: bool) -> None:
        """The experts' arithmetic of the calls that follow: this library's F32 one, or the official one
        (s14_first_real_token/executor.py:712-743: E4M3FN activation quantisation per 128 elements, BF16
        results, the route weight before w2, y = moe_branch in BF16 values).  One GPU only."""
        check(L.lib().s14_block_set_semantics(self._h, 1 if official else 0))

    def last_counts(self):
        """(chunks, up items, down items, bad id flag) of the last call; synchronise the stream first."""
        out = (C.c_uint32 * 4)()
        check(L.lib().s14_block_last_counts(self._h, out))
        return tuple(int(v) for v in out)

    def close(self) -> None:
        if getattr(self, "_h", None):
            # a connected exchange is closed here (the process is leaving); ranks that go on after this one
            # follow the order of the header: disconnect everywhere, a host barrier, then destroy
            L.lib().s14_block_ep_disconnect(self._h)
            check(L.lib().s14_block_destroy(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RoutedLayerHostCall:
    """A bound routed layer call on host buffers (see S14Context.bind_routed_moe_layer_host)."""

    def __init__(self, ctx: "S14Context", desc, keep_alive):
        self._ctx, self._desc, self._keep = ctx, desc, keep_alive
        self._ref = C.byref(desc)
        self._fn = L.lib().s14_routed_moe_layer_host

    def run_addresses(self, host_x: int, host_y: int, host_ids: int = 0, host_weights: int = 0) -> None:
        """host_x / host_y: addresses of hidden F32 values (pinned memory for speed); host_ids /
        host_weights: addresses of top_k int32 / F32 values, or 0."""
        rc = self._fn(self._ctx._h, self._ref, host_x, host_y, host_ids or None, host_weights or None)
        if rc:
            check(rc)

    def __call__(self, host_x: np.ndarray, host_y: np.ndarray, host_ids: Optional[np.ndarray] = None,
                 host_weights: Optional[np.ndarray] = None) -> None:
        self.run_addresses(host_x.ctypes.data, host_y.ctypes.data,
                           host_ids.ctypes.data if host_ids is not None else 0,
                           host_weights.ctypes.data if host_weights is not None else 0)


def _router_desc(x, wr_bf16, bias, ids_out, weights_out, score_fn, top_k, route_scale):
    d = L.RouterDesc()
    d.n_experts, d.hidden = wr_bf16.shape[0], wr_bf16.shape[1]
    d.n_tokens = 1 if x.dim() == 1 else x.shape[0]
    d.top_k, d.score_fn, d.route_scale = top_k, score_fn, route_scale
    d.x = x.data_ptr()
    d.router_weight_bf16 = wr_bf16.data_ptr()
    d.bias = bias.data_ptr() if bias is not None else None
    d.ids_out = ids_out.data_ptr() if ids_out is not None else None
    d.weights_out = weights_out.data_ptr() if weights_out is not None else None
    return d


class S14NumericPipelines:
    """The five primitive operators (s14_vulkan.rs:187-425): ``bind_*`` validates shapes
    and capacities and returns a dispatch record, ``cmd_*`` enqueues it on a stream."""

    def __init__(self, ctx: S14Context):
        self._ctx = ctx

    def _h(self):
        return self._ctx.handle

    def bind_mxfp4(self, shape: S14MatvecShape, x, packed_weight, weight_scale, y) -> L.Mxfp4Dispatch:
        d = L.Mxfp4Dispatch()
        bx, bw, bs, by = _buf(x), _buf(packed_weight), _buf(weight_scale), _buf(y)
        check(L.lib().s14_bind_mxfp4(self._h(), shape._c, C.byref(bx), C.byref(bw), C.byref(bs),
                                     C.byref(by), C.byref(d)))
        return d

    def bind_fp8(self, shape: S14MatvecShape, x, weight, weight_scale, y, *,
                 scale_format: int = L.SCALE_UE8M0, n_tokens: int = 1) -> L.Fp8Dispatch:
        d = L.Fp8Dispatch()
        bx, bw, bs, by = _buf(x), _buf(weight), _buf(weight_scale), _buf(y)
        check(L.lib().s14_bind_fp8_ex(self._h(), shape._c, scale_format, n_tokens, C.byref(bx),
                                      C.byref(bw), C.byref(bs), C.byref(by), C.byref(d)))
        return d

    def bind_swiglu_limit(self, n: int, gate, up, y) -> L.SwigluLimitDispatch:
        d = L.SwigluLimitDispatch()
        bg, bu, by = _buf(gate), _buf(up), _buf(y)
        check(L.lib().s14_bind_swiglu_limit(self._h(), n, C.byref(bg), C.byref(bu), C.byref(by),
                                            C.byref(d)))
        return d

    def bind_route_mix(self, n: int, route_weight: float, expert, routed) -> L.RouteMixDispatch:
        d = L.RouteMixDispatch()
        be, br = _buf(expert), _buf(routed)
        check(L.lib().s14_bind_route_mix(self._h(), n, route_weight, C.byref(be), C.byref(br),
                                         C.byref(d)))
        return d

    def bind_moe_accumulate(self, n: int, weight: float, expert, accumulator) -> L.MoeAccumulateDispatch:
        d = L.MoeAccumulateDispatch()
        be, ba = _buf(expert), _buf(accumulator)
        check(L.lib().s14_bind_moe_accumulate(self._h(), n, weight, C.byref(be), C.byref(ba),
                                              C.byref(d)))
        return d

    def _stream(self, stream):
        return stream if stream is not None else _torch_stream()

    def cmd_mxfp4_matvec(self, dispatch, stream=None) -> None:
        check(L.lib().s14_cmd_mxfp4_matvec(self._h(), self._stream(stream), C.byref(dispatch)))

    def cmd_fp8_matvec(self, dispatch, stream=None) -> None:
        check(L.lib().s14_cmd_fp8_matvec(self._h(), self._stream(stream), C.byref(dispatch)))

    def cmd_swiglu_limit(self, dispatch, stream=None) -> None:
        check(L.lib().s14_cmd_swiglu_limit(self._h(), self._stream(stream), C.byref(dispatch)))

    def cmd_route_mix(self, dispatch, stream=None) -> None:
        check(L.lib().s14_cmd_route_mix(self._h(), self._stream(stream), C.byref(dispatch)))

    def cmd_moe_accumulate(self, dispatch, stream=None) -> None:
        check(L.lib().s14_cmd_moe_accumulate(self._h(), self._stream(stream), C.byref(dispatch)))


def _key(layer: int, kind: int, slot: int) -> L.ExpertKey:
    return L.ExpertKey(layer, kind, slot)


class VramPool:
    """Fixed-slot page pool (vram_pool.rs:62-422).  ``ctx=None`` gives the bookkeeping-only
    pool the reference's unit tests build with ``new_for_tests``."""

    def __init__(self, ctx: Optional[S14Context], n_slots: int, slot_bytes: int):
        h = C.c_void_p()
        check(L.lib().s14_pool_create(ctx.handle if ctx is not None else None, n_slots, slot_bytes,
                                      C.byref(h)))
        self._h = h
        self._ctx = ctx

    def close(self) -> None:
        if self._h:
            L.lib().s14_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def capacity(self) -> int:
        return L.lib().s14_pool_capacity(self._h)

    def slot_bytes(self) -> int:
        return L.lib().s14_pool_slot_bytes(self._h)

    def n_loaded(self) -> int:
        return L.lib().s14_pool_n_loaded(self._h)

    def total_bytes(self) -> int:
        return L.lib().s14_pool_total_bytes(self._h)

    def slot_offset(self, slot: int) -> int:
        return L.lib().s14_pool_slot_offset(self._h, slot)

    def slot_ptr(self, slot: int) -> Optional[int]:
        return L.lib().s14_pool_slot_ptr(self._h, slot)

    def lookup(self, key: L.ExpertKey) -> Optional[int]:
        found, slot = C.c_int32(), C.c_uint32()
        check(L.lib().s14_pool_lookup(self._h, key, C.byref(found), C.byref(slot)))
        return slot.value if found.value else None

    def lookup_and_pin(self, key: L.ExpertKey) -> Optional[L.SlotBinding]:
        found, lease = C.c_int32(), L.SlotBinding()
        check(L.lib().s14_pool_lookup_and_pin(self._h, key, C.byref(found), C.byref(lease)))
        return lease if found.value else None

    def reserve_loading_generation(self, key: L.ExpertKey) -> L.LoadingReservation:
        r = L.LoadingReservation()
        check(L.lib().s14_pool_reserve_loading_generation(self._h, key, C.byref(r)))
        return r

    def reserve_loading(self, key: L.ExpertKey):
        """(slot, evicted key or None), vram_pool.rs:172-175."""
        r = self.reserve_loading_generation(key)
        return r.slot, (r.evicted if r.has_evicted else None)

    def mark_ready(self, slot: int, key: L.ExpertKey) -> None:
        check(L.lib().s14_pool_mark_ready(self._h, slot, key))

    @staticmethod
    def _arr(reservations):
        arr = (L.LoadingReservation * max(1, len(reservations)))()
        for i, r in enumerate(reservations):
            arr[i] = r
        return arr

    def validate_publish_batch(self, reservations) -> None:
        check(L.lib().s14_pool_validate_publish_batch(self._h, self._arr(reservations), len(reservations)))

    def publish_batch_and_pin(self, reservations) -> List[L.SlotBinding]:
        out = (L.SlotBinding * max(1, len(reservations)))()
        check(L.lib().s14_pool_publish_batch_and_pin(self._h, self._arr(reservations),
                                                     len(reservations), out))
        return [L.SlotBinding.from_buffer_copy(out[i]) for i in range(len(reservations))]

    def validate_binding(self, binding: L.SlotBinding) -> None:
        check(L.lib().s14_pool_validate_binding(self._h, binding))

    def release_after_compute_fence(self, lease: L.SlotBinding) -> None:
        check(L.lib().s14_pool_release_after_compute_fence(self._h, lease))

    def cancel_loading(self, slot: int, key: L.ExpertKey) -> None:
        check(L.lib().s14_pool_cancel_loading(self._h, slot, key))

    def cancel_reservation(self, reservation: L.LoadingReservation) -> None:
        check(L.lib().s14_pool_cancel_reservation(self._h, reservation))

    # upload engine (the reference's ExpertLoader on a transfer queue)
    def upload_page_async(self, reservation: L.LoadingReservation, host_ptr: int, nbytes: int) -> None:
        check(L.lib().s14_pool_upload_page_async(self._h, C.byref(reservation), host_ptr, nbytes))

    def transfer_fence(self) -> None:
        check(L.lib().s14_pool_transfer_fence(self._h))

    def wait_transfer_fence(self) -> None:
        check(L.lib().s14_pool_wait_transfer_fence(self._h))

    def compute_wait_transfer(self, stream: Optional[int] = None) -> None:
        check(L.lib().s14_pool_compute_wait_transfer(
            self._h, stream if stream is not None else _torch_stream()))


ExpertKey = _key


@dataclass
class RouteDecision:
    """runner.rs:121-126.  ``kind``: 0 hash router (layers 0-2), 1 score router."""

    layer: int
    kind: int
    expert_ids: List[int] = field(default_factory=list)
    weights: List[float] = field(default_factory=list)

    def _c(self) -> L.RouteDecisionC:
        c = L.RouteDecisionC()
        c.layer, c.kind = self.layer, self.kind
        n = min(len(self.expert_ids), len(self.weights))
        if len(self.expert_ids) != len(self.weights) or n > L.EXPERTS_PER_TOKEN:
            c.n = 0xFFFF  # rejected by the library: not six ids and six weights
            return c
        c.n = n
        for i in range(n):
            c.expert_ids[i] = self.expert_ids[i]
            c.weights[i] = self.weights[i]
        return c

    def validate_for(self, profile: int = L.PROFILE_S14_TOP6) -> None:
        c = self._c()
        check(L.lib().s14_route_validate_for(C.byref(c), profile))


class RouteLoadBatch:
    def __init__(self, handle, route: RouteDecision):
        self._h = handle
        self.layer = route.layer
        self.expert_ids = list(route.expert_ids)
        self.route_weights = list(route.weights)

    def missing(self):
        """[(reservation, is_shared)] for the pages that still need an upload."""
        res = (L.LoadingReservation * 7)()
        shared = (C.c_int32 * 7)()
        n = C.c_uint32()
        check(L.lib().s14_route_load_batch_missing(self._h, res, shared, C.byref(n)))
        return [(L.LoadingReservation.from_buffer_copy(res[i]), bool(shared[i])) for i in range(n.value)]


class S14MoeComputeLeaseBatch:
    def __init__(self, handle):
        self._h = handle
        routed = (L.SlotBinding * L.EXPERTS_PER_TOKEN)()
        shared = L.SlotBinding()
        ids = (C.c_uint16 * L.EXPERTS_PER_TOKEN)()
        w = (C.c_float * L.EXPERTS_PER_TOKEN)()
        check(L.lib().s14_moe_compute_lease_bindings(handle, routed, C.byref(shared), ids, w))
        self._routed = [L.SlotBinding.from_buffer_copy(routed[i]) for i in range(L.EXPERTS_PER_TOKEN)]
        self._shared = shared
        self._ids = [int(v) for v in ids]
        self._w = [float(v) for v in w]

    def routed_bindings(self):
        return self._routed

    def shared_binding(self):
        return self._shared

    def expert_ids(self):
        return self._ids

    def route_weights(self):
        return self._w


class S14MoePages:
    """All-or-nothing page transaction over six routed pages and the shared page
    (S14VulkanMoePages, s14_vulkan.rs:703-819)."""

    def __init__(self, routed_pool: VramPool, shared_pool: VramPool, profile: int = L.PROFILE_S14_TOP6,
                 min_routed_bytes: int = L.EXPERT_PAGE_BYTES,
                 min_shared_bytes: int = L.SHARED_EXPERT_PAGE_BYTES):
        h = C.c_void_p()
        check(L.lib().s14_moe_pages_create_ex(routed_pool.handle, shared_pool.handle, profile,
                                              min_routed_bytes, min_shared_bytes, C.byref(h)))
        self._h = h
        self.routed_pool, self.shared_pool = routed_pool, shared_pool

    def __del__(self):
        try:
            if self._h:
                L.lib().s14_moe_pages_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def begin_after_official_route(self, route: RouteDecision) -> RouteLoadBatch:
        c = route._c()
        h = C.c_void_p()
        check(L.lib().s14_moe_pages_begin_after_official_route(self._h, C.byref(c), C.byref(h)))
        return RouteLoadBatch(h, route)

    def publish_after_transfer_fence(self, batch: RouteLoadBatch) -> S14MoeComputeLeaseBatch:
        h = C.c_void_p()
        handle, batch._h = batch._h, None  # consumed either way
        check(L.lib().s14_moe_pages_publish_after_transfer_fence(self._h, handle, C.byref(h)))
        return S14MoeComputeLeaseBatch(h)

    def release_after_compute_fence(self, lease: S14MoeComputeLeaseBatch) -> None:
        check(L.lib().s14_moe_pages_release_after_compute_fence(self._h, lease._h))
        lease._h = None

    def cancel(self, batch: RouteLoadBatch) -> None:
        handle, batch._h = batch._h, None
        check(L.lib().s14_moe_pages_cancel(self._h, handle))
