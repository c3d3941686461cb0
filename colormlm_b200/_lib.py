"""ctypes binding of libpolaris_s14_cuda.so (the C ABI in include/polaris_s14_cuda.h).

Loading never falls back to anything else: if the library is missing the import
fails with the build command to run.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpolaris_s14_cuda.so")

OK, ERR_CONTRACT, ERR_CUDA, ERR_POOL, ERR_CODE, ERR_DEVICE = 0, 1, 2, 3, 4, 5
EXPERT_PAGE_BYTES = 13_369_344
SHARED_EXPERT_PAGE_BYTES = 25_167_360
ROUTED_EXPERT_KIND, SHARED_EXPERT_KIND = 0x53, 0x54
EXPERTS_PER_TOKEN = 6
MAX_BLOCK_TOKENS = 8
PAGE_MXFP4, PAGE_FP8 = 0, 1
ACCUM_PAIRWISE, ACCUM_REFERENCE = 0, 1
LAYER_PATH_TENSOR, LAYER_PATH_TENSOR_PER_TOKEN, LAYER_PATH_TENSOR_STACK, LAYER_PATH_F32, LAYER_PATH_REFERENCE = 1, 2, 3, 4, 5
LAYER_PATH_ROUTER_KERNEL = 0x100
LAYER_PATH_TENSOR_BLOCK = 6
STREAM_F32, STREAM_BF16 = 0, 1
EP_SHARED_BY_TOKEN = 0xFFFFFFFF
SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS = 0, 1
SCALE_UE8M0, SCALE_F32 = 0, 1
PROFILE_S14_TOP6, PROFILE_FULL_DEPTH43_NATIVE_TOP6 = 0, 1


class MatvecShape(C.Structure):
    _fields_ = [("n", C.c_uint32), ("k", C.c_uint32)]


class Buffer(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("size", C.c_uint64)]


class Mxfp4Dispatch(C.Structure):
    _fields_ = [("shape", MatvecShape), ("x", C.c_void_p), ("packed_weight", C.c_void_p),
                ("weight_scale", C.c_void_p), ("y", C.c_void_p)]


class Fp8Dispatch(C.Structure):
    _fields_ = [("shape", MatvecShape), ("scale_format", C.c_uint32), ("n_tokens", C.c_uint32),
                ("x", C.c_void_p), ("weight", C.c_void_p), ("weight_scale", C.c_void_p),
                ("y", C.c_void_p)]


class SwigluLimitDispatch(C.Structure):
    _fields_ = [("n", C.c_uint32), ("gate", C.c_void_p), ("up", C.c_void_p), ("y", C.c_void_p)]


class RouteMixDispatch(C.Structure):
    _fields_ = [("n", C.c_uint32), ("route_weight", C.c_float), ("expert", C.c_void_p),
                ("routed", C.c_void_p)]


class MoeAccumulateDispatch(C.Structure):
    _fields_ = [("n", C.c_uint32), ("weight", C.c_float), ("expert", C.c_void_p),
                ("accumulator", C.c_void_p)]


class TokenRoute(C.Structure):
    _fields_ = [("n_routed", C.c_uint32), ("expert_ids", C.c_uint16 * EXPERTS_PER_TOKEN),
                ("weights", C.c_float * EXPERTS_PER_TOKEN), ("pages", C.c_void_p * EXPERTS_PER_TOKEN)]


class MoeLayerDesc(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("inter", C.c_uint32), ("n_tokens", C.c_uint32),
                ("shared_kind", C.c_uint32), ("shared_page", C.c_void_p),
                ("routes", C.POINTER(TokenRoute)), ("x", C.c_void_p), ("y", C.c_void_p)]


class RouterDesc(C.Structure):
    _fields_ = [("n_experts", C.c_uint32), ("hidden", C.c_uint32), ("n_tokens", C.c_uint32),
                ("top_k", C.c_uint32), ("score_fn", C.c_uint32), ("route_scale", C.c_float),
                ("x", C.c_void_p), ("router_weight_bf16", C.c_void_p), ("bias", C.c_void_p),
                ("ids_out", C.c_void_p), ("weights_out", C.c_void_p)]


class HcParams(C.Structure):
    _fields_ = [("n_tokens", C.c_uint32), ("hc", C.c_uint32), ("hidden", C.c_uint32), ("dtype", C.c_uint32),
                ("sinkhorn_iters", C.c_uint32), ("norm_eps", C.c_float), ("hc_eps", C.c_float),
                ("hc_fn", C.c_void_p), ("hc_scale", C.c_void_p), ("hc_base", C.c_void_p)]


class ExecMoeDesc(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("inter", C.c_uint32), ("shared_kind", C.c_uint32), ("route", C.c_void_p),
                ("shared_page", C.c_void_p), ("ffn_input_bf16", C.c_void_p), ("residual_bf16", C.c_void_p),
                ("post", C.c_void_p), ("comb", C.c_void_p), ("state_out_bf16", C.c_void_p),
                ("moe_branch_out_bf16", C.c_void_p)]


class RoutedLayerDesc(C.Structure):
    _fields_ = [("router", RouterDesc), ("inter", C.c_uint32), ("shared_kind", C.c_uint32),
                ("page_table", C.c_void_p), ("shared_page", C.c_void_p), ("y", C.c_void_p)]


class StackLayer(C.Structure):
    _fields_ = [("router_weight_bf16", C.c_void_p), ("bias", C.c_void_p), ("page_table", C.c_void_p),
                ("shared_page", C.c_void_p), ("ids_out", C.c_void_p), ("weights_out", C.c_void_p),
                ("y_out", C.c_void_p)]


class StackConfig(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("n_experts", C.c_uint32), ("hidden", C.c_uint32), ("inter", C.c_uint32),
                ("top_k", C.c_uint32), ("score_fn", C.c_uint32), ("route_scale", C.c_float),
                ("shared_kind", C.c_uint32), ("residual", C.c_uint32)]


class ExpertKey(C.Structure):
    _fields_ = [("layer", C.c_uint32), ("kind", C.c_uint8), ("slot", C.c_uint32)]


class SlotBinding(C.Structure):
    _fields_ = [("key", ExpertKey), ("slot", C.c_uint32), ("generation", C.c_uint64)]


class LoadingReservation(C.Structure):
    _fields_ = [("key", ExpertKey), ("slot", C.c_uint32), ("generation", C.c_uint64),
                ("has_evicted", C.c_int32), ("evicted", ExpertKey)]


class RouteDecisionC(C.Structure):
    _fields_ = [("layer", C.c_uint8), ("kind", C.c_uint8), ("expert_ids", C.c_uint16 * EXPERTS_PER_TOKEN),
                ("weights", C.c_float * EXPERTS_PER_TOKEN), ("n", C.c_uint32)]


# name -> (restype, argtypes); every symbol the header declares is listed here, and the
# CPU test-suite checks that the built library exports each of them.
_VP, _U32, _U64, _I32, _F32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float
_P = C.POINTER
SIGNATURES = {
    "s14_last_error": (C.c_char_p, []),
    "s14_ctx_create": (_I32, [_I32, _P(_VP)]),
    "s14_ctx_destroy": (_I32, [_VP]),
    "s14_ctx_compute_stream": (_VP, [_VP]),
    "s14_ctx_copy_stream": (_VP, [_VP]),
    "s14_ctx_synchronize": (_I32, [_VP]),
    "s14_ctx_set_accumulation": (_I32, [_VP, _U32]),
    "s14_ctx_accumulation": (_U32, [_VP]),
    "s14_ctx_sm_count": (_I32, [_VP]),
    "s14_ctx_device_status": (_I32, [_VP, _P(_U32)]),
    "s14_ctx_launch_count": (_U64, [_VP]),
    "s14_ctx_last_layer_path": (_U32, [_VP]),
    "s14_ctx_set_layer_trace": (_I32, [_VP, _I32]),
    "s14_ctx_read_layer_trace": (_I32, [_VP, _VP, _U32, _P(_U32), _P(_U32)]),
    "s14_ctx_set_kernel_timing": (_I32, [_VP, _I32]),
    "s14_ctx_kernel_times": (_I32, [_VP, _P(C.c_double), _P(_U64)]),
    "s14_shape_new": (_I32, [_U32, _U32, _P(MatvecShape)]),
    "s14_shape_validate_mxfp4": (_I32, [MatvecShape]),
    "s14_shape_validate_fp8": (_I32, [MatvecShape]),
    "s14_shape_fp32_input_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_shape_fp32_output_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_shape_mxfp4_weight_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_shape_mxfp4_scale_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_shape_fp8_weight_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_shape_fp8_scale_bytes": (_I32, [MatvecShape, _P(_U64)]),
    "s14_stack_create": (_I32, [_VP, _P(StackConfig), _P(StackLayer), _P(_VP)]),
    "s14_stack_destroy": (_I32, [_VP]),
    "s14_cmd_stack_decode": (_I32, [_VP, _VP, _VP, _VP, _VP]),
    "s14_stack_decode_host": (_I32, [_VP, _VP, _VP, _VP]),
    "s14_block_create": (_I32, [_VP, _U32, _U32, _U32, _P(_VP)]),
    "s14_block_destroy": (_I32, [_VP]),
    "s14_block_set_residual": (_I32, [_VP, _I32]),
    "s14_block_set_semantics": (_I32, [_VP, _U32]),
    "s14_cmd_moe_block": (_I32, [_VP, _VP, _VP, _P(MoeLayerDesc)]),
    "s14_cmd_routed_moe_block": (_I32, [_VP, _VP, _VP, _P(RoutedLayerDesc)]),
    "s14_block_last_counts": (_I32, [_VP, _P(_U32)]),
    "s14_block_ep_create": (_I32, [_VP, _U32, _U32, _VP]),
    "s14_block_ep_connect": (_I32, [_VP, _VP]),
    "s14_block_ep_connect_local": (_I32, [_VP, _P(_VP)]),
    "s14_block_ep_set_wait_limit": (_I32, [_VP, _U32]),
    "s14_block_ep_disconnect": (_I32, [_VP]),
    "s14_cmd_routed_moe_block_ep": (_I32, [_VP, _VP, _VP, _P(RoutedLayerDesc), _U32, _I32]),
    "s14_cmd_routed_moe_block_experts_ep": (_I32, [_VP, _VP, _VP, _P(RoutedLayerDesc), _U32, _U32, _U32, _VP]),
    "s14_cmd_moe_block_mix": (_I32, [_VP, _VP, _VP, _VP, _VP, _VP, _U32, _U32, _I32, _VP, _VP]),
    "s14_cmd_hc_pre": (_I32, [_VP, _VP, _P(HcParams), _VP, _VP, _VP, _VP]),
    "s14_cmd_hc_post": (_I32, [_VP, _VP, _U32, _U32, _U32, _U32, _VP, _VP, _VP, _VP, _VP]),
    "s14_cmd_rms_norm": (_I32, [_VP, _VP, _U32, _U32, _U32, _VP, _VP, _F32, _VP]),
    "s14_cmd_hc_head_reduce": (_I32, [_VP, _VP, _P(HcParams), _VP, _VP, _VP]),
    "s14_cmd_router_hash": (_I32, [_VP, _VP, _P(RouterDesc), _VP]),
    "s14_exec_routed_and_shared_moe_then_hc_post": (_I32, [_VP, _VP, _P(ExecMoeDesc)]),
    "s14_exec_hc_head_norm_full_logits": (_I32, [_VP, _VP, _P(HcParams), _VP, _VP, _U32, _VP, _VP]),
    "s14_layer_work_list": (_I32, [_U32, _U32, _U32, _U32, _U32, _U32, _VP, _U32, _VP]),
    "s14_mxfp4_expert_page_from_tensors": (_I32, [_U32, _U32, _VP, _VP]),
    "s14_mxfp4_expert_page_to_tensors": (_I32, [_U32, _U32, _VP, _VP]),
    "s14_validate_ue8m0_codes": (_I32, [_VP, _U64, _P(_U64)]),
    "s14_validate_e4m3fn_codes": (_I32, [_VP, _U64, _P(_U64)]),
    "s14_bind_mxfp4": (_I32, [_VP, MatvecShape, _P(Buffer), _P(Buffer), _P(Buffer), _P(Buffer),
                              _P(Mxfp4Dispatch)]),
    "s14_cmd_mxfp4_matvec": (_I32, [_VP, _VP, _P(Mxfp4Dispatch)]),
    "s14_bind_fp8": (_I32, [_VP, MatvecShape, _P(Buffer), _P(Buffer), _P(Buffer), _P(Buffer),
                            _P(Fp8Dispatch)]),
    "s14_bind_fp8_ex": (_I32, [_VP, MatvecShape, _U32, _U32, _P(Buffer), _P(Buffer), _P(Buffer),
                               _P(Buffer), _P(Fp8Dispatch)]),
    "s14_cmd_fp8_matvec": (_I32, [_VP, _VP, _P(Fp8Dispatch)]),
    "s14_bind_swiglu_limit": (_I32, [_VP, _U32, _P(Buffer), _P(Buffer), _P(Buffer),
                                     _P(SwigluLimitDispatch)]),
    "s14_cmd_swiglu_limit": (_I32, [_VP, _VP, _P(SwigluLimitDispatch)]),
    "s14_bind_route_mix": (_I32, [_VP, _U32, _F32, _P(Buffer), _P(Buffer), _P(RouteMixDispatch)]),
    "s14_cmd_route_mix": (_I32, [_VP, _VP, _P(RouteMixDispatch)]),
    "s14_bind_moe_accumulate": (_I32, [_VP, _U32, _F32, _P(Buffer), _P(Buffer),
                                       _P(MoeAccumulateDispatch)]),
    "s14_cmd_moe_accumulate": (_I32, [_VP, _VP, _P(MoeAccumulateDispatch)]),
    "s14_cmd_moe_layer": (_I32, [_VP, _VP, _P(MoeLayerDesc)]),
    "s14_cmd_router": (_I32, [_VP, _VP, _P(RouterDesc)]),
    "s14_cmd_routed_moe_layer": (_I32, [_VP, _VP, _P(RoutedLayerDesc)]),
    "s14_cmd_routed_moe_experts_ep": (_I32, [_VP, _VP, _P(RoutedLayerDesc), _U32, _U32, _U32, _VP]),
    "s14_cmd_moe_mix_slots": (_I32, [_VP, _VP, _VP, _VP, _U32, _I32, _VP, _U32]),
    "s14_ep_exchange_create": (_I32, [_VP, _U32, _U32, _U32, _VP]),
    "s14_ep_exchange_connect": (_I32, [_VP, _VP]),
    "s14_ep_exchange_connect_local": (_I32, [_VP, _P(_VP)]),
    "s14_ep_exchange_destroy": (_I32, [_VP]),
    "s14_ep_exchange_disconnect": (_I32, [_VP]),
    "s14_ep_exchange_set_wait_limit": (_I32, [_VP, _U32]),
    "s14_cmd_routed_moe_layer_ep": (_I32, [_VP, _VP, _P(RoutedLayerDesc), _U32, _I32]),
    "s14_routed_moe_layer_host": (_I32, [_VP, _P(RoutedLayerDesc), _VP, _VP, _VP, _VP]),
    "s14_cmd_head_logits": (_I32, [_VP, _VP, _VP, _U32, _VP, _U32, _U32, _VP, _U32]),
    "s14_cmd_greedy_argmax": (_I32, [_VP, _VP, _VP, _U32, _VP]),
    "s14_moe_layer_noalloc": (_I32, [_I32, _VP, _U32, _P(MoeLayerDesc)]),
    "s14_moe_layer_host": (_I32, [_VP, _P(MoeLayerDesc), _VP, _VP]),
    "s14_pool_create": (_I32, [_VP, _U32, _U64, _P(_VP)]),
    "s14_pool_create_host": (_I32, [_U32, _U64, _P(_VP)]),
    "s14_pool_destroy": (_I32, [_VP]),
    "s14_loader_create": (_I32, [_VP, _U32, _P(_VP)]),
    "s14_loader_destroy": (_I32, [_VP]),
    "s14_loader_enqueue_from_buf": (_I32, [_VP, ExpertKey, _VP, _U64, _P(_U32)]),
    "s14_loader_batch_enqueue_from_bufs": (_I32, [_VP, _VP, _VP, _VP, _U32, _VP]),
    "s14_loader_wait_all": (_I32, [_VP]),
    "s14_loader_in_flight": (_U32, [_VP]),
    "s14_loader_stat_loads": (_U64, [_VP]),
    "s14_loader_stat_bytes": (_U64, [_VP]),
    "s14_pool_capacity": (_U32, [_VP]),
    "s14_pool_slot_bytes": (_U64, [_VP]),
    "s14_pool_n_loaded": (_U32, [_VP]),
    "s14_pool_total_bytes": (_U64, [_VP]),
    "s14_pool_slot_offset": (_U64, [_VP, _U32]),
    "s14_pool_slot_ptr": (_VP, [_VP, _U32]),
    "s14_pool_lookup": (_I32, [_VP, ExpertKey, _P(_I32), _P(_U32)]),
    "s14_pool_lookup_and_pin": (_I32, [_VP, ExpertKey, _P(_I32), _P(SlotBinding)]),
    "s14_pool_reserve_loading_generation": (_I32, [_VP, ExpertKey, _P(LoadingReservation)]),
    "s14_pool_mark_ready": (_I32, [_VP, _U32, ExpertKey]),
    "s14_pool_validate_publish_batch": (_I32, [_VP, _P(LoadingReservation), _U32]),
    "s14_pool_publish_batch_and_pin": (_I32, [_VP, _P(LoadingReservation), _U32, _P(SlotBinding)]),
    "s14_pool_validate_binding": (_I32, [_VP, SlotBinding]),
    "s14_pool_release_after_compute_fence": (_I32, [_VP, SlotBinding]),
    "s14_pool_cancel_loading": (_I32, [_VP, _U32, ExpertKey]),
    "s14_pool_cancel_reservation": (_I32, [_VP, LoadingReservation]),
    "s14_pool_upload_page_async": (_I32, [_VP, _P(LoadingReservation), _VP, _U64]),
    "s14_pool_transfer_fence": (_I32, [_VP]),
    "s14_pool_wait_transfer_fence": (_I32, [_VP]),
    "s14_pool_compute_wait_transfer": (_I32, [_VP, _VP]),
    "s14_host_alloc_pinned": (_I32, [_U64, _P(_VP)]),
    "s14_host_free_pinned": (_I32, [_VP]),
    "s14_route_validate_for": (_I32, [_P(RouteDecisionC), _U32]),
    "s14_moe_pages_create": (_I32, [_VP, _VP, _U32, _P(_VP)]),
    "s14_moe_pages_create_ex": (_I32, [_VP, _VP, _U32, _U64, _U64, _P(_VP)]),
    "s14_moe_pages_destroy": (_I32, [_VP]),
    "s14_moe_pages_begin_after_official_route": (_I32, [_VP, _P(RouteDecisionC), _P(_VP)]),
    "s14_route_load_batch_missing": (_I32, [_VP, _P(LoadingReservation), _P(_I32), _P(_U32)]),
    "s14_moe_pages_publish_after_transfer_fence": (_I32, [_VP, _VP, _P(_VP)]),
    "s14_moe_compute_lease_bindings": (_I32, [_VP, _P(SlotBinding), _P(SlotBinding),
                                              _P(C.c_uint16), _P(_F32)]),
    "s14_moe_pages_release_after_compute_fence": (_I32, [_VP, _VP]),
    "s14_moe_pages_cancel": (_I32, [_VP, _VP]),
}

_lib = None


class S14Error(RuntimeError):
    """A non-zero status from the C ABI; ``code`` is the S14_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[s14 status {code}] {message}")
        self.code = code
        self.message = message


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m colormlm_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise S14Error(status, lib().s14_last_error().decode("utf-8", "replace"))
