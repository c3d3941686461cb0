"""ctypes loader for the CPU oracle (``s14_oracle.c``).

TEST INFRASTRUCTURE ONLY.  The package under ``colormlm_b200/`` never imports
this module; it is used by ``tests/``, by the smoke check and by the benchmark's
CPU-baseline leg, as the checker or as the timed CPU reference.

Every wrapper takes and returns numpy arrays and forwards to the C function of
the same name; see the C file for the reference lines each one restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libs14_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc, OpenMP, no FMA contraction)."""
    src = os.path.join(_HERE, "s14_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libs14_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.s14o_e2m1.restype = C.c_float
        _lib.s14o_e2m1.argtypes = [C.c_uint8]
        _lib.s14o_ue8m0.restype = C.c_float
        _lib.s14o_ue8m0.argtypes = [C.c_uint8]
        _lib.s14o_e4m3fn.restype = C.c_float
        _lib.s14o_e4m3fn.argtypes = [C.c_uint8]
        _lib.s14o_max_threads.restype = C.c_int
        _lib.s14o_greedy_argmax.restype = C.c_int64
        _lib.s14o_error_stats.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def max_threads() -> int:
    return int(lib().s14o_max_threads())


def set_threads(n: int) -> None:
    lib().s14o_set_threads(C.c_int(n))


def e2m1(code: int) -> float:
    return float(lib().s14o_e2m1(code))


def ue8m0(code: int) -> float:
    return float(lib().s14o_ue8m0(code))


def e4m3fn(code: int) -> float:
    return float(lib().s14o_e4m3fn(code))


def mxfp4_matvec(x, packed_weight, scale, n: int, k: int) -> np.ndarray:
    x, w, s = _f32(x), _u8(packed_weight), _u8(scale)
    assert x.size == k and w.size == n * k // 2 and s.size == n * k // 32
    y = np.empty(n, np.float32)
    lib().s14o_mxfp4_matvec(_p(x), _p(w), _p(s), C.c_uint32(n), C.c_uint32(k), _p(y))
    return y


def mxfp4_matvec_f64(x, packed_weight, scale, n: int, k: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    w, s = _u8(packed_weight), _u8(scale)
    assert x.size == k and w.size == n * k // 2 and s.size == n * k // 32
    y = np.empty(n, np.float64)
    lib().s14o_mxfp4_matvec_f64(_p(x), _p(w), _p(s), C.c_uint32(n), C.c_uint32(k), _p(y))
    return y


def fp8_scale_count(n: int, k: int) -> int:
    return ((n + 127) // 128) * ((k + 127) // 128)


def fp8_matvec(x, weight, scale, n: int, k: int) -> np.ndarray:
    """scale: uint8 UE8M0 codes or float32 block scales (one per 128x128 block)."""
    x, w = _f32(x), _u8(weight)
    scale = np.ascontiguousarray(scale)
    assert x.size == k and w.size == n * k and scale.size == fp8_scale_count(n, k)
    y = np.empty(n, np.float32)
    if scale.dtype == np.uint8:
        lib().s14o_fp8_matvec(_p(x), _p(w), _p(scale), C.c_uint32(n), C.c_uint32(k), _p(y))
    else:
        scale = _f32(scale)
        lib().s14o_fp8_matvec_f32scale(_p(x), _p(w), _p(scale), C.c_uint32(n), C.c_uint32(k), _p(y))
    return y


def fp8_matvec_f64(x, weight, scale, n: int, k: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    w = _u8(weight)
    scale = np.ascontiguousarray(scale)
    is_f32 = 0 if scale.dtype == np.uint8 else 1
    if is_f32:
        scale = _f32(scale)
    y = np.empty(n, np.float64)
    lib().s14o_fp8_matvec_f64(_p(x), _p(w), _p(scale), C.c_int(is_f32), C.c_uint32(n),
                              C.c_uint32(k), _p(y))
    return y


def swiglu_limit(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    assert gate.size == up.size
    y = np.empty(gate.size, np.float32)
    lib().s14o_swiglu_limit(_p(gate), _p(up), C.c_uint32(gate.size), _p(y))
    return y


def swiglu_limit_libm(gate, up) -> np.ndarray:
    """The same with the C library's expf (not correctly rounded in rare cases)."""
    gate, up = _f32(gate), _f32(up)
    y = np.empty(gate.size, np.float32)
    lib().s14o_swiglu_limit_libm(_p(gate), _p(up), C.c_uint32(gate.size), _p(y))
    return y


def expert_chain_mxfp4(x, page, hidden: int, inter: int, route_weight: float):
    """Returns (route_weight * down, down)."""
    x, page = _f32(x), _u8(page)
    work = np.empty(3 * inter, np.float32)
    down = np.empty(hidden, np.float32)
    y = np.empty(hidden, np.float32)
    lib().s14o_expert_chain_mxfp4(_p(x), _p(page), C.c_uint32(hidden), C.c_uint32(inter),
                                  C.c_float(route_weight), _p(work), _p(down), _p(y))
    return y, down


def _page_ptrs(pages):
    pages = [_u8(p) for p in pages]
    arr = (C.c_void_p * len(pages))(*[p.ctypes.data for p in pages])
    return pages, arr


def moe_layer(x, routed_pages, route_weights, shared_page, shared_kind: int, hidden: int,
              inter: int) -> np.ndarray:
    """shared_kind: 0 MXFP4 page, 1 FP8 page, 2 none."""
    x = _f32(x)
    pages, arr = _page_ptrs(routed_pages)
    rw = _f32(route_weights)
    shared = _u8(shared_page) if shared_page is not None else np.zeros(1, np.uint8)
    work = np.empty(3 * inter + hidden, np.float32)
    y = np.empty(hidden, np.float32)
    lib().s14o_moe_layer(_p(x), arr, _p(rw), C.c_uint32(len(pages)), _p(shared),
                         C.c_int(shared_kind), C.c_uint32(hidden), C.c_uint32(inter), _p(work), _p(y))
    return y


def moe_layer_acc64(x, routed_pages, route_weights, shared_page, shared_kind: int, hidden: int,
                    inter: int) -> np.ndarray:
    """The layer with double accumulators inside each matvec and F32 everywhere else."""
    x = _f32(x)
    pages, arr = _page_ptrs(routed_pages)
    rw = _f32(route_weights)
    shared = _u8(shared_page) if shared_page is not None else np.zeros(1, np.uint8)
    work = np.empty(3 * inter + hidden, np.float32)
    work64 = np.empty(2 * max(hidden, inter), np.float64)
    y = np.empty(hidden, np.float32)
    lib().s14o_moe_layer_acc64(_p(x), arr, _p(rw), C.c_uint32(len(pages)), _p(shared),
                               C.c_int(shared_kind), C.c_uint32(hidden), C.c_uint32(inter), _p(work),
                               _p(work64), _p(y))
    return y


def act_quant(x) -> np.ndarray:
    """l42_reference.py:389-403: the E4M3FN quantisation of activations per 128 elements (last axis)."""
    x = _f32(x)
    assert x.shape[-1] % 128 == 0
    out = np.empty_like(x)
    lib().s14o_act_quant(_p(x), C.c_uint32(x.size), _p(out))
    return out


def official_moe_layer(x, routed_pages, route_weights, shared_page, shared_kind: int, hidden: int,
                       inter: int) -> np.ndarray:
    """executor.py:712-743: moe_branch of one token with the official roundings (exact dot products)."""
    x = _f32(x)
    pages, arr = _page_ptrs(routed_pages)
    rw = _f32(route_weights)
    shared = _u8(shared_page) if shared_page is not None else np.zeros(1, np.uint8)
    work = np.empty(2 * hidden + 4 * inter, np.float32)
    work64 = np.empty(2 * max(hidden, inter), np.float64)
    y = np.empty(hidden, np.float32)
    lib().s14o_official_moe_layer(_p(x), arr, _p(rw), C.c_uint32(len(pages)), _p(shared),
                                  C.c_int(shared_kind), C.c_uint32(hidden), C.c_uint32(inter), _p(work),
                                  _p(work64), _p(y))
    return y


def router(x, wr_bf16_bits, bias, score_fn: int = 0, top_k: int = 6, route_scale: float = 1.0):
    """Returns (ids int32[top_k], weights f32[top_k], scores f32[E], select f32[E])."""
    x = _f32(x)
    wr = np.ascontiguousarray(wr_bf16_bits, dtype=np.uint16)
    n_experts, hidden = wr.shape
    assert x.size == hidden
    b = _f32(bias) if bias is not None else None
    ids = np.empty(top_k, np.int32)
    w = np.empty(top_k, np.float32)
    scores = np.empty(n_experts, np.float32)
    select = np.empty(n_experts, np.float32)
    lib().s14o_router(_p(x), _p(wr), _p(b) if b is not None else None, C.c_uint32(n_experts),
                      C.c_uint32(hidden), C.c_int(score_fn), C.c_uint32(top_k),
                      C.c_float(route_scale), _p(ids), _p(w), _p(scores), _p(select))
    return ids, w, scores, select


def head_logits(x, w_bf16_bits) -> np.ndarray:
    x = _f32(x)
    w = np.ascontiguousarray(w_bf16_bits, dtype=np.uint16)
    vocab, hidden = w.shape
    out = np.empty(vocab, np.float32)
    lib().s14o_head_logits(_p(x), _p(w), C.c_uint32(vocab), C.c_uint32(hidden), _p(out))
    return out


def greedy_argmax(logits) -> int:
    logits = _f32(logits)
    return int(lib().s14o_greedy_argmax(_p(logits), C.c_uint32(logits.size)))


def error_stats(actual, expected) -> dict:
    """max_abs / mean_abs / rmse / max_rel(|ref|>1e-5), as the reference reports them."""
    a, e = _f32(actual).ravel(), _f32(expected).ravel()
    assert a.size == e.size
    out = (C.c_double * 4)()
    rc = lib().s14o_error_stats(_p(a), _p(e), C.c_uint64(a.size), out)
    if rc != 0:
        raise ValueError("error_stats: empty input or non-finite value")
    return {"max_abs": out[0], "mean_abs": out[1], "rmse": out[2], "max_rel": out[3]}


# ---- the steps on either side of the MoE inside one layer (hc.py, final_head.py) ----------------
# Streams are F32 arrays, or BF16 bit patterns in uint16 arrays (dtype=1), as the reference's state is.

def _stream(a, dtype: int) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16 if dtype else np.float32)


def hc_split_sinkhorn(mixes, scale, base, hc: int = 4, iters: int = 20, eps: float = 1e-6):
    """mixes [(2 + hc) * hc] -> (pre [hc], post [hc], comb [hc, hc])."""
    mixes, scale, base = _f32(mixes), _f32(scale), _f32(base)
    pre, post, comb = np.empty(hc, np.float32), np.empty(hc, np.float32), np.empty((hc, hc), np.float32)
    lib().s14o_hc_split_sinkhorn(_p(mixes), _p(scale), _p(base), C.c_uint32(hc), C.c_uint32(iters), C.c_float(eps),
                                 _p(pre), _p(post), _p(comb))
    return pre, post, comb


def hc_pre(x, hc_fn, hc_scale, hc_base, dtype: int = 0, norm_eps: float = 1e-6, iters: int = 20, hc_eps: float = 1e-6):
    """x [T, hc, hidden] -> (reduced [T, hidden], post [T, hc], comb [T, hc, hc])."""
    x = _stream(x, dtype)
    n_tok, hc, hidden = x.shape
    fn, sc, ba = _f32(hc_fn), _f32(hc_scale), _f32(hc_base)
    assert fn.shape == ((2 + hc) * hc, hc * hidden)
    red = np.empty((n_tok, hidden), x.dtype)
    post, comb = np.empty((n_tok, hc), np.float32), np.empty((n_tok, hc, hc), np.float32)
    for t in range(n_tok):
        lib().s14o_hc_pre(_p(x[t]), C.c_int(dtype), _p(fn), _p(sc), _p(ba), C.c_uint32(hc), C.c_uint32(hidden),
                          C.c_float(norm_eps), C.c_uint32(iters), C.c_float(hc_eps), _p(red[t]), _p(post[t]), _p(comb[t]))
    return red, post, comb


def hc_post(branch, residual, post, comb, dtype: int = 0):
    """branch [T, hidden], residual [T, hc, hidden], post [T, hc], comb [T, hc, hc] -> merged [T, hc, hidden]."""
    branch, residual = _stream(branch, dtype), _stream(residual, dtype)
    n_tok, hc, hidden = residual.shape
    post, comb = _f32(post), _f32(comb)
    out = np.empty_like(residual)
    for t in range(n_tok):
        lib().s14o_hc_post(_p(branch[t]), _p(residual[t]), C.c_int(dtype), _p(post[t]), _p(comb[t]), C.c_uint32(hc),
                           C.c_uint32(hidden), _p(out[t]))
    return out


def rms_norm(x, w, dtype: int = 0, eps: float = 1e-6):
    """x [T, hidden] -> w * x * rsqrt(mean(x^2) + eps)."""
    x, w = _stream(x, dtype), _f32(w)
    out = np.empty_like(x)
    for t in range(x.shape[0]):
        lib().s14o_rms_norm(_p(x[t]), C.c_int(dtype), _p(w), C.c_uint32(x.shape[1]), C.c_float(eps), _p(out[t]))
    return out


def hc_head_reduce(x, fn, scale, base, dtype: int = 0, norm_eps: float = 1e-6, hc_eps: float = 1e-6):
    """x [T, hc, hidden] -> (reduced [T, hidden], pre [T, hc])."""
    x = _stream(x, dtype)
    n_tok, hc, hidden = x.shape
    fn, sc, ba = _f32(fn), _f32(scale), _f32(base)
    red, pre = np.empty((n_tok, hidden), x.dtype), np.empty((n_tok, hc), np.float32)
    for t in range(n_tok):
        lib().s14o_hc_head_reduce(_p(x[t]), C.c_int(dtype), _p(fn), _p(sc), _p(ba), C.c_uint32(hc), C.c_uint32(hidden),
                                  C.c_float(norm_eps), C.c_float(hc_eps), _p(red[t]), _p(pre[t]))
    return red, pre


def router_hash(x, wr_bf16_bits, tid2eid_row, score_fn: int = 1, route_scale: float = 1.5):
    """The hash-routed layers: ids from the token's tid2eid row, weights from the router's scores of them."""
    x = _f32(x)
    wr = np.ascontiguousarray(wr_bf16_bits, dtype=np.uint16)
    row = np.ascontiguousarray(tid2eid_row, dtype=np.int64)
    ids, w = np.empty(row.size, np.int32), np.empty(row.size, np.float32)
    lib().s14o_router_hash(_p(x), _p(wr), C.c_uint32(wr.shape[0]), C.c_uint32(wr.shape[1]), C.c_int(score_fn),
                           C.c_uint32(row.size), C.c_float(route_scale), _p(row), _p(ids), _p(w))
    return ids, w
