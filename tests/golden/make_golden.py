"""Generates tests/golden/s14_golden.npz by running the reference's importable Python
code (``fast16/research/polaris_meridian_v1``) on small seeded inputs.

Run from the repository root where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The resulting file is committed; the tests only read it and never need the reference
itself.  Small inputs are stored next to the outputs; large random inputs are rebuilt by
the tests from the same seeds with ``colormlm_b200.synth`` and checked against a SHA-256
stored here.  Cases:

* decode tables of all E2M1, UE8M0 and E4M3FN codes (``decode_*`` of the reference);
* the reference's own deterministic MXFP4 fixture
  (local_s14_primitives/tests/test_primitives.py:58-72) through ``fp4_linear`` with F32
  and F64 accumulation;
* a seeded MXFP4 matvec with the benchmark's value distribution through ``fp4_linear``;
* the reference's FP8 fixture (test_primitives.py:97-112, seed 7) through
  ``fp8_weight_linear`` with UE8M0 and with F32 block scales;
* one expert chain and one 6+1 expert layer composed from ``fp4_linear``,
  ``fp8_weight_linear`` and the reference's ``_limited_swiglu``
  (s14_first_real_token/executor.py:706-710) in the order of
  examples/s14_vulkan_numeric.rs:929-947, with F64 accumulation;
* router outputs from the torch expressions of executor.py:638-668 (both score
  functions);
* LM-head logits through ``bf16_checkpoint_head_logits`` on the reference's seed-731
  fixture (tests/test_final_head.py:22-30);
* the hyper-connection reduce / expand, RMSNorm and the head's reduce (``hc_split_sinkhorn``,
  ``hc_pre``, ``hc_post``, ``hc_head_reduce``, ``official_rms_norm``) on the reference's own
  fixtures (tests/test_primitives.py:126-141, tests/test_final_head.py:22-46) and on seeded streams
  of the model's size in F32 and BF16; the hash-routed layers' weights from the torch expressions
  of executor.py:638-668;
* the official expert arithmetic: ``_activation_quant`` (l42_reference.py:389-403) on seeded rows and
  ``finish_layer`` (s14_first_real_token/executor.py:712-743) itself on synthetic pages of hidden 4096 x
  intermediate 512, with an MXFP4 and with an FP8 shared expert.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def _digest(*arrays) -> bytes:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.digest()


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from fast16.research.polaris_meridian_v1.local_s14_primitives import (
        FP4_E2M1_VALUES, decode_fp8_e4m3fn, decode_ue8m0, fp4_linear, fp8_weight_linear)
    from fast16.research.polaris_meridian_v1.local_s14_primitives.final_head import (
        bf16_checkpoint_head_logits)
    from fast16.research.polaris_meridian_v1.s14_first_real_token.executor import (
        NativeLayerReference)

    from colormlm_b200 import synth
    from colormlm_b200.pages import ExpertPageLayout

    swiglu = NativeLayerReference._limited_swiglu
    out = {}

    # decode tables
    out["e2m1_table"] = np.asarray(FP4_E2M1_VALUES, dtype=np.float32)
    out["ue8m0_table"] = decode_ue8m0(torch.arange(255, dtype=torch.uint8)).numpy()
    codes = torch.tensor([c for c in range(256) if c not in (0x7F, 0xFF)], dtype=torch.uint8)
    out["e4m3_codes"] = codes.numpy()
    out["e4m3_table"] = decode_fp8_e4m3fn(codes).numpy()

    # the reference's deterministic MXFP4 fixture
    packed = torch.arange(3 * 64, dtype=torch.uint8).reshape(3, 64)
    scales = torch.tensor([[126, 127, 128, 129], [127, 128, 126, 127], [128, 126, 127, 128]],
                          dtype=torch.uint8)
    x = torch.sin(torch.arange(2 * 128, dtype=torch.float32).reshape(2, 128) * 0.013)
    out["fx_packed"], out["fx_scales"], out["fx_x"] = packed.numpy(), scales.numpy(), x.numpy()
    out["fx_y_f32"] = fp4_linear(x, packed, scales, output_dtype=torch.float32).numpy()
    out["fx_y_f64"] = fp4_linear(x.double(), packed, scales, accumulation_dtype=torch.float64,
                                 output_dtype=torch.float64).numpy()

    # seeded MXFP4 matvec, benchmark distribution
    g = synth.rng(1001)
    n, k = 96, 1024
    w = synth.mxfp4_codes(g, n, k)
    s = synth.mxfp4_scales(g, n, k)
    xv = synth.activations(g, 2, k)
    out["mx_inputs_sha256"] = np.frombuffer(_digest(w, s, xv), dtype=np.uint8)
    out["mx_y_f32"] = fp4_linear(torch.from_numpy(xv), torch.from_numpy(w), torch.from_numpy(s),
                                 output_dtype=torch.float32).numpy()
    out["mx_y_f64"] = fp4_linear(torch.from_numpy(xv).double(), torch.from_numpy(w), torch.from_numpy(s),
                                 accumulation_dtype=torch.float64, output_dtype=torch.float64).numpy()

    # the reference's FP8 fixture (seed 7), ragged 129 x 130
    torch.manual_seed(7)
    _raw_x = torch.randint(0, 255, (2, 130), dtype=torch.uint8)  # consumed to keep the stream aligned
    raw_w = torch.randint(0, 255, (129, 130), dtype=torch.uint8)
    raw_w[raw_w == 0x7F] = 0x7E
    scale_w = torch.tensor([[127, 128], [126, 127]], dtype=torch.uint8)
    logical_x = torch.sin(torch.arange(260, dtype=torch.float32).reshape(2, 130) * 0.01)
    out["f8_w"], out["f8_s"], out["f8_x"] = raw_w.numpy(), scale_w.numpy(), logical_x.numpy()
    out["f8_y"] = fp8_weight_linear(logical_x, raw_w, scale_w, output_chunk_size=41).numpy()
    out["f8_y_f64"] = fp8_weight_linear(logical_x.double(), raw_w, scale_w, output_chunk_size=41,
                                        accumulation_dtype=torch.float64,
                                        output_dtype=torch.float64).numpy()
    scale_f = torch.tensor([[0.011, 0.0071], [0.0093, 0.0127]], dtype=torch.float32)
    out["f8_sf"] = scale_f.numpy()
    out["f8_y_sf"] = fp8_weight_linear(logical_x, raw_w, scale_f, output_chunk_size=41).numpy()

    # aligned FP8 projection, benchmark distribution (wq_a-like, smaller)
    g = synth.rng(1002)
    n8, k8 = 256, 512
    w8 = synth.e4m3_codes(g, n8, k8)
    s8 = synth.fp8_block_scales_ue8m0(g, n8, k8)
    s8f = synth.fp8_block_scales_f32(g, n8, k8)
    x8 = synth.activations(g, 4, k8)
    out["p8_inputs_sha256"] = np.frombuffer(_digest(w8, s8, s8f, x8), dtype=np.uint8)
    out["p8_y"] = fp8_weight_linear(torch.from_numpy(x8), torch.from_numpy(w8), torch.from_numpy(s8)).numpy()
    out["p8_y_sf"] = fp8_weight_linear(torch.from_numpy(x8), torch.from_numpy(w8), torch.from_numpy(s8f)).numpy()

    # expert chain and layer, F64 accumulation, hidden 1024 / inter 1024
    hidden, inter = 1024, 1024
    g = synth.rng(1003)
    lay4 = ExpertPageLayout(hidden, inter, 0)
    lay8 = ExpertPageLayout(hidden, inter, 1)
    pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(7)]
    page8 = synth.fp8_expert_page(g, hidden, inter)
    xl = synth.activations(g, 1, hidden)[0]
    weights = np.asarray([0.31, 0.22, 0.17, 0.13, 0.1, 0.07], dtype=np.float32)
    # the pages are not stored (random bytes do not compress): the tests regenerate them
    # from seed 1003 and check this digest
    out["ly_inputs_sha256"] = np.frombuffer(_digest(*pages, page8, xl), dtype=np.uint8)
    out["ly_w"] = weights

    def t(a, shape):
        return torch.from_numpy(np.ascontiguousarray(a)).reshape(shape)

    def chain4(page, xin):
        p = lay4.split(page)
        xd = torch.from_numpy(xin).double()
        kw = dict(accumulation_dtype=torch.float64, output_dtype=torch.float64)
        gate = fp4_linear(xd, t(p["w1"], (inter, hidden // 2)), t(p["s1"], (inter, hidden // 32)), **kw)
        up = fp4_linear(xd, t(p["w3"], (inter, hidden // 2)), t(p["s3"], (inter, hidden // 32)), **kw)
        # the reference's SwiGLU runs in F32 (it calls .float()); keep that
        h = swiglu(gate.float(), up.float())
        return fp4_linear(h.double(), t(p["w2"], (hidden, inter // 2)), t(p["s2"], (hidden, inter // 32)), **kw)

    def chain8(page, xin):
        p = lay8.split(page)
        xd = torch.from_numpy(xin).double()
        nb_u = ((inter + 127) // 128, (hidden + 127) // 128)
        nb_d = ((hidden + 127) // 128, (inter + 127) // 128)
        gate = fp8_weight_linear(xd, t(p["w1"], (inter, hidden)), t(p["s1"], nb_u), accumulation_dtype=torch.float64, output_dtype=torch.float64)
        up = fp8_weight_linear(xd, t(p["w3"], (inter, hidden)), t(p["s3"], nb_u), accumulation_dtype=torch.float64, output_dtype=torch.float64)
        h = swiglu(gate.float(), up.float())
        return fp8_weight_linear(h.double(), t(p["w2"], (hidden, inter)), t(p["s2"], nb_d), accumulation_dtype=torch.float64,
                                 output_dtype=torch.float64)

    downs = [chain4(p, xl) for p in pages]
    out["ly_chain0_down"] = downs[0].numpy()
    acc = torch.zeros(hidden, dtype=torch.float64)
    for e in range(6):
        acc += float(weights[e]) * downs[e]
    out["ly_y_mxfp4_shared"] = (acc + downs[6]).numpy()
    out["ly_y_fp8_shared"] = (acc + chain8(page8, xl)).numpy()

    # router: executor.py:638-668 with both score functions, scale 1.5 and 1.0
    g = synth.rng(1004)
    n_exp, hid = 256, 1024
    wr_bits = synth.router_weight_bf16(g, n_exp, hid)
    bias = synth.router_bias(g, n_exp)
    xr = synth.activations(g, 4, hid)
    out["rt_inputs_sha256"] = np.frombuffer(_digest(wr_bits, bias, xr), dtype=np.uint8)
    wr = torch.from_numpy(synth.bf16_bits_to_f32(wr_bits))
    logits = F.linear(torch.from_numpy(xr).float(), wr.float())
    for name, scores in (("sig", torch.sigmoid(logits)), ("ssp", F.softplus(logits).sqrt())):
        indices = (scores + torch.from_numpy(bias)).topk(6, dim=-1).indices
        w6 = scores.gather(1, indices)
        w6 = w6 / w6.sum(dim=-1, keepdim=True) * 1.5
        out[f"rt_{name}_ids"] = indices.numpy().astype(np.int32)
        out[f"rt_{name}_w"] = w6.numpy()
        sel = (scores + torch.from_numpy(bias)).sort(dim=-1, descending=True).values
        out[f"rt_{name}_gap"] = (sel[:, 5] - sel[:, 6]).numpy()

    # LM head on the reference's seed-731 fixture
    torch.manual_seed(731)
    hx = torch.randn(2, 3, 4, 8, dtype=torch.float32).to(torch.bfloat16)
    _ = torch.randn(4, 32, dtype=torch.float32)
    head_weight = torch.randn(13, 8, dtype=torch.float32).to(torch.bfloat16)
    hid_states = hx[:, :, 0]
    out["hd_x"] = hid_states.float().numpy()
    out["hd_w"] = head_weight.view(torch.int16).numpy().view(np.uint16)
    out["hd_logits"] = bf16_checkpoint_head_logits(hid_states, head_weight, full_logits=True,
                                                   output_chunk_size=5).numpy()

    # ---- the steps on either side of the MoE: hc.py:19-148, final_head.py:43-110 ----
    from fast16.research.polaris_meridian_v1.local_s14_primitives.hc import hc_post, hc_pre, hc_split_sinkhorn
    from fast16.research.polaris_meridian_v1.local_s14_primitives.final_head import hc_head_reduce, official_rms_norm

    # the reference's own deterministic fixture (tests/test_primitives.py:126-141)
    mixes = torch.linspace(-1000, 1000, 24, dtype=torch.float32).reshape(1, 1, 24)
    hscale = torch.tensor([0.5, -0.25, 0.01])
    hbase = torch.linspace(-1, 1, 24)
    pre, post, comb = hc_split_sinkhorn(mixes, hscale, hbase, sinkhorn_iters=20)
    out["hcf_pre"], out["hcf_post"], out["hcf_comb"] = pre.numpy().ravel(), post.numpy().ravel(), comb.numpy().reshape(4, 4)
    fx = torch.sin(torch.arange(32, dtype=torch.float32) * 0.1).reshape(1, 1, 4, 8)
    ffn = torch.linspace(-0.2, 0.2, 24 * 32).reshape(24, 32)
    red, post2, comb2 = hc_pre(fx, ffn, hscale, hbase)
    fbranch = torch.cos(torch.arange(8, dtype=torch.float32)).reshape(1, 1, 8)
    out["hcf_reduced"], out["hcf_post2"], out["hcf_comb2"] = red.numpy().reshape(8), post2.numpy().ravel(), comb2.numpy().reshape(4, 4)
    out["hcf_merged"] = hc_post(fbranch, fx, post2, comb2).numpy().reshape(4, 8)
    out["hcf_mixes"], out["hcf_base"], out["hcf_fn"] = mixes.numpy().ravel(), hbase.numpy(), ffn.numpy()   # torch's linspace
    out["hcf_x"], out["hcf_branch"] = fx.numpy().reshape(1, 4, 8), fbranch.numpy().reshape(1, 8)
    # the reference's seed-731 fixture of the head (tests/test_final_head.py:22-46): BF16 streams
    torch.manual_seed(731)
    hx = torch.randn(2, 3, 4, 8, dtype=torch.float32).to(torch.bfloat16)
    hfn = torch.randn(4, 32, dtype=torch.float32) * 0.1
    hsc = torch.tensor([0.7], dtype=torch.float32)
    hba = torch.linspace(-0.3, 0.3, 4, dtype=torch.float32)
    nw = torch.linspace(0.8, 1.2, 8, dtype=torch.float32)
    hred, hpre = hc_head_reduce(hx, hfn, hsc, hba)
    out["hh_x"] = hx.view(torch.int16).numpy().view(np.uint16).reshape(6, 4, 8)
    out["hh_fn"], out["hh_base"], out["hh_nw"] = hfn.numpy(), hba.numpy(), nw.numpy()
    out["hh_reduced"] = hred.view(torch.int16).numpy().view(np.uint16).reshape(6, 8)
    out["hh_pre"] = hpre.numpy().reshape(6, 4)
    out["hh_norm"] = official_rms_norm(hx[:, :, 0], nw).view(torch.int16).numpy().view(np.uint16).reshape(6, 8)
    # seeded streams of the model's size (3 tokens x 4 x 4096), F32 and BF16
    g = synth.rng(1005)
    hfn_np, hsc_np, hba_np = synth.hc_params(g, 4096)
    xs_np = synth.hc_streams(g, 3, 4096)
    br_np = synth.activations(g, 3, 4096)
    nw_np = g.uniform(0.5, 1.5, size=4096).astype(np.float32)
    out["hc_inputs_sha256"] = np.frombuffer(_digest(hfn_np, hsc_np, hba_np, xs_np, br_np, nw_np), dtype=np.uint8)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        xs_t = torch.from_numpy(xs_np).to(dt).reshape(1, 3, 4, 4096)
        br_t = torch.from_numpy(br_np).to(dt).reshape(1, 3, 4096)
        red, post, comb = hc_pre(xs_t, torch.from_numpy(hfn_np), torch.from_numpy(hsc_np), torch.from_numpy(hba_np))
        merged = hc_post(br_t, xs_t, post, comb)
        normed = official_rms_norm(red, torch.from_numpy(nw_np))
        out[f"hc_{name}_reduced"] = red.float().numpy().reshape(3, 4096)
        out[f"hc_{name}_post"], out[f"hc_{name}_comb"] = post.numpy().reshape(3, 4), comb.numpy().reshape(3, 4, 4)
        out[f"hc_{name}_merged"] = merged.float().numpy().reshape(3, 4, 4096)
        out[f"hc_{name}_normed"] = normed.float().numpy().reshape(3, 4096)
    # the hash-routed layers (executor.py:638-668 with layer < 3): ids from tid2eid, weights from the scores
    g = synth.rng(1006)
    wr_bits = synth.router_weight_bf16(g, 256, 1024)
    xr = synth.activations(g, 3, 1024)
    tid2eid = np.stack([g.permutation(256)[:6] for _ in range(3)]).astype(np.int64)
    out["rh_inputs_sha256"] = np.frombuffer(_digest(wr_bits, xr, tid2eid), dtype=np.uint8)
    scores = F.softplus(F.linear(torch.from_numpy(xr).float(), torch.from_numpy(synth.bf16_bits_to_f32(wr_bits)).float())).sqrt()
    w6 = scores.gather(1, torch.from_numpy(tid2eid))
    out["rh_w"] = (w6 / w6.sum(dim=-1, keepdim=True) * 1.5).numpy()

    # the final path (final_head.py:152-191: head reduce -> RMSNorm -> BF16 head) at hidden 1024, vocabulary 768
    from fast16.research.polaris_meridian_v1.local_s14_primitives.final_head import native_final_logits

    g = synth.rng(1007)
    nfn, nsc, nba = synth.hc_params(g, 1024, head=True)
    nx = synth.hc_streams(g, 2, 1024)
    nnw = g.uniform(0.5, 1.5, size=1024).astype(np.float32)
    nhw = synth.head_weight_bf16(g, 768, 1024)
    out["nf_inputs_sha256"] = np.frombuffer(_digest(nfn, nsc, nba, nx, nnw, nhw), dtype=np.uint8)
    head_t = torch.from_numpy(synth.bf16_bits_to_f32(nhw)).to(torch.bfloat16)
    logits, normalized, npre = native_final_logits(
        torch.from_numpy(nx).to(torch.bfloat16).reshape(1, 2, 4, 1024), torch.from_numpy(nfn), torch.from_numpy(nsc),
        torch.from_numpy(nba), torch.from_numpy(nnw), head_t, full_logits=True, enforce_official_shape=False)
    out["nf_logits"] = logits.numpy().reshape(2, 768)
    out["nf_normalized"] = normalized.float().numpy().reshape(2, 1024)
    out["nf_pre"] = npre.numpy().reshape(2, 4)

    # official expert semantics: the reference's own _activation_quant, _linear_fp4 / _linear_fp8 and
    # finish_layer (l42_reference.py:389-419, s14_first_real_token/executor.py:712-743) run on synthetic
    # pages; only the two weight loaders (which read checkpoint files and return the dequantised F32 matrix,
    # l42_reference.py:360-387) are replaced by the dequantisation of the synthetic tensors
    from fast16.research.polaris_meridian_v1.s14_first_real_token import executor as ex

    g = synth.rng(1011)
    aq_x = synth.activations(g, 6, 512)
    aq_x[1] *= np.float32(1e-5)          # below the 1e-4 floor of amax
    aq_x[2] *= np.float32(300.0)
    aq_x[3, :128] = 0.0                  # an all-zero group
    aq_x[4, :128] = np.clip(aq_x[4, :128], -1.0, 1.0) * np.float32(100.0)
    aq_x[4, 0] = np.float32(112.0)       # amax / 448 an exact power of two
    aq_x[5] = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(aq_x[5]))
    out["aq_x"] = aq_x
    out["aq_y"] = ex.NativeLayerReference._activation_quant(aq_x)

    hidden, inter = 4096, 512            # finish_layer fixes the hidden size
    g = synth.rng(1012)
    lay4 = ExpertPageLayout(hidden, inter, 0)
    lay8 = ExpertPageLayout(hidden, inter, 1)
    of_pages = [synth.mxfp4_expert_page(g, hidden, inter) for _ in range(7)]
    of_page8 = synth.fp8_expert_page(g, hidden, inter)
    of_x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(synth.activations(g, 2, hidden)))
    of_w = np.asarray([[0.52, 0.33, 0.27, 0.18, 0.12, 0.08], [0.29, 0.26, 0.25, 0.24, 0.23, 0.23]], dtype=np.float32)
    out["of_inputs_sha256"] = np.frombuffer(_digest(*of_pages, of_page8, of_x), dtype=np.uint8)
    out["of_w"] = of_w

    e2m1 = np.asarray(FP4_E2M1_VALUES, dtype=np.float32)
    all_codes = np.arange(256, dtype=np.uint8)
    finite = (all_codes & 0x7F) != 0x7F      # 0x7F and 0xFF are NaN and never occur in the synthetic pages
    e4m3 = np.zeros(256, dtype=np.float32)
    e4m3[finite] = decode_fp8_e4m3fn(torch.from_numpy(all_codes[finite])).numpy()

    def dense4(packed, scales):
        # [n, k/2] bytes (low nibble = even k) and [n, k/32] UE8M0 codes -> [n, k] F32 (exact: powers of two)
        codes = np.stack([packed & 15, packed >> 4], axis=-1).reshape(packed.shape[0], -1)
        return np.ldexp(e2m1[codes], np.repeat(scales.astype(np.int32) - 127, 32, axis=1)).astype(np.float32)

    def dense8(packed, scales):
        # [n, k] E4M3FN codes and one UE8M0 code per 128 x 128 block -> [n, k] F32
        expo = np.kron(scales.astype(np.int32) - 127, np.ones((128, 128), dtype=np.int32))
        return np.ldexp(e4m3[packed], expo[: packed.shape[0], : packed.shape[1]]).astype(np.float32)

    shapes = {"w1": (inter, hidden), "w3": (inter, hidden), "w2": (hidden, inter)}
    table = {}
    for e, page in enumerate(of_pages):
        parts = lay4.split(page)
        for name, (n, k) in shapes.items():
            prefix = ("layers.5.ffn.experts.%d." % e if e < 6 else "mxfp4_shared.") + name
            table[prefix] = dense4(np.ascontiguousarray(parts[name]).reshape(n, k // 2),
                                   np.ascontiguousarray(parts["s" + name[1]]).reshape(n, k // 32))
    parts = lay8.split(of_page8)
    for name, (n, k) in shapes.items():
        table["fp8_shared." + name] = dense8(np.ascontiguousarray(parts[name]).reshape(n, k),
                                             np.ascontiguousarray(parts["s" + name[1]]).reshape((n + 127) // 128, (k + 127) // 128))

    for shared_name in ("mxfp4_shared", "fp8_shared"):
        ref = object.__new__(ex.NativeLayerReference)
        ref.layer = 5
        ref._weight_fp4 = lambda prefix: table[prefix]
        ref._weight_fp8 = lambda prefix, _s=shared_name: table[prefix.replace("layers.5.ffn.shared_experts", _s)]
        branches = []
        for tok in range(2):
            pending = ex.PendingLayer(
                post_attention_state=torch.zeros(1, 1, 4, hidden, dtype=torch.bfloat16),
                post_ffn=torch.ones(1, 1, 4), comb_ffn=torch.eye(4).reshape(1, 1, 4, 4),
                ffn_input=torch.from_numpy(of_x[tok]).to(torch.bfloat16).reshape(1, 1, hidden),
                route_ids=[0, 1, 2, 3, 4, 5], route_weights=[float(v) for v in of_w[tok]], route_source="golden",
                attention_branch=None, runtime_state=None)
            branch, _ = ref.finish_layer(pending)
            branches.append(branch.float().numpy().reshape(hidden))
        out["of_branch_" + shared_name] = np.stack(branches)

    path = os.path.join(HERE, "s14_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
