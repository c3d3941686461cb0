"""The allocation-free layer entry point, for callers that cannot call cudaMalloc (a frozen
memory plan, someone else's graph capture) and so cannot build a context: it must give exactly
what the context-based entry point gives, on repeated calls that reuse the library's built-in
scratch.  Collected last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from colormlm_b200 import _lib as L
from colormlm_b200 import synth
from colormlm_b200.pages import ExpertPageLayout
from colormlm_b200.s14 import S14Context, S14Error, TokenRoute, _layer_desc

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("cuda_lib")]


def _noalloc(routes, shared, hidden, inter, x, y, mode):
    desc, keep = _layer_desc(routes, shared, L.PAGE_MXFP4, hidden, inter)
    desc.x, desc.y = x.data_ptr(), y.data_ptr()
    L.check(L.lib().s14_moe_layer_noalloc(0, torch.cuda.current_stream().cuda_stream, mode, C.byref(desc)))
    del keep


@pytest.mark.parametrize("hidden,inter", [(2048, 1024), (4096, 2048)])
def test_noalloc_layer_matches_context_layer_on_repeated_calls(hidden, inter):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    g = synth.rng(4711 + hidden)
    lay = ExpertPageLayout(hidden, inter)
    pages = [torch.from_numpy(lay.to_expert_page(synth.mxfp4_expert_page(g, hidden, inter))).cuda() for _ in range(8)]
    xs = torch.from_numpy(synth.activations(g, 2, hidden)).cuda()
    w = [0.3, 0.25, 0.15, 0.12, 0.1, 0.08]
    # the entry point without a context runs the F32 pairwise kernels; the context it is compared
    # with is told to run the same ones (it prefers the tcgen05 kernel otherwise)
    os.environ["S14_TENSOR_PATH"] = "off"
    try:
        ctx = S14Context(0)
    finally:
        del os.environ["S14_TENSOR_PATH"]
    try:
        for mode in (L.ACCUM_PAIRWISE, L.ACCUM_REFERENCE):
            ctx.set_accumulation(mode)
            # two calls in a row with different routes and tokens: the second one finds the scratch
            # and the counters as the first one left them
            for call, ids in enumerate(([0, 1, 2, 3, 4, 5], [6, 3, 0, 5, 2, 1])):
                route = [TokenRoute(ids, w, [pages[i].data_ptr() for i in ids])]
                x = xs[call:call + 1].contiguous()
                want, got = torch.empty_like(x), torch.full_like(x, float("nan"))
                ctx.cmd_moe_layer(x, want, route, pages[7].data_ptr(), L.PAGE_MXFP4, hidden, inter)
                _noalloc(route, pages[7].data_ptr(), hidden, inter, x, got, mode)
                torch.cuda.synchronize()
                # same kernels, same order of operations: the tolerance of the other tests is met exactly
                assert torch.equal(want, got), (mode, call, (want - got).abs().max().item())
    finally:
        ctx.close()


def test_noalloc_layer_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    hidden, inter = 1024, 1024
    page = torch.zeros(synth.mxfp4_expert_page(synth.rng(1), hidden, inter).size, dtype=torch.uint8, device="cuda")
    x = torch.zeros((2, hidden), device="cuda")
    y = torch.empty_like(x)
    two_tokens = [TokenRoute([0], [1.0], [page.data_ptr()])] * 2
    with pytest.raises(S14Error) as e:
        _noalloc(two_tokens, None, hidden, inter, x, y, L.ACCUM_PAIRWISE)
    assert e.value.code == L.ERR_CONTRACT and "one token" in e.value.message
    with pytest.raises(S14Error):
        _noalloc(two_tokens[:1], None, 8192, inter, x, y, L.ACCUM_PAIRWISE)
    torch.cuda.synchronize()


def test_noalloc_layer_names_the_sizes_it_takes():
    """hidden and intermediate are 1024, 2048 or 4096, as the header says; 3072 fits the scratch but
    no layer kernel is built for it, and the refusal says which sizes are taken."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    page = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    x = torch.zeros((1, 4096), device="cuda")
    y = torch.empty_like(x)
    one = [TokenRoute([0], [1.0], [page.data_ptr()])]
    for hidden, inter in ((3072, 1024), (1024, 3072), (512, 1024)):
        with pytest.raises(S14Error) as e:
            _noalloc(one, None, hidden, inter, x, y, L.ACCUM_PAIRWISE)
        assert e.value.code == L.ERR_CONTRACT and "1024, 2048 or 4096" in e.value.message


def test_noalloc_layer_leaves_the_current_device_as_it_was():
    """The call makes `device` current for itself only: afterwards cudaGetDevice gives what it gave
    before, after a good call and after a refused one.  With two GPUs the call goes to the other one."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    target = 1 if torch.cuda.device_count() > 1 else 0
    before = torch.cuda.current_device()
    hidden, inter = 1024, 1024
    lay = ExpertPageLayout(hidden, inter)
    with torch.cuda.device(target):
        page = torch.from_numpy(lay.to_expert_page(synth.mxfp4_expert_page(synth.rng(5), hidden, inter))).cuda()
        x = torch.from_numpy(synth.activations(synth.rng(6), 1, hidden)).cuda()
        y = torch.empty_like(x)
        torch.cuda.synchronize()
    desc, keep = _layer_desc([TokenRoute([0], [1.0], [page.data_ptr()])], None, L.PAGE_MXFP4, hidden, inter)
    desc.x, desc.y = x.data_ptr(), y.data_ptr()
    assert torch.cuda.current_device() == before
    L.check(L.lib().s14_moe_layer_noalloc(target, None, L.ACCUM_PAIRWISE, C.byref(desc)))
    assert torch.cuda.current_device() == before
    desc.n_tokens = 2  # refused
    assert L.lib().s14_moe_layer_noalloc(target, None, L.ACCUM_PAIRWISE, C.byref(desc)) == L.ERR_CONTRACT
    assert torch.cuda.current_device() == before
    with torch.cuda.device(target):
        torch.cuda.synchronize()
        assert bool(torch.isfinite(y).all())
    del keep
