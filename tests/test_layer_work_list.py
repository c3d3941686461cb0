"""The deal of a layer's work to the CTAs of the tensor-core kernel (host arithmetic, no GPU):
every up item (job, slice) and every down item (job, row tile) belongs to exactly one CTA, a
CTA runs its up items before its down items (so no wait of a down item on another CTA's up
items can form a cycle), and the units of 16 KB per CTA are level."""
import ctypes as C

import numpy as np
import pytest

from colormlm_b200 import _lib as L


def work_list(cta, n_ctas, n_jobs, hidden, inter, cap=1024, n_early=0):
    items = (C.c_uint32 * cap)()
    count = C.c_uint32(0)
    L.check(L.lib().s14_layer_work_list(cta, n_ctas, n_jobs, n_early, hidden, inter, items, cap, C.byref(count)))
    return [int(v) for v in items[:min(count.value, cap)]], count.value


@pytest.mark.parametrize("n_early", [0, 1])
@pytest.mark.parametrize("n_ctas", [148, 132, 64, 7])
@pytest.mark.parametrize("n_jobs", [1, 2, 5, 7])
@pytest.mark.parametrize("hidden,inter", [(4096, 2048), (2048, 1024), (1024, 1024), (1024, 4096), (512, 512)])
def test_every_item_once_up_before_down(cuda_lib, n_ctas, n_jobs, hidden, inter, n_early):
    S, RT = inter // 64, hidden // 128
    seen = {}
    for c in range(n_ctas):
        items, count = work_list(c, n_ctas, n_jobs, hidden, inter, n_early=n_early)
        ups = [it for it in items if not it >> 31]
        # the early jobs' up items lead the list
        assert [((it >> 8) & 0xFF) < n_early for it in ups] == sorted(((it >> 8) & 0xFF) < n_early for it in ups)[::-1]
        assert count == len(items)
        downs_started = False
        last_down = -1
        for it in items:
            down, job, idx = it >> 31, (it >> 8) & 0xFF, it & 0xFF
            assert job < n_jobs and idx < (RT if down else S)
            assert (down, job, idx) not in seen
            seen[(down, job, idx)] = c
            if down:
                downs_started = True
                assert job * RT + idx > last_down  # a CTA's down items keep the job order
                last_down = job * RT + idx
            else:
                assert not downs_started
    assert len(seen) == n_jobs * (S + RT)


def test_benchmark_layer_is_level(cuda_lib):
    """7 experts at 4096 x 2048 on 148 CTAs: 36.3 units per CTA on average, no CTA above 40; the
    shared expert (job 0 of a routed call) has its 32 up items on CTAs 0-31."""
    hidden, inter, n_ctas = 4096, 2048, 148
    loads = []
    for c in range(n_ctas):
        items, _ = work_list(c, n_ctas, 7, hidden, inter)
        loads.append(sum((inter // 256) if it >> 31 else (hidden // 256) for it in items))
        if c < 32:
            assert items[0] == c  # up item of job 0, slice c
        assert len(items) <= 5
    assert sum(loads) == 7 * (32 * 16 + 32 * 8)
    assert max(loads) <= 40 and min(loads) >= 24
    assert max(loads) / np.mean(loads) < 1.11


def test_routed_benchmark_layer_is_level(cuda_lib):
    """The same layer when it picks its own routes: the shared expert's 32 up items lead the lists of
    CTAs 0-31 and run during the selection; the other 4864 units are level (32.9 per CTA on average, no
    CTA above 40); CTAs 32-75 hold two routed up items, and the first down items of the first 32 CTAs
    after them are the shared expert's, which are ready first."""
    hidden, inter, n_ctas = 4096, 2048, 148
    loads = []
    for c in range(n_ctas):
        items, _ = work_list(c, n_ctas, 7, hidden, inter, n_early=1)
        if c < 32:
            assert items[0] == c
            items = items[1:]
        ups = [it for it in items if not it >> 31]
        assert all(((it >> 8) & 0xFF) > 0 for it in ups)
        assert len(ups) == (2 if 32 <= c < 76 else 1)
        loads.append(sum((inter // 256) if it >> 31 else (hidden // 256) for it in items))
        if 76 <= c < 108:
            downs = [it for it in items if it >> 31]
            assert downs[0] == (0x80000000 | (c - 76))
    assert sum(loads) == 6 * 32 * 16 + 7 * 32 * 8
    assert max(loads) <= 40 and min(loads) >= 32
    assert max(loads) / np.mean(loads) < 1.22


def test_rejects_bad_arguments(cuda_lib):
    count = C.c_uint32(0)
    for args in ((148, 148, 7, 0, 4096, 2048), (0, 0, 7, 0, 4096, 2048), (0, 148, 7, 0, 4000, 2048), (0, 148, 7, 0, 4096, 0)):
        with pytest.raises(L.S14Error):
            L.check(L.lib().s14_layer_work_list(*args, None, 0, C.byref(count)))
