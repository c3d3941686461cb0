"""Host-side contract of the S14 page pool and operator shapes, through the C ABI, without
a GPU.  Each test restates a unit test of the reference (file:line in the docstring)."""
import ctypes as C

import numpy as np
import pytest

from colormlm_b200 import _lib as L
from colormlm_b200.s14 import (ExpertKey, RouteDecision, S14Error, S14MatvecShape, S14MoePages,
                               VramPool, validate_e4m3fn_codes, validate_ue8m0_codes)

pytestmark = pytest.mark.usefixtures("cuda_lib")

ROUTED, SHARED = L.ROUTED_EXPERT_KIND, L.SHARED_EXPERT_KIND


def route(ids, weights=None, layer=42, kind=1):
    return RouteDecision(layer=layer, kind=kind, expert_ids=list(ids),
                         weights=list(weights) if weights is not None else [0.25] * 6)


def test_real_sample_shapes_have_exact_byte_contracts():
    """s14_vulkan.rs:835-856"""
    w1 = S14MatvecShape(2048, 4096).validate_mxfp4()
    assert w1.mxfp4_weight_bytes() == 4_194_304 and w1.mxfp4_scale_bytes() == 262_144
    w2 = S14MatvecShape(4096, 2048).validate_mxfp4()
    assert w2.mxfp4_weight_bytes() == 4_194_304 and w2.mxfp4_scale_bytes() == 262_144
    wq_a = S14MatvecShape(1024, 4096).validate_fp8()
    assert wq_a.fp8_weight_bytes() == 4_194_304 and wq_a.fp8_scale_bytes() == 256
    assert w1.fp32_input_bytes() == 16384 and w1.fp32_output_bytes() == 8192
    assert 3 * 4_194_304 + 3 * 262_144 == L.EXPERT_PAGE_BYTES
    shared_up = S14MatvecShape(2048, 4096).validate_fp8()
    assert 3 * shared_up.fp8_weight_bytes() + 3 * shared_up.fp8_scale_bytes() == L.SHARED_EXPERT_PAGE_BYTES


def test_rejects_invalid_quantized_codes():
    """s14_vulkan.rs:859-865"""
    validate_ue8m0_codes(bytes([0, 127, 254]))
    with pytest.raises(S14Error) as e:
        validate_ue8m0_codes(bytes([127, 255]))
    assert e.value.code == L.ERR_CODE and "byte 1" in e.value.message
    validate_e4m3fn_codes(bytes([0x00, 0x01, 0x7E, 0xFE]))
    for bad in (0x7F, 0xFF):
        with pytest.raises(S14Error):
            validate_e4m3fn_codes(bytes([bad]))
    validate_ue8m0_codes(b"")


def test_mxfp4_rejects_non_native_k_alignment_and_zero_shapes():
    """s14_vulkan.rs:868-873, 46-50"""
    with pytest.raises(S14Error):
        S14MatvecShape(1, 32).validate_mxfp4()
    with pytest.raises(S14Error):
        S14MatvecShape(0, 128)
    with pytest.raises(S14Error):
        S14MatvecShape(4, 0)
    S14MatvecShape(1, 128).validate_mxfp4()
    assert S14MatvecShape(129, 130).validate_fp8().fp8_scale_bytes() == 4  # ragged: ceil on both axes


def test_reserve_eviction_logic():
    """vram_pool.rs:437-489"""
    p = VramPool(None, 3, 1024)
    k1, k2, k3, k4 = (ExpertKey(0, 0, i) for i in (1, 2, 3, 4))
    for i, k in enumerate((k1, k2, k3)):
        slot, evicted = p.reserve_loading(k)
        assert slot == i and evicted is None
        assert p.lookup(k) is None  # hidden while Loading
        p.mark_ready(slot, k)
    assert p.n_loaded() == 3
    p.lookup(k2)  # k1 becomes the oldest
    slot, evicted = p.reserve_loading(k4)
    assert slot == 0 and (evicted.layer, evicted.kind, evicted.slot) == (0, 0, 1)
    assert p.lookup(k4) is None
    p.mark_ready(slot, k4)
    assert p.n_loaded() == 3
    assert p.lookup(k1) is None
    assert p.lookup(k2) is not None and p.lookup(k3) is not None and p.lookup(k4) is not None
    assert p.capacity() == 3 and p.slot_bytes() == 1024 and p.total_bytes() == 3072
    assert p.slot_offset(2) == 2048 and p.slot_ptr(2) is None


def test_loading_slots_are_hidden_and_never_evicted():
    """vram_pool.rs:492-522"""
    p = VramPool(None, 1, 1024)
    loading, other = ExpertKey(1, 0, 7), ExpertKey(1, 0, 8)
    slot, _ = p.reserve_loading(loading)
    assert p.lookup(loading) is None
    with pytest.raises(S14Error) as e:
        p.reserve_loading(other)
    assert e.value.code == L.ERR_POOL
    with pytest.raises(S14Error):
        p.reserve_loading(loading)  # already loading
    p.cancel_loading(slot, loading)
    replacement, _ = p.reserve_loading(other)
    assert replacement == slot
    p.mark_ready(replacement, other)
    assert p.lookup(other) == slot
    with pytest.raises(S14Error):
        p.reserve_loading(other)  # already ready


def test_pinned_ready_slot_cannot_be_evicted_until_compute_fence_release():
    """vram_pool.rs:525-551"""
    p = VramPool(None, 1, 1024)
    resident, replacement = ExpertKey(42, ROUTED, 126), ExpertKey(42, ROUTED, 12)
    lease = p.publish_batch_and_pin([p.reserve_loading_generation(resident)])[0]
    with pytest.raises(S14Error):
        p.reserve_loading_generation(replacement)
    p.release_after_compute_fence(lease)
    r = p.reserve_loading_generation(replacement)
    assert r.has_evicted and r.evicted.slot == 126


def test_stale_generation_is_rejected_after_slot_reuse():
    """vram_pool.rs:554-586"""
    p = VramPool(None, 1, 1024)
    first, second = ExpertKey(42, ROUTED, 126), ExpertKey(42, ROUTED, 12)
    lease = p.publish_batch_and_pin([p.reserve_loading_generation(first)])[0]
    stale = L.SlotBinding.from_buffer_copy(lease)
    p.release_after_compute_fence(lease)
    p.publish_batch_and_pin([p.reserve_loading_generation(second)])
    with pytest.raises(S14Error):
        p.validate_binding(stale)
    with pytest.raises(S14Error):
        p.release_after_compute_fence(stale)


def test_batch_publish_preflight_prevents_partial_visibility():
    """vram_pool.rs:589-616"""
    p = VramPool(None, 2, 1024)
    first, second = ExpertKey(42, ROUTED, 126), ExpertKey(42, ROUTED, 12)
    r1, r2 = p.reserve_loading_generation(first), p.reserve_loading_generation(second)
    stale2 = L.LoadingReservation.from_buffer_copy(r2)
    stale2.generation += 1
    with pytest.raises(S14Error):
        p.publish_batch_and_pin([r1, stale2])
    assert p.lookup(first) is None and p.lookup(second) is None
    with pytest.raises(S14Error):
        p.publish_batch_and_pin([])  # an empty batch is an error
    with pytest.raises(S14Error):
        p.publish_batch_and_pin([r1, r1])  # duplicate slot / key
    p.cancel_reservation(r1)
    p.cancel_reservation(r2)
    with pytest.raises(S14Error):
        p.cancel_reservation(r1)  # already cancelled
    assert p.n_loaded() == 0


def test_pool_rejects_degenerate_sizes():
    """vram_pool.rs:77-85"""
    for n, b in ((0, 1024), (4, 0), (0xFFFFFFFF, 1 << 62)):
        with pytest.raises(S14Error):
            VramPool(None, n, b)


def test_route_decision_validate_for():
    """s14_runner/src/runner.rs:128-180"""
    good = route([126, 12, 205, 149, 227, 174])
    good.validate_for(L.PROFILE_S14_TOP6)
    good.validate_for(L.PROFILE_FULL_DEPTH43_NATIVE_TOP6)
    bad_cases = [
        route([126, 12, 205, 149, 227, 174], layer=3),             # not an S14 layer
        route([126, 12, 205, 149, 227]),                           # five ids
        route([126, 12, 205, 149, 227, 174], kind=0),              # score layer with hash kind
        route([126, 12, 205, 149, 227, 256]),                      # id out of range
        route([126, 126, 205, 149, 227, 174]),                     # duplicate
        route([126, 12, 205, 149, 227, 174], [0.25] * 5 + [float("nan")]),
        route([126, 12, 205, 149, 227, 174], [0.25] * 5 + [-0.25]),
        route([126, 12, 205, 149, 227, 174], [0.0] + [0.25] * 5),  # sum 1.25
    ]
    for r in bad_cases:
        with pytest.raises(S14Error) as e:
            r.validate_for(L.PROFILE_S14_TOP6)
        assert e.value.code == L.ERR_CONTRACT
    route([1, 2, 3, 4, 5, 6], layer=3).validate_for(L.PROFILE_FULL_DEPTH43_NATIVE_TOP6)
    route([1, 2, 3, 4, 5, 6], layer=1, kind=0).validate_for(L.PROFILE_S14_TOP6)  # hash layers 0-2


def _pools(n_routed):
    return (VramPool(None, n_routed, L.EXPERT_PAGE_BYTES), VramPool(None, 1, L.SHARED_EXPERT_PAGE_BYTES))


def test_moe_pages_require_full_size_slots():
    """s14_vulkan.rs:709-734"""
    small = VramPool(None, 6, L.EXPERT_PAGE_BYTES - 1)
    shared = VramPool(None, 1, L.SHARED_EXPERT_PAGE_BYTES)
    with pytest.raises(S14Error):
        S14MoePages(small, shared)
    with pytest.raises(S14Error):
        S14MoePages(VramPool(None, 6, L.EXPERT_PAGE_BYTES), VramPool(None, 1, L.EXPERT_PAGE_BYTES))
    # an MXFP4 shared expert only needs a routed-size slot
    S14MoePages(VramPool(None, 6, L.EXPERT_PAGE_BYTES), VramPool(None, 1, L.EXPERT_PAGE_BYTES),
                min_shared_bytes=L.EXPERT_PAGE_BYTES)


def test_route_load_batch_rolls_back_every_reservation_on_capacity_failure():
    """s14_vulkan.rs:876-889"""
    routed, shared = _pools(5)
    pages = S14MoePages(routed, shared)
    with pytest.raises(S14Error):
        pages.begin_after_official_route(route([126, 12, 205, 149, 227, 174]))
    assert routed.n_loaded() == 0 and shared.n_loaded() == 0


def test_route_load_batch_rejects_duplicate_or_weight_drift_before_reservation():
    """s14_vulkan.rs:892-908"""
    routed, shared = _pools(6)
    pages = S14MoePages(routed, shared)
    with pytest.raises(S14Error):
        pages.begin_after_official_route(route([126, 126, 205, 149, 227, 174]))
    with pytest.raises(S14Error):
        pages.begin_after_official_route(route([126, 12, 205, 149, 227, 174], [0.0] + [0.25] * 5))
    assert routed.n_loaded() == 0 and shared.n_loaded() == 0


def test_route_load_batch_capacity_failure_releases_cached_pin():
    """s14_vulkan.rs:911-939"""
    resident = ExpertKey(42, ROUTED, 126)
    routed, shared = _pools(1)
    lease = routed.publish_batch_and_pin([routed.reserve_loading_generation(resident)])[0]
    routed.release_after_compute_fence(lease)
    pages = S14MoePages(routed, shared)
    with pytest.raises(S14Error):
        pages.begin_after_official_route(route([126, 12, 205, 149, 227, 174]))
    routed.reserve_loading_generation(ExpertKey(42, ROUTED, 7))  # the cached pin was given back


def test_route_load_batch_publishes_all_then_holds_compute_fence_pins():
    """s14_vulkan.rs:942-963"""
    routed, shared = _pools(6)
    pages = S14MoePages(routed, shared)
    ids = [126, 12, 205, 149, 227, 174]
    batch = pages.begin_after_official_route(route(ids))
    missing = batch.missing()
    assert len(missing) == 7 and [m[1] for m in missing] == [False] * 6 + [True]
    compute = pages.publish_after_transfer_fence(batch)
    assert len(compute.routed_bindings()) == 6 and compute.expert_ids() == ids
    assert compute.route_weights() == [0.25] * 6
    assert compute.shared_binding().key.kind == SHARED
    with pytest.raises(S14Error):
        pages.begin_after_official_route(route([1, 2, 3, 4, 5, 6]))  # everything is pinned
    pages.release_after_compute_fence(compute)
    replacement = pages.begin_after_official_route(route([1, 2, 3, 4, 5, 6]))
    pages.cancel(replacement)
    # a second pass over the first route now hits the shared page and misses the evicted ones
    again = pages.begin_after_official_route(route(ids))
    assert not any(is_shared for _, is_shared in again.missing())
    pages.cancel(again)


def test_stale_shared_generation_prevents_partial_routed_publication():
    """s14_vulkan.rs:966-996"""
    ids = [126, 12, 205, 149, 227, 174]
    routed, shared = _pools(6)
    pages = S14MoePages(routed, shared)
    batch = pages.begin_after_official_route(route(ids))
    stale_shared = [r for r, is_shared in batch.missing() if is_shared][0]
    shared.cancel_reservation(stale_shared)
    unrelated = shared.reserve_loading_generation(ExpertKey(42, SHARED, 1))
    with pytest.raises(S14Error):
        pages.publish_after_transfer_fence(batch)
    for e in ids:
        assert routed.lookup(ExpertKey(42, ROUTED, e)) is None
    assert routed.n_loaded() == 0
    shared.cancel_reservation(unrelated)


def test_upload_needs_a_device_pool():
    p = VramPool(None, 1, 1024)
    r = p.reserve_loading_generation(ExpertKey(0, ROUTED, 0))
    buf = np.zeros(16, np.uint8)
    with pytest.raises(S14Error):
        p.upload_page_async(r, buf.ctypes.data, 16)


def test_expert_page_from_tensors_matches_the_numpy_mirror_and_the_stated_offsets():
    """The MXFP4 expert page: the C conversion, the numpy mirror and the byte offsets stated in
    the header agree, and converting back returns the tensors."""
    import ctypes as C

    import numpy as np

    from colormlm_b200 import _lib as L
    from colormlm_b200 import synth
    from colormlm_b200.pages import ExpertPageLayout

    for hidden, inter in ((1024, 1024), (2048, 1024), (512, 256)):
        lay = ExpertPageLayout(hidden, inter)
        tensor_page = synth.mxfp4_expert_page(synth.rng(9 + hidden), hidden, inter)
        want = lay.to_expert_page(tensor_page)
        got = np.empty_like(want)
        L.check(L.lib().s14_mxfp4_expert_page_from_tensors(hidden, inter, tensor_page.ctypes.data_as(C.c_void_p),
                                                           got.ctypes.data_as(C.c_void_p)))
        assert np.array_equal(want, got)
        assert not np.array_equal(want, tensor_page)
        t, o = lay.split(tensor_page), lay.offsets
        g = np.random.default_rng(1)

        unit = 16384 + 1024  # codes, then two scale atoms

        def in_unit(m, kb):  # 128 rows of 128 bytes, the 16-byte chunks of row m at chunk ^ (m % 8)
            return m * 128 + (((kb % 8) ^ (m % 8)) << 4)

        def scale_in_unit(m, kb):
            return 16384 + ((kb // 4) % 2) * 512 + (m % 32) * 16 + (m // 32) * 4 + kb % 4

        down0 = (inter // 64) * (hidden // 256) * unit
        for _ in range(200):
            n, kb = int(g.integers(hidden)), int(g.integers(inter // 32))
            base = down0 + ((n // 128) * (inter // 256) + kb // 8) * unit
            off = base + in_unit(n % 128, kb)
            assert np.array_equal(got[off:off + 16], t["w2"].reshape(hidden, inter // 2)[n, kb * 16:kb * 16 + 16])
            assert got[base + scale_in_unit(n % 128, kb)] == t["s2"].reshape(hidden, inter // 32)[n, kb]
            i, kb = int(g.integers(inter)), int(g.integers(hidden // 32))
            for mat, name, wname in ((0, "s1", "w1"), (1, "s3", "w3")):
                m = i % 64 + 64 * mat
                base = ((i // 64) * (hidden // 256) + kb // 8) * unit
                assert got[base + scale_in_unit(m, kb)] == t[name].reshape(inter, hidden // 32)[i, kb]
                off = base + in_unit(m, kb)
                assert np.array_equal(got[off:off + 16], t[wname].reshape(inter, hidden // 2)[i, kb * 16:kb * 16 + 16])
        back = np.empty_like(tensor_page)
        L.check(L.lib().s14_mxfp4_expert_page_to_tensors(hidden, inter, got.ctypes.data_as(C.c_void_p),
                                                         back.ctypes.data_as(C.c_void_p)))
        assert np.array_equal(back, tensor_page)
    with pytest.raises(L.S14Error):
        L.check(L.lib().s14_mxfp4_expert_page_from_tensors(100, 256, None, None))


# ---- ExpertLoader (expert_loader.rs:163-442): staging ring, per-entry fences, waves ------------

def _host_pool(n_slots, slot_bytes):
    pool = C.c_void_p()
    L.check(L.lib().s14_pool_create_host(n_slots, slot_bytes, C.byref(pool)))
    return pool


def _loader(pool, depth):
    ld = C.c_void_p()
    L.check(L.lib().s14_loader_create(pool, depth, C.byref(ld)))
    return ld


def _page(tag, nbytes):
    return (np.arange(nbytes, dtype=np.uint32) * 2654435761 + tag * 97).astype(np.uint8)


def _slot_bytes_of(pool, slot, nbytes):
    ptr = L.lib().s14_pool_slot_ptr(pool, slot)
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(nbytes,)).copy()


def _lookup(pool, key):
    slot = C.c_uint32()
    found = C.c_int32()
    L.check(L.lib().s14_pool_lookup(pool, key, C.byref(found), C.byref(slot)))
    return slot.value if found.value else None


def test_loader_page_is_hidden_until_its_transfer_is_complete(cuda_lib):
    slot_bytes = 256
    pool, ld = _host_pool(4, slot_bytes), None
    try:
        ld = _loader(pool, 2)
        key = L.ExpertKey(3, 0, 17)
        data = _page(1, slot_bytes)
        slot = C.c_uint32()
        L.check(L.lib().s14_loader_enqueue_from_buf(ld, key, data.ctypes.data, data.size, C.byref(slot)))
        assert L.lib().s14_loader_in_flight(ld) == 1
        assert _lookup(pool, key) is None  # Loading: not visible
        L.check(L.lib().s14_loader_wait_all(ld))
        assert L.lib().s14_loader_in_flight(ld) == 0
        assert _lookup(pool, key) == slot.value
        assert np.array_equal(_slot_bytes_of(pool, slot.value, slot_bytes), data)
        # a page that is Ready is not loaded again
        again = C.c_uint32()
        L.check(L.lib().s14_loader_enqueue_from_buf(ld, key, data.ctypes.data, data.size, C.byref(again)))
        assert again.value == slot.value and L.lib().s14_loader_stat_loads(ld) == 1
        assert L.lib().s14_loader_stat_bytes(ld) == slot_bytes
    finally:
        L.lib().s14_loader_destroy(ld)
        L.lib().s14_pool_destroy(pool)


def test_loader_reclaims_a_ring_entry_before_reusing_its_staging_buffer(cuda_lib):
    """Three pages through a ring of two: the third takes the first entry again, which publishes the
    first page; every page arrives intact although the host engine copies as late as the wait."""
    slot_bytes = 128
    pool, ld = _host_pool(8, slot_bytes), None
    try:
        ld = _loader(pool, 2)
        keys = [L.ExpertKey(0, 0, i) for i in range(3)]
        pages = [_page(10 + i, slot_bytes) for i in range(3)]
        slots = []
        for k, p in zip(keys, pages):
            s = C.c_uint32()
            L.check(L.lib().s14_loader_enqueue_from_buf(ld, k, p.ctypes.data, p.size, C.byref(s)))
            slots.append(s.value)
        assert _lookup(pool, keys[0]) == slots[0]      # published when its entry was reclaimed
        assert _lookup(pool, keys[1]) is None and _lookup(pool, keys[2]) is None
        assert L.lib().s14_loader_in_flight(ld) == 2
        # asking for a page that is in flight settles it instead of loading it twice
        s = C.c_uint32()
        L.check(L.lib().s14_loader_enqueue_from_buf(ld, keys[1], pages[1].ctypes.data, slot_bytes, C.byref(s)))
        assert s.value == slots[1] and _lookup(pool, keys[1]) == slots[1]
        L.check(L.lib().s14_loader_wait_all(ld))
        for k, p, sl in zip(keys, pages, slots):
            assert _lookup(pool, k) == sl
            assert np.array_equal(_slot_bytes_of(pool, sl, slot_bytes), p)
        assert L.lib().s14_loader_stat_loads(ld) == 3
    finally:
        L.lib().s14_loader_destroy(ld)
        L.lib().s14_pool_destroy(pool)


def test_loader_batch_runs_in_waves_no_deeper_than_the_ring(cuda_lib):
    """Seven requests with two duplicates through a ring of two (expert_loader.rs:299-358): five
    loads, every input gets its page's slot, all but the last wave are Ready on return, and no page
    was overwritten in a staging buffer."""
    slot_bytes = 64
    pool, ld = _host_pool(8, slot_bytes), None
    try:
        ld = _loader(pool, 2)
        ids = [4, 1, 4, 9, 2, 1, 7]
        keys = (L.ExpertKey * len(ids))(*[L.ExpertKey(5, 0, i) for i in ids])
        pages = {i: _page(i, slot_bytes) for i in set(ids)}
        datas = (C.c_void_p * len(ids))(*[pages[i].ctypes.data for i in ids])
        sizes = (C.c_uint64 * len(ids))(*[slot_bytes] * len(ids))
        slots = (C.c_uint32 * len(ids))()
        L.check(L.lib().s14_loader_batch_enqueue_from_bufs(ld, keys, datas, sizes, len(ids), slots))
        assert L.lib().s14_loader_stat_loads(ld) == 5
        assert slots[0] == slots[2] and slots[1] == slots[5] and len({slots[i] for i in range(len(ids))}) == 5
        assert L.lib().s14_loader_in_flight(ld) == 1  # the last wave (one page) is still in flight
        assert _lookup(pool, L.ExpertKey(5, 0, 7)) is None and _lookup(pool, L.ExpertKey(5, 0, 2)) is not None
        L.check(L.lib().s14_loader_wait_all(ld))
        for pos, i in enumerate(ids):
            assert np.array_equal(_slot_bytes_of(pool, slots[pos], slot_bytes), pages[i]), i
    finally:
        L.lib().s14_loader_destroy(ld)
        L.lib().s14_pool_destroy(pool)


def test_loader_refusals_leave_the_pool_as_it_was(cuda_lib):
    slot_bytes = 64
    pool, ld = _host_pool(2, slot_bytes), None
    try:
        ld = _loader(pool, 2)
        big = _page(1, 2 * slot_bytes)
        s = C.c_uint32()
        rc = L.lib().s14_loader_enqueue_from_buf(ld, L.ExpertKey(0, 0, 1), big.ctypes.data, big.size, C.byref(s))
        assert rc == L.ERR_POOL and L.lib().s14_pool_n_loaded(pool) == 0 and L.lib().s14_loader_in_flight(ld) == 0
        # more distinct pages than the pool has slots: refused before anything is issued
        ids = [1, 2, 3]
        keys = (L.ExpertKey * 3)(*[L.ExpertKey(0, 0, i) for i in ids])
        pages = [_page(i, slot_bytes) for i in ids]
        datas = (C.c_void_p * 3)(*[p.ctypes.data for p in pages])
        sizes = (C.c_uint64 * 3)(*[slot_bytes] * 3)
        slots = (C.c_uint32 * 3)()
        rc = L.lib().s14_loader_batch_enqueue_from_bufs(ld, keys, datas, sizes, 3, slots)
        assert rc == L.ERR_POOL and b"distinct experts" in L.lib().s14_last_error()
        assert L.lib().s14_loader_stat_loads(ld) == 0 and L.lib().s14_pool_n_loaded(pool) == 0
        # a loader on a bookkeeping-only pool is refused
        bare = C.c_void_p()
        L.check(L.lib().s14_pool_create(None, 2, slot_bytes, C.byref(bare)))
        none = C.c_void_p()
        assert L.lib().s14_loader_create(bare, 2, C.byref(none)) == L.ERR_POOL
        L.lib().s14_pool_destroy(bare)
        assert L.lib().s14_loader_create(pool, 0, C.byref(none)) == L.ERR_POOL
    finally:
        L.lib().s14_loader_destroy(ld)
        L.lib().s14_pool_destroy(pool)
