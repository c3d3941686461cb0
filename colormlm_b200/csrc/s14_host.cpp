// Host-side bookkeeping of the S14 MoE path: byte contracts, code validation,
// the slot pool and the route page transaction.  See s14_host.hpp for the
// reference types each class stands in for.
#include "s14_host.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <sstream>
#include <unordered_set>

#include "../../include/polaris_s14_cuda.h"

namespace s14 {

namespace {
constexpr uint32_t kFp4Group = 32;
constexpr uint32_t kFp8Tile = 128;
constexpr uint8_t kSelectedLayers[14] = {0, 1, 2, 6, 7, 14, 15, 22, 23, 30, 31, 40, 41, 42};
constexpr uint8_t kNumLayers = 43;

std::string key_str(const ExpertKey &k) {
    std::ostringstream os;
    os << "ExpertKey{layer=" << k.layer << ", kind=0x" << std::hex << (int)k.kind << std::dec
       << ", slot=" << k.slot << "}";
    return os.str();
}
}  // namespace

// ---- S14MatvecShape ---------------------------------------------------------

S14MatvecShape S14MatvecShape::make(uint32_t n, uint32_t k) {
    if (n == 0 || k == 0) throw ContractError("S14 matvec requires non-zero N and K");
    S14MatvecShape s;
    s.n = n;
    s.k = k;
    return s;
}

S14MatvecShape S14MatvecShape::validate_mxfp4() const {
    if (n == 0 || k == 0) throw ContractError("S14 matvec requires non-zero N and K");
    if (k % kFp8Tile != 0)
        throw ContractError("S14 MXFP4 K=" + std::to_string(k) + " must be a multiple of 128");
    (void)mxfp4_weight_bytes();
    (void)mxfp4_scale_bytes();
    return *this;
}

S14MatvecShape S14MatvecShape::validate_fp8() const {
    if (n == 0 || k == 0) throw ContractError("S14 matvec requires non-zero N and K");
    (void)fp8_scale_bytes();
    return *this;
}

uint64_t S14MatvecShape::mxfp4_weight_bytes() const {
    if (k % 2 != 0) throw ContractError("S14 MXFP4 K=" + std::to_string(k) + " must be even");
    return (uint64_t)n * k / 2;
}

uint64_t S14MatvecShape::mxfp4_scale_bytes() const {
    if (k % kFp4Group != 0)
        throw ContractError("S14 MXFP4 K=" + std::to_string(k) + " must be a multiple of 32");
    return (uint64_t)n * (k / kFp4Group);
}

uint64_t S14MatvecShape::fp8_scale_bytes() const {
    const uint64_t n_tiles = ((uint64_t)n + kFp8Tile - 1) / kFp8Tile;
    const uint64_t k_tiles = ((uint64_t)k + kFp8Tile - 1) / kFp8Tile;
    return n_tiles * k_tiles;
}

void validate_ue8m0_codes(const uint8_t *codes, uint64_t len) {
    for (uint64_t i = 0; i < len; ++i)
        if (codes[i] == 0xff)
            throw CodeError("UE8M0 scale contains 0xff NaN at byte " + std::to_string(i), i);
}

static void check_page_shape(uint32_t hidden, uint32_t inter, const void *a, const void *b) {
    if (hidden == 0 || inter == 0 || (hidden & 255u) || (inter & 255u))
        throw ContractError("MXFP4 expert page: hidden and intermediate must be non-zero multiples of 256");
    if (!a || !b) throw ContractError("MXFP4 expert page: NULL buffer");
}

// forward = true: tensors -> page order; false: page order -> tensors
static void reorder_page(uint32_t hidden, uint32_t inter, const uint8_t *src, uint8_t *dst, bool forward) {
    const size_t wb = (size_t)hidden * inter / 2, sb = (size_t)hidden * inter / 32;
    const uint32_t kb_down = inter >> 5, kb_up = hidden >> 5;
    auto move16 = [&](size_t tensor_at, size_t page_at) {
        std::memcpy(forward ? dst + page_at : dst + tensor_at, forward ? src + tensor_at : src + page_at, 16);
    };
    auto move1 = [&](size_t tensor_at, size_t page_at) {
        if (forward) dst[page_at] = src[tensor_at];
        else dst[tensor_at] = src[page_at];
    };
    for (uint32_t n = 0; n < hidden; ++n)
        for (uint32_t kb = 0; kb < kb_down; ++kb) {
            move16(2 * wb + (size_t)n * (inter >> 1) + (size_t)kb * 16u, mxfp4_down_chunk_offset(n, kb, hidden, inter));
            move1(3 * wb + 2 * sb + (size_t)n * kb_down + kb, mxfp4_down_scale_offset(n, kb, hidden, inter));
        }
    for (uint32_t mat = 0; mat < 2; ++mat)
        for (uint32_t i = 0; i < inter; ++i)
            for (uint32_t kb = 0; kb < kb_up; ++kb) {
                move16((size_t)mat * wb + (size_t)i * (hidden >> 1) + (size_t)kb * 16u,
                       mxfp4_up_chunk_offset(mat, i, kb, hidden));
                move1(3 * wb + (size_t)mat * sb + (size_t)i * kb_up + kb, mxfp4_up_scale_offset(mat, i, kb, hidden, inter));
            }
}

void mxfp4_expert_page_from_tensors(uint32_t hidden, uint32_t inter, const uint8_t *tensor_page, uint8_t *page) {
    check_page_shape(hidden, inter, tensor_page, page);
    reorder_page(hidden, inter, tensor_page, page, true);
}

void mxfp4_expert_page_to_tensors(uint32_t hidden, uint32_t inter, const uint8_t *page, uint8_t *tensor_page) {
    check_page_shape(hidden, inter, page, tensor_page);
    reorder_page(hidden, inter, page, tensor_page, false);
}

void validate_e4m3fn_codes(const uint8_t *codes, uint64_t len) {
    for (uint64_t i = 0; i < len; ++i)
        if (codes[i] == 0x7f || codes[i] == 0xff)
            throw CodeError("E4M3FN weight contains NaN code at byte " + std::to_string(i), i);
}

// ---- VramPool ---------------------------------------------------------------

VramPool::VramPool(uint32_t n_slots, uint64_t slot_bytes, uint8_t *base)
    : base_(base), slot_bytes_(slot_bytes), n_slots_(n_slots) {
    if (n_slots == 0) throw PoolError("VRAM pool must contain at least one slot");
    if (slot_bytes == 0) throw PoolError("VRAM slot size must be greater than zero");
    if (slot_bytes > std::numeric_limits<uint64_t>::max() / n_slots)
        throw PoolError("VRAM pool size overflow");
    slots_.resize(n_slots);
    index_.reserve(n_slots);
}

std::optional<uint32_t> VramPool::lookup(const ExpertKey &key) {
    auto it = index_.find(key);
    if (it == index_.end()) return std::nullopt;
    if (clock_ != std::numeric_limits<uint64_t>::max()) ++clock_;
    slots_[it->second].last_access = clock_;
    return it->second;
}

std::optional<SlotLease> VramPool::lookup_and_pin(const ExpertKey &key) {
    auto it = index_.find(key);
    if (it == index_.end()) return std::nullopt;
    const uint32_t slot = it->second;
    if (!is(slot, State::Ready, key))
        throw PoolError("VRAM index for " + key_str(key) + " points at non-ready slot " +
                        std::to_string(slot));
    Slot &s = slots_[slot];
    if (s.pin_count == std::numeric_limits<uint32_t>::max())
        throw PoolError("VRAM slot " + std::to_string(slot) + " pin count overflow");
    ++s.pin_count;
    if (clock_ != std::numeric_limits<uint64_t>::max()) ++clock_;
    s.last_access = clock_;
    return SlotLease{key, slot, s.generation};
}

LoadingReservation VramPool::reserve_loading_generation(const ExpertKey &key) {
    if (index_.count(key)) throw PoolError("expert " + key_str(key) + " is already ready");
    for (uint32_t i = 0; i < n_slots_; ++i)
        if (is(i, State::Loading, key))
            throw PoolError("expert " + key_str(key) + " is already loading");

    int64_t chosen = -1;
    for (uint32_t i = 0; i < n_slots_; ++i)
        if (slots_[i].state == State::Empty) {
            chosen = i;
            break;
        }
    if (chosen < 0) {
        // least recently used among Ready slots nobody has pinned; first one on ties
        for (uint32_t i = 0; i < n_slots_; ++i) {
            const Slot &s = slots_[i];
            if (s.state != State::Ready || s.pin_count != 0) continue;
            if (chosen < 0 || s.last_access < slots_[chosen].last_access) chosen = i;
        }
        if (chosen < 0)
            throw PoolError("all " + std::to_string(n_slots_) +
                            " VRAM slots are Loading or pinned Ready");
    }
    Slot &s = slots_[chosen];
    LoadingReservation r;
    if (s.state == State::Ready) {
        index_.erase(s.key);
        r.evicted = s.key;
    } else {
        ++n_loaded_;
    }
    if (s.generation == std::numeric_limits<uint64_t>::max())
        throw PoolError("VRAM slot " + std::to_string(chosen) + " generation overflow");
    ++s.generation;
    s.pin_count = 0;
    s.state = State::Loading;
    s.key = key;
    r.key = key;
    r.slot = (uint32_t)chosen;
    r.generation = s.generation;
    return r;
}

void VramPool::mark_ready(uint32_t slot, const ExpertKey &key) {
    if (slot >= n_slots_) throw PoolError("invalid VRAM slot " + std::to_string(slot));
    if (!is(slot, State::Loading, key))
        throw PoolError("slot " + std::to_string(slot) + " cannot publish " + key_str(key) +
                        ": it is not loading that key");
    LoadingReservation r;
    r.key = key;
    r.slot = slot;
    r.generation = slots_[slot].generation;
    auto leases = publish_batch_and_pin({r});
    release_after_compute_fence(leases[0]);
}

void VramPool::validate_publish_batch(const std::vector<LoadingReservation> &reservations) const {
    if (reservations.empty()) throw PoolError("cannot publish an empty VRAM batch");
    std::unordered_set<uint32_t> seen_slots;
    std::unordered_set<ExpertKey, ExpertKeyHash> seen_keys;
    for (const LoadingReservation &r : reservations) {
        const bool new_slot = seen_slots.insert(r.slot).second;
        if (!new_slot || !seen_keys.insert(r.key).second)
            throw PoolError("VRAM publish batch contains a duplicate slot or key");
        if (r.slot >= n_slots_) throw PoolError("invalid VRAM slot " + std::to_string(r.slot));
        const Slot &s = slots_[r.slot];
        if (!is(r.slot, State::Loading, r.key) || s.generation != r.generation)
            throw PoolError("stale VRAM generation for " + key_str(r.key) +
                            ": slot=" + std::to_string(r.slot) +
                            " generation=" + std::to_string(r.generation) +
                            " current_generation=" + std::to_string(s.generation));
        if (s.pin_count != 0)
            throw PoolError("Loading slot " + std::to_string(r.slot) + " unexpectedly has compute pins");
        if (index_.count(r.key))
            throw PoolError("cannot publish " + key_str(r.key) + ": key is already visible");
    }
}

std::vector<SlotLease> VramPool::publish_batch_and_pin(
    const std::vector<LoadingReservation> &reservations) {
    validate_publish_batch(reservations);
    return publish_prevalidated_batch_and_pin(reservations);
}

std::vector<SlotLease> VramPool::publish_prevalidated_batch_and_pin(
    const std::vector<LoadingReservation> &reservations) {
    std::vector<SlotLease> leases;
    leases.reserve(reservations.size());
    for (const LoadingReservation &r : reservations) {
        Slot &s = slots_[r.slot];
        s.state = State::Ready;
        s.key = r.key;
        index_[r.key] = r.slot;
        s.pin_count = 1;
        if (clock_ != std::numeric_limits<uint64_t>::max()) ++clock_;
        s.last_access = clock_;
        leases.push_back(SlotLease{r.key, r.slot, r.generation});
    }
    return leases;
}

void VramPool::validate_binding(const SlotBinding &b) const {
    if (b.slot >= n_slots_) throw PoolError("invalid VRAM slot " + std::to_string(b.slot));
    const Slot &s = slots_[b.slot];
    if (!is(b.slot, State::Ready, b.key) || s.generation != b.generation || s.pin_count == 0)
        throw PoolError("stale or unpinned VRAM binding for " + key_str(b.key) +
                        ": slot=" + std::to_string(b.slot) +
                        " generation=" + std::to_string(b.generation));
}

void VramPool::release_after_compute_fence(const SlotLease &lease) {
    validate_binding(lease);
    --slots_[lease.slot].pin_count;
}

void VramPool::cancel_loading(uint32_t slot, const ExpertKey &key) {
    if (slot < n_slots_ && is(slot, State::Loading, key)) {
        slots_[slot].state = State::Empty;
        slots_[slot].pin_count = 0;
        if (n_loaded_ > 0) --n_loaded_;
    }
}

void VramPool::cancel_reservation(const LoadingReservation &r) {
    if (r.slot >= n_slots_) throw PoolError("invalid VRAM slot " + std::to_string(r.slot));
    Slot &s = slots_[r.slot];
    if (!is(r.slot, State::Loading, r.key) || s.generation != r.generation)
        throw PoolError("stale VRAM cancellation for " + key_str(r.key) +
                        ": slot=" + std::to_string(r.slot) +
                        " generation=" + std::to_string(r.generation));
    s.state = State::Empty;
    s.pin_count = 0;
    if (n_loaded_ > 0) --n_loaded_;
}

// ---- RouteDecision ----------------------------------------------------------

// ---- ExpertLoader ---------------------------------------------------------------------

ExpertLoader::ExpertLoader(VramPool &pool, TransferEngine &engine, uint32_t pipeline_depth, uint64_t staging_bytes)
    : pool_(pool), engine_(engine), depth_(pipeline_depth), staging_bytes_(staging_bytes), pending_(pipeline_depth) {
    if (pipeline_depth == 0) throw PoolError("expert loader needs a staging ring of at least one buffer");
    if (staging_bytes == 0 || staging_bytes > pool.slot_bytes())
        throw PoolError("staging buffers must hold one page and no more than a VRAM slot: " + std::to_string(staging_bytes) +
                        " bytes against slots of " + std::to_string(pool.slot_bytes()));
}

uint32_t ExpertLoader::in_flight() const {
    uint32_t n = 0;
    for (const Pending &p : pending_) n += p.active ? 1u : 0u;
    return n;
}

// Waits for the entry's transfer and publishes its page.
void ExpertLoader::complete_entry(uint32_t entry) {
    Pending &p = pending_[entry];
    if (!p.active) return;
    engine_.wait(entry);
    p.active = false;  // whatever mark_ready says, the entry is free again
    pool_.mark_ready(p.slot, p.key);
}

uint32_t ExpertLoader::enqueue_from_buf(const ExpertKey &key, const uint8_t *data, uint64_t bytes) {
    if (auto slot = pool_.lookup(key)) return *slot;
    for (uint32_t e = 0; e < depth_; ++e) {
        if (pending_[e].active && pending_[e].key == key) {  // in flight already: settle it
            complete_entry(e);
            if (auto slot = pool_.lookup(key)) return *slot;
        }
    }
    if (!data) throw PoolError("expert page bytes are NULL");
    if (bytes == 0 || bytes > staging_bytes_ || bytes > pool_.slot_bytes())
        throw PoolError("expert page of " + std::to_string(bytes) + " bytes does not fit a staging buffer of " +
                        std::to_string(staging_bytes_) + " / a VRAM slot of " + std::to_string(pool_.slot_bytes()));
    const uint32_t entry = next_;
    next_ = (next_ + 1) % depth_;
    complete_entry(entry);  // the ring entry's earlier transfer no longer reads its staging buffer
    const LoadingReservation r = pool_.reserve_loading_generation(key);  // may evict; hidden until published
    try {
        std::memcpy(engine_.staging(entry), data, bytes);
        engine_.submit(entry, pool_.slot_ptr(r.slot), bytes);
    } catch (...) {
        pool_.cancel_loading(r.slot, key);
        throw;
    }
    pending_[entry].active = true;
    pending_[entry].key = key;
    pending_[entry].slot = r.slot;
    ++stat_loads;
    stat_bytes += bytes;
    return r.slot;
}

void ExpertLoader::wait_all() {
    for (uint32_t e = 0; e < depth_; ++e) complete_entry(e);
}

std::vector<uint32_t> ExpertLoader::batch_enqueue_from_bufs(const std::vector<ExpertKey> &keys,
                                                            const std::vector<const uint8_t *> &datas,
                                                            const std::vector<uint64_t> &sizes) {
    if (keys.size() != datas.size() || keys.size() != sizes.size())
        throw PoolError("expert loader batch: keys, buffers and sizes differ in number");
    if (keys.empty()) return {};
    wait_all();  // earlier work is Ready before duplicates are looked for
    std::vector<size_t> unique;             // first input index of every distinct key
    std::vector<size_t> to_unique(keys.size());
    for (size_t i = 0; i < keys.size(); ++i) {
        size_t u = 0;
        while (u < unique.size() && !(keys[unique[u]] == keys[i])) ++u;
        if (u == unique.size()) unique.push_back(i);
        to_unique[i] = u;
    }
    if (unique.size() > pool_.capacity())
        throw PoolError("batch requests " + std::to_string(unique.size()) + " distinct experts but VRAM pool has only " +
                        std::to_string(pool_.capacity()) + " slots");
    std::vector<uint32_t> slots(unique.size());
    for (size_t base = 0; base < unique.size(); base += depth_) {
        const size_t end = std::min(unique.size(), base + depth_);
        for (size_t u = base; u < end; ++u) slots[u] = enqueue_from_buf(keys[unique[u]], datas[unique[u]], sizes[unique[u]]);
        // the next wave reuses the staging buffers: this one is published and drained first; the last
        // wave stays in flight until the caller's wait_all
        if (end < unique.size()) wait_all();
    }
    std::vector<uint32_t> out(keys.size());
    for (size_t i = 0; i < keys.size(); ++i) out[i] = slots[to_unique[i]];
    return out;
}

void RouteDecision::validate_for(GraphProfile profile) const {
    bool in_profile = false;
    if (profile == GraphProfile::S14Top6) {
        in_profile = std::binary_search(std::begin(kSelectedLayers), std::end(kSelectedLayers), layer);
    } else {
        in_profile = layer < kNumLayers;
    }
    if (!in_profile)
        throw ContractError("route layer " + std::to_string(layer) +
                            " is not part of the registered profile");
    if (expert_ids.size() != S14_EXPERTS_PER_TOKEN || weights.size() != S14_EXPERTS_PER_TOKEN)
        throw ContractError("profile requires top-6, got ids=" + std::to_string(expert_ids.size()) +
                            " weights=" + std::to_string(weights.size()));
    if (layer >= kNumLayers) throw ContractError("layer outside 0..42");
    const RouterKind expected = layer < 3 ? RouterKind::Hash : RouterKind::Score;
    if (kind != expected)
        throw ContractError("L" + std::to_string(layer) + " router kind should be " +
                            (expected == RouterKind::Hash ? "hash" : "score"));
    for (size_t i = 0; i < expert_ids.size(); ++i) {
        if (expert_ids[i] >= S14_N_ROUTED_EXPERTS)
            throw ContractError("route[" + std::to_string(i) + "] expert " +
                                std::to_string(expert_ids[i]) + " out of range");
        if (!std::isfinite(weights[i]) || weights[i] < 0.0f)
            throw ContractError("route[" + std::to_string(i) + "] weight is not finite and non-negative");
        for (size_t j = 0; j < i; ++j)
            if (expert_ids[j] == expert_ids[i])
                throw ContractError("route expert " + std::to_string(expert_ids[i]) + " repeated");
    }
    float sum = 0.0f;
    for (float w : weights) sum += w;
    if (std::fabs(sum - 1.5f) > 1e-4f)
        throw ContractError("normalized weights * route_scale should sum to 1.5, got " +
                            std::to_string(sum));
}

// ---- S14MoePages --------------------------------------------------------------

namespace {

PageState acquire_page(VramPool &pool, const ExpertKey &key) {
    PageState p;
    if (auto lease = pool.lookup_and_pin(key)) {
        p.loading = false;
        p.lease = *lease;
    } else {
        p.loading = true;
        p.reservation = pool.reserve_loading_generation(key);
    }
    return p;
}

std::vector<LoadingReservation> loading_reservations(const std::vector<PageState> &pages) {
    std::vector<LoadingReservation> out;
    for (const PageState &p : pages)
        if (p.loading) out.push_back(p.reservation);
    return out;
}

void validate_page_publish(const VramPool &pool, const std::vector<PageState> &pages) {
    auto r = loading_reservations(pages);
    if (!r.empty()) pool.validate_publish_batch(r);
}

std::vector<SlotLease> publish_prevalidated_pages(VramPool &pool, const std::vector<PageState> &pages) {
    auto r = loading_reservations(pages);
    std::vector<SlotLease> published;
    if (!r.empty()) published = pool.publish_prevalidated_batch_and_pin(r);
    std::vector<SlotLease> out;
    size_t next = 0;
    for (const PageState &p : pages) out.push_back(p.loading ? published.at(next++) : p.lease);
    return out;
}

// Gives back every pin / reservation; returns the first error message ("" = none).
std::string rollback_pages(VramPool &pool, const std::vector<PageState> &pages) {
    std::string first;
    for (const PageState &p : pages) {
        try {
            if (p.loading)
                pool.cancel_reservation(p.reservation);
            else
                pool.release_after_compute_fence(p.lease);
        } catch (const std::exception &e) {
            if (first.empty()) first = e.what();
        }
    }
    return first;
}

}  // namespace

S14MoePages::S14MoePages(VramPool &routed_pool, VramPool &shared_pool, GraphProfile profile,
                         uint64_t min_routed_bytes, uint64_t min_shared_bytes)
    : routed_(routed_pool), shared_(shared_pool), profile_(profile) {
    if (routed_pool.slot_bytes() < min_routed_bytes)
        throw ContractError("S14 routed slot is " + std::to_string(routed_pool.slot_bytes()) +
                            " B, requires at least " + std::to_string(min_routed_bytes) + " B");
    if (shared_pool.slot_bytes() < min_shared_bytes)
        throw ContractError("S14 shared slot is " + std::to_string(shared_pool.slot_bytes()) +
                            " B, requires at least " + std::to_string(min_shared_bytes) + " B");
}

RouteLoadBatch S14MoePages::begin_after_official_route(const RouteDecision &route) {
    route.validate_for(profile_);
    RouteLoadBatch batch;
    batch.layer = route.layer;
    batch.expert_ids = route.expert_ids;
    batch.route_weights = route.weights;
    for (uint16_t expert : route.expert_ids) {
        const ExpertKey key{route.layer, S14_ROUTED_EXPERT_KIND, expert};
        try {
            batch.routed_pages.push_back(acquire_page(routed_, key));
        } catch (...) {
            rollback_pages(routed_, batch.routed_pages);
            throw;
        }
    }
    const ExpertKey shared_key{route.layer, S14_SHARED_EXPERT_KIND, 0};
    try {
        batch.shared_page = acquire_page(shared_, shared_key);
    } catch (...) {
        rollback_pages(routed_, batch.routed_pages);
        throw;
    }
    return batch;
}

S14MoeComputeLeaseBatch S14MoePages::publish_after_transfer_fence(RouteLoadBatch batch) {
    const std::vector<PageState> shared_pages{batch.shared_page};
    try {
        validate_page_publish(routed_, batch.routed_pages);
        validate_page_publish(shared_, shared_pages);
    } catch (...) {
        rollback_pages(routed_, batch.routed_pages);
        rollback_pages(shared_, shared_pages);
        throw;
    }
    S14MoeComputeLeaseBatch out;
    out.layer = batch.layer;
    out.expert_ids = batch.expert_ids;
    out.route_weights = batch.route_weights;
    out.routed = publish_prevalidated_pages(routed_, batch.routed_pages);
    out.shared = publish_prevalidated_pages(shared_, shared_pages).at(0);
    return out;
}

void S14MoePages::release_after_compute_fence(S14MoeComputeLeaseBatch batch) {
    for (const SlotLease &l : batch.routed) routed_.validate_binding(l);
    shared_.validate_binding(batch.shared);
    for (const SlotLease &l : batch.routed) routed_.release_after_compute_fence(l);
    shared_.release_after_compute_fence(batch.shared);
}

void S14MoePages::cancel(RouteLoadBatch batch) {
    const std::string routed_err = rollback_pages(routed_, batch.routed_pages);
    const std::string shared_err = rollback_pages(shared_, {batch.shared_page});
    if (!routed_err.empty()) throw PoolError(routed_err);
    if (!shared_err.empty()) throw PoolError(shared_err);
}

}  // namespace s14
