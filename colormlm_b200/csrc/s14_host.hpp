// C++ host-side mirror of the reference's operator / page-pool interface for the
// S14 MoE path.  Names, argument meaning and error behaviour follow the Rust
// types they stand in for; each class cites them.  Everything here is plain
// host bookkeeping: device memory is a base address handed in by the caller.
#ifndef S14_HOST_HPP
#define S14_HOST_HPP

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "s14_page_layout.h"

namespace s14 {

// Error classes map onto the C ABI status codes.
struct ContractError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct PoolError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct CodeError : std::runtime_error {
    uint64_t index;
    CodeError(const std::string &m, uint64_t i) : std::runtime_error(m), index(i) {}
};

// S14MatvecShape (ssd_inference/src/s14_vulkan.rs:40-114).
struct S14MatvecShape {
    uint32_t n = 0, k = 0;
    static S14MatvecShape make(uint32_t n, uint32_t k);
    S14MatvecShape validate_mxfp4() const;
    S14MatvecShape validate_fp8() const;
    uint64_t fp32_input_bytes() const { return (uint64_t)k * 4; }
    uint64_t fp32_output_bytes() const { return (uint64_t)n * 4; }
    uint64_t mxfp4_weight_bytes() const;
    uint64_t mxfp4_scale_bytes() const;
    uint64_t fp8_weight_bytes() const { return (uint64_t)n * k; }
    uint64_t fp8_scale_bytes() const;
};

// storage_bytes (s14_vulkan.rs:128-130): byte counts rounded up to whole 32-bit words.
inline uint64_t storage_bytes(uint64_t logical) { return (logical + 3) / 4 * 4; }

// The MXFP4 expert page the GPU reads (byte order: s14_page_layout.h) against the *tensor page*, the
// six checkpoint tensors in their own ABI one after the other (w1 | w3 | w2 | s1 | s3 | s2, weights
// [N, K/2] bytes, scales [N, K/32] codes), which the loader receives.  Same size; hidden and
// intermediate must be multiples of 256.  No counterpart in the reference, which fixes no page layout.
// src and dst must not overlap.
void mxfp4_expert_page_from_tensors(uint32_t hidden, uint32_t inter, const uint8_t *tensor_page, uint8_t *page);
void mxfp4_expert_page_to_tensors(uint32_t hidden, uint32_t inter, const uint8_t *page, uint8_t *tensor_page);

// validate_ue8m0_codes / validate_e4m3fn_codes (s14_vulkan.rs:143-156).
void validate_ue8m0_codes(const uint8_t *codes, uint64_t len);
void validate_e4m3fn_codes(const uint8_t *codes, uint64_t len);

// ExpertKey (vram_pool.rs:16-21).
struct ExpertKey {
    uint32_t layer = 0;
    uint8_t kind = 0;
    uint32_t slot = 0;
    bool operator==(const ExpertKey &o) const {
        return layer == o.layer && kind == o.kind && slot == o.slot;
    }
};
struct ExpertKeyHash {
    size_t operator()(const ExpertKey &k) const {
        uint64_t v = ((uint64_t)k.layer << 40) ^ ((uint64_t)k.kind << 32) ^ k.slot;
        v ^= v >> 33;
        v *= 0xff51afd7ed558ccdull;
        v ^= v >> 33;
        return (size_t)v;
    }
};

// SlotBinding / SlotLease / LoadingReservation (vram_pool.rs:30-60).  A lease is a
// binding whose pin the holder must give back through release_after_compute_fence.
struct SlotBinding {
    ExpertKey key;
    uint32_t slot = 0;
    uint64_t generation = 0;
};
using SlotLease = SlotBinding;
struct LoadingReservation {
    ExpertKey key;
    uint32_t slot = 0;
    uint64_t generation = 0;
    std::optional<ExpertKey> evicted;
};

// VramPool (vram_pool.rs:62-422): fixed slots, Empty -> Loading -> Ready, LRU among
// unpinned Ready slots, generation stamp per reservation, pin count per slot.
class VramPool {
public:
    // base == nullptr gives the bookkeeping-only pool of the reference's unit tests.
    VramPool(uint32_t n_slots, uint64_t slot_bytes, uint8_t *base);
    uint32_t capacity() const { return n_slots_; }
    uint64_t slot_bytes() const { return slot_bytes_; }
    uint32_t n_loaded() const { return n_loaded_; }
    uint64_t total_bytes() const { return (uint64_t)n_slots_ * slot_bytes_; }
    uint64_t slot_offset(uint32_t slot) const { return (uint64_t)slot * slot_bytes_; }
    uint8_t *slot_ptr(uint32_t slot) const { return base_ ? base_ + slot_offset(slot) : nullptr; }
    uint8_t *base() const { return base_; }

    std::optional<uint32_t> lookup(const ExpertKey &key);
    std::optional<SlotLease> lookup_and_pin(const ExpertKey &key);
    LoadingReservation reserve_loading_generation(const ExpertKey &key);
    void mark_ready(uint32_t slot, const ExpertKey &key);
    void validate_publish_batch(const std::vector<LoadingReservation> &reservations) const;
    std::vector<SlotLease> publish_batch_and_pin(const std::vector<LoadingReservation> &reservations);
    std::vector<SlotLease> publish_prevalidated_batch_and_pin(
        const std::vector<LoadingReservation> &reservations);
    void validate_binding(const SlotBinding &binding) const;
    void release_after_compute_fence(const SlotLease &lease);
    void cancel_loading(uint32_t slot, const ExpertKey &key);
    void cancel_reservation(const LoadingReservation &reservation);

private:
    enum class State : uint8_t { Empty, Loading, Ready };
    struct Slot {
        State state = State::Empty;
        ExpertKey key;
        uint64_t last_access = 0;
        uint32_t pin_count = 0;
        uint64_t generation = 0;
    };
    bool is(uint32_t slot, State st, const ExpertKey &key) const {
        return slots_[slot].state == st && slots_[slot].key == key;
    }
    uint8_t *base_;
    uint64_t slot_bytes_;
    uint32_t n_slots_;
    std::vector<Slot> slots_;
    std::unordered_map<ExpertKey, uint32_t, ExpertKeyHash> index_;
    uint64_t clock_ = 0;
    uint32_t n_loaded_ = 0;
};

// ExpertLoader (ssd_inference/src/expert_loader.rs:163-442): expert pages go to pool slots through a
// ring of `pipeline_depth` staging buffers, each with a fence of its own.  An entry of the ring is
// reused only after its transfer has completed and its page has been published (Loading -> Ready); a
// page is not visible through VramPool::lookup before that.  batch_enqueue works in waves no deeper
// than the ring, so that a later page never overwrites staging memory an earlier transfer still
// reads (expert_loader.rs:299-358).  The transfers themselves are behind an interface: CUDA copies
// on the context's copy stream in the library, host copies that run as late as the wait in the CPU
// tests (which is what shows a staging buffer that was reused too early).
struct TransferEngine {
    virtual ~TransferEngine() = default;
    virtual uint8_t *staging(uint32_t entry) = 0;                          // host memory of the ring entry
    virtual void submit(uint32_t entry, uint8_t *dst, uint64_t bytes) = 0; // start staging -> dst; throws on failure
    virtual void wait(uint32_t entry) = 0;                                 // that entry's last transfer is complete
};

class ExpertLoader {
public:
    ExpertLoader(VramPool &pool, TransferEngine &engine, uint32_t pipeline_depth, uint64_t staging_bytes);
    // The page of `key` from bytes in host memory: returns the pool slot.  A page that is Ready, or
    // in flight (its entry is completed first), is not loaded again.  Blocks only to reclaim the
    // ring entry it takes (enqueue_from_buf, expert_loader.rs:362-442).
    uint32_t enqueue_from_buf(const ExpertKey &key, const uint8_t *data, uint64_t bytes);
    // Several pages: earlier work is settled, duplicates are loaded once, more distinct pages than
    // the pool has slots are refused before anything is issued; waves of pipeline_depth, every wave but
    // the last drained before the next one starts (batch_enqueue, expert_loader.rs:299-358).
    std::vector<uint32_t> batch_enqueue_from_bufs(const std::vector<ExpertKey> &keys,
                                                  const std::vector<const uint8_t *> &datas,
                                                  const std::vector<uint64_t> &sizes);
    void wait_all();  // every transfer complete, every page published (expert_loader.rs:291-297)
    uint32_t in_flight() const;
    uint32_t pipeline_depth() const { return depth_; }
    uint64_t stat_loads = 0, stat_bytes = 0;

private:
    struct Pending {
        bool active = false;
        ExpertKey key;
        uint32_t slot = 0;
    };
    void complete_entry(uint32_t entry);
    VramPool &pool_;
    TransferEngine &engine_;
    uint32_t depth_;
    uint64_t staging_bytes_;
    uint32_t next_ = 0;
    std::vector<Pending> pending_;
};

// RouterKind / GraphProfile / RouteDecision (s14_runner/src/contract.rs:27-52,
// runner.rs:121-180).
enum class RouterKind : uint8_t { Hash = 0, Score = 1 };
enum class GraphProfile : uint32_t { S14Top6 = 0, FullDepth43NativeTop6 = 1 };
struct RouteDecision {
    uint8_t layer = 0;
    RouterKind kind = RouterKind::Score;
    std::vector<uint16_t> expert_ids;
    std::vector<float> weights;
    void validate_for(GraphProfile profile) const;
};

// One page of a route transaction: either a pinned cached page or a reservation
// that still needs its upload (PageState, s14_vulkan.rs:499-503).
struct PageState {
    bool loading = false;
    SlotLease lease;
    LoadingReservation reservation;
};

// RouteLoadBatch / S14MoeComputeLeaseBatch (s14_vulkan.rs:663-701).
struct RouteLoadBatch {
    uint8_t layer = 0;
    std::vector<uint16_t> expert_ids;
    std::vector<float> route_weights;
    std::vector<PageState> routed_pages;
    PageState shared_page;
};
struct S14MoeComputeLeaseBatch {
    uint8_t layer = 0;
    std::vector<uint16_t> expert_ids;
    std::vector<float> route_weights;
    std::vector<SlotLease> routed;
    SlotLease shared;
};

// S14VulkanMoePages (s14_vulkan.rs:703-819): all-or-nothing transaction over the six
// routed pages and the layer's shared page, across two pools.
class S14MoePages {
public:
    // min_*_bytes default to EXPERT_PAGE_BYTES / S14_SHARED_EXPERT_PAGE_BYTES
    // (s14_runner/src/memory.rs:3, s14_vulkan.rs:18); other values serve small test shapes
    // and the MXFP4 shared expert.
    S14MoePages(VramPool &routed_pool, VramPool &shared_pool, GraphProfile profile,
                uint64_t min_routed_bytes = 13369344ull, uint64_t min_shared_bytes = 25167360ull);
    RouteLoadBatch begin_after_official_route(const RouteDecision &route);
    S14MoeComputeLeaseBatch publish_after_transfer_fence(RouteLoadBatch batch);
    void release_after_compute_fence(S14MoeComputeLeaseBatch batch);
    void cancel(RouteLoadBatch batch);
    VramPool &routed_pool() { return routed_; }
    VramPool &shared_pool() { return shared_; }

private:
    VramPool &routed_;
    VramPool &shared_;
    GraphProfile profile_;
};

}  // namespace s14

#endif
