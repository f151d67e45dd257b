// Host side of the path: VRAM page pool with a frozen resident snapshot, and the query planner
// that turns router output into per-expert page lists.
//
// Mirrors, for VRAM-resident weights only:
//   PageId / key()                         src/core/types.rs:199-265
//   PageBufferManager (T1 pool, page table, preload, resident snapshot, get_page_resident)
//                                          src/storage/buffer_manager.rs:206-288, :622-761, :883-899
//   LayerPlan / ExpertPlan / ResolvedPage, QueryPlanner::plan_layer (resident fast path)
//                                          src/runtime/query_planner.rs:19-46, :235-272
// The reference allocates one cudaMalloc(2 MiB) per slot (buffer_manager.rs:1237-1242); here the
// pool is one allocation cut into 2 MiB slots, so a 180 GB device holds the slots back to back
// and page addresses stay 2 MiB aligned.  RAM/NVMe tiers, eviction and prefetch are absent: a
// page that is not resident is an error (Error::PageNotFound), never a fault.
#pragma once
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace vib3 {

constexpr size_t kPageSize = 2u * 1024u * 1024u;  // PAGE_SIZE, src/core/types.rs:14
constexpr uint16_t kExpertShared = 0xFFFF;        // EXPERT_SHARED, src/core/types.rs:170
// shared-expert segment ids (src/storage/convert.rs:2014-2032)
constexpr uint16_t kSegSharedUp = 14, kSegSharedGate = 15, kSegSharedDown = 16;

struct PageId {
    uint16_t layer, expert, segment, page_idx;
    static PageId shared(uint16_t layer, uint16_t segment, uint16_t page_idx) {
        return PageId{layer, kExpertShared, segment, page_idx};
    }
    uint64_t key() const {
        return (uint64_t)layer << 48 | (uint64_t)expert << 32 | (uint64_t)segment << 16 | (uint64_t)page_idx;
    }
    static PageId from_key(uint64_t k) {
        return PageId{(uint16_t)(k >> 48), (uint16_t)(k >> 32), (uint16_t)(k >> 16), (uint16_t)k};
    }
};

// What get_page_resident returns (PageHandle, buffer_manager.rs:883-899) plus the catalog's row
// range (format.rs:113-114), which the planner copies into ResolvedPage.
struct ResidentPage {
    void* device_ptr;
    uint32_t size;
    uint16_t row_start, row_count;
    int64_t slot;
};

struct ResolvedPage {
    PageId id;
    void* device_ptr;
    uint16_t row_start, row_count;
};

struct ExpertPlan {
    uint16_t expert_id;
    float weight;
    std::vector<ResolvedPage> pages;
    bool fully_resident;
};

struct LayerPlan {
    uint16_t layer;
    std::vector<ExpertPlan> experts;
    bool all_resident;
};

// Device form of a ResolvedPage; layout shared with the kernels (vib3_page_entry).
struct DevicePageEntry {
    uint64_t ptr;
    uint16_t row_start, row_count;
    uint32_t reserved;
};

class PageBufferManager {
public:
    // device_base == nullptr: allocate capacity_pages * 2 MiB; else adopt caller-owned memory.
    PageBufferManager(void* device_base, size_t capacity_pages, uint64_t slot_seed);
    ~PageBufferManager();
    PageBufferManager(const PageBufferManager&) = delete;
    PageBufferManager& operator=(const PageBufferManager&) = delete;

    bool ok() const { return base_ != nullptr; }
    size_t capacity() const { return capacity_; }
    void* slot_ptr(int64_t slot) const;

    // Place one page (preload_all's per-page step): free slot, optional H2D copy, table entry.
    // Returns the slot or a negative VIB3_ERR_* code.
    int64_t load_page(PageId id, uint16_t row_start, uint16_t row_count, const void* host_data, size_t nbytes);
    // Freeze into the resident snapshot (buffer_manager.rs:746-757).
    int freeze();
    bool frozen() const { return frozen_; }
    size_t resident_pages() const { return table_.size(); }
    // Snapshot lookup; nullptr when absent or not frozen.
    const ResidentPage* get_page_resident(PageId id) const;
    // Number of pages the catalog holds for the segment of `id` (highest loaded page_idx + 1).
    int segment_page_count(PageId id) const;

    // Device table [num_experts][3][pages] for a layer (or [3][pages] for its shared expert),
    // built once and cached; absent pages become ptr = 0.
    int device_page_table(uint16_t layer, int num_experts, int pages, bool shared, void** out);

private:
    unsigned char* base_ = nullptr;
    bool owns_ = false;
    size_t capacity_ = 0;
    std::vector<int64_t> free_slots_;  // handed out from the back
    std::unordered_map<uint64_t, ResidentPage> table_;
    std::unordered_map<uint64_t, int> segment_counts_;
    bool frozen_ = false;
    std::mutex mu_;
    std::unordered_map<uint64_t, void*> device_tables_;
};

class QueryPlanner {
public:
    explicit QueryPlanner(const PageBufferManager* pool, int pages_per_segment)
        : pool_(pool), pages_(pages_per_segment) {}
    // plan_layer_resident (query_planner.rs:235-272).  Returns 0, or VIB3_ERR_RANGE when a page of
    // an active expert is missing (the reference's Error::PageNotFound), VIB3_ERR_STATE before freeze.
    int plan_layer(uint16_t layer, const uint16_t* expert_ids, const float* weights, int n, LayerPlan* out) const;

private:
    const PageBufferManager* pool_;
    int pages_;
};

}  // namespace vib3
