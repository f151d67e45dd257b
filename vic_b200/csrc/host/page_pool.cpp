#include "page_pool.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "../launch_common.h"

namespace vib3 {

namespace {
// splitmix64: seeds the slot permutation
uint64_t splitmix(uint64_t& s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// key of a segment's page counter (the catalog's "how many pages does this segment have")
uint64_t count_key(PageId id) { return PageId{id.layer, id.expert, id.segment, 0xFFFF}.key(); }
}  // namespace

PageBufferManager::PageBufferManager(void* device_base, size_t capacity_pages, uint64_t slot_seed)
    : capacity_(capacity_pages) {
    if (capacity_pages == 0) return;
    if (device_base) {
        if ((uintptr_t)device_base & 255) return;  // slots must keep 16-byte code rows aligned
        base_ = static_cast<unsigned char*>(device_base);
    } else {
        void* p = nullptr;
        if (cudaMalloc(&p, capacity_pages * kPageSize) != cudaSuccess) {
            cudaGetLastError();
            return;
        }
        base_ = static_cast<unsigned char*>(p);
        owns_ = true;
    }
    free_slots_.resize(capacity_pages);
    for (size_t i = 0; i < capacity_pages; ++i) free_slots_[i] = (int64_t)(capacity_pages - 1 - i);
    if (slot_seed != 0) {
        uint64_t s = slot_seed;
        for (size_t i = capacity_pages - 1; i > 0; --i) {
            size_t j = (size_t)(splitmix(s) % (i + 1));
            std::swap(free_slots_[i], free_slots_[j]);
        }
    }
}

PageBufferManager::~PageBufferManager() {
    for (auto& kv : device_tables_) cudaFree(kv.second);
    if (owns_ && base_) cudaFree(base_);
}

void* PageBufferManager::slot_ptr(int64_t slot) const {
    if (!base_ || slot < 0 || (size_t)slot >= capacity_) return nullptr;
    return base_ + (size_t)slot * kPageSize;
}

int64_t PageBufferManager::load_page(PageId id, uint16_t row_start, uint16_t row_count, const void* host_data,
                                     size_t nbytes) {
    std::lock_guard<std::mutex> lock(mu_);
    if (!base_ || frozen_) return VIB3_ERR_STATE;
    if (nbytes == 0 || nbytes > kPageSize) return VIB3_ERR_SHAPE;
    if (id.page_idx == 0xFFFF) return VIB3_ERR_RANGE;
    if (table_.count(id.key())) return VIB3_ERR_STATE;  // already resident
    if (free_slots_.empty()) return VIB3_ERR_COUNT;     // the reference's Error::TierFull
    const int64_t slot = free_slots_.back();
    void* dst = slot_ptr(slot);
    if (host_data) {
        // a pool over host memory (tests of the host logic without a GPU) takes a plain copy
        cudaPointerAttributes attr;
        const bool on_device = cudaPointerGetAttributes(&attr, dst) == cudaSuccess &&
                               (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
        if (!on_device) {
            (void)cudaGetLastError();
            memcpy(dst, host_data, nbytes);
        } else if (cudaMemcpy(dst, host_data, nbytes, cudaMemcpyHostToDevice) != cudaSuccess) {
            return VIB3_ERR_STATE;
        }
    }
    free_slots_.pop_back();
    table_[id.key()] = ResidentPage{dst, (uint32_t)nbytes, row_start, row_count, slot};
    int& cnt = segment_counts_[count_key(id)];
    cnt = std::max(cnt, (int)id.page_idx + 1);
    return slot;
}

int PageBufferManager::freeze() {
    std::lock_guard<std::mutex> lock(mu_);
    if (!base_) return VIB3_ERR_STATE;
    frozen_ = true;
    return VIB3_OK;
}

int PageBufferManager::segment_page_count(PageId id) const {
    auto it = segment_counts_.find(count_key(id));
    return it == segment_counts_.end() ? 0 : it->second;
}

const ResidentPage* PageBufferManager::get_page_resident(PageId id) const {
    if (!frozen_ || id.page_idx == 0xFFFF) return nullptr;
    auto it = table_.find(id.key());
    return it == table_.end() ? nullptr : &it->second;
}

int PageBufferManager::device_page_table(uint16_t layer, int num_experts, int pages, bool shared, void** out) {
    if (!out) return VIB3_ERR_NULL;
    if (!frozen_) return VIB3_ERR_STATE;
    if (pages <= 0 || pages > 0xFFFE || (!shared && (num_experts <= 0 || num_experts > 0xFFFE))) return VIB3_ERR_COUNT;
    std::lock_guard<std::mutex> lock(mu_);
    const uint64_t ck = ((uint64_t)layer << 40) | ((uint64_t)(shared ? 1 : 0) << 39) | ((uint64_t)num_experts << 16) | (uint64_t)pages;
    auto it = device_tables_.find(ck);
    if (it != device_tables_.end()) {
        *out = it->second;
        return VIB3_OK;
    }
    const int experts = shared ? 1 : num_experts;
    std::vector<DevicePageEntry> host((size_t)experts * 3 * pages, DevicePageEntry{0, 0, 0, 0});
    const uint16_t shared_seg[3] = {kSegSharedUp, kSegSharedGate, kSegSharedDown};
    for (int e = 0; e < experts; ++e)
        for (int seg = 0; seg < 3; ++seg)
            for (int p = 0; p < pages; ++p) {
                PageId id = shared ? PageId::shared(layer, shared_seg[seg], (uint16_t)p)
                                   : PageId{layer, (uint16_t)e, (uint16_t)seg, (uint16_t)p};
                auto f = table_.find(id.key());
                if (f == table_.end()) continue;
                host[((size_t)e * 3 + seg) * pages + p] =
                    DevicePageEntry{(uint64_t)(uintptr_t)f->second.device_ptr, f->second.row_start, f->second.row_count, 0};
            }
    void* dev = nullptr;
    cudaError_t err = cudaMalloc(&dev, host.size() * sizeof(DevicePageEntry));
    if (err != cudaSuccess) return (int)err;
    err = cudaMemcpy(dev, host.data(), host.size() * sizeof(DevicePageEntry), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        cudaFree(dev);
        return (int)err;
    }
    device_tables_[ck] = dev;
    *out = dev;
    return VIB3_OK;
}

int QueryPlanner::plan_layer(uint16_t layer, const uint16_t* expert_ids, const float* weights, int n,
                             LayerPlan* out) const {
    if (!pool_ || !out || (n > 0 && !expert_ids)) return VIB3_ERR_NULL;
    if (!pool_->frozen()) return VIB3_ERR_STATE;
    out->layer = layer;
    out->experts.clear();
    out->all_resident = true;
    for (int i = 0; i < n; ++i) {
        ExpertPlan ep{expert_ids[i], weights ? weights[i] : 0.f, {}, true};
        const bool shared = expert_ids[i] == kExpertShared;
        const uint16_t segs[3] = {shared ? kSegSharedUp : (uint16_t)0, shared ? kSegSharedGate : (uint16_t)1,
                                  shared ? kSegSharedDown : (uint16_t)2};
        for (int s = 0; s < 3; ++s) {
            // pages of a segment in catalog order (segment, page_idx): format.rs:881-892
            int found = 0;
            for (int p = 0; p < pages_; ++p) {
                const ResidentPage* rp = pool_->get_page_resident(PageId{layer, expert_ids[i], segs[s], (uint16_t)p});
                if (!rp) break;
                ep.pages.push_back(ResolvedPage{PageId{layer, expert_ids[i], segs[s], (uint16_t)p}, rp->device_ptr,
                                                rp->row_start, rp->row_count});
                ++found;
            }
            if (found == 0 || pool_->segment_page_count(PageId{layer, expert_ids[i], segs[s], 0}) != found)
                return VIB3_ERR_RANGE;  // Error::PageNotFound
        }
        out->experts.push_back(std::move(ep));
    }
    return VIB3_OK;
}

}  // namespace vib3

// ── C view ─────────────────────────────────────────────────────────────────────────────────

using namespace vib3;

struct vib3_pool {
    PageBufferManager mgr;
    vib3_pool(void* base, size_t cap, uint64_t seed) : mgr(base, cap, seed) {}
};

struct vib3_resolved_page_c {
    uint64_t key;
    void* device_ptr;
    uint16_t expert_id, segment, row_start, row_count;
};

extern "C" {

vib3_pool* vib3_pool_create(void* device_base, size_t capacity_pages, uint64_t slot_seed) {
    vib3_pool* p = new vib3_pool(device_base, capacity_pages, slot_seed);
    if (!p->mgr.ok()) {
        delete p;
        return nullptr;
    }
    return p;
}

void vib3_pool_destroy(vib3_pool* pool) { delete pool; }

long long vib3_pool_load_page(vib3_pool* pool, uint16_t layer, uint16_t expert, uint16_t segment, uint16_t page_idx,
                              uint16_t row_start, uint16_t row_count, const void* host_data, size_t nbytes) {
    if (!pool) return VIB3_ERR_NULL;
    return pool->mgr.load_page(PageId{layer, expert, segment, page_idx}, row_start, row_count, host_data, nbytes);
}

void* vib3_pool_slot_ptr(const vib3_pool* pool, long long slot) { return pool ? pool->mgr.slot_ptr(slot) : nullptr; }

int vib3_pool_freeze(vib3_pool* pool) { return pool ? pool->mgr.freeze() : VIB3_ERR_NULL; }

int vib3_pool_get_page_resident(const vib3_pool* pool, uint64_t page_key, void** device_ptr, uint16_t* row_start,
                                uint16_t* row_count, uint32_t* size) {
    if (!pool) return VIB3_ERR_NULL;
    if (!pool->mgr.frozen()) return VIB3_ERR_STATE;
    const ResidentPage* rp = pool->mgr.get_page_resident(PageId::from_key(page_key));
    if (!rp) return VIB3_ERR_RANGE;
    if (device_ptr) *device_ptr = rp->device_ptr;
    if (row_start) *row_start = rp->row_start;
    if (row_count) *row_count = rp->row_count;
    if (size) *size = rp->size;
    return VIB3_OK;
}

size_t vib3_pool_resident_pages(const vib3_pool* pool) { return pool ? pool->mgr.resident_pages() : 0; }

int vib3_pool_device_page_table(vib3_pool* pool, uint16_t layer, int num_experts, int pages_per_segment, int shared,
                                void** device_table) {
    if (!pool) return VIB3_ERR_NULL;
    return pool->mgr.device_page_table(layer, num_experts, pages_per_segment, shared != 0, device_table);
}

uint64_t vib3_page_key(uint16_t layer, uint16_t expert, uint16_t segment, uint16_t page_idx) {
    return PageId{layer, expert, segment, page_idx}.key();
}

int vib3_planner_plan_layer(const vib3_pool* pool, uint16_t layer, const uint16_t* expert_ids, int num_active,
                            int pages_per_segment, vib3_resolved_page_c* out_pages, int max_pages) {
    if (!pool || (!out_pages && max_pages > 0)) return VIB3_ERR_NULL;
    QueryPlanner planner(&pool->mgr, pages_per_segment);
    LayerPlan plan;
    if (int e = planner.plan_layer(layer, expert_ids, nullptr, num_active, &plan)) return e;
    int n = 0;
    for (const auto& ep : plan.experts)
        for (const auto& rp : ep.pages) {
            if (n >= max_pages) return VIB3_ERR_COUNT;
            out_pages[n++] = vib3_resolved_page_c{rp.id.key(), rp.device_ptr, ep.expert_id, rp.id.segment, rp.row_start,
                                                  rp.row_count};
        }
    return n;
}

const char* vib3_b200_version(void) { return "vib3-b200 0.1 (sm_100a)"; }

}  // extern "C"
