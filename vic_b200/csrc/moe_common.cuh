// Argument block, limits and page-table helpers shared by the MoE sublayer kernels.
#pragma once
#include "int4_math.cuh"
#include "launch_common.h"
#include <atomic>

namespace vib3 {

constexpr int kMaxSlots = 17;   // MAX_ACTIVE_EXPERTS (src/core/types.rs:26) + one shared expert
constexpr int kMaxPages = 16;   // pages per segment the kernels accept (Mixtral-shape needs 16)
constexpr int kSegUp = 0, kSegGate = 1, kSegDown = 2;

struct MoeLayerArgs {
    const void* x;                 // [H] activations
    int x_dtype;                   // XDType
    const PageEntry* page_table;   // [num_experts][3][P]
    const PageEntry* shared_pages; // [3][P] or null
    const unsigned short* expert_ids;  // [top_k], device
    const float* expert_weights;       // [top_k], device
    int top_k;
    const int* num_active_dev;     // optional device int: use only the first min(top_k, *num_active_dev) routed slots
    int num_experts;
    float shared_weight;
    __half* act;                   // [slots][I] scratch, in act_slot() order
    float* out;                    // [H]
    int out_accumulate;            // 0: out = layer output; 1: out += layer output (residual add)
    int H, I, P;
    int rpp_gu, rpp_dn;            // rows per page of gate/up and of down
    int* status;                   // device status word, or null
    // Grouped mode (slot_token != null): the routed slots are (token, expert) PAIRS of several tokens,
    // listed in ascending token order; x and out have one row per token.
    const unsigned short* slot_token;  // [top_k] token of each routed slot, or null
    int n_tokens;                  // rows of x / out
    int shared_token;              // the token the shared expert (if any) belongs to
    int x_stride;                  // bytes between the tokens' activation vectors
    int out_stride;                // floats between the tokens' output rows
    int slot_begin;                // pairs of the device-side count that earlier launches have taken
};

enum StatusBits : int { kStatusMissingPage = 1, kStatusBadExpert = 2, kStatusTimeout = 4 };

// Routed slots actually used by this launch (see MoeLayerArgs::num_active_dev).
__device__ __forceinline__ int active_top_k(const MoeLayerArgs& a) {
    if (a.num_active_dev == nullptr) return a.top_k;
    return min(a.top_k, max(0, *a.num_active_dev - a.slot_begin));
}

__device__ __forceinline__ void flag(int* status, int bit) {
    if (status) atomicOr(status, bit);
}

// One warp lists the (token, expert, weight) triples, token-major, whose expert lies in [lo, hi): the pairs of a step
// that an expert-parallel rank owns.  ids / w: n_tokens rows of top_k entries, row strides in bytes.  The lists have
// room for `capacity` entries; *count_out receives the number of pairs found, even if it exceeds the capacity.
__device__ __forceinline__ void select_local_pairs_warp(const unsigned char* ids, int ids_stride, const unsigned char* w, int w_stride,
                                                        int n_tokens, int top_k, int lo, int hi, unsigned short* pe, float* pw,
                                                        unsigned short* pt, int capacity, int* count_out) {
    const int lane = threadIdx.x & 31;
    const int total = n_tokens * top_k;
    int n = 0;
    for (int base = 0; base < total; base += 32) {
        const int i = base + lane;
        int e = -1, tk = 0;
        float wv = 0.f;
        if (i < total) {
            tk = i / top_k;
            const int j = i - tk * top_k;
            e = reinterpret_cast<const unsigned short*>(ids + (size_t)tk * ids_stride)[j];
            wv = reinterpret_cast<const float*>(w + (size_t)tk * w_stride)[j];
        }
        const bool keep = e >= lo && e < hi;
        const unsigned m = __ballot_sync(0xffffffffu, keep);
        const int pos = n + __popc(m & ((1u << lane) - 1u));
        if (keep && pos < capacity) {
            pe[pos] = (unsigned short)e;
            pw[pos] = wv;
            pt[pos] = (unsigned short)tk;
        }
        n += __popc(m);
    }
    if (lane == 0) *count_out = n;
}

// Position of slot s's activations in the scratch buffer: the shared expert (slot top_k in plan
// order) is stored FIRST, so that where it lives does not depend on the routing — the gate/up kernel
// can then work on the shared expert before the router has finished.  `a.top_k` is the active count.
__device__ __forceinline__ int act_slot(const MoeLayerArgs& a, int s) {
    const int nsh = a.shared_pages ? 1 : 0;
    return s < a.top_k ? s + nsh : 0;
}

// Resolve the page-table block ([3][P] entries) of slot s: routed expert or the shared expert.
__device__ __forceinline__ const PageEntry* slot_pages(const MoeLayerArgs& a, int s) {
    if (s < a.top_k) {
        unsigned e = __ldcg(a.expert_ids + s);  // (from L2: the router may have stored it moments ago)
        if (e >= (unsigned)a.num_experts) return nullptr;
        return a.page_table + (size_t)e * 3 * a.P;
    }
    return a.shared_pages;
}


// Pipelined (bulk-copy staged) variants, defined in moe_pipe.cu.  They return VIB3_ERR_UNSUPPORTED
// without launching when the shape does not meet their alignment rules; the caller then uses the
// direct-load kernels.
struct RouterArgs;
int launch_gateup_pipelined(const MoeLayerArgs& a, cudaStream_t st, const RouterArgs* router = nullptr);
int launch_down_pipelined(const MoeLayerArgs& a, cudaStream_t st);
int sm_count();

// Run-time switch: 1 (default) = staged kernels where the shape allows, 0 = direct-load kernels only.
extern std::atomic<int> g_use_pipeline;
// 1 (default) = staged kernels are launched with programmatic dependent launch.
extern std::atomic<int> g_use_pdl;
// Shared memory the gate/up kernel leaves free on an SM so that a router CTA (43 KB static plus the
// per-CTA reservation) fits beside it.
constexpr size_t kRouterCtaSmem = 46 * 1024;

}  // namespace vib3
