// vib3_launch_moe_layer_int4_paged_noalloc: the fused MoE sublayer for callers that cannot hand
// over a scratch buffer.
//
// Who needs it: a host that gives all free VRAM to its page pool at start-up (the reference sizes
// its T1 pool from free device memory, src/runtime/engine.rs:593-662, so a cudaMalloc made later by a
// plugin can fail), a serving loop that forbids allocation after warm-up because cudaMalloc and
// cudaFree may synchronise the device, or a binding layer that has no allocator of its own.  Such a
// caller still passes its inputs and its output; only the fp16 intermediate that travels from the
// gate/up kernel to the down kernel comes from an array that is part of this library's image.
//
// The array is a file-scope __device__ array: every GPU on which this part of the library gets loaded
// keeps kNoAllocMaxHalves * 2 bytes (544 KiB) for it until the process exits.  With the CUDA runtime's
// lazy module loading that happens at the first call on a device, not when the library is opened: the
// first call may therefore synchronise the device and, on a device without 544 KiB free, fails with
// the runtime's out-of-memory error.  A caller that hands all free VRAM to a pool makes one call
// (any valid arguments) BEFORE it sizes the pool.  In host code the array's name is only a handle, not
// a device address, so the address is asked for once per device with cudaGetSymbolAddress (with that
// device current) and then passed to the kernels like any buffer.
//
// Rules for callers:
//   * (top_k + 1 if a shared expert is given) * expert_hidden_dim must not exceed 278,528 values;
//     larger requests return VIB3_ERR_CAPACITY and launch nothing.
//   * The first call on a device loads the array and looks its address up.  Make that call outside any
//     stream capture and before free VRAM is given away.
//   * All calls on a device share the one array and each call overwrites what the previous one left
//     (nothing has to be cleared: the second kernel reads only what the first kernel of the same call
//     wrote).  Two calls whose kernels can overlap on the GPU — different streams without an ordering
//     between them — race on it; order them, or use vib3_launch_moe_layer_int4_paged with one
//     scratch buffer per stream.
//   * No cudaMalloc, cudaFree or other allocating call is made here or below.
#include <cuda_fp16.h>
#include <mutex>

#include "launch_common.h"

extern "C" int vib3_launch_moe_layer_int4_paged(const void* x, int x_dtype, const void* page_table, int num_experts,
                                                const void* shared_pages, const unsigned short* expert_ids,
                                                const float* expert_weights, int top_k, float shared_weight,
                                                void* act_scratch, float* out, int out_accumulate, int hidden_dim,
                                                int expert_hidden_dim, int pages_per_segment,
                                                int rows_per_page_gate_up, int rows_per_page_down, int group_size,
                                                int* status, void* stream);

namespace {

constexpr size_t kNoAllocMaxHalves = 17u * 16384u;  // 278,528 fp16 values = 544 KiB
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) __half g_noalloc_act[kNoAllocMaxHalves];

std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kNoAllocMaxDevices] = {};

// Device address of the array on the current device; looked up on first use.
int noalloc_scratch(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return VIB3_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_act);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return VIB3_ERR_STATE;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return VIB3_OK;
}

}  // namespace

extern "C" int vib3_launch_moe_layer_int4_paged_noalloc(const void* x, int x_dtype, const void* page_table,
                                                        int num_experts, const void* shared_pages,
                                                        const unsigned short* expert_ids, const float* expert_weights,
                                                        int top_k, float shared_weight, float* out, int out_accumulate,
                                                        int hidden_dim, int expert_hidden_dim, int pages_per_segment,
                                                        int rows_per_page_gate_up, int rows_per_page_down,
                                                        int group_size, int* status, void* stream) {
    if (top_k < 0) return VIB3_ERR_COUNT;   // (the codes of vib3_launch_moe_layer_int4_paged)
    if (expert_hidden_dim <= 0) return VIB3_ERR_SHAPE;
    const size_t slots = (size_t)top_k + (shared_pages ? 1u : 0u);
    if (slots * (size_t)expert_hidden_dim > kNoAllocMaxHalves) return VIB3_ERR_CAPACITY;
    void* scratch = nullptr;
    if (int e = noalloc_scratch(&scratch)) return e;
    return vib3_launch_moe_layer_int4_paged(x, x_dtype, page_table, num_experts, shared_pages, expert_ids,
                                            expert_weights, top_k, shared_weight, scratch, out, out_accumulate,
                                            hidden_dim, expert_hidden_dim, pages_per_segment, rows_per_page_gate_up,
                                            rows_per_page_down, group_size, status, stream);
}
