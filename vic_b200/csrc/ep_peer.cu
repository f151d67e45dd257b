// Expert-parallel exchange over peer memory (NVLink): the two small exchanges of a decode step — every rank's
// token message to every rank, and every rank's partial output row of token t to rank t — as plain stores into
// the peers' buffers followed by a flag, instead of two NCCL collectives (whose latency, about 10 microseconds
// each for messages of 14 to 28 KB, is a fifth of the step).
//
// One process per GPU.  Each rank allocates one exchange buffer with vib3_peer_alloc, which also returns a 64-byte
// inter-process handle; the ranks exchange the handles on the host (any transport) and map each other's buffers
// with vib3_peer_open.  Device code then sees a table of `world` pointers, entry r = rank r's buffer (its own
// allocation for r == rank).  Only plain peer loads and stores are used: no multicast objects, no TMA from peer
// memory.
//
// Ordering.  A sender's kernel stores its data into the peer's buffer, makes the stores visible system-wide
// (__threadfence_system) and then stores the step number into the peer's flag word for this sender.  The
// receiver polls its own flag words with acquire loads at system scope (a kernel of its own, or the first warp of
// the kernel that consumes the data: the pair selection after the messages, the row sum after the partial rows);
// the data is then read from the receiver's own memory.  Step numbers come from a counter in the rank's device
// memory that the wait for the messages advances (the rows of a step carry the advanced number), so a CUDA graph
// of a step can be replayed.
//
// Every poll loop is bounded (kPeerSpinLimit polls with a sleep between them, about two seconds): a peer that
// never arrives sets VIB3_STATUS_TIMEOUT in the status word and the kernel returns; the context stays usable.
//
// Flow control needs no second buffer: a rank publishes the message of step s only after its own step s-1 has
// finished, which needed every rank's partial rows of step s-1, which those ranks wrote after they had read all
// messages of step s-1; and a rank's partial rows of step s are written after it has seen the owner's message
// of step s, which the owner sent after it had summed the rows of step s-1.
#include <cuda_runtime.h>
#include <cstdint>

#include "launch_common.h"
#include "moe_common.cuh"

namespace vib3 {

constexpr unsigned kPeerSpinLimit = 1u << 24;

// grid = world (one CTA per destination).  Destination d receives `bytes` bytes from src + d * src_stride at
// dst_table[d] + rank * dst_stride, then the step number in flag_table[d][rank].  bytes may be 0 (a bare signal).
// add_src (optional; rows of fp32 values, bytes a multiple of 16): when *add_count > add_threshold, row d of add_src is
// added to what is sent — the partial sums of the launch windows beyond the first, which a step almost never needs.
__global__ void __launch_bounds__(256) peer_publish_kernel(const unsigned char* src, size_t src_stride, int bytes,
                                                           unsigned char* const* dst_table, size_t dst_stride,
                                                           unsigned int* const* flag_table, const unsigned int* step_counter,
                                                           unsigned step_offset, int rank, const unsigned char* add_src,
                                                           const int* add_count, int add_threshold) {
    const int d = blockIdx.x;
    const unsigned char* s = src + (size_t)d * src_stride;
    unsigned char* t = dst_table[d] + (size_t)rank * dst_stride;
    const int n16 = bytes >> 4;
    if (add_src != nullptr && *add_count > add_threshold) {
        const float4* s2 = reinterpret_cast<const float4*>(add_src + (size_t)d * src_stride);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(s)[i];
            const float4 w = s2[i];
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
            reinterpret_cast<float4*>(t)[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(t)[i] = reinterpret_cast<const uint4*>(s)[i];
    }
    for (int i = (n16 << 4) + threadIdx.x; i < bytes; i += blockDim.x) t[i] = s[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned step = *step_counter + step_offset;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_table[d] + rank), "r"(step) : "memory");
    }
}

// One warp: lane r (and r + 32, ...) polls flags[r] until it has reached `step`; false if a poll loop ran out.
__device__ __forceinline__ bool peer_wait_warp(const unsigned int* flags, unsigned step, int world) {
    bool ok = true;
    for (int r = threadIdx.x & 31; r < world; r += 32) {
        unsigned seen = 0;
        unsigned it = 0;
        for (;; ++it) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
            if ((int)(seen - step) >= 0 || it >= kPeerSpinLimit) break;
            __nanosleep(100);
        }
        if ((int)(seen - step) < 0) ok = false;
    }
    return __all_sync(0xffffffffu, ok);
}

// The wait for the messages of the next step and the list of this rank's pairs in one launch (one warp).
__global__ void __launch_bounds__(32) peer_select_pairs_kernel(const unsigned int* flags, unsigned int* step_counter, int world, int* status,
                                                               const unsigned char* ids, int ids_stride, const unsigned char* w, int w_stride,
                                                               int top_k, int lo, int hi, unsigned short* pe, float* pw, unsigned short* pt,
                                                               int capacity, int* count_out) {
    // The expert kernels behind this launch may become resident now: what they do before their own dependency wait
    // (barriers, the shared expert of the rank's own token, whose vector an earlier launch wrote) needs no message.
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned step = *step_counter + 1u;
    if (!peer_wait_warp(flags, step, world) && threadIdx.x == 0) flag(status, kStatusTimeout);
    __syncwarp();
    if (threadIdx.x == 0) *step_counter = step;
    select_local_pairs_warp(ids, ids_stride, w, w_stride, world, top_k, lo, hi, pe, pw, pt, capacity, count_out);
}

// The wait for the partial rows of the CURRENT step (*step_counter: the message wait of the step advanced it) and
// their sum in row order in one launch: the first warp of every CTA polls the flags itself.
__global__ void __launch_bounds__(128) peer_sum_rows_kernel(const unsigned int* flags, const unsigned int* step_counter, int world, int* status,
                                                            const float* in, int rows, int cols, int row_stride, float* out) {
    if (threadIdx.x < 32) {
        if (!peer_wait_warp(flags, *step_counter, world) && threadIdx.x == 0) flag(status, kStatusTimeout);
    }
    __syncthreads();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c + 3 < cols) {
        float4 acc = __ldcg(reinterpret_cast<const float4*>(in + c));
        for (int r = 1; r < rows; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(in + (size_t)r * row_stride + c));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + c) = acc;
    } else {
        for (int k = c; k < cols; ++k) {
            float acc = __ldcg(in + k);
            for (int r = 1; r < rows; ++r) acc += __ldcg(in + (size_t)r * row_stride + k);
            out[k] = acc;
        }
    }
}

// One warp: waits until every flag has reached the step after *step_counter, then the counter advances
// (advance != 0).
__global__ void __launch_bounds__(32) peer_wait_kernel(const unsigned int* flags, unsigned int* step_counter, int world, int advance,
                                                       int* status) {
    const unsigned step = *step_counter + 1u;
    if (!peer_wait_warp(flags, step, world) && threadIdx.x == 0) flag(status, kStatusTimeout);
    __syncwarp();
    if (threadIdx.x == 0 && advance) *step_counter = step;
}

}  // namespace vib3

using namespace vib3;

// A device allocation that other processes on this node can map, zero-filled, with its inter-process handle.
extern "C" int vib3_peer_alloc(size_t bytes, void** ptr_out, unsigned char* handle_out) {
    if (!ptr_out || !handle_out || bytes == 0) return VIB3_ERR_NULL;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return (int)e;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    for (int i = 0; i < 64; ++i) handle_out[i] = reinterpret_cast<const unsigned char*>(&h)[i];
    *ptr_out = p;
    return VIB3_OK;
}

extern "C" int vib3_peer_open(const unsigned char* handle, void** ptr_out) {
    if (!handle || !ptr_out) return VIB3_ERR_NULL;
    cudaIpcMemHandle_t h;
    for (int i = 0; i < 64; ++i) reinterpret_cast<unsigned char*>(&h)[i] = handle[i];
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *ptr_out = p;
    return VIB3_OK;
}

extern "C" int vib3_peer_close(void* ptr) { return ptr ? (int)cudaIpcCloseMemHandle(ptr) : VIB3_OK; }
extern "C" int vib3_peer_free(void* ptr) { return ptr ? (int)cudaFree(ptr) : VIB3_OK; }

extern "C" int vib3_launch_peer_publish(const void* src, size_t src_stride_bytes, int bytes, void* const* dst_table,
                                        size_t dst_stride_bytes, unsigned int* const* flag_table, const unsigned int* step_counter,
                                        int step_offset, int rank, int world, void* stream) {
    if (!dst_table || !flag_table || !step_counter || (bytes > 0 && !src)) return VIB3_ERR_NULL;
    if (world <= 0 || rank < 0 || rank >= world || bytes < 0) return VIB3_ERR_COUNT;
    if (bytes > 0 && (((uintptr_t)src | src_stride_bytes | dst_stride_bytes) & 15)) return VIB3_ERR_ALIGN;
    peer_publish_kernel<<<world, 256, 0, (cudaStream_t)stream>>>((const unsigned char*)src, src_stride_bytes, bytes,
                                                                (unsigned char* const*)dst_table, dst_stride_bytes, flag_table,
                                                                step_counter, (unsigned)step_offset, rank, nullptr, nullptr, 0);
    return (int)cudaGetLastError();
}

// vib3_launch_peer_publish for rows of fp32 values with a second addend: destination d receives
// src[d] + (*add_count > add_threshold ? add_src[d] : 0), rows src_stride_bytes apart in both sources.
extern "C" int vib3_launch_peer_publish_rows(const float* src, const float* add_src, size_t src_stride_bytes, int bytes,
                                             const int* add_count, int add_threshold, void* const* dst_table,
                                             size_t dst_stride_bytes, unsigned int* const* flag_table,
                                             const unsigned int* step_counter, int step_offset, int rank, int world, void* stream) {
    if (!src || !add_src || !add_count || !dst_table || !flag_table || !step_counter) return VIB3_ERR_NULL;
    if (world <= 0 || rank < 0 || rank >= world || bytes <= 0) return VIB3_ERR_COUNT;
    if ((((uintptr_t)src | (uintptr_t)add_src | src_stride_bytes | dst_stride_bytes) & 15) || (bytes & 15)) return VIB3_ERR_ALIGN;
    peer_publish_kernel<<<world, 256, 0, (cudaStream_t)stream>>>((const unsigned char*)src, src_stride_bytes, bytes,
                                                                (unsigned char* const*)dst_table, dst_stride_bytes, flag_table,
                                                                step_counter, (unsigned)step_offset, rank,
                                                                (const unsigned char*)add_src, add_count, add_threshold);
    return (int)cudaGetLastError();
}

extern "C" int vib3_launch_peer_wait(const unsigned int* flags, unsigned int* step_counter, int world, int advance, int* status,
                                     void* stream) {
    if (!flags || !step_counter) return VIB3_ERR_NULL;
    if (world <= 0) return VIB3_ERR_COUNT;
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, step_counter, world, advance, status);
    return (int)cudaGetLastError();
}

// vib3_launch_peer_wait for the messages (the counter advances) followed by vib3_launch_select_local_pairs over the
// `world` received messages, as one launch.
extern "C" int vib3_launch_peer_select_pairs(const unsigned int* flags, unsigned int* step_counter, int world, int* status,
                                             const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                             int weights_stride_bytes, int top_k, int expert_lo, int expert_hi,
                                             unsigned short* pair_experts, float* pair_weights, unsigned short* pair_tokens,
                                             int capacity, int* count_out, void* stream) {
    if (!flags || !step_counter || !ids || !weights || !pair_experts || !pair_weights || !pair_tokens || !count_out) return VIB3_ERR_NULL;
    if (world <= 0 || world > 65535 || top_k <= 0 || top_k > kMaxSlots - 1 || capacity <= 0 || expert_lo < 0 || expert_hi < expert_lo)
        return VIB3_ERR_COUNT;
    if ((ids_stride_bytes & 1) || (weights_stride_bytes & 3)) return VIB3_ERR_ALIGN;
    peer_select_pairs_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, step_counter, world, status, (const unsigned char*)ids,
                                                                 ids_stride_bytes, (const unsigned char*)weights, weights_stride_bytes,
                                                                 top_k, expert_lo, expert_hi, pair_experts, pair_weights, pair_tokens,
                                                                 capacity, count_out);
    return (int)cudaGetLastError();
}

// The wait for the rows of the current step (flags must have reached *step_counter) followed by
// vib3_launch_sum_rows_f32, as one launch.
extern "C" int vib3_launch_peer_sum_rows(const unsigned int* flags, const unsigned int* step_counter, int world, int* status,
                                         const float* in, int rows, int cols, int row_stride, float* out, void* stream) {
    if (!flags || !step_counter || !in || !out) return VIB3_ERR_NULL;
    if (world <= 0 || rows <= 0 || cols <= 0 || row_stride < cols) return VIB3_ERR_SHAPE;
    if (((uintptr_t)in & 15) || ((uintptr_t)out & 15) || (row_stride & 3)) return VIB3_ERR_ALIGN;
    const int threads = 128, per_block = threads * 4;
    peer_sum_rows_kernel<<<(cols + per_block - 1) / per_block, threads, 0, (cudaStream_t)stream>>>(flags, step_counter, world, status, in,
                                                                                                 rows, cols, row_stride, out);
    return (int)cudaGetLastError();
}
