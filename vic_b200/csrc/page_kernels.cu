// Per-page entry points with the reference's own launcher signatures, so that the reference's
// Rust wrappers (src/compute/kernels.rs) can link against this library unchanged.
//
//   vib3_launch_partial_matmul_int4        cuda/src/kernels.cu:1043  (x fp16)
//   vib3_launch_partial_matmul_int4_f32    cuda/src/kernels.cu:1202  (x fp32)
//   vib3_launch_fused_swiglu_int4_f32      cuda/src/kernels.cu:1278
//   vib3_launch_silu_mul                   cuda/src/kernels.cu:1069
//   vib3_launch_weighted_accumulate[_f32[_f32]]  cuda/src/kernels.cu:1108, :1120, :2513
//   vib3_launch_residual_add_f32_f32       cuda/src/kernels.cu:1132
//
// Two code paths per GEMV: a fast one (K a multiple of 32, group size 32, 16-byte aligned code
// rows: one 16-byte load = one scale group) and a general one for any K / group size /
// alignment (the reference's tests use K = 2 and K = 4, tests/integration_test.rs:1709-1831).
#include "int4_math.cuh"
#include "launch_common.h"

#include <atomic>

namespace vib3 {
extern std::atomic<int> g_use_pdl;   // 1 = launches may be programmatic dependents (moe_layer.cu)

enum Epilogue : int { EPI_F16 = 0, EPI_SWIGLU_F16 = 1 };

struct PageGemvArgs {
    const void* x;
    int x_dtype;
    const unsigned char* codes[2];       // [0] the matrix (or gate), [1] up (fused SwiGLU only)
    const unsigned short* scales[2];
    __half* y;
    int K, M, group_size;
};

// Fast path: one warp per row (NR = 2: the gate row and the up row together).
template <class MATH, int NR, int B>
__global__ void __launch_bounds__(256) page_gemv_kernel(PageGemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    typename MATH::XS* xs = reinterpret_cast<typename MATH::XS*>(smem_raw);
    stage_x<MATH>(xs, a.x, a.x_dtype, a.K, threadIdx.x, blockDim.x);
    __syncthreads();
    const int nchunks = a.K / kGroupSize;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.M) return;
    const uint4* codes[NR];
    const unsigned short* sc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        codes[r] = reinterpret_cast<const uint4*>(a.codes[r] + (size_t)row * (a.K / 2));
        sc[r] = a.scales[r] + (size_t)row * nchunks;
    }
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    for (int c0 = lane; c0 < nchunks; c0 += 32 * B) {
        uint4 q[B][NR];
        unsigned short sb[B][NR];
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int c = c0 + 32 * i;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                if (c < nchunks) {
                    q[i][r] = ldg_stream16(codes[r] + c);
                    sb[i][r] = ldg_stream2(sc[r] + c);
                } else {
                    q[i][r] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
                    sb[i][r] = 0;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int c = min(c0 + 32 * i, nchunks - 1);
            float s[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) s[r] = scale_to_f32(sb[i][r]);
            MATH::template chunk<NR>(q[i], s, xs + (size_t)c * MATH::kStride, acc);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
        if (NR == 1) a.y[row] = __float2half_rn(acc[0]);
        else a.y[row] = __float2half_rn(silu_mul_f32(acc[0], acc[NR - 1]));  // one rounding, as kernels.cu:355-357
    }
}

// General path: any K, any group size, byte-granular loads; lane l takes bytes l, l+32, ...
template <int NR>
__global__ void __launch_bounds__(256) page_gemv_general_kernel(PageGemvArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.M) return;
    const int packed_k = (a.K + 1) / 2;
    const int groups = (a.K + a.group_size - 1) / a.group_size;
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    for (int b = lane; b < packed_k; b += 32) {
        const int col = 2 * b;
        const float x0 = load_x_as_f32(a.x, a.x_dtype, col);
        const float x1 = col + 1 < a.K ? load_x_as_f32(a.x, a.x_dtype, col + 1) : 0.f;
        const int g0 = col / a.group_size;
        const int g1 = min((col + 1) / a.group_size, groups - 1);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const unsigned char p = a.codes[r][(size_t)row * packed_k + b];
            // scales may sit at an odd address (K/2 * M odd): read them bytewise
            const unsigned char* sb = reinterpret_cast<const unsigned char*>(a.scales[r]);
            const size_t i0 = ((size_t)row * groups + g0) * 2, i1 = ((size_t)row * groups + g1) * 2;
            const float s0 = scale_to_f32((unsigned short)(sb[i0] | (sb[i0 + 1] << 8)));
            const float s1 = scale_to_f32((unsigned short)(sb[i1] | (sb[i1 + 1] << 8)));
            acc[r] = fmaf(x0, (float)((int)(p & 0xF) - 8) * s0, acc[r]);
            acc[r] = fmaf(x1, (float)((int)(p >> 4) - 8) * s1, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
        if (NR == 1) a.y[row] = __float2half_rn(acc[0]);
        else a.y[row] = __float2half_rn(silu_mul_f32(acc[0], acc[NR - 1]));
    }
}

template <class MATH, int NR, int B>
static int launch_fast(const PageGemvArgs& a, cudaStream_t st) {
    const size_t smem = (size_t)(a.K / kGroupSize) * MATH::kStride * sizeof(typename MATH::XS);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(page_gemv_kernel<MATH, NR, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    page_gemv_kernel<MATH, NR, B><<<(a.M + 7) / 8, 256, smem, st>>>(a);
    return (int)cudaGetLastError();
}

template <class MATH, int NR>
static int launch_page_gemv(const PageGemvArgs& a, cudaStream_t st) {
    bool fast = a.group_size == kGroupSize && a.K % kGroupSize == 0 && a.K <= 65536 && (((uintptr_t)a.x) & 15) == 0;
    for (int r = 0; r < NR; ++r) fast = fast && (((uintptr_t)a.codes[r]) & 15) == 0 && (((uintptr_t)a.scales[r]) & 1) == 0;
    if (!fast) {
        page_gemv_general_kernel<NR><<<(a.M + 7) / 8, 256, 0, st>>>(a);
        return (int)cudaGetLastError();
    }
    const int per_lane = (a.K / kGroupSize + 31) / 32;
    if (per_lane % 7 == 0) return launch_fast<MATH, NR, 7>(a, st);
    if (per_lane % 4 == 0) return launch_fast<MATH, NR, 4>(a, st);
    if (per_lane % 2 == 0) return launch_fast<MATH, NR, 2>(a, st);
    return launch_fast<MATH, NR, 1>(a, st);
}

static int check_gemv(const void* x, const void* w, const void* s, const void* y, int K, int M, int group_size) {
    if (!x || !w || !s || !y) return VIB3_ERR_NULL;
    if (K <= 0 || M < 0 || group_size <= 0) return VIB3_ERR_SHAPE;
    if ((uintptr_t)y & 1) return VIB3_ERR_ALIGN;
    return VIB3_OK;
}

__global__ void silu_mul_kernel(const __half* a, const __half* b, __half* y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(silu_mul_f32(__half2float(a[i]), __half2float(b[i])));
}
__global__ void wacc_f16_kernel(__half* out, const __half* y, float w, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(fmaf(w, __half2float(y[i]), __half2float(out[i])));
}
__global__ void wacc_f32_kernel(float* out, const __half* y, float w, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fmaf(w, __half2float(y[i]), out[i]);
}
__global__ void wacc_f32_f32_kernel(float* out, const float* y, float w, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fmaf(w, y[i], out[i]);
}
__global__ void residual_add_kernel(float* acc, const float* y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] += y[i];
}

}  // namespace vib3

using namespace vib3;

extern "C" int vib3_launch_partial_matmul_int4(const void* x_f16, const void* w_packed, const void* scales,
                                               void* y_f16, int K, int M_slice, int group_size, void* stream) {
    if (int e = check_gemv(x_f16, w_packed, scales, y_f16, K, M_slice, group_size)) return e;
    if (M_slice == 0) return VIB3_OK;
    if ((uintptr_t)x_f16 & 1) return VIB3_ERR_ALIGN;
    PageGemvArgs a{x_f16, X_F16, {(const unsigned char*)w_packed, nullptr}, {(const unsigned short*)scales, nullptr},
                   (__half*)y_f16, K, M_slice, group_size};
    return launch_page_gemv<MathF16, 1>(a, (cudaStream_t)stream);
}

extern "C" int vib3_launch_partial_matmul_int4_f32(const void* x_f32, const void* w_packed, const void* scales,
                                                   void* y_f16, int K, int M_slice, int group_size, void* stream) {
    if (int e = check_gemv(x_f32, w_packed, scales, y_f16, K, M_slice, group_size)) return e;
    if (M_slice == 0) return VIB3_OK;
    if ((uintptr_t)x_f32 & 3) return VIB3_ERR_ALIGN;
    PageGemvArgs a{x_f32, X_F32, {(const unsigned char*)w_packed, nullptr}, {(const unsigned short*)scales, nullptr},
                   (__half*)y_f16, K, M_slice, group_size};
    return launch_page_gemv<MathF32, 1>(a, (cudaStream_t)stream);
}

extern "C" int vib3_launch_fused_swiglu_int4_f32(const void* x_f32, const void* up_w, const void* up_s,
                                                 const void* gate_w, const void* gate_s, void* y_f16, int K,
                                                 int M_slice, int group_size, void* stream) {
    if (int e = check_gemv(x_f32, up_w, up_s, y_f16, K, M_slice, group_size)) return e;
    if (int e = check_gemv(x_f32, gate_w, gate_s, y_f16, K, M_slice, group_size)) return e;
    if (M_slice == 0) return VIB3_OK;
    if ((uintptr_t)x_f32 & 3) return VIB3_ERR_ALIGN;
    PageGemvArgs a{x_f32, X_F32, {(const unsigned char*)gate_w, (const unsigned char*)up_w},
                   {(const unsigned short*)gate_s, (const unsigned short*)up_s}, (__half*)y_f16, K, M_slice, group_size};
    return launch_page_gemv<MathF32, 2>(a, (cudaStream_t)stream);
}

static int check_vec(const void* a, const void* b, int dim) {
    if (!a || !b) return VIB3_ERR_NULL;
    if (dim < 0) return VIB3_ERR_SHAPE;
    return VIB3_OK;
}

// The first operand receives the SiLU (the reference's C parameter names say otherwise, its
// kernel and its Rust caller agree on this order: kernels.cu:772-785, kernels.rs:529-537).
extern "C" int vib3_launch_silu_mul(const void* silu_operand_f16, const void* mul_operand_f16, void* y_f16, int dim,
                                    void* stream) {
    if (int e = check_vec(silu_operand_f16, mul_operand_f16, dim)) return e;
    if (!y_f16) return VIB3_ERR_NULL;
    if (dim == 0) return VIB3_OK;
    silu_mul_kernel<<<(dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const __half*)silu_operand_f16,
                                                                        (const __half*)mul_operand_f16, (__half*)y_f16, dim);
    return (int)cudaGetLastError();
}

extern "C" int vib3_launch_weighted_accumulate(void* out_f16, const void* y_f16, float w, int dim, void* stream) {
    if (int e = check_vec(out_f16, y_f16, dim)) return e;
    if (dim == 0) return VIB3_OK;
    wacc_f16_kernel<<<(dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>((__half*)out_f16, (const __half*)y_f16, w, dim);
    return (int)cudaGetLastError();
}

extern "C" int vib3_launch_weighted_accumulate_f32(void* out_f32, const void* y_f16, float w, int dim, void* stream) {
    if (int e = check_vec(out_f32, y_f16, dim)) return e;
    if (dim == 0) return VIB3_OK;
    wacc_f32_kernel<<<(dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>((float*)out_f32, (const __half*)y_f16, w, dim);
    return (int)cudaGetLastError();
}

extern "C" int vib3_launch_weighted_accumulate_f32_f32(void* out_f32, const void* y_f32, float w, int dim, void* stream) {
    if (int e = check_vec(out_f32, y_f32, dim)) return e;
    if (dim == 0) return VIB3_OK;
    wacc_f32_f32_kernel<<<(dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>((float*)out_f32, (const float*)y_f32, w, dim);
    return (int)cudaGetLastError();
}

extern "C" int vib3_launch_residual_add_f32_f32(void* acc_f32, const void* layer_out_f32, int dim, void* stream) {
    if (int e = check_vec(acc_f32, layer_out_f32, dim)) return e;
    if (dim == 0) return VIB3_OK;
    residual_add_kernel<<<(dim + 255) / 256, 256, 0, (cudaStream_t)stream>>>((float*)acc_f32, (const float*)layer_out_f32, dim);
    return (int)cudaGetLastError();
}

// ── RMS norm in front of the MoE sublayer ──────────────────────────────────────────────────
// Sum of squares: 256 partial sums (fused multiply-add), then a halving tree in shared memory, as the reference
// kernel (cuda/src/kernels.cu:921-953); square root and reciprocal are IEEE (the reference's CPU path,
// src/compute/kernels.rs:2591-2603; its CUDA build uses the fast-math approximations).
// Sum over the CTA (a whole number of warps, at most 32): butterfly inside each warp, then the warps' sums in
// warp order by every thread — the same value, bit for bit, in all threads.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int tid = threadIdx.x, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // (red may still be read from an earlier call)
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += red[w];
    return s;
}
__device__ __forceinline__ float block_inv_rms(float ss, int H, float eps, float* red) {
    const float rms = sqrtf(block_sum(ss, red) / (float)H + eps);
    return 1.0f / rms;
}

__device__ __forceinline__ void store_x(void* out, int dtype, int d, float v) {
    if (dtype == X_F32) reinterpret_cast<float*>(out)[d] = v;
    else if (dtype == X_F16) reinterpret_cast<__half*>(out)[d] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(out)[d] = __float2bfloat16_rn(v);
}

// One CTA per token: hidden += delta (optional), x = cast(hidden * inv_rms * weight).
// VEC (1024 threads): H a multiple of 4 and at most 8192, 16-byte aligned rows: a thread keeps its (at most two)
// 4-column items in registers — every load is requested before anything is stored, one pass over the row.  Two items
// per thread rather than eight in a quarter of the threads: the kernel runs once per layer on cold instruction caches,
// and its time is the code it has to fetch.  Otherwise 256 threads and three passes.
template <bool VEC>
__global__ void __launch_bounds__(VEC ? 1024 : 256) residual_rms_norm_kernel(float* __restrict__ hidden, int hidden_stride, const void* __restrict__ delta,
                                                                int delta_dtype, int delta_stride, const float* __restrict__ delta2,
                                                                int delta2_stride, const __half* __restrict__ weight, float eps,
                                                                int flags, void* __restrict__ x_out, int x_dtype, int x_stride, int H) {
    __shared__ float red[256];
    const int t = blockIdx.x, tid = threadIdx.x;
    // flags bit 1: the kernels behind this one may start now (they must wait for it before they read x_out or hidden)
    if ((flags & 2) && tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int center = flags & 1;
    float* row = hidden + (size_t)t * hidden_stride;
    const unsigned char* drow = delta ? reinterpret_cast<const unsigned char*>(delta) + (size_t)t * delta_stride : nullptr;
    const float* d2row = delta2 ? delta2 + (size_t)t * delta2_stride : nullptr;
    unsigned char* xrow = reinterpret_cast<unsigned char*>(x_out) + (size_t)t * x_stride;
    if (VEC) {
        constexpr int kItems = 2, kThreads = 1024;
        const int n4 = H >> 2;
        float4 h[kItems], dl[kItems];
        uint2 wv[kItems];
        // The norm weights are nobody's output: they are requested before the wait for the predecessor (the kernel
        // may be launched as a programmatic dependent, e.g. of the previous sublayer's last kernel).
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            const int it = tid + kThreads * i;
            wv[i] = make_uint2(0x3C003C00u, 0x3C003C00u);   // 1.0
            if (it < n4 && weight) wv[i] = reinterpret_cast<const uint2*>(weight)[it];
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            const int it = tid + kThreads * i;
            h[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            dl[i] = h[i];
            if (it < n4) {
                h[i] = reinterpret_cast<const float4*>(row)[it];
                if (drow) {
                    if (delta_dtype == X_F32) dl[i] = reinterpret_cast<const float4*>(drow)[it];
                    else {
                        const uint2 r2 = reinterpret_cast<const uint2*>(drow)[it];
                        if (delta_dtype == X_F16) {
                            const __half2 p0 = *reinterpret_cast<const __half2*>(&r2.x), p1 = *reinterpret_cast<const __half2*>(&r2.y);
                            dl[i] = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
                        } else {
                            dl[i] = make_float4(__uint_as_float(r2.x << 16), __uint_as_float(r2.x & 0xFFFF0000u), __uint_as_float(r2.y << 16),
                                                __uint_as_float(r2.y & 0xFFFF0000u));
                        }
                    }
                }
                if (d2row) {
                    const float4 e = reinterpret_cast<const float4*>(d2row)[it];
                    dl[i].x += e.x; dl[i].y += e.y; dl[i].z += e.z; dl[i].w += e.w;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            h[i].x += dl[i].x; h[i].y += dl[i].y; h[i].z += dl[i].z; h[i].w += dl[i].w;
        }
        float mean = 0.f;
        if (center) {
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < kItems; ++i) sum += (h[i].x + h[i].y) + (h[i].z + h[i].w);
            mean = block_sum(sum, red) / (float)H;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            if (tid + kThreads * i < n4) {
                ss = fmaf(h[i].x - mean, h[i].x - mean, ss);
                ss = fmaf(h[i].y - mean, h[i].y - mean, ss);
                ss = fmaf(h[i].z - mean, h[i].z - mean, ss);
                ss = fmaf(h[i].w - mean, h[i].w - mean, ss);
            }
        }
        const float inv_rms = block_inv_rms(ss, H, eps, red);
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            const int it = tid + kThreads * i;
            if (it < n4) {
                if (drow || d2row) reinterpret_cast<float4*>(row)[it] = h[i];
                const __half2 w0 = *reinterpret_cast<const __half2*>(&wv[i].x), w1 = *reinterpret_cast<const __half2*>(&wv[i].y);
                float v[4] = {(h[i].x - mean) * inv_rms, (h[i].y - mean) * inv_rms, (h[i].z - mean) * inv_rms, (h[i].w - mean) * inv_rms};
                if (weight) {
                    v[0] *= __low2float(w0); v[1] *= __high2float(w0); v[2] *= __low2float(w1); v[3] *= __high2float(w1);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) store_x(xrow, x_dtype, 4 * it + c, v[c]);
            }
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (drow || d2row)
            for (int d = tid; d < H; d += 256)   // (a thread re-reads only its own columns)
                row[d] += (drow ? load_x_as_f32(drow, delta_dtype, d) : 0.f) + (d2row ? d2row[d] : 0.f);
        float mean = 0.f;
        if (center) {
            float sum = 0.f;
            for (int d = tid; d < H; d += 256) sum += row[d];
            mean = block_sum(sum, red) / (float)H;
        }
        float ss = 0.f;
        for (int d = tid; d < H; d += 256) ss = fmaf(row[d] - mean, row[d] - mean, ss);
        const float inv_rms = block_inv_rms(ss, H, eps, red);
        for (int d = tid; d < H; d += 256) {
            float v = (row[d] - mean) * inv_rms;
            if (weight) v *= __half2float(weight[d]);
            store_x(xrow, x_dtype, d, v);
        }
    }
}

static int launch_norm(float* hidden, int hidden_stride, const void* delta, int delta_dtype, int delta_stride, const float* delta2,
                       int delta2_stride, const void* weight, float eps, int center, void* x_out, int x_dtype, int x_stride, int H,
                       int n_tokens, cudaStream_t st) {
    const bool vec = H % 4 == 0 && H <= 8192 && ((uintptr_t)hidden & 15) == 0 && (hidden_stride & 3) == 0 && ((uintptr_t)delta & 15) == 0 &&
                     (delta_stride & 15) == 0 && ((uintptr_t)delta2 & 15) == 0 && (delta2_stride & 3) == 0 && ((uintptr_t)weight & 7) == 0 &&
                     ((uintptr_t)x_out & 15) == 0 && (x_stride & 15) == 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tokens); cfg.blockDim = dim3(vec ? 1024 : 256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_use_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const __half* w16 = (const __half*)weight;
    if (vec)
        return (int)cudaLaunchKernelEx(&cfg, residual_rms_norm_kernel<true>, hidden, hidden_stride, delta, delta_dtype, delta_stride, delta2,
                                       delta2_stride, w16, eps, center, x_out, x_dtype, x_stride, H);
    return (int)cudaLaunchKernelEx(&cfg, residual_rms_norm_kernel<false>, hidden, hidden_stride, delta, delta_dtype, delta_stride, delta2,
                                   delta2_stride, w16, eps, center, x_out, x_dtype, x_stride, H);
}

// Reference signature (cuda/src/kernels.cu:1178): fp32 in, fp32 out, fp16 weight, one vector.
extern "C" int vib3_launch_rms_norm_f32(const void* input, void* output, const void* weight, int hidden_dim, float eps,
                                        void* stream) {
    if (!input || !output || !weight) return VIB3_ERR_NULL;
    if (hidden_dim <= 0) return VIB3_ERR_SHAPE;
    if (input != output)
        if (cudaMemcpyAsync(output, input, (size_t)hidden_dim * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) != cudaSuccess)
            return (int)cudaGetLastError();
    // normalise in place on the copy: the kernel reads and writes the same row
    return launch_norm((float*)output, hidden_dim, nullptr, 0, 0, nullptr, 0, weight, eps, 0, output, X_F32, 0, hidden_dim, 1,
                       (cudaStream_t)stream);
}

// The two steps either side of the MoE sublayer in the reference's layer loop (residual_add_f32_f32, then
// rms_norm_f32 of the next sublayer: src/runtime/engine.rs:5302, :5072) as ONE launch for n_tokens rows:
//   hidden[t] += delta[t] + delta2[t]   (delta: the other sublayer's output, fp32 / fp16 / bf16, or NULL; delta2: fp32 or
//                                        NULL, e.g. the sum over expert-parallel ranks of the previous MoE sublayer's outputs)
//   x_out[t]   = cast(hidden[t] * inv_rms(hidden[t]) * weight)      (weight fp16 or NULL; x_out fp32 / fp16 / bf16)
// center != 0 (not in the reference): the row's mean is removed first, x = (hidden - mean) * inv_rms(hidden - mean) * weight.
// For stacks of SYNTHETIC layers: INT4 codes drawn uniformly from [-8, 7] have mean -0.5, so every output row of such a
// matrix carries a common term proportional to the sum of its input; through a residual stream that term feeds itself and
// after a few layers every token routes alike.  Trained weights have no such mean.
// The MoE sublayer that follows adds its own output to hidden (out_accumulate = 1), so a layer costs this
// launch plus the MoE launches.
extern "C" int vib3_launch_residual_rms_norm(float* hidden, int hidden_stride, const void* delta, int delta_dtype,
                                             int delta_stride_bytes, const float* delta2, int delta2_stride,
                                             const void* weight_f16, float eps, int center, void* x_out, int x_dtype,
                                             int x_stride_bytes, int hidden_dim, int n_tokens, void* stream) {
    if (!hidden || !x_out) return VIB3_ERR_NULL;
    if (hidden_dim <= 0 || n_tokens <= 0 || hidden_stride < hidden_dim) return VIB3_ERR_SHAPE;
    if (x_dtype < X_F32 || x_dtype > X_BF16 || (delta && (delta_dtype < X_F32 || delta_dtype > X_BF16))) return VIB3_ERR_UNSUPPORTED;
    if ((void*)hidden == x_out) return VIB3_ERR_UNSUPPORTED;
    if (delta2 && delta2_stride < hidden_dim) return VIB3_ERR_SHAPE;
    return launch_norm(hidden, hidden_stride, delta, delta_dtype, delta_stride_bytes, delta2, delta2_stride, weight_f16, eps, center, x_out,
                       x_dtype, x_stride_bytes, hidden_dim, n_tokens, (cudaStream_t)stream);
}
