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

namespace vib3 {

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
