// INT4 group-32 dequantisation and dot-product building blocks shared by every kernel of the
// MoE decode path.
//
// Weight format (reference: cuda/src/kernels.cu:126-145, src/compute/kernels.rs:94-98):
// a page holds `rows` rows of K/2 code bytes followed by `rows` rows of K/32 fp16 scales.
// A code byte carries two columns, low nibble = even column; the weight is (nibble - 8) * scale.
// One 16-byte load is therefore exactly one scale group: 32 codes, columns 32c .. 32c+31,
// word j of the load = columns 32c+8j .. 32c+8j+7, nibble p of a word = column 8j+p.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace vib3 {

constexpr int kGroupSize = 32;
constexpr int kWarp = 32;
// Activation vectors are staged in shared memory chunk by chunk (32 values) with padding so
// that 32 lanes reading 32 different chunks with 16-byte loads hit every bank group once:
// 80-byte stride for halves (5 x 16 B, 5 is odd), 144-byte stride for floats (9 x 16 B).
constexpr int kXStrideH = 40;  // halves per staged chunk
constexpr int kXStrideF = 36;  // floats per staged chunk

enum XDType : int { X_F32 = 0, X_F16 = 1, X_BF16 = 2 };

// Device page-table entry: where a page lives and which rows of its matrix it holds.
// Mirrors ResolvedPage{device_ptr,row_start,row_count} (src/runtime/query_planner.rs:36-42).
struct PageEntry {
    unsigned long long ptr;
    unsigned short row_start;
    unsigned short row_count;
    unsigned int reserved;
};
static_assert(sizeof(PageEntry) == 16, "PageEntry is 16 bytes");

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}

// Streaming 16-byte load: weights are read exactly once per token, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned short ldg_stream2(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// fp16 x fp16 -> exact product, added to an fp32 accumulator with one rounding (sm_100 mixed
// precision FMA).  The four variants pick the low or high half of each 32-bit operand.
#define VIB3_FMA_MIX(NAME, AH, BH)                                                       \
    __device__ __forceinline__ float NAME(uint32_t a, uint32_t b, float c) {             \
        asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"                                         \
            "mov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"                         \
            "fma.rn.f32.f16 %0, " AH ", " BH ", %0;\n\t}"                                \
            : "+f"(c)                                                                    \
            : "r"(a), "r"(b));                                                           \
        return c;                                                                        \
    }
VIB3_FMA_MIX(fma_mix_ll, "al", "bl")
VIB3_FMA_MIX(fma_mix_lh, "al", "bh")
VIB3_FMA_MIX(fma_mix_hl, "ah", "bl")
VIB3_FMA_MIX(fma_mix_hh, "ah", "bh")
#undef VIB3_FMA_MIX

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// ── Math policy F16: activations held as fp16 (exact for fp16 input, exact for bf16 input
// inside fp16's normal range), codes turned into exact fp16 integers with the 0x6400 trick:
// (w & 0x000F000F) | 0x64006400 is the half2 (1024 + n0, 1024 + n4); subtracting 1032 gives
// n - 8 exactly.  (w & 0x00F000F0) | 0x64006400 is (1024 + 16 n1, 1024 + 16 n5); times 1/16
// minus 72 gives n - 8 exactly.  Products with the activation are exact inside the mixed
// FMA, so the only roundings are the fp32 accumulations.
struct MathF16 {
    using XS = __half;
    static constexpr int kStride = kXStrideH;

    // acc[r] += scale[r] * sum_{i<32} (n_i - 8) * x_i for NR rows sharing the same x chunk.
    template <int NR>
    static __device__ __forceinline__ void chunk(const uint4 (&q)[NR], const float (&s)[NR],
                                                 const XS* xchunk, float (&acc)[NR]) {
        const uint4* xp = reinterpret_cast<const uint4*>(xchunk);
        float p0[NR], p1[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { p0[r] = 0.f; p1[r] = 0.f; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 xv = xp[j];  // halves (0,1) (2,3) (4,5) (6,7) of word j's columns
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = j == 0 ? q[r].x : j == 1 ? q[r].y : j == 2 ? q[r].z : q[r].w;
                const uint32_t w8 = w >> 8;
                const uint32_t d04 = h2_sub(lop3_and_or(w, 0x000F000Fu, 0x64006400u), 0x64086408u);
                const uint32_t d15 = h2_fma(lop3_and_or(w, 0x00F000F0u, 0x64006400u), 0x2C002C00u, 0xD480D480u);
                const uint32_t d26 = h2_sub(lop3_and_or(w8, 0x000F000Fu, 0x64006400u), 0x64086408u);
                const uint32_t d37 = h2_fma(lop3_and_or(w8, 0x00F000F0u, 0x64006400u), 0x2C002C00u, 0xD480D480u);
                p0[r] = fma_mix_ll(d04, xv.x, p0[r]);  // col 0
                p1[r] = fma_mix_lh(d15, xv.x, p1[r]);  // col 1
                p0[r] = fma_mix_ll(d26, xv.y, p0[r]);  // col 2
                p1[r] = fma_mix_lh(d37, xv.y, p1[r]);  // col 3
                p0[r] = fma_mix_hl(d04, xv.z, p0[r]);  // col 4
                p1[r] = fma_mix_hh(d15, xv.z, p1[r]);  // col 5
                p0[r] = fma_mix_hl(d26, xv.w, p0[r]);  // col 6
                p1[r] = fma_mix_hh(d37, xv.w, p1[r]);  // col 7
            }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = fmaf(s[r], p0[r] + p1[r], acc[r]);
    }

    static __device__ __forceinline__ XS from_f32(float v) {
        return __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
    }
};

// ── Math policy F32: activations held as fp32; codes turned into fp32 with the 2^23 trick
// (0x4B000000 | n is the float 8388608 + n).
struct MathF32 {
    using XS = float;
    static constexpr int kStride = kXStrideF;

    template <int NR>
    static __device__ __forceinline__ void chunk(const uint4 (&q)[NR], const float (&s)[NR],
                                                 const XS* xchunk, float (&acc)[NR]) {
        const float4* xp = reinterpret_cast<const float4*>(xchunk);
        float p0[NR], p1[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { p0[r] = 0.f; p1[r] = 0.f; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 xa = xp[2 * j], xb = xp[2 * j + 1];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = j == 0 ? q[r].x : j == 1 ? q[r].y : j == 2 ? q[r].z : q[r].w;
                const float k = 8388616.f;  // 2^23 + 8
                const float w0 = __uint_as_float(lop3_and_or(w, 0xFu, 0x4B000000u)) - k;
                const float w1 = __uint_as_float(lop3_and_or(w >> 4, 0xFu, 0x4B000000u)) - k;
                const float w2 = __uint_as_float(lop3_and_or(w >> 8, 0xFu, 0x4B000000u)) - k;
                const float w3 = __uint_as_float(lop3_and_or(w >> 12, 0xFu, 0x4B000000u)) - k;
                const float w4 = __uint_as_float(lop3_and_or(w >> 16, 0xFu, 0x4B000000u)) - k;
                const float w5 = __uint_as_float(lop3_and_or(w >> 20, 0xFu, 0x4B000000u)) - k;
                const float w6 = __uint_as_float(lop3_and_or(w >> 24, 0xFu, 0x4B000000u)) - k;
                const float w7 = __uint_as_float(lop3_and_or(w >> 28, 0xFu, 0x4B000000u)) - k;
                p0[r] = fmaf(w0, xa.x, p0[r]);
                p1[r] = fmaf(w1, xa.y, p1[r]);
                p0[r] = fmaf(w2, xa.z, p0[r]);
                p1[r] = fmaf(w3, xa.w, p1[r]);
                p0[r] = fmaf(w4, xb.x, p0[r]);
                p1[r] = fmaf(w5, xb.y, p1[r]);
                p0[r] = fmaf(w6, xb.z, p0[r]);
                p1[r] = fmaf(w7, xb.w, p1[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = fmaf(s[r], p0[r] + p1[r], acc[r]);
    }

    static __device__ __forceinline__ XS from_f32(float v) { return v; }
};

__device__ __forceinline__ float load_x_as_f32(const void* x, int dtype, int i) {
    if (dtype == X_F32) return reinterpret_cast<const float*>(x)[i];
    if (dtype == X_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
}

// Copy an activation vector of n values (n a multiple of 32) into padded chunk layout.
template <class MATH>
__device__ __forceinline__ void stage_x(typename MATH::XS* dst, const void* x, int dtype, int n, int tid,
                                        int nthreads) {
    for (int i = tid; i < n; i += nthreads) {
        dst[(i >> 5) * MATH::kStride + (i & 31)] = MATH::from_f32(load_x_as_f32(x, dtype, i));
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float scale_to_f32(unsigned short bits) {
    return __half2float(__ushort_as_half(bits));
}

// silu(g) * u with the reference's formula g / (1 + exp(-g)) (cuda/src/kernels.cu:783).
__device__ __forceinline__ float silu_mul_f32(float g, float u) {
    return (g / (1.0f + expf(-g))) * u;
}

}  // namespace vib3
