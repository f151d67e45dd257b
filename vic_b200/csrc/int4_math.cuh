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
// inside fp16's normal range).  Codes become fp16 numbers with one logic op per two weights:
// (w & 0x000F000F) | 0x64006400 is the half2 (1024 + n_a, 1024 + n_b) for two even columns,
// (w & 0x00F000F0) | 0x64006400 is (1024 + 16 n_a, 1024 + 16 n_b) for two odd columns.
// The offsets are not subtracted per weight.  The mixed-precision FMA forms the exact product
// x * (1024 + n) and accumulates it in fp32; per 32-column chunk the staged activation carries
// Se = sum of its even-column values and So = sum of its odd-column values, and
//     sum_i (n_i - 8) x_i = (P_even - 1032 Se) + (P_odd - 1152 So) / 16
// is formed with two fused multiply-adds (the cancellation is exact inside the FMA).  The only
// roundings are the 16 fp32 accumulations of P_even and of P_odd at magnitude ~1e3, a relative
// error of a few 1e-5 of the chunk sum.
struct MathF16 {
    using XS = __half;
    static constexpr int kStride = kXStrideH;

    // acc[r] += scale[r] * sum_{i<32} (n_i - 8) * x_i for NR rows sharing the same x chunk.
    template <int NR>
    static __device__ __forceinline__ void chunk(const uint4 (&q)[NR], const float (&s)[NR],
                                                 const XS* xchunk, float (&acc)[NR]) {
        const uint4* xp = reinterpret_cast<const uint4*>(xchunk);
        float pe[NR], po[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { pe[r] = 0.f; po[r] = 0.f; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 xv = xp[j];  // halves (0,1) (2,3) (4,5) (6,7) of word j's columns
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = j == 0 ? q[r].x : j == 1 ? q[r].y : j == 2 ? q[r].z : q[r].w;
                const uint32_t w8 = w >> 8;
                const uint32_t d04 = lop3_and_or(w, 0x000F000Fu, 0x64006400u);   // cols 0,4: 1024 + n
                const uint32_t d15 = lop3_and_or(w, 0x00F000F0u, 0x64006400u);   // cols 1,5: 1024 + 16 n
                const uint32_t d26 = lop3_and_or(w8, 0x000F000Fu, 0x64006400u);  // cols 2,6
                const uint32_t d37 = lop3_and_or(w8, 0x00F000F0u, 0x64006400u);  // cols 3,7
                pe[r] = fma_mix_ll(d04, xv.x, pe[r]);  // col 0
                po[r] = fma_mix_lh(d15, xv.x, po[r]);  // col 1
                pe[r] = fma_mix_ll(d26, xv.y, pe[r]);  // col 2
                po[r] = fma_mix_lh(d37, xv.y, po[r]);  // col 3
                pe[r] = fma_mix_hl(d04, xv.z, pe[r]);  // col 4
                po[r] = fma_mix_hh(d15, xv.z, po[r]);  // col 5
                pe[r] = fma_mix_hl(d26, xv.w, pe[r]);  // col 6
                po[r] = fma_mix_hh(d37, xv.w, po[r]);  // col 7
            }
        }
        const float2 sums = *reinterpret_cast<const float2*>(xchunk + 32);  // (Se, So) in the chunk's padding
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const float te = fmaf(-1032.f, sums.x, pe[r]);
            const float to = fmaf(-1152.f, sums.y, po[r]);
            acc[r] = fmaf(s[r], fmaf(to, 0.0625f, te), acc[r]);
        }
    }

    static __device__ __forceinline__ XS from_f32(float v) {
        return __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
    }
    static __device__ __forceinline__ float to_f32(XS v) { return __half2float(v); }
    static constexpr bool kChunkSums = true;
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
    static __device__ __forceinline__ float to_f32(XS v) { return v; }
    static constexpr bool kChunkSums = false;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ unsigned short lds16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// ── Math policy Q16 (integer dot products).  The activation chunk (32 values) is held as 16-bit
// fixed point relative to the chunk's largest magnitude, x_i = sx * q_i with |q_i| <= 32512 and
// q_i = 256 * hi_i + lo_i (hi signed, lo in 0..255).  One dp4a multiplies four 4-bit codes
// (isolated with one AND as bytes) by four hi or four lo bytes and accumulates in int32, exactly.
// Per chunk and row:  sum_i (n_i - 8) x_i = sx * (256 * D_hi + D_lo - 8 * sum_i q_i),  converted to
// fp32 once per 32 weights and scaled by sx * (fp16 group scale).  Everything up to that
// conversion is exact integer arithmetic; the only approximation is the 16-bit rounding of the
// activations, at most 2^-16 of the chunk maximum per value (fp16 keeps 2^-11, bf16 2^-8).
// All work sits on the integer pipe at about one instruction per weight.
//
// Shared-memory layout of a staged chunk (80 bytes): for word j = 0..3 of the code load (columns
// 8j..8j+7) one uint4 {hi of even columns, hi of odd columns, lo of even columns, lo of odd
// columns}, then the float sx and the int 8 * sum q.
// Byte B (0: low, 1: second) of each of four integers as the four bytes of a word, a in the lowest: three byte permutes
// (the shift-mask-or form is eleven instructions, and the quantisation code runs once, cold, at the start of a kernel).
template <int B>
__device__ __forceinline__ uint32_t pack_bytes(int a, int b, int c, int d) {
    const uint32_t lo = __byte_perm((uint32_t)a, (uint32_t)b, B == 0 ? 0x0040u : 0x0051u);
    const uint32_t hi = __byte_perm((uint32_t)c, (uint32_t)d, B == 0 ? 0x0040u : 0x0051u);
    return __byte_perm(lo, hi, 0x5410u);
}

struct MathQ16 {
    using XS = unsigned char;
    static constexpr int kStride = 80;  // bytes per staged chunk

    static __device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
        int d;
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
        return d;
    }
    static __device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
        int d;
        asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
        return d;
    }

    template <int NR>
    static __device__ __forceinline__ void chunk(const uint4 (&q)[NR], const float (&s)[NR],
                                                 const XS* xchunk, float (&acc)[NR]) {
        const uint4* xp = reinterpret_cast<const uint4*>(xchunk);
        int dh[NR], dl[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { dh[r] = 0; dl[r] = 0; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 xv = xp[j];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = j == 0 ? q[r].x : j == 1 ? q[r].y : j == 2 ? q[r].z : q[r].w;
                const uint32_t we = w & 0x0F0F0F0Fu;         // codes of columns 0,2,4,6
                const uint32_t wo = (w >> 4) & 0x0F0F0F0Fu;  // codes of columns 1,3,5,7
                dh[r] = dp4a_us(we, xv.x, dh[r]);
                dl[r] = dp4a_uu(we, xv.z, dl[r]);
                dh[r] = dp4a_us(wo, xv.y, dh[r]);
                dl[r] = dp4a_uu(wo, xv.w, dl[r]);
            }
        }
        const float sx = *reinterpret_cast<const float*>(xchunk + 64);
        const int sq8 = *reinterpret_cast<const int*>(xchunk + 68);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int t = dh[r] * 256 + dl[r] - sq8;
            acc[r] = fmaf((float)t, s[r] * sx, acc[r]);
        }
    }

    // Same arithmetic with the quantised activation chunk held in registers (xv[j] = the uint4 of
    // word j, sx, sq8 as in the staged layout).
    static __device__ __forceinline__ float chunk_r(const uint4& q, float s, const uint4 (&xv)[4], float sx, int sq8,
                                                    float acc) {
        int dh = 0, dl = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t w = j == 0 ? q.x : j == 1 ? q.y : j == 2 ? q.z : q.w;
            const uint32_t we = w & 0x0F0F0F0Fu;
            const uint32_t wo = (w >> 4) & 0x0F0F0F0Fu;
            dh = dp4a_us(we, xv[j].x, dh);
            dl = dp4a_uu(we, xv[j].z, dl);
            dh = dp4a_us(wo, xv[j].y, dh);
            dl = dp4a_uu(wo, xv[j].w, dl);
        }
        const int t = dh * 256 + dl - sq8;
        return fmaf((float)t, s * sx, acc);
    }

    // Quantise one chunk (32 consecutive fp16 values at `src`, 16-byte aligned) into registers, with
    // exactly the arithmetic of stage_x_q16.
    static __device__ __forceinline__ void quantize_chunk(const __half* src, uint4 (&xv)[4], float& sx, int& sq8) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 r = *reinterpret_cast<const uint4*>(src + 8 * j);
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
                v[8 * j + 2 * k] = __low2float(h);
                v[8 * j + 2 * k + 1] = __high2float(h);
            }
        }
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) m = fmaxf(m, fabsf(v[i]));
        const float inv = m > 0.f ? 32512.f / m : 0.f;
        int sq = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int q[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                q[k] = max(-32512, min(32512, __float2int_rn(v[8 * j + k] * inv)));
                sq += q[k];
            }
            xv[j].x = pack_bytes<1>(q[0], q[2], q[4], q[6]);
            xv[j].y = pack_bytes<1>(q[1], q[3], q[5], q[7]);
            xv[j].z = pack_bytes<0>(q[0], q[2], q[4], q[6]);
            xv[j].w = pack_bytes<0>(q[1], q[3], q[5], q[7]);
        }
        sx = m * (1.0f / 32512.f);
        sq8 = 8 * sq;
    }

    // Same arithmetic with the staged chunk given as a 32-bit shared-memory address: explicit
    // ld.shared, offsets that are constants after unrolling fold into the instruction.
    template <int NR>
    static __device__ __forceinline__ void chunk_s(const uint4 (&q)[NR], const float (&s)[NR], uint32_t xaddr,
                                                   float (&acc)[NR]) {
        int dh[NR], dl[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) { dh[r] = 0; dl[r] = 0; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 xv = lds128(xaddr + 16 * j);
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = j == 0 ? q[r].x : j == 1 ? q[r].y : j == 2 ? q[r].z : q[r].w;
                const uint32_t we = w & 0x0F0F0F0Fu;
                const uint32_t wo = (w >> 4) & 0x0F0F0F0Fu;
                dh[r] = dp4a_us(we, xv.x, dh[r]);
                dl[r] = dp4a_uu(we, xv.z, dl[r]);
                dh[r] = dp4a_us(wo, xv.y, dh[r]);
                dl[r] = dp4a_uu(wo, xv.w, dl[r]);
            }
        }
        const uint2 tail = lds64(xaddr + 64);  // {sx, 8 * sum q}
        const float sx = __uint_as_float(tail.x);
        const int sq8 = (int)tail.y;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int t = dh[r] * 256 + dl[r] - sq8;
            acc[r] = fmaf((float)t, s[r] * sx, acc[r]);
        }
    }
};

__device__ __forceinline__ float load_x_as_f32(const void* x, int dtype, int i) {
    if (dtype == X_F32) return reinterpret_cast<const float*>(x)[i];
    if (dtype == X_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
}

// Load 8 consecutive activations (index 8*item .. 8*item+7) as fp32 with 16-byte loads.  The
// vector must be 16-byte aligned for 16-bit types and for fp32 (launchers check this).
__device__ __forceinline__ void load_x8(const void* x, int dtype, int item, float (&v)[8]) {
    if (dtype == X_F32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * item);
        const float4 b = __ldg(reinterpret_cast<const float4*>(x) + 2 * item + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(x) + item);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (dtype == X_F16) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
                v[2 * k] = __low2float(h);
                v[2 * k + 1] = __high2float(h);
            } else {
                v[2 * k] = __uint_as_float(w[k] << 16);
                v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
    }
}

// Copy an activation vector of n values (n a multiple of 32) into padded chunk layout.  Must
// be called by whole warps with nthreads a multiple of 32.  A thread handles 8 consecutive
// values (one quarter of a chunk); up to U such items per thread are requested before any is
// used, so the whole vector costs one or two round trips to L2.  For MathF16 each chunk's padding
// receives the sums of its even and of its odd columns (as staged, i.e. after the conversion to
// fp16).  The caller synchronises.
template <class MATH, int U = 4>
__device__ __forceinline__ void stage_x(typename MATH::XS* dst, const void* x, int dtype, int n, int tid,
                                        int nthreads) {
    const int nitems = n >> 3;
    for (int base = 0; base < nitems; base += U * nthreads) {
        float v[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int item = base + u * nthreads + tid;
            if (item < nitems) load_x8(x, dtype, item, v[u]);
            else {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[u][k] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int item = base + u * nthreads + tid;
            const bool live = item < nitems;
            const int c = item >> 2, jj = item & 3;
            float se = 0.f, so = 0.f;
            typename MATH::XS t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                t[k] = MATH::from_f32(v[u][k]);
                if (k & 1) so += MATH::to_f32(t[k]);
                else se += MATH::to_f32(t[k]);
            }
            if (live) {
#pragma unroll
                for (int k = 0; k < 8; ++k) dst[(size_t)c * MATH::kStride + jj * 8 + k] = t[k];
            }
            if (MATH::kChunkSums) {
                se += __shfl_xor_sync(0xffffffffu, se, 1);
                so += __shfl_xor_sync(0xffffffffu, so, 1);
                se += __shfl_xor_sync(0xffffffffu, se, 2);
                so += __shfl_xor_sync(0xffffffffu, so, 2);
                if (live && jj == 0) {
                    float* sums = reinterpret_cast<float*>(dst + (size_t)c * MATH::kStride + 32);
                    sums[0] = se;
                    sums[1] = so;
                }
            }
        }
    }
}

// Quantise an activation vector of n values (n a multiple of 32) into the MathQ16 chunk layout.
// Same work split as stage_x: a thread owns 8 consecutive values = one uint4 of the layout; the 4
// threads of a chunk agree on its maximum and on the sum of its codes with two shuffles.
template <int U = 4>
__device__ __forceinline__ void stage_x_q16(unsigned char* dst, const void* x, int dtype, int n, int tid, int nthreads) {
    const int nitems = n >> 3;
    for (int base = 0; base < nitems; base += U * nthreads) {
        float v[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int item = base + u * nthreads + tid;
            if (item < nitems) load_x8(x, dtype, item, v[u]);
            else {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[u][k] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int item = base + u * nthreads + tid;
            const bool live = item < nitems;
            const int c = item >> 2, jj = item & 3;
            float m = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[u][k]));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            const float inv = m > 0.f ? 32512.f / m : 0.f;
            int q[8], sq = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                q[k] = max(-32512, min(32512, __float2int_rn(v[u][k] * inv)));
                sq += q[k];
            }
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            uint4 o;
            o.x = pack_bytes<1>(q[0], q[2], q[4], q[6]);
            o.y = pack_bytes<1>(q[1], q[3], q[5], q[7]);
            o.z = pack_bytes<0>(q[0], q[2], q[4], q[6]);
            o.w = pack_bytes<0>(q[1], q[3], q[5], q[7]);
            if (live) {
                unsigned char* chunk = dst + (size_t)c * MathQ16::kStride;
                *reinterpret_cast<uint4*>(chunk + 16 * jj) = o;
                if (jj == 0) {
                    *reinterpret_cast<float*>(chunk + 64) = m * (1.0f / 32512.f);
                    *reinterpret_cast<int*>(chunk + 68) = 8 * sq;
                }
            }
        }
    }
}

// Uniform entry: stage (and for MathQ16 quantise) an activation vector for the given math policy.
template <class MATH>
__device__ __forceinline__ void stage_activation(typename MATH::XS* dst, const void* x, int dtype, int n, int tid, int nthreads) {
    stage_x<MATH>(dst, x, dtype, n, tid, nthreads);
}
template <>
__device__ __forceinline__ void stage_activation<MathQ16>(unsigned char* dst, const void* x, int dtype, int n, int tid, int nthreads) {
    stage_x_q16<2>(dst, x, dtype, n, tid, nthreads);   // (two items per thread and trip: less code for a freshly launched kernel to fetch)
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
