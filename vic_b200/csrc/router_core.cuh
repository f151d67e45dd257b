// Device code of the router shared by the stand-alone router kernel (router.cu) and by the expert
// kernel that routes in its own prologue (moe_pipe.cu): the chain arithmetic of a logit, scoring,
// selection, the near-tie recomputation in the CPU router's summation order, and the weights.
#pragma once
#include "int4_math.cuh"
#include "launch_common.h"

namespace vib3 {

constexpr int kRouterMaxExperts = 512;  // MAX_EXPERTS, src/core/types.rs:20
constexpr int kRouterMaxTopK = 16;      // MAX_ACTIVE_EXPERTS, src/core/types.rs:26
constexpr int kRouterXMax = 8192;       // widest activation vector staged in shared memory
constexpr int kSeqCands = 4;            // near-tied experts recomputed side by side (more take further rounds)
constexpr int kSeqBlock = 512;          // products per hand-over between the warps of a recomputation
constexpr unsigned kRouterSpinLimit = 1u << 22;

enum WDType : int { W_F16 = 0, W_F32 = 1 };

struct RouterArgs {
    const void* x;
    int x_dtype;
    const void* W;
    int w_dtype;
    float* scores;        // [E] logits; [2E] when exact_order (second half: sum |x*w|); [3E] single launch, sigmoid
    const float* bias;    // [E] or null: added to the score for selection only
    const float* logit_offset;  // [E] or null: added to the logit before scoring (a pre-activation bias)
    unsigned short* out_ids;
    float* out_weights;
    unsigned int* counter;  // workspace words (single-launch paths only)
    int H, E, top_k, mode;
    float scaling;
    int normalize;
    int exact_order;
    int hold_dependents;  // the first kernel lets its dependents start only after its own dependency wait (see make_router_args)
    // batched launch (grid y = token): distances between the tokens' vectors / buffers; zero for one token
    int x_stride;        // bytes
    int scores_stride;   // floats
    int ids_stride;      // entries
    int weights_stride;  // entries
    int counter_stride;  // words
};

// The arguments of token blockIdx.y of a batched launch.
__device__ __forceinline__ void router_args_of_token(RouterArgs& a, int t) {
    a.x = reinterpret_cast<const unsigned char*>(a.x) + (size_t)t * a.x_stride;
    a.scores += (size_t)t * a.scores_stride;
    if (a.out_ids) a.out_ids += (size_t)t * a.ids_stride;
    if (a.out_weights) a.out_weights += (size_t)t * a.weights_stride;
    if (a.counter) a.counter += (size_t)t * a.counter_stride;
}

__device__ __forceinline__ float load_w(const void* W, int w_dtype, size_t i) {
    return w_dtype == W_F32 ? reinterpret_cast<const float*>(W)[i]
                            : __half2float(reinterpret_cast<const __half*>(W)[i]);
}

// Four consecutive weights of a row (item i = columns 4i .. 4i+3) with one streaming load.
template <int WD> struct WItem;
template <> struct WItem<W_F32> {
    using T = uint4;
    static __device__ __forceinline__ T load(const void* row, int i) { return ldg_stream16(reinterpret_cast<const uint4*>(row) + i); }
    static __device__ __forceinline__ float4 cvt(const T& v) {
        return make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
    }
};
template <> struct WItem<W_F16> {
    using T = uint2;
    static __device__ __forceinline__ T load(const void* row, int i) {
        uint2 v;
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(reinterpret_cast<const uint2*>(row) + i));
        return v;
    }
    static __device__ __forceinline__ float4 cvt(const T& v) {
        const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
};

// Four consecutive activations (item i = columns 4i .. 4i+3) as fp32 from the raw copy of the vector in
// shared memory.
template <int XD>
__device__ __forceinline__ float4 x_item(const unsigned char* xraw, int i) {
    if (XD == X_F32) return reinterpret_cast<const float4*>(xraw)[i];
    const uint2 v = reinterpret_cast<const uint2*>(xraw)[i];
    if (XD == X_F16) {
        const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xFFFF0000u));
}

__device__ __forceinline__ unsigned int orderable(float v) {
    const unsigned int b = __float_as_uint(v + 0.0f);  // -0 -> +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float exp_rn(float v) { return (float)exp((double)v); }

__device__ __forceinline__ float sigmoid_ref(float z) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_rn(-z)));
}


// Scratch of scoring and selection.  `ring` holds the products of a sequential-order recomputation:
// per candidate two halves of kSeqBlock products.
struct __align__(16) TopKSmem {
    float logit[kRouterMaxExperts];
    float sig[kRouterMaxExperts];
    float sel[kRouterMaxExperts];
    float wid[kRouterMaxExperts];
    int cand[kRouterMaxExperts];
    int chosen[kRouterMaxTopK + 1];
    int redo;
    int ncand;
    int failed;
    unsigned long long seq_full[2], seq_empty[2];  // mbarriers of the recomputation's two ring halves
    unsigned seq_blocks;                           // blocks handed over so far (phase bookkeeping)
};
constexpr int kSeqRingFloats = kSeqCands * 2 * kSeqBlock;  // 16 KB

// The reference kernel's reduction of an expert's 128 chain sums (kernels.cu:52-57, :682-705) when lane l
// holds chains 4l .. 4l+3: its shfl_down tree over each group of 32 chains is, in this layout, three
// shuffles by 4, 2, 1 lanes per component followed by (c0 + c2) + (c1 + c3) inside a lane; the four group
// sums s0..s3 then meet as (s0 + s2) + (s1 + s3).  Same pairs, same order, so the same bits; valid in lane 0.
__device__ __forceinline__ float chain_tree(const float (&acc)[4]) {
    float v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        v[c] = acc[c];
        v[c] += __shfl_down_sync(0xffffffffu, v[c], 4);
        v[c] += __shfl_down_sync(0xffffffffu, v[c], 2);
        v[c] += __shfl_down_sync(0xffffffffu, v[c], 1);
    }
    float s = __fadd_rn(__fadd_rn(v[0], v[2]), __fadd_rn(v[1], v[3]));   // group sum, valid in lanes 0, 8, 16, 24
    s = __fadd_rn(s, 0.0f);  // the reference adds zeros from its idle lanes (turns -0 into +0)
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 16));
    s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, 8));
    return s;
}

__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The best `nsel` entries of sm.sel[0 .. E) in descending order, ties towards the lower expert index,
// found by ONE warp: lane l keeps the keys of experts l, l + 32, ... in registers; a round is two
// warp-wide integer reductions (largest key, then lowest index holding it).  Lane i returns the
// i-th selected expert (-1 when fewer exist).
// kPerLane: keys per lane, at least E / 32 (the loops over them are unrolled: the narrower form is less code for a
// freshly launched kernel to fetch).
template <int kPerLane>
__device__ __forceinline__ int warp_select_n(const RouterArgs& a, const TopKSmem& sm, int nsel) {
    const int lane = threadIdx.x & 31;
    unsigned key[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        const int e = lane + 32 * j;
        key[j] = e < a.E ? orderable(sm.sel[e]) : 0u;
    }
    int mine = -1;
    for (int round = 0; round < nsel; ++round) {
        unsigned m = key[0];
#pragma unroll
        for (int j = 1; j < kPerLane; ++j) m = max(m, key[j]);
        const unsigned best = __reduce_max_sync(0xffffffffu, m);
        unsigned idx = 0xFFFFu;
#pragma unroll
        for (int j = kPerLane - 1; j >= 0; --j)
            if (key[j] == best) idx = (unsigned)(lane + 32 * j);
        const unsigned who = __reduce_min_sync(0xffffffffu, idx);
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
            if ((unsigned)(lane + 32 * j) == who) key[j] = 0u;
        if (lane == round) mine = best ? (int)who : -1;
    }
    return mine;
}
__device__ inline int warp_select(const RouterArgs& a, const TopKSmem& sm, int nsel) {
    return a.E <= 384 ? warp_select_n<12>(a, sm, nsel) : warp_select_n<kRouterMaxExperts / 32>(a, sm, nsel);
}


// Barrier among the `nthreads` threads (a multiple of 32) that run the selection together; id 2 is not
// used by anything else in the kernels that include this file.
__device__ __forceinline__ void group_sync(int nthreads) {
    if (nthreads == 32) __syncwarp();
    else asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
}

__device__ __forceinline__ void seq_bar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void seq_bar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"((uint32_t)__cvta_generic_to_shared(bar)) : "memory");
}
__device__ __forceinline__ bool seq_bar_wait(unsigned long long* bar, unsigned parity) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(bar);
    for (unsigned it = 0; it < kRouterSpinLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// Called once by one thread before the group's first selection (followed by a group_sync).
__device__ __forceinline__ void topk_smem_init(TopKSmem& sm, int helper_warps) {
    for (int h = 0; h < 2; ++h) {
        seq_bar_init(&sm.seq_full[h], helper_warps);
        seq_bar_init(&sm.seq_empty[h], 1);
    }
    sm.seq_blocks = 0;
    sm.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Logits of up to kSeqCands experts in the CPU router's order (kernels.rs:2346-2350): per expert a single
// chain, multiply then add, d = 0 .. H-1.  The 7168 dependent additions of the Kimi shape are the cost
// (about 18 us on B200, whatever the number of candidates); everything else hides under them: the group's
// first warp only adds — lane c owns candidate c's chain — while the other warps form the rounded products
// a block of kSeqBlock ahead into a two-half ring in shared memory.  `warp` is the caller's index in the
// group, `nwarps` >= 2 its size.  Lane c < nc of warp 0 returns candidate c's sum.
__device__ inline float sequential_logits(const RouterArgs& a, TopKSmem& sm, float* ring, const int* cands, int nc, int warp,
                                   int nwarps, int lane) {
    const int nblocks = (a.H + kSeqBlock - 1) / kSeqBlock;
    const unsigned first = sm.seq_blocks;  // (read before anybody advances it: the caller synchronised)
    float acc = 0.f;
    if (warp == 0) {
        for (int b = 0; b < nblocks; ++b) {
            const unsigned gb = first + b;
            const int half = gb & 1;
            if (!seq_bar_wait(&sm.seq_full[half], (gb >> 1) & 1)) { sm.failed = 1; break; }
            if (lane < nc) {
                const float* p = ring + (lane * 2 + half) * kSeqBlock;
                const int n = min(kSeqBlock, a.H - b * kSeqBlock);
                int i = 0;
                for (; i + 32 <= n; i += 32) {
                    float4 q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) q[j] = *reinterpret_cast<const float4*>(p + i + 4 * j);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc = __fadd_rn(acc, q[j].x);
                        acc = __fadd_rn(acc, q[j].y);
                        acc = __fadd_rn(acc, q[j].z);
                        acc = __fadd_rn(acc, q[j].w);
                    }
                }
                for (; i < n; ++i) acc = __fadd_rn(acc, p[i]);
            }
            __syncwarp();
            if (lane == 0) seq_bar_arrive(&sm.seq_empty[half]);
        }
    } else {
        const int hw = warp - 1, nh = nwarps - 1;
        for (int b = 0; b < nblocks; ++b) {
            const unsigned gb = first + b;
            const int half = gb & 1;
            if (gb >= 2 && !seq_bar_wait(&sm.seq_empty[half], ((gb >> 1) - 1) & 1)) { sm.failed = 1; break; }
            const int n = min(kSeqBlock, a.H - b * kSeqBlock);
            // (candidate, 4-element item) pairs of the block: one 16-byte (fp16 weights: 8-byte) load of the
            // weights and one of the activations per item, all of a lane's items requested before any is used
            // (one round trip per block); rows that are not 16-byte aligned take the scalar path
            const bool vec = a.H % 4 == 0 && ((uintptr_t)a.x & 15) == 0 && ((uintptr_t)a.W & 15) == 0 && n % 4 == 0;
            if (vec) {
                const int n4 = n >> 2, total = nc * n4;
                constexpr int U = 4;
                for (int t0 = hw * 32 + lane; t0 < total; t0 += nh * 32 * U) {
                    float4 xv[U], wv[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int t = t0 + u * nh * 32;
                        const bool in = t < total;
                        const int c = in ? t / n4 : 0, i = in ? t - c * n4 : 0;
                        const int item = (b * kSeqBlock >> 2) + i;
                        if (a.x_dtype == X_F32) xv[u] = __ldg(reinterpret_cast<const float4*>(a.x) + item);
                        else {
                            const uint2 r2 = __ldg(reinterpret_cast<const uint2*>(a.x) + item);
                            if (a.x_dtype == X_F16) {
                                const __half2 p0 = *reinterpret_cast<const __half2*>(&r2.x), p1 = *reinterpret_cast<const __half2*>(&r2.y);
                                xv[u] = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
                            } else {
                                xv[u] = make_float4(__uint_as_float(r2.x << 16), __uint_as_float(r2.x & 0xFFFF0000u),
                                                    __uint_as_float(r2.y << 16), __uint_as_float(r2.y & 0xFFFF0000u));
                            }
                        }
                        const size_t wi = ((size_t)cands[c] * a.H >> 2) + item;
                        if (a.w_dtype == W_F32) wv[u] = __ldcg(reinterpret_cast<const float4*>(a.W) + wi);
                        else wv[u] = WItem<W_F16>::cvt(__ldcg(reinterpret_cast<const uint2*>(a.W) + wi));
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int t = t0 + u * nh * 32;
                        if (t < total) {
                            const int c = t / n4, i = t - c * n4;
                            *reinterpret_cast<float4*>(ring + (c * 2 + half) * kSeqBlock + 4 * i) =
                                make_float4(__fmul_rn(xv[u].x, wv[u].x), __fmul_rn(xv[u].y, wv[u].y), __fmul_rn(xv[u].z, wv[u].z),
                                            __fmul_rn(xv[u].w, wv[u].w));
                        }
                    }
                }
            } else {
                const int total = nc * n;
                for (int t0 = (hw * 32 + lane); t0 < total; t0 += nh * 32 * 8) {
                    float xv[8], wv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int t = t0 + u * nh * 32;
                        const bool in = t < total;
                        const int c = in ? t / n : 0, i = in ? t - c * n : 0;
                        const int d = b * kSeqBlock + i;
                        xv[u] = in ? load_x_as_f32(a.x, a.x_dtype, d) : 0.f;
                        wv[u] = in ? load_w(a.W, a.w_dtype, (size_t)cands[c] * a.H + d) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int t = t0 + u * nh * 32;
                        if (t < total) {
                            const int c = t / n, i = t - c * n;
                            ring[(c * 2 + half) * kSeqBlock + i] = __fmul_rn(xv[u], wv[u]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) seq_bar_arrive(&sm.seq_full[half]);
        }
    }
    return acc;
}

__device__ __forceinline__ void group_score(const RouterArgs& a, TopKSmem& sm, int tid, int nthreads) {
    for (int e = tid; e < a.E; e += nthreads) {
        const float z = sm.logit[e];
        if (a.mode == 0) {
            sm.sig[e] = z;
            sm.sel[e] = z;
        } else {
            const float s = sigmoid_ref(z);
            sm.sig[e] = s;
            sm.sel[e] = a.bias ? __fadd_rn(s, a.bias[e]) : s;
        }
    }
    group_sync(nthreads);
}

// Scoring, selection and weights from the logits in a.scores, by a group of `nthreads` threads (whole
// warps; `tid` = index in the group; at least two warps when a.exact_order is set) that all call this
// together; the group's first warp selects.  have_sig: a.scores[2E ..] already holds the sigmoid of every
// logit.  write_global: store ids, weights (and recomputed logits) to a.out_ids / a.out_weights / a.scores.
// ids_smem / w_smem (optional, shared memory, kRouterMaxTopK entries): receive the same results.
__device__ inline void router_finish(const RouterArgs& a, TopKSmem& sm, float* ring, int tid, int nthreads, bool have_sig,
                              bool write_global, unsigned short* ids_smem, float* w_smem) {
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int k = min(a.top_k, a.E);
    const int nsel = min(k + 1, a.E);
    const bool exact = a.exact_order && nsel > 1 && nwarps >= 2;
    // one round trip: logits and (exact-order mode) the sums of |x w| together; then scoring and,
    // in exact-order mode, the half-width of each expert's selection score under a change of
    // summation order.  The logits of two fp32 summation orders of H products differ by less than
    //     eps = 8 * 2^-24 * (sqrt(H) * |S| + sum |x w|)
    // (a statistical bound, not a worst-case one: over 57,600 expert-token samples of the Kimi shape the
    // largest observed difference is 0.18 eps and the root mean square 0.025 eps; the oracle's tests
    // check a 4x margin); a selection score moves by at most eps
    // times the local slope of the scoring function (1 for raw logits, s (1 - s) for the sigmoid,
    // taken 1.25x for the curvature) plus a few ulps of rounding.
    for (int e0 = 0; e0 < a.E; e0 += 4 * nthreads) {
        float z[4], ab[4], sg[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // all loads first: one round trip
            const int e = e0 + tid + nthreads * j;
            z[j] = e < a.E ? __ldcg(a.scores + e) : 0.f;
            ab[j] = (exact && e < a.E) ? __ldcg(a.scores + a.E + e) : 0.f;
            sg[j] = (have_sig && e < a.E) ? __ldcg(a.scores + 2 * a.E + e) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = e0 + tid + nthreads * j;
            if (e >= a.E) continue;
            float s = z[j], sel = z[j];
            if (a.mode != 0) {
                s = have_sig ? sg[j] : sigmoid_ref(z[j]);
                sel = a.bias ? __fadd_rn(s, a.bias[e]) : s;
            }
            sm.logit[e] = z[j];
            sm.sig[e] = s;
            sm.sel[e] = sel;
            if (exact) {
                const float eps = 8.f * 5.9604645e-8f * (sqrtf((float)a.H) * fabsf(z[j]) + ab[j]);
                const float slope = a.mode == 0 ? 1.f : 1.25f * s * (1.f - s);
                sm.wid[e] = eps * slope + 2.f * 1.1920929e-7f * fmaxf(fabsf(sel), 1e-30f);
            }
        }
    }
    if (tid == 0) sm.redo = 0;
    group_sync(nthreads);

    int mine = -1;  // warp 0: lane i holds the i-th selected expert
    if (warp == 0) {
        mine = warp_select(a, sm, nsel);
        if (exact) {
            // adjacent scores among the best k+1 closer than their widths: the order may differ
            const int next = __shfl_down_sync(0xffffffffu, mine, 1);
            bool close = false;
            if (lane + 1 < nsel && mine >= 0 && next >= 0)
                close = sm.sel[mine] - sm.sel[next] <= sm.wid[mine] + sm.wid[next];
            if (__ballot_sync(0xffffffffu, close)) {
                if (lane < nsel) sm.chosen[lane] = mine;
                if (lane == 0) sm.redo = 1;
            }
        }
    }
    group_sync(nthreads);

    if (sm.redo) {
        // candidates: every expert whose score interval overlaps that of one of the best k+1
        const int last = sm.chosen[nsel - 1];
        if (tid == 0) sm.ncand = 0;
        group_sync(nthreads);
        for (int e = tid; e < a.E; e += nthreads) {
            bool cand = false;
            if (last < 0 || sm.sel[e] + sm.wid[e] >= sm.sel[last] - sm.wid[last])
                for (int i = 0; i < nsel; ++i) {
                    const int c = sm.chosen[i];
                    if (c >= 0 && c != e && fabsf(sm.sel[e] - sm.sel[c]) <= sm.wid[e] + sm.wid[c]) cand = true;
                }
            if (cand) sm.cand[atomicAdd(&sm.ncand, 1)] = e;
        }
        group_sync(nthreads);
        const int nblocks = (a.H + kSeqBlock - 1) / kSeqBlock;
        for (int c0 = 0; c0 < sm.ncand; c0 += kSeqCands) {
            const int nc = min(kSeqCands, sm.ncand - c0);
            const float acc = sequential_logits(a, sm, ring, sm.cand + c0, nc, warp, nwarps, lane);
            if (warp == 0 && lane < nc) {
                const int e = sm.cand[c0 + lane];
                const float v = a.logit_offset ? __fadd_rn(acc, a.logit_offset[e]) : acc;
                sm.logit[e] = v;
                if (write_global) a.scores[e] = v;
            }
            group_sync(nthreads);
            if (tid == 0) sm.seq_blocks += nblocks;
            group_sync(nthreads);
        }
        if (tid == 0 && write_global && a.counter) a.counter[1] += 1u;  // diagnostics: near-tie recomputations so far
        group_score(a, sm, tid, nthreads);
        if (warp == 0) mine = warp_select(a, sm, k);
    }

    if (warp != 0) return;
    // weights, lane i for the i-th selected expert; sums run in selection order
    const bool live = lane < k && mine >= 0;
    float wout = 0.f;
    if (a.mode == 0) {
        const float zl = live ? sm.logit[mine] : -INFINITY;
        float mx = zl;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float ex = live ? exp_rn(__fsub_rn(zl, mx)) : 0.f;
        float sum = 0.f;
        for (int i = 0; i < k; ++i) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, i));
        wout = __fdiv_rn(ex, sum);
    } else {
        const float w = live ? sm.sig[mine] : 0.f;
        float total = 0.f;
        for (int i = 0; i < k; ++i) total = __fadd_rn(total, __shfl_sync(0xffffffffu, w, i));
        const bool norm = a.normalize && total > 1e-20f;
        wout = __fmul_rn(norm ? __fdiv_rn(w, total) : w, a.scaling);
    }
    if (live && write_global) {
        a.out_ids[lane] = (unsigned short)mine;
        a.out_weights[lane] = wout;
    }
    if (ids_smem && lane < kRouterMaxTopK) {
        ids_smem[lane] = live ? (unsigned short)mine : (unsigned short)0xFFFF;
        w_smem[lane] = live ? wout : 0.f;
    }
}

// Logit of one expert row held in shared memory (16-byte aligned), by one warp: lane l owns the chains
// 4l .. 4l+3 (see chain_tree).  xraw: the activation vector as given (XD) in shared memory.  H a multiple
// of 8 (fp32 x: of 4).  logit is valid in lane 0, absum in every lane.
template <int XD, int WD>
__device__ __forceinline__ void row_logit_smem(const unsigned char* wrow, const unsigned char* xraw, int H, int lane,
                                               float& logit, float& absum) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float aabs[4] = {0.f, 0.f, 0.f, 0.f};
    const int n4 = H >> 2;
    for (int it = lane; it < n4; it += 32) {
        float4 wv;
        if (WD == W_F32) wv = reinterpret_cast<const float4*>(wrow)[it];
        else wv = WItem<W_F16>::cvt(reinterpret_cast<const uint2*>(wrow)[it]);
        const float4 xv = x_item<XD>(xraw, it);
        acc[0] = fmaf(xv.x, wv.x, acc[0]);
        acc[1] = fmaf(xv.y, wv.y, acc[1]);
        acc[2] = fmaf(xv.z, wv.z, acc[2]);
        acc[3] = fmaf(xv.w, wv.w, acc[3]);
        aabs[0] += fabsf(xv.x * wv.x);
        aabs[1] += fabsf(xv.y * wv.y);
        aabs[2] += fabsf(xv.z * wv.z);
        aabs[3] += fabsf(xv.w * wv.w);
    }
    logit = chain_tree(acc);
    absum = warp_total((aabs[0] + aabs[1]) + (aabs[2] + aabs[3]));
}

}  // namespace vib3
