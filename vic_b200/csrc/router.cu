// Router: logits GEMV, scoring (softmax / sigmoid), stable top-k, normalise and scale.
//
// Reference entry points kept with identical signatures:
//   vib3_launch_router_gemv       cuda/src/kernels.cu:1143  (x fp16, W fp16)
//   vib3_launch_router_gemv_f32   cuda/src/kernels.cu:1477  (x fp32, W fp16)
//   vib3_launch_router_topk       cuda/src/kernels.cu:4075  (GEMV + top-k, results stay on device)
// and one extended launcher, vib3_launch_router_topk_ex, that also accepts fp32 router weights
// and fp16/bf16 activations, any expert count up to 512 (the reference's bitonic kernel needs a
// power of two, kernels.cu:3899), and finishes in a single launch.
//
// Summation order of the logits: exactly the reference CUDA kernel's (kernels.cu:665-707) — 128
// chains per expert, chain t adds d = t, t+128, ... with fused multiply-add, a shfl_down tree
// per warp, then (s0+s2)+(s1+s3) — so logits are bit-identical to the reference's on a GPU.
//
// Scoring and selection follow the reference's CPU router (src/compute/kernels.rs:2364-2437),
// which is the only well-defined reference for 384 experts: softmax over the selected k only;
// sigmoid with optional selection bias, weights from the unbiased sigmoid, divided by their sum
// when it exceeds 1e-20, times the scaling factor; ties resolved towards the lower expert index
// (stable sort).  exp() is evaluated in double and rounded once, sums and divisions are IEEE
// fp32 in selection order.
//
// Bit-exact indices against the CPU router's sequential summation order: when any two adjacent
// selection scores among the best k+1 are closer than a bound on the summation-order
// difference, the near-tied experts' logits are recomputed with one sequential multiply-then-add
// chain per expert (the CPU order) before the final selection.  This costs tens of microseconds
// and happens for a few percent of tokens.
#include "int4_math.cuh"
#include "launch_common.h"

namespace vib3 {

constexpr int kRouterMaxExperts = 512;  // MAX_EXPERTS, src/core/types.rs:20
constexpr int kRouterMaxTopK = 16;      // MAX_ACTIVE_EXPERTS, src/core/types.rs:26
constexpr int kChains = 128;

enum WDType : int { W_F16 = 0, W_F32 = 1 };

struct RouterArgs {
    const void* x;
    int x_dtype;
    const void* W;
    int w_dtype;
    float* scores;        // [E] logits; [2E] when exact_order (second half: sum |x*w|)
    const float* bias;    // [E] or null: added to the score for selection only
    const float* logit_offset;  // [E] or null: added to the logit before scoring (a pre-activation bias)
    unsigned short* out_ids;
    float* out_weights;
    unsigned int* counter;  // two words of workspace (single-launch path only)
    int H, E, top_k, mode;
    float scaling;
    int normalize;
    int exact_order;
};

__device__ __forceinline__ float load_w(const void* W, int w_dtype, size_t i) {
    return w_dtype == W_F32 ? reinterpret_cast<const float*>(W)[i]
                            : __half2float(reinterpret_cast<const __half*>(W)[i]);
}
template <int WD>
__device__ __forceinline__ float load_w_t(const void* W, size_t i) {
    if (WD == W_F32) {
        float v;
        asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(reinterpret_cast<const float*>(W) + i));
        return v;
    }
    return __half2float(__ushort_as_half(ldg_stream2(reinterpret_cast<const __half*>(W) + i)));
}
template <int XD>
__device__ __forceinline__ float load_x_t(const void* x, int i) {
    if (XD == X_F32) return __ldg(reinterpret_cast<const float*>(x) + i);
    if (XD == X_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(x) + i));
    return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(x) + i));
}

// shfl_down tree of the reference (kernels.cu:52-57); only lane 0's value is meaningful.
__device__ __forceinline__ float warp_sum_down(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

// Logit of one expert with 128 threads (lane = chain index); result valid in chain 0.
// All of a thread's weight loads (NW = ceil(H / 128) <= U) are requested first; while they are in
// flight the CTA copies the activation vector into shared memory as fp32, so the whole row costs one
// round trip to memory.  The per-chain order of additions (d = chain, chain + 128, ...) is kept.
template <int U, int XD, int WD>
__device__ __forceinline__ void expert_logit(const RouterArgs& a, int expert, int chain, float* smem4, float* smem4_abs,
                                             float* xs, float& logit, float& absum) {
    const size_t base = (size_t)expert * a.H;
    float acc = 0.f, aabs = 0.f;
    bool staged = xs == nullptr;
    for (int d0 = chain; d0 < a.H; d0 += U * kChains) {
        float w[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int d = d0 + i * kChains;
            w[i] = d < a.H ? load_w_t<WD>(a.W, base + d) : 0.f;
        }
        if (!staged) {  // first batch of weight loads is in flight: copy the activations meanwhile
            for (int i = threadIdx.x; i < a.H; i += blockDim.x) xs[i] = load_x_t<XD>(a.x, i);
            __syncthreads();
            staged = true;
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int d = d0 + i * kChains;
            if (d < a.H) {
                const float xv = xs ? xs[d] : load_x_t<XD>(a.x, d);
                acc = fmaf(xv, w[i], acc);
                aabs += fabsf(xv * w[i]);
            }
        }
    }
    acc = warp_sum_down(acc);
    aabs = warp_sum_down(aabs);
    const int wid = chain >> 5, wl = chain & 31;
    if (wl == 0) { smem4[wid] = acc; smem4_abs[wid] = aabs; }
    __syncthreads();
    if (wid == 0) {
        float f = wl < 4 ? smem4[wl] : 0.f;
        float g = wl < 4 ? smem4_abs[wl] : 0.f;
        f = warp_sum_down(f);
        g = warp_sum_down(g);
        logit = f;
        absum = g;
    }
}

__device__ __forceinline__ unsigned int orderable(float v) {
    const unsigned int b = __float_as_uint(v + 0.0f);  // -0 -> +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float exp_rn(float v) { return (float)exp((double)v); }

__device__ __forceinline__ float sigmoid_ref(float z) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_rn(-z)));
}

// Scoring by one CTA of 256 threads, selection and weights by its first warp.
struct __align__(16) TopKSmem {
    float prod[8][1024];   // per-warp products of the sequential-order recomputation (16-byte aligned: read as float4)
    float logit[kRouterMaxExperts];
    float sig[kRouterMaxExperts];
    float sel[kRouterMaxExperts];
    int chosen[kRouterMaxTopK + 1];
    float wid[kRouterMaxExperts];
    int redo;
    int ncand;
    int cand[kRouterMaxExperts];
};

// The best `nsel` entries of sm.sel[0 .. E) in descending order, ties towards the lower expert index,
// found by ONE warp: lane l keeps the keys of experts l, l + 32, ... in registers; a round is two
// warp-wide integer reductions (largest key, then lowest index holding it).  Lane i returns the
// i-th selected expert (-1 when fewer exist).
__device__ int warp_select(const RouterArgs& a, const TopKSmem& sm, int nsel) {
    const int lane = threadIdx.x & 31;
    constexpr int kPerLane = kRouterMaxExperts / 32;
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

__device__ void block_score(const RouterArgs& a, TopKSmem& sm) {
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
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
    __syncthreads();
}

__device__ void router_finish(const RouterArgs& a, TopKSmem& sm) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = min(a.top_k, a.E);
    const int nsel = min(k + 1, a.E);
    const bool exact = a.exact_order && nsel > 1;
    // one round trip: logits and (exact-order mode) the sums of |x w| together; then scoring and,
    // in exact-order mode, the half-width of each expert's selection score under a change of
    // summation order.  The logits of two fp32 summation orders of H products differ by less than
    //     eps = 8 * 2^-24 * (sqrt(H) * |S| + sum |x w|)
    // (a statistical bound, not a worst-case one: over 57,600 expert-token samples of the Kimi shape the
    // largest observed difference is 0.18 eps and the root mean square 0.025 eps; the oracle's tests
    // check a 4x margin); a selection score moves by at most eps
    // times the local slope of the scoring function (1 for raw logits, s (1 - s) for the sigmoid,
    // taken 1.25x for the curvature) plus a few ulps of rounding.
    // (single-launch path, sigmoid mode: the GEMV CTAs have already stored the sigmoid of their logits)
    const bool have_sig = a.counter != nullptr && a.mode != 0;
    constexpr int kPerThread = kRouterMaxExperts / 256;
    float z[kPerThread], ab[kPerThread], sg[kPerThread];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {  // all loads first: one round trip
        const int e = tid + 256 * j;
        z[j] = e < a.E ? __ldcg(a.scores + e) : 0.f;
        ab[j] = (exact && e < a.E) ? __ldcg(a.scores + a.E + e) : 0.f;
        sg[j] = (have_sig && e < a.E) ? __ldcg(a.scores + 2 * a.E + e) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        const int e = tid + 256 * j;
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
    if (tid == 0) sm.redo = 0;
    __syncthreads();

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
    __syncthreads();

    if (sm.redo) {
        // candidates: every expert whose score interval overlaps that of one of the best k+1
        const int last = sm.chosen[nsel - 1];
        if (tid == 0) sm.ncand = 0;
        __syncthreads();
        for (int e = tid; e < a.E; e += blockDim.x) {
            bool cand = false;
            if (last < 0 || sm.sel[e] + sm.wid[e] >= sm.sel[last] - sm.wid[last])
                for (int i = 0; i < nsel; ++i) {
                    const int c = sm.chosen[i];
                    if (c >= 0 && c != e && fabsf(sm.sel[e] - sm.sel[c]) <= sm.wid[e] + sm.wid[c]) cand = true;
                }
            if (cand) sm.cand[atomicAdd(&sm.ncand, 1)] = e;
        }
        __syncthreads();
        // the CPU router's order: one chain per expert, multiply then add, d = 0 .. H-1
        // (kernels.rs:2346-2350).  A warp forms 1024 rounded products at a time in parallel;
        // lane 0 then adds them in order.
        for (int ci = warp; ci < sm.ncand; ci += 8) {
            const int e = sm.cand[ci];
            const size_t base = (size_t)e * a.H;
            float acc = 0.f;
            for (int d0 = 0; d0 < a.H; d0 += 1024) {
                const int n = min(1024, a.H - d0);
                for (int i = lane; i < n; i += 32)
                    sm.prod[warp][i] = __fmul_rn(load_x_as_f32(a.x, a.x_dtype, d0 + i), load_w(a.W, a.w_dtype, base + d0 + i));
                __syncwarp();
                if (lane == 0) {
                    int i = 0;
                    for (; i + 4 <= n; i += 4) {
                        const float4 p = *reinterpret_cast<const float4*>(&sm.prod[warp][i]);
                        acc = __fadd_rn(acc, p.x);
                        acc = __fadd_rn(acc, p.y);
                        acc = __fadd_rn(acc, p.z);
                        acc = __fadd_rn(acc, p.w);
                    }
                    for (; i < n; ++i) acc = __fadd_rn(acc, sm.prod[warp][i]);
                }
                __syncwarp();
            }
            if (lane == 0) {
                if (a.logit_offset) acc = __fadd_rn(acc, a.logit_offset[e]);
                sm.logit[e] = acc;
                a.scores[e] = acc;
            }
        }
        __syncthreads();
        if (tid == 0 && a.counter) a.counter[1] += 1u;  // diagnostics: near-tie recomputations so far
        block_score(a, sm);
        if (warp == 0) mine = warp_select(a, sm, k);
    }

    if (warp != 0) return;
    // weights, lane i for the i-th selected expert; sums run in selection order
    const bool live = lane < k && mine >= 0;
    if (a.mode == 0) {
        const float z = live ? sm.logit[mine] : -INFINITY;
        float mx = z;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float ex = live ? exp_rn(__fsub_rn(z, mx)) : 0.f;
        float sum = 0.f;
        for (int i = 0; i < k; ++i) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, i));
        if (live) {
            a.out_ids[lane] = (unsigned short)mine;
            a.out_weights[lane] = __fdiv_rn(ex, sum);
        }
    } else {
        const float w = live ? sm.sig[mine] : 0.f;
        float total = 0.f;
        for (int i = 0; i < k; ++i) total = __fadd_rn(total, __shfl_sync(0xffffffffu, w, i));
        const bool norm = a.normalize && total > 1e-20f;
        if (live) {
            const float v = norm ? __fdiv_rn(w, total) : w;
            a.out_ids[lane] = (unsigned short)mine;
            a.out_weights[lane] = __fmul_rn(v, a.scaling);
        }
    }
}

// GEMV: 2 experts per CTA, 128 threads each.  When `a.counter` is set, the CTA that finishes
// last also does the scoring and selection (single launch).
template <int U, int XD, int WD, bool XSMEM>
__global__ void __launch_bounds__(256) router_kernel(RouterArgs a) {
    __shared__ float red[2][4], red_abs[2][4];
    __shared__ TopKSmem sm;
    __shared__ int is_last;
    // let a dependent kernel (launched with programmatic stream serialization) begin its prologue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int local = threadIdx.x >> 7, chain = threadIdx.x & 127;
    const int expert = blockIdx.x * 2 + local;
    float logit = 0.f, absum = 0.f;
    // the activation vector as fp32 in shared memory; the selection phase has not started yet, so
    // the product buffer of TopKSmem (8192 floats) is free to hold it
    float* xs = (XSMEM && a.H <= 8 * 1024) ? &sm.prod[0][0] : nullptr;
    // both halves of the CTA must reach the __syncthreads inside expert_logit
    const int e_clamped = min(expert, a.E - 1);
    expert_logit<U, XD, WD>(a, e_clamped, chain, red[local], red_abs[local], xs, logit, absum);
    if (chain == 0 && expert < a.E) {
        if (a.logit_offset) logit = __fadd_rn(logit, a.logit_offset[expert]);
        a.scores[expert] = logit;
        if (a.exact_order) a.scores[a.E + expert] = absum;
        // single launch, sigmoid scoring: the double-precision exponential runs here, in parallel over
        // the CTAs, instead of in the last CTA's serial tail
        if (a.counter != nullptr && a.mode != 0) a.scores[2 * a.E + expert] = sigmoid_ref(logit);
    }
    if (a.counter == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        // release this CTA's logits and acquire everybody else's in one operation
        unsigned int ticket;
        asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(a.counter) : "memory");
        is_last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    router_finish(a, sm);
    if (threadIdx.x == 0) *a.counter = 0u;  // ready for the next launch
}

__global__ void __launch_bounds__(256) router_topk_kernel(RouterArgs a) {
    __shared__ TopKSmem sm;
    router_finish(a, sm);
}

// 0 (default): 14 loads per batch, activations from global memory; 1: whole row in one batch,
// activations via shared memory; 2: two batches.  Set through vib3_config_set(2, v).
int g_router_variant = 0;

static int launch_router(const RouterArgs& a, cudaStream_t st) {
    const int grid = (a.E + 1) / 2;
    // The default variant asks for the largest shared-memory carve-out: the gate/up kernel that follows
    // sizes itself to fit beside one router CTA, which only works if both want the same SM configuration.
#define VIB3_ROUTER_CASE(XD, WD)                                                      \
    if (a.x_dtype == XD && a.w_dtype == WD) {                                         \
        static const cudaError_t carve = cudaFuncSetAttribute(router_kernel<14, XD, WD, false>,    \
            cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);  \
        (void)carve;                                                                  \
        if (g_router_variant == 0) router_kernel<14, XD, WD, false><<<grid, 256, 0, st>>>(a);      \
        else if (g_router_variant == 2) router_kernel<28, XD, WD, true><<<grid, 256, 0, st>>>(a);  \
        else if (g_router_variant == 3) router_kernel<56, XD, WD, false><<<grid, 256, 0, st>>>(a); \
        else if (g_router_variant == 4) router_kernel<28, XD, WD, false><<<grid, 256, 0, st>>>(a); \
        else router_kernel<56, XD, WD, true><<<grid, 256, 0, st>>>(a);                \
        return (int)cudaGetLastError();                                               \
    }
    VIB3_ROUTER_CASE(X_F32, W_F16)
    VIB3_ROUTER_CASE(X_F32, W_F32)
    VIB3_ROUTER_CASE(X_F16, W_F16)
    VIB3_ROUTER_CASE(X_F16, W_F32)
    VIB3_ROUTER_CASE(X_BF16, W_F16)
    VIB3_ROUTER_CASE(X_BF16, W_F32)
#undef VIB3_ROUTER_CASE
    return VIB3_ERR_UNSUPPORTED;
}

static int check_router(const RouterArgs& a) {
    if (!a.x || !a.W || !a.scores) return VIB3_ERR_NULL;
    if (a.H <= 0 || a.E <= 0) return VIB3_ERR_SHAPE;
    return VIB3_OK;
}

static int check_topk(const RouterArgs& a) {
    if (!a.out_ids || !a.out_weights) return VIB3_ERR_NULL;
    if (a.E > kRouterMaxExperts) return VIB3_ERR_COUNT;
    if (a.top_k <= 0 || a.top_k > kRouterMaxTopK || a.top_k > a.E) return VIB3_ERR_COUNT;
    if (a.mode != 0 && a.mode != 1) return VIB3_ERR_UNSUPPORTED;
    return VIB3_OK;
}

}  // namespace vib3

using namespace vib3;

extern "C" int vib3_router_config_set(int value) {
    const int old = g_router_variant;
    g_router_variant = value;
    return old;
}

extern "C" int vib3_launch_router_gemv(const void* x_f16, const void* W_f16, float* scores, int hidden_dim,
                                       int num_experts, void* stream) {
    RouterArgs a{};
    a.x = x_f16; a.x_dtype = X_F16; a.W = W_f16; a.w_dtype = W_F16; a.scores = scores; a.H = hidden_dim; a.E = num_experts;
    if (int e = check_router(a)) return e;
    return launch_router(a, (cudaStream_t)stream);
}

extern "C" int vib3_launch_router_gemv_f32(const void* x_f32, const void* W_f16, float* scores, int hidden_dim,
                                           int num_experts, void* stream) {
    RouterArgs a{};
    a.x = x_f32; a.x_dtype = X_F32; a.W = W_f16; a.w_dtype = W_F16; a.scores = scores; a.H = hidden_dim; a.E = num_experts;
    if (int e = check_router(a)) return e;
    return launch_router(a, (cudaStream_t)stream);
}

// Reference signature: two launches (GEMV, then selection), weights always normalised in
// sigmoid mode as the reference's kernel does (kernels.cu:4056-4062).
extern "C" int vib3_launch_router_topk(const void* x_f32, const void* W_f16, float* scores_buf, const float* bias,
                                       unsigned short* out_ids, float* out_weights, int hidden_dim, int num_experts,
                                       int top_k, int scoring_mode, float scaling_factor, void* stream) {
    RouterArgs a{};
    a.x = x_f32; a.x_dtype = X_F32; a.W = W_f16; a.w_dtype = W_F16; a.scores = scores_buf; a.bias = bias;
    a.out_ids = out_ids; a.out_weights = out_weights; a.H = hidden_dim; a.E = num_experts; a.top_k = top_k;
    a.mode = scoring_mode; a.scaling = scaling_factor; a.normalize = 1; a.exact_order = 0;
    if (int e = check_router(a)) return e;
    if (int e = check_topk(a)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    if (int e = launch_router(a, st)) return e;
    router_topk_kernel<<<1, 256, 0, st>>>(a);
    return (int)cudaGetLastError();
}

// Extended launcher: one launch.  scores_buf holds 3E floats ([0, E) receives the logits, the rest is scratch);
// workspace is two 32-bit words, zero before the first call: [0] is an arrival counter that every
// call leaves at zero, [1] counts the near-tie recomputations done so far (diagnostics).
extern "C" int vib3_launch_router_topk_ex(const void* x, int x_dtype, const void* W, int w_dtype, float* scores_buf,
                                          const float* bias, const float* logit_offset, unsigned short* out_ids,
                                          float* out_weights,
                                          int hidden_dim, int num_experts, int top_k, int scoring_mode,
                                          float scaling_factor, int normalize, int exact_order,
                                          unsigned int* workspace, void* stream) {
    RouterArgs a{};
    a.x = x; a.x_dtype = x_dtype; a.W = W; a.w_dtype = w_dtype; a.scores = scores_buf; a.bias = bias;
    a.logit_offset = logit_offset;
    a.out_ids = out_ids; a.out_weights = out_weights; a.counter = workspace; a.H = hidden_dim; a.E = num_experts;
    a.top_k = top_k; a.mode = scoring_mode; a.scaling = scaling_factor; a.normalize = normalize; a.exact_order = exact_order;
    if (int e = check_router(a)) return e;
    if (int e = check_topk(a)) return e;
    if (!workspace) return VIB3_ERR_NULL;
    if (x_dtype < X_F32 || x_dtype > X_BF16 || (w_dtype != W_F16 && w_dtype != W_F32)) return VIB3_ERR_UNSUPPORTED;
    return launch_router(a, (cudaStream_t)stream);
}
