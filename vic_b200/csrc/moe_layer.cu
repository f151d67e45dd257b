// Batch-1 MoE sublayer over buffer-manager pages: two launches for the whole layer.
//
//   gate/up kernel : for every selected expert (plus the shared expert) and every row of its
//                    gate and up matrices: act = f16( silu(f16(Wg x)) * f16(Wu x) )
//   down kernel    : out[r] = sum over experts, in plan order, of w_e * f16(Wd_e[r,:] . act_e)
//
// This replaces the reference's per-page launch sequence for INT4 experts
// (src/runtime/engine.rs:6094-6107, :6215-6223, :6290-6296; src/compute/kernels.rs:493-541):
// about 150 launches per layer there, 2 here, with the same rounding points (fp16 after each
// projection and after the SiLU product, fp32 accumulation across experts).
//
// Pages are addressed through a device page table: entry [expert][segment][page] holds the
// page's device pointer and row range (segment 0 = up, 1 = gate, 2 = down,
// src/core/types.rs:204).  The experts of the token are read from device memory (router
// output), so no host synchronisation sits between the router and the experts.
#include "moe_common.cuh"
#include "router_core.cuh"

#include <cstring>
#include <new>

namespace vib3 {

// ── gate/up + SiLU ─────────────────────────────────────────────────────────────────────────
// One warp per (slot, row).  Lane l takes chunks l, l+32, ... of the row: one 16-byte load of
// codes and one 2-byte scale per chunk for gate and for up; B chunks per lane are requested
// before any is consumed.
template <class MATH, int B>
__global__ void __launch_bounds__(256, 2) moe_gateup_kernel(MoeLayerArgs a) {
    a.top_k = active_top_k(a);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    typename MATH::XS* xs = reinterpret_cast<typename MATH::XS*>(smem_raw);
    const int nchunks = a.H / kGroupSize;
    PageEntry* tab = reinterpret_cast<PageEntry*>(smem_raw + (size_t)nchunks * MATH::kStride * sizeof(typename MATH::XS));
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);

    // page entries of gate and up for every slot: tab[(s*2 + seg)*P + p], seg 0 = up, 1 = gate
    for (int i = threadIdx.x; i < slots * 2 * a.P; i += blockDim.x) {
        const int s = i / (2 * a.P), rem = i % (2 * a.P);
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[rem];  // segments 0 and 1 are the first 2*P entries
        else if (rem == 0) flag(a.status, kStatusBadExpert);
        tab[i] = e;
    }
    stage_activation<MATH>(xs, a.x, a.x_dtype, a.H, threadIdx.x, blockDim.x);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int total_rows = slots * a.I;
    const size_t code_row_bytes = (size_t)a.H / 2;
    const int scale_row = nchunks;  // u16 per row

    for (int g = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); g < total_rows; g += gridDim.x * warps_per_cta) {
        const int s = g / a.I, row = g - s * a.I;
        const int p = row / a.rpp_gu, rin = row - p * a.rpp_gu;
        const PageEntry eu = tab[(s * 2 + kSegUp) * a.P + p];
        const PageEntry eg = tab[(s * 2 + kSegGate) * a.P + p];
        float acc[2] = {0.f, 0.f};  // [0] gate, [1] up
        if (eu.ptr != 0 && eg.ptr != 0 && rin < eu.row_count && rin < eg.row_count) {
            const unsigned char* gbase = reinterpret_cast<const unsigned char*>(eg.ptr);
            const unsigned char* ubase = reinterpret_cast<const unsigned char*>(eu.ptr);
            const uint4* gcodes = reinterpret_cast<const uint4*>(gbase + (size_t)rin * code_row_bytes);
            const uint4* ucodes = reinterpret_cast<const uint4*>(ubase + (size_t)rin * code_row_bytes);
            const unsigned short* gsc = reinterpret_cast<const unsigned short*>(gbase + (size_t)eg.row_count * code_row_bytes) + (size_t)rin * scale_row;
            const unsigned short* usc = reinterpret_cast<const unsigned short*>(ubase + (size_t)eu.row_count * code_row_bytes) + (size_t)rin * scale_row;
            for (int c0 = lane; c0 < nchunks; c0 += 32 * B) {
                uint4 q[B][2];
                unsigned short sc[B][2];
#pragma unroll
                for (int i = 0; i < B; ++i) {
                    const int c = c0 + 32 * i;
                    if (c < nchunks) {
                        q[i][0] = ldg_stream16(gcodes + c);
                        q[i][1] = ldg_stream16(ucodes + c);
                        sc[i][0] = ldg_stream2(gsc + c);
                        sc[i][1] = ldg_stream2(usc + c);
                    } else {
                        q[i][0] = q[i][1] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
                        sc[i][0] = sc[i][1] = 0;
                    }
                }
#pragma unroll
                for (int i = 0; i < B; ++i) {
                    const int c = min(c0 + 32 * i, nchunks - 1);
                    const float s2[2] = {scale_to_f32(sc[i][0]), scale_to_f32(sc[i][1])};
                    MATH::template chunk<2>(q[i], s2, xs + (size_t)c * MATH::kStride, acc);
                }
            }
        } else if (lane == 0) {
            flag(a.status, kStatusMissingPage);
        }
        const float gsum = warp_sum(acc[0]);
        const float usum = warp_sum(acc[1]);
        if (lane == 0) {
            // the reference rounds each projection to fp16 before silu_mul, and its result again
            const float g16 = __half2float(__float2half_rn(gsum));
            const float u16 = __half2float(__float2half_rn(usum));
            a.act[(size_t)act_slot(a, s) * a.I + row] = __float2half_rn(silu_mul_f32(g16, u16));
        }
    }
}

// ── down + routing weight + accumulate ─────────────────────────────────────────────────────
// One warp per output row r, all slots: y_s = f16(Wd_s[r,:] . act_s), out[r] = sum_s w_s * y_s
// accumulated in plan order, so the result does not depend on scheduling.
template <int B, int SB>
__global__ void __launch_bounds__(384, 1) moe_down_kernel(MoeLayerArgs a) {
    a.top_k = active_top_k(a);
    using MATH = MathQ16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int nchunks = a.I / kGroupSize;
    MATH::XS* acts = reinterpret_cast<MATH::XS*>(smem_raw);  // [slots][nchunks * kStride]
    PageEntry* tab = reinterpret_cast<PageEntry*>(smem_raw + (size_t)slots * nchunks * MATH::kStride * sizeof(MATH::XS));
    float* wts = reinterpret_cast<float*>(tab + slots * a.P);

    for (int i = threadIdx.x; i < slots * a.P; i += blockDim.x) {
        const int s = i / a.P, p = i - s * a.P;
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[kSegDown * a.P + p];
        tab[i] = e;
    }
    for (int s = threadIdx.x; s < slots; s += blockDim.x) wts[s] = s < a.top_k ? a.expert_weights[s] : a.shared_weight;
    // act is [slots][I] and the staged layout is [slots][chunks]: one vector of slots * I values,
    // both in act_slot() order
    stage_activation<MATH>(acts, a.act, X_F16, slots * a.I, threadIdx.x, blockDim.x);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const size_t code_row_bytes = (size_t)a.I / 2;
    const uint4 kZeroCodes = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);

    for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < a.H; r += gridDim.x * warps_per_cta) {
        const int p = r / a.rpp_dn, rin = r - p * a.rpp_dn;
        float out = 0.f;
        for (int s0 = 0; s0 < slots; s0 += SB) {
            // SB slots at a time: SB*B independent 16-byte loads per lane are requested before use
            const uint4* codes[SB];
            const unsigned short* sc[SB];
            float acc[SB];
#pragma unroll
            for (int ss = 0; ss < SB; ++ss) {
                acc[ss] = 0.f;
                codes[ss] = nullptr;
                sc[ss] = nullptr;
                if (s0 + ss < slots) {
                    const PageEntry e = tab[(s0 + ss) * a.P + p];
                    if (e.ptr != 0 && rin < e.row_count) {
                        const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                        codes[ss] = reinterpret_cast<const uint4*>(base + (size_t)rin * code_row_bytes);
                        sc[ss] = reinterpret_cast<const unsigned short*>(base + (size_t)e.row_count * code_row_bytes) + (size_t)rin * nchunks;
                    } else if (lane == 0) {
                        flag(a.status, kStatusMissingPage);
                    }
                }
            }
            for (int c0 = lane; c0 < nchunks; c0 += 32 * B) {
                uint4 q[SB][B];
                unsigned short sb[SB][B];
#pragma unroll
                for (int ss = 0; ss < SB; ++ss) {
#pragma unroll
                    for (int i = 0; i < B; ++i) {
                        const int c = c0 + 32 * i;
                        if (codes[ss] != nullptr && c < nchunks) {
                            q[ss][i] = ldg_stream16(codes[ss] + c);
                            sb[ss][i] = ldg_stream2(sc[ss] + c);
                        } else {
                            q[ss][i] = kZeroCodes;
                            sb[ss][i] = 0;
                        }
                    }
                }
#pragma unroll
                for (int ss = 0; ss < SB; ++ss) {
                    const MATH::XS* xs = acts + (size_t)act_slot(a, min(s0 + ss, slots - 1)) * nchunks * MATH::kStride;
#pragma unroll
                    for (int i = 0; i < B; ++i) {
                        const int c = min(c0 + 32 * i, nchunks - 1);
                        const uint4 q1[1] = {q[ss][i]};
                        const float s1[1] = {scale_to_f32(sb[ss][i])};
                        float a1[1] = {acc[ss]};
                        MATH::template chunk<1>(q1, s1, xs + (size_t)c * MATH::kStride, a1);
                        acc[ss] = a1[0];
                    }
                }
            }
#pragma unroll
            for (int ss = 0; ss < SB; ++ss) {
                const float y = warp_sum(acc[ss]);
                // fp16 rounding of the down projection, then out += w * y (cuda/src/kernels.cu:803-813)
                if (s0 + ss < slots) out = fmaf(wts[s0 + ss], __half2float(__float2half_rn(y)), out);
            }
        }
        if (lane == 0) {
            if (a.out_accumulate) a.out[r] += out;
            else a.out[r] = out;
        }
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────────

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

std::atomic<int> g_use_pipeline{1};
std::atomic<int> g_use_pdl{1};
// 1 = vib3_launch_moe_layer_routed_int4_paged lets the gate/up kernel route the token in its prologue where the
// shapes allow; 0 (default: measured 2 us per layer-token faster on the Kimi shape) = the router is a launch of its own.
std::atomic<int> g_route_in_kernel{0};

template <class K>
static int ensure_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

template <class MATH, int B>
static int launch_gateup(const MoeLayerArgs& a, cudaStream_t st) {
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t smem = (size_t)(a.H / kGroupSize) * MATH::kStride * sizeof(typename MATH::XS) + (size_t)slots * 2 * a.P * sizeof(PageEntry);
    if (int e = ensure_smem(moe_gateup_kernel<MATH, B>, smem)) return e;
    const int total_rows = slots * a.I;
    int grid = min(2 * sm_count(), (total_rows + 7) / 8);
    moe_gateup_kernel<MATH, B><<<grid, 256, smem, st>>>(a);
    return (int)cudaGetLastError();
}

template <int B, int SB>
static int launch_down(const MoeLayerArgs& a, cudaStream_t st) {
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t smem = (size_t)slots * (a.I / kGroupSize) * MathQ16::kStride + (size_t)slots * a.P * sizeof(PageEntry) + slots * sizeof(float);
    if (int e = ensure_smem(moe_down_kernel<B, SB>, smem)) return e;
    int grid = min(sm_count(), (a.H + 11) / 12);
    moe_down_kernel<B, SB><<<grid, 384, smem, st>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace vib3

namespace vib3 {
int make_router_args(const void* x, int x_dtype, const void* W, int w_dtype, float* scores_buf, const float* bias,
                     const float* logit_offset, unsigned short* out_ids, float* out_weights, int hidden_dim, int num_experts,
                     int top_k, int scoring_mode, float scaling_factor, int normalize, int exact_order,
                     unsigned int* workspace, RouterArgs& a);  // router.cu
int launch_router_args(const RouterArgs& a, cudaStream_t st);  // router.cu
}  // namespace vib3

using namespace vib3;

static int moe_layer_dispatch(int phases, const int* num_active_dev, const RouterArgs* router, const void* x, int x_dtype, const void* page_table, int num_experts,
                              const void* shared_pages, const unsigned short* expert_ids, const float* expert_weights,
                              int top_k, float shared_weight, void* act_scratch, float* out, int out_accumulate,
                              int hidden_dim, int expert_hidden_dim, int pages_per_segment, int rows_per_page_gate_up,
                              int rows_per_page_down, int group_size, int* status, void* stream) {
    if (!x || !page_table || !expert_ids || !expert_weights || !act_scratch || !out) return VIB3_ERR_NULL;
    if (group_size != kGroupSize) return VIB3_ERR_UNSUPPORTED;
    if (x_dtype < X_F32 || x_dtype > X_BF16) return VIB3_ERR_UNSUPPORTED;
    if (hidden_dim <= 0 || expert_hidden_dim <= 0 || hidden_dim % kGroupSize || expert_hidden_dim % kGroupSize) return VIB3_ERR_SHAPE;
    if (top_k < 0 || top_k > kMaxSlots - 1 || num_experts <= 0) return VIB3_ERR_COUNT;
    if (top_k + (shared_pages ? 1 : 0) == 0) return VIB3_ERR_COUNT;
    if (pages_per_segment <= 0 || pages_per_segment > kMaxPages) return VIB3_ERR_COUNT;
    if (rows_per_page_gate_up <= 0 || rows_per_page_down <= 0) return VIB3_ERR_SHAPE;
    if ((long long)rows_per_page_gate_up * pages_per_segment < expert_hidden_dim) return VIB3_ERR_SHAPE;
    if ((long long)rows_per_page_down * pages_per_segment < hidden_dim) return VIB3_ERR_SHAPE;
    if (((uintptr_t)x & 15) || ((uintptr_t)page_table & 15) || ((uintptr_t)shared_pages & 15) ||
        ((uintptr_t)act_scratch & 15) || ((uintptr_t)out & 3)) return VIB3_ERR_ALIGN;

    MoeLayerArgs a;
    a.x = x; a.x_dtype = x_dtype;
    a.page_table = (const PageEntry*)page_table; a.shared_pages = (const PageEntry*)shared_pages;
    a.expert_ids = expert_ids; a.expert_weights = expert_weights; a.top_k = top_k; a.num_experts = num_experts;
    a.num_active_dev = num_active_dev;
    a.shared_weight = shared_weight; a.act = (__half*)act_scratch; a.out = out; a.out_accumulate = out_accumulate;
    a.H = hidden_dim; a.I = expert_hidden_dim; a.P = pages_per_segment;
    a.rpp_gu = rows_per_page_gate_up; a.rpp_dn = rows_per_page_down; a.status = status;
    a.slot_token = nullptr; a.n_tokens = 1; a.shared_token = 0; a.x_stride = 0; a.out_stride = 0; a.slot_begin = 0;
    cudaStream_t st = (cudaStream_t)stream;

    const bool use_pipe = g_use_pipeline.load(std::memory_order_relaxed) != 0;
    int err = 0;
    if (router) {
        // the gate/up kernel routes the token itself where the shapes allow; otherwise the router is a launch of its own
        err = ((phases & 1) && use_pipe && g_route_in_kernel.load(std::memory_order_relaxed)) ? launch_gateup_pipelined(a, st, router)
                                                                                               : VIB3_ERR_UNSUPPORTED;
        if (err == 0) phases &= ~1;
        else if (err != VIB3_ERR_UNSUPPORTED) return err;
        else if ((err = launch_router_args(*router, st)) != 0) return err;
    }
    if ((phases & 1) && use_pipe) {
        err = launch_gateup_pipelined(a, st);
        if (err == 0) phases &= ~1;
        else if (err != VIB3_ERR_UNSUPPORTED) return err;
    }
    if ((phases & 2) && !(phases & 1) && use_pipe) {
        err = launch_down_pipelined(a, st);
        if (err == 0) phases &= ~2;
        else if (err != VIB3_ERR_UNSUPPORTED) return err;
    }
    err = 0;
    if (phases & 1) {
        const int lane_chunks_gu = (hidden_dim / kGroupSize + 31) / 32;
        err = lane_chunks_gu % 7 == 0 ? launch_gateup<MathQ16, 7>(a, st)
            : lane_chunks_gu % 4 == 0 ? launch_gateup<MathQ16, 4>(a, st)
            : lane_chunks_gu % 2 == 0 ? launch_gateup<MathQ16, 2>(a, st) : launch_gateup<MathQ16, 1>(a, st);
        if (err) return err;
    }
    if (phases & 2) {
        const int lane_chunks_dn = (expert_hidden_dim / kGroupSize + 31) / 32;
        err = lane_chunks_dn % 7 == 0 ? launch_down<7, 2>(a, st)
            : lane_chunks_dn % 4 == 0 ? launch_down<4, 4>(a, st)
            : lane_chunks_dn % 2 == 0 ? launch_down<2, 9>(a, st) : launch_down<1, 9>(a, st);
    }
    return err;
}

#define VIB3_MOE_ARGS                                                                                               \
    const void *x, int x_dtype, const void *page_table, int num_experts, const void *shared_pages,                   \
        const unsigned short *expert_ids, const float *expert_weights, int top_k, float shared_weight,              \
        void *act_scratch, float *out, int out_accumulate, int hidden_dim, int expert_hidden_dim,                   \
        int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down, int group_size, int *status,      \
        void *stream
#define VIB3_MOE_PASS                                                                                               \
    x, x_dtype, page_table, num_experts, shared_pages, expert_ids, expert_weights, top_k, shared_weight, act_scratch, \
        out, out_accumulate, hidden_dim, expert_hidden_dim, pages_per_segment, rows_per_page_gate_up,               \
        rows_per_page_down, group_size, status, stream

// key 0: staged (bulk-copy) kernels on/off; key 1: programmatic dependent launch of the staged
// kernels on/off; key 2: routing inside the gate/up kernel on/off.  Atomic exchanges: safe against concurrent launches from other threads (a launch
// sees the old or the new value).  Returns the previous value, or VIB3_ERR_UNSUPPORTED.
extern "C" int vib3_config_set(int key, int value) {
    if (key == 0) return g_use_pipeline.exchange(value ? 1 : 0);
    if (key == 1) return g_use_pdl.exchange(value ? 1 : 0);
    if (key == 2) return g_route_in_kernel.exchange(value ? 1 : 0);
    return VIB3_ERR_UNSUPPORTED;
}

extern "C" int vib3_launch_moe_layer_int4_paged(VIB3_MOE_ARGS) { return moe_layer_dispatch(3, nullptr, nullptr, VIB3_MOE_PASS); }
extern "C" int vib3_launch_moe_gate_up_int4_paged(VIB3_MOE_ARGS) { return moe_layer_dispatch(1, nullptr, nullptr, VIB3_MOE_PASS); }
extern "C" int vib3_launch_moe_down_int4_paged(VIB3_MOE_ARGS) { return moe_layer_dispatch(2, nullptr, nullptr, VIB3_MOE_PASS); }
// Same as vib3_launch_moe_layer_int4_paged, but only the first min(top_k, *num_active_dev) routed slots
// are used (a device-side count, e.g. the experts of a token that are resident on this GPU).
extern "C" int vib3_launch_moe_layer_int4_paged_var(VIB3_MOE_ARGS, const int* num_active_dev) {
    if (!num_active_dev) return VIB3_ERR_NULL;
    return moe_layer_dispatch(3, num_active_dev, nullptr, VIB3_MOE_PASS);
}

// Router and experts of one token: the routing (ids, weights; device) is an OUTPUT.  Where the shapes allow,
// the gate/up kernel routes the token in its own prologue (two launches for the layer); otherwise the router
// is launched first (three).  workspace: four 32-bit words, zero before the first call and left zero at
// [0] and [2]; calls that share one must not overlap on the GPU.  scores_buf: 3 * num_experts floats.
extern "C" int vib3_launch_moe_layer_routed_int4_paged(
    const void* x, int x_dtype, const void* router_w, int w_dtype, float* scores_buf, const float* bias,
    const float* logit_offset, unsigned short* ids_out, float* weights_out, int num_experts, int top_k, int scoring_mode,
    float scaling_factor, int normalize, int exact_order, unsigned int* workspace, const void* page_table,
    const void* shared_pages, float shared_weight, void* act_scratch, float* out, int out_accumulate, int hidden_dim,
    int expert_hidden_dim, int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down, int group_size,
    int* status, void* stream) {
    RouterArgs r;
    if (int e = make_router_args(x, x_dtype, router_w, w_dtype, scores_buf, bias, logit_offset, ids_out, weights_out, hidden_dim,
                                 num_experts, top_k, scoring_mode, scaling_factor, normalize, exact_order, workspace, r)) return e;
    return moe_layer_dispatch(3, nullptr, &r, x, x_dtype, page_table, num_experts, shared_pages, ids_out, weights_out, top_k,
                              shared_weight, act_scratch, out, out_accumulate, hidden_dim, expert_hidden_dim, pages_per_segment,
                              rows_per_page_gate_up, rows_per_page_down, group_size, status, stream);
}

// One token through one MoE sublayer FROM AND TO HOST MEMORY: copies the token to the device, launches
// the router and the two expert kernels, and waits for the stream.  The only entry point of this library
// that copies or synchronises.  x_host: hidden_dim values of x_dtype in ordinary or pinned host memory.
// The result goes to out_host: if out_dev is null, out_host must be device-addressable (pinned) memory
// and the last kernel stores into it directly; otherwise the kernels write out_dev and a copy follows.
// All other arguments as for vib3_launch_router_topk_ex and vib3_launch_moe_layer_int4_paged.
extern "C" int vib3_moe_layer_step_host(const void* x_host, int x_dtype, void* x_dev, const void* router_w, int w_dtype,
                                        float* scores_buf, const float* bias, unsigned short* ids_dev, float* weights_dev,
                                        int num_experts, int top_k, int scoring_mode, float scaling_factor, int normalize,
                                        int exact_order, unsigned int* workspace, const void* page_table,
                                        const void* shared_pages, float shared_weight, void* act_scratch, float* out_dev,
                                        float* out_host, int hidden_dim, int expert_hidden_dim, int pages_per_segment,
                                        int rows_per_page_gate_up, int rows_per_page_down, int group_size, int* status,
                                        void* stream) {
    if (!x_host || !x_dev || !out_host) return VIB3_ERR_NULL;
    if (x_dtype < X_F32 || x_dtype > X_BF16 || hidden_dim <= 0) return VIB3_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t xbytes = (size_t)hidden_dim * (x_dtype == X_F32 ? 4 : 2);
    cudaError_t ce = cudaMemcpyAsync(x_dev, x_host, xbytes, cudaMemcpyHostToDevice, st);
    if (ce != cudaSuccess) return (int)ce;
    float* out = out_dev ? out_dev : out_host;
    int err = vib3_launch_moe_layer_routed_int4_paged(x_dev, x_dtype, router_w, w_dtype, scores_buf, bias, nullptr, ids_dev, weights_dev,
                                                      num_experts, top_k, scoring_mode, scaling_factor, normalize, exact_order, workspace,
                                                      page_table, shared_pages, shared_weight, act_scratch, out, 0, hidden_dim,
                                                      expert_hidden_dim, pages_per_segment, rows_per_page_gate_up, rows_per_page_down,
                                                      group_size, status, stream);
    if (err) return err;
    if (out_dev) {
        ce = cudaMemcpyAsync(out_host, out_dev, (size_t)hidden_dim * sizeof(float), cudaMemcpyDeviceToHost, st);
        if (ce != cudaSuccess) return (int)ce;
    }
    ce = cudaStreamSynchronize(st);
    return ce == cudaSuccess ? 0 : (int)ce;
}

// ── One token from and to host memory as ONE graph launch ──────────────────────────────────────
// vib3_moe_layer_step_host costs the host a copy, three launches and a synchronisation per token.  A caller
// that decodes many tokens through the same layer binds the layer once: vib3_moe_step_create records the copy of
// the token from a pinned staging buffer, the router and the two expert kernels (the last one storing the fp32
// output straight into the caller's pinned buffer) into a CUDA graph, after one eager run that also takes care
// of one-time kernel attributes; vib3_moe_step_run then copies the token into the staging buffer (host to host),
// launches the graph and waits for the stream.  Create allocates (pinned staging memory, the graph): call it at
// start-up and outside any stream capture, like vib3_moe_prewarm_gpu_bufs (cuda/src/kernels.cu:6507).
namespace {
struct StepHandle {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    void* x_pin = nullptr;
    size_t xbytes = 0;
};
}  // namespace

extern "C" void vib3_moe_step_destroy(void* handle) {
    StepHandle* h = static_cast<StepHandle*>(handle);
    if (!h) return;
    if (h->exec) cudaGraphExecDestroy(h->exec);
    if (h->graph) cudaGraphDestroy(h->graph);
    if (h->x_pin) cudaFreeHost(h->x_pin);
    delete h;
}

extern "C" int vib3_moe_step_create(int x_dtype, void* x_dev, const void* router_w, int w_dtype, float* scores_buf, const float* bias,
                                    unsigned short* ids_dev, float* weights_dev, int num_experts, int top_k, int scoring_mode,
                                    float scaling_factor, int normalize, int exact_order, unsigned int* workspace,
                                    const void* page_table, const void* shared_pages, float shared_weight, void* act_scratch,
                                    float* out_host_pinned, int hidden_dim, int expert_hidden_dim, int pages_per_segment,
                                    int rows_per_page_gate_up, int rows_per_page_down, int group_size, int* status, void* stream,
                                    void** handle_out) {
    if (!x_dev || !out_host_pinned || !handle_out) return VIB3_ERR_NULL;
    if (x_dtype < X_F32 || x_dtype > X_BF16 || hidden_dim <= 0) return VIB3_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (!st) return VIB3_ERR_UNSUPPORTED;   // the legacy default stream cannot be captured
    StepHandle* h = new (std::nothrow) StepHandle();
    if (!h) return VIB3_ERR_STATE;
    h->xbytes = (size_t)hidden_dim * (x_dtype == X_F32 ? 4 : 2);
    cudaError_t ce = cudaHostAlloc(&h->x_pin, h->xbytes, cudaHostAllocDefault);
    if (ce != cudaSuccess) {
        delete h;
        return (int)ce;
    }
    memset(h->x_pin, 0, h->xbytes);
    auto body = [&]() -> int {
        cudaError_t e = cudaMemcpyAsync(x_dev, h->x_pin, h->xbytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return (int)e;
        return vib3_launch_moe_layer_routed_int4_paged(x_dev, x_dtype, router_w, w_dtype, scores_buf, bias, nullptr, ids_dev, weights_dev,
                                                       num_experts, top_k, scoring_mode, scaling_factor, normalize, exact_order, workspace,
                                                       page_table, shared_pages, shared_weight, act_scratch, out_host_pinned, 0,
                                                       hidden_dim, expert_hidden_dim, pages_per_segment, rows_per_page_gate_up,
                                                       rows_per_page_down, group_size, status, stream);
    };
    int err = body();   // eager: validates the arguments, sets one-time kernel attributes
    if (!err && (ce = cudaStreamSynchronize(st)) != cudaSuccess) err = (int)ce;
    if (!err && (ce = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal)) != cudaSuccess) err = (int)ce;
    if (!err) {
        err = body();
        ce = cudaStreamEndCapture(st, &h->graph);
        if (!err && ce != cudaSuccess) err = (int)ce;
    }
    if (!err && (ce = cudaGraphInstantiate(&h->exec, h->graph, 0)) != cudaSuccess) err = (int)ce;
    if (err) {
        vib3_moe_step_destroy(h);
        return err;
    }
    *handle_out = h;
    return VIB3_OK;
}

extern "C" int vib3_moe_step_run(void* handle, const void* x_host, void* stream) {
    StepHandle* h = static_cast<StepHandle*>(handle);
    if (!h || !x_host) return VIB3_ERR_NULL;
    memcpy(h->x_pin, x_host, h->xbytes);
    cudaError_t ce = cudaGraphLaunch(h->exec, (cudaStream_t)stream);
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaStreamSynchronize((cudaStream_t)stream);
    return ce == cudaSuccess ? 0 : (int)ce;
}

// Grouped form for expert parallelism: the routed slots are (token, expert) pairs of several tokens in
// ascending token order (vib3_launch_select_local_pairs makes such a list); x has n_tokens rows
// x_stride_bytes apart, out has n_tokens rows out_stride floats apart.  This launch takes the pairs
// [pair_begin, pair_begin + pair_capacity) of the list whose length is *num_pairs_dev; the pointers
// pair_experts / pair_weights / pair_tokens are the START of the lists.  The shared expert (if given)
// belongs to token shared_token.  Staged kernels only: VIB3_ERR_UNSUPPORTED for other shapes.
extern "C" int vib3_launch_moe_layer_int4_paged_grouped(
    const void* x, int x_dtype, int x_stride_bytes, int n_tokens, const void* page_table, int num_experts,
    const void* shared_pages, int shared_token, const unsigned short* pair_experts, const float* pair_weights,
    const unsigned short* pair_tokens, int pair_capacity, int pair_begin, const int* num_pairs_dev, float shared_weight,
    void* act_scratch, float* out, int out_stride, int out_accumulate, int hidden_dim, int expert_hidden_dim,
    int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down, int group_size, int* status, void* stream) {
    if (!x || !page_table || !pair_experts || !pair_weights || !pair_tokens || !num_pairs_dev || !act_scratch || !out) return VIB3_ERR_NULL;
    if (group_size != kGroupSize) return VIB3_ERR_UNSUPPORTED;
    if (x_dtype < X_F32 || x_dtype > X_BF16) return VIB3_ERR_UNSUPPORTED;
    if (hidden_dim <= 0 || expert_hidden_dim <= 0 || hidden_dim % kGroupSize || expert_hidden_dim % kGroupSize) return VIB3_ERR_SHAPE;
    if (pair_capacity <= 0 || pair_capacity > kMaxSlots - 1 || pair_begin < 0 || num_experts <= 0) return VIB3_ERR_COUNT;
    if (n_tokens <= 0 || n_tokens > 65535 || shared_token < 0 || shared_token >= n_tokens) return VIB3_ERR_COUNT;
    if (pages_per_segment <= 0 || pages_per_segment > kMaxPages) return VIB3_ERR_COUNT;
    if (rows_per_page_gate_up <= 0 || rows_per_page_down <= 0) return VIB3_ERR_SHAPE;
    if ((long long)rows_per_page_gate_up * pages_per_segment < expert_hidden_dim) return VIB3_ERR_SHAPE;
    if ((long long)rows_per_page_down * pages_per_segment < hidden_dim) return VIB3_ERR_SHAPE;
    if (out_stride < hidden_dim || x_stride_bytes <= 0) return VIB3_ERR_SHAPE;
    if (((uintptr_t)x & 15) || (x_stride_bytes & 15) || ((uintptr_t)page_table & 15) || ((uintptr_t)shared_pages & 15) ||
        ((uintptr_t)act_scratch & 15) || ((uintptr_t)out & 3)) return VIB3_ERR_ALIGN;
    if (!g_use_pipeline.load(std::memory_order_relaxed)) return VIB3_ERR_UNSUPPORTED;

    MoeLayerArgs a;
    a.x = x; a.x_dtype = x_dtype;
    a.page_table = (const PageEntry*)page_table; a.shared_pages = (const PageEntry*)shared_pages;
    a.expert_ids = pair_experts + pair_begin; a.expert_weights = pair_weights + pair_begin;
    a.top_k = pair_capacity; a.num_experts = num_experts; a.num_active_dev = num_pairs_dev;
    a.shared_weight = shared_weight; a.act = (__half*)act_scratch; a.out = out; a.out_accumulate = out_accumulate;
    a.H = hidden_dim; a.I = expert_hidden_dim; a.P = pages_per_segment;
    a.rpp_gu = rows_per_page_gate_up; a.rpp_dn = rows_per_page_down; a.status = status;
    a.slot_token = pair_tokens + pair_begin; a.n_tokens = n_tokens; a.shared_token = shared_token;
    a.x_stride = x_stride_bytes; a.out_stride = out_stride; a.slot_begin = pair_begin;
    cudaStream_t st = (cudaStream_t)stream;
    int err = launch_gateup_pipelined(a, st);
    if (err) return err;
    return launch_down_pipelined(a, st);
}

// The (token, expert, weight) triples, in token-major order, whose expert lies in [expert_lo, expert_hi):
// the pairs of a step that an expert-parallel rank owns.  ids / weights: n_tokens rows of top_k entries,
// row strides in bytes.  The lists have room for `capacity` entries (n_tokens * top_k suffices);
// *count_out receives the number of pairs found, even if it exceeds the capacity.
__global__ void select_local_pairs_kernel(const unsigned char* ids, int ids_stride, const unsigned char* w, int w_stride,
                                          int n_tokens, int top_k, int lo, int hi, unsigned short* pe, float* pw,
                                          unsigned short* pt, int capacity, int* count_out) {
    select_local_pairs_warp(ids, ids_stride, w, w_stride, n_tokens, top_k, lo, hi, pe, pw, pt, capacity, count_out);
}

extern "C" int vib3_launch_select_local_pairs(const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                              int weights_stride_bytes, int n_tokens, int top_k, int expert_lo,
                                              int expert_hi, unsigned short* pair_experts, float* pair_weights,
                                              unsigned short* pair_tokens, int capacity, int* count_out, void* stream) {
    if (!ids || !weights || !pair_experts || !pair_weights || !pair_tokens || !count_out) return VIB3_ERR_NULL;
    if (n_tokens <= 0 || n_tokens > 65535 || top_k <= 0 || top_k > kMaxSlots - 1 || capacity <= 0 || expert_lo < 0 ||
        expert_hi < expert_lo) return VIB3_ERR_COUNT;
    if ((ids_stride_bytes & 1) || (weights_stride_bytes & 3)) return VIB3_ERR_ALIGN;
    select_local_pairs_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const unsigned char*>(ids), ids_stride_bytes, reinterpret_cast<const unsigned char*>(weights),
        weights_stride_bytes, n_tokens, top_k, expert_lo, expert_hi, pair_experts, pair_weights, pair_tokens, capacity, count_out);
    return (int)cudaGetLastError();
}

// out[c] = in[0][c] + in[1][c] + ... in row order (fp32): the last step of an expert-parallel layer when
// every rank has received the other ranks' partial sums for its token.
__global__ void sum_rows_kernel(const float* in, int rows, int cols, int row_stride, float* out) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c + 3 < cols) {
        float4 acc = *reinterpret_cast<const float4*>(in + c);
        for (int r = 1; r < rows; ++r) {
            const float4 v = *reinterpret_cast<const float4*>(in + (size_t)r * row_stride + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + c) = acc;
    } else {
        for (int k = c; k < cols; ++k) {
            float acc = in[k];
            for (int r = 1; r < rows; ++r) acc += in[(size_t)r * row_stride + k];
            out[k] = acc;
        }
    }
}

extern "C" int vib3_launch_sum_rows_f32(const float* in, int rows, int cols, int row_stride, float* out, void* stream) {
    if (!in || !out) return VIB3_ERR_NULL;
    if (rows <= 0 || cols <= 0 || row_stride < cols) return VIB3_ERR_SHAPE;
    if (((uintptr_t)in & 15) || ((uintptr_t)out & 15) || (row_stride & 3)) return VIB3_ERR_ALIGN;
    const int threads = 128, per_block = threads * 4;
    sum_rows_kernel<<<(cols + per_block - 1) / per_block, threads, 0, (cudaStream_t)stream>>>(in, rows, cols, row_stride, out);
    return (int)cudaGetLastError();
}

// Keep, in order, the (expert, weight) pairs whose expert lies in [expert_lo, expert_hi): the slots of
// a token that an expert-parallel rank owns.  ids_out/weights_out have room for top_k entries; the
// rest is filled with expert_lo / 0; *count_out receives the number kept.
__global__ void select_local_experts_kernel(const unsigned short* ids, const float* w, int top_k, int lo, int hi,
                                            unsigned short* ids_out, float* w_out, int* count_out) {
    if (threadIdx.x != 0) return;
    int n = 0;
    for (int i = 0; i < top_k; ++i) {
        const int e = ids[i];
        if (e >= lo && e < hi) {
            ids_out[n] = (unsigned short)e;
            w_out[n] = w[i];
            ++n;
        }
    }
    *count_out = n;
    for (int i = n; i < top_k; ++i) {
        ids_out[i] = (unsigned short)lo;
        w_out[i] = 0.f;
    }
}

extern "C" int vib3_launch_select_local_experts(const unsigned short* ids, const float* weights, int top_k,
                                                int expert_lo, int expert_hi, unsigned short* ids_out,
                                                float* weights_out, int* count_out, void* stream) {
    if (!ids || !weights || !ids_out || !weights_out || !count_out) return VIB3_ERR_NULL;
    if (top_k <= 0 || top_k > kMaxSlots - 1 || expert_lo < 0 || expert_hi < expert_lo) return VIB3_ERR_COUNT;
    select_local_experts_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ids, weights, top_k, expert_lo, expert_hi, ids_out,
                                                                   weights_out, count_out);
    return (int)cudaGetLastError();
}
