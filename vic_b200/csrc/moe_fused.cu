// The whole expert part of a batch-1 MoE sublayer in ONE persistent kernel: gate/up + SiLU, a grid
// barrier, down + routing weight + accumulate.
//
// Why: the two-kernel version pays a second prologue (page-table lookup, activation quantisation,
// an empty copy ring) and a launch boundary between the phases — about 6 us of a 50 us layer.  Here
// the producer warp runs straight from the last gate/up tiles into the first down tiles (the down
// weights depend only on the routing, not on the gate/up results), so HBM stays busy across the
// phase change; the consumers only wait at the grid barrier for the other CTAs' activations.
//
// Shape of the kernel: one CTA per SM, cooperative launch (all CTAs resident, which the grid barrier
// needs), 19 warps: warp 18 produces, warps 0..15 consume gate/up tiles exactly as
// moe_gateup_pipe_kernel does (8 groups of 2 warps, 4 rows per warp sharing each activation load),
// warps 0..2*slots-1 consume down tiles exactly as moe_down_pipe_kernel does (two warps per expert slot,
// activations in registers).  Shared memory holds two rings: 3 gate/up stages and 2 down stages.
// The arithmetic is the same code as in the two-kernel version: identical bits.
//
// The grid barrier is a counter pair in global memory (caller-provided, zero before first use, left
// zero by every launch): arrive with release, poll with acquire under an iteration limit, and the
// last CTA to leave resets both counters.  A CTA that gives up sets VIB3_STATUS_TIMEOUT and returns.
#include "pipe_common.cuh"

namespace vib3 {

constexpr int kFusedConsumerWarps = 18;
constexpr int kFusedThreads = (kFusedConsumerWarps + 1) * 32;  // 608
constexpr int kFusedGStages = 3;
constexpr int kFusedDStages = 2;
constexpr int kFDownRows = 4;
constexpr int kFDownWarpsPerSlot = 2;
constexpr unsigned kGridSpinLimit = 1u << 21;

// Called by one thread per CTA.  ws[0] counts arrivals, ws[1] departures.
__device__ __forceinline__ bool grid_barrier(unsigned* ws, unsigned nblocks) {
    unsigned v;
    asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;" : "=r"(v) : "l"(ws) : "memory");
    ++v;
    for (unsigned it = 0; v < nblocks; ++it) {
        if (it > kGridSpinLimit) return false;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(ws) : "memory");
    }
    unsigned d;
    asm volatile("atom.add.relaxed.gpu.u32 %0, [%1], 1;" : "=r"(d) : "l"(ws + 1) : "memory");
    if (d == nblocks - 1) {  // everybody has seen the full count: clean up for the next launch
        ws[1] = 0;
        __threadfence();
        ws[0] = 0;
    }
    return true;
}

template <int NCHG, int NCHD>
__global__ void __launch_bounds__(kFusedThreads, 1) moe_layer_fused_kernel(MoeLayerArgs a, unsigned* gws) {
    using MATH = MathQ16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nchunks_h = a.H / kGroupSize;
    const int max_slots = a.top_k + (a.shared_pages ? 1 : 0);
    const unsigned g_code_row = (unsigned)a.H / 2, g_scale_row = (unsigned)a.H / 16;
    const unsigned g_stage_bytes = 2 * kTileRows * (g_code_row + g_scale_row);
    const unsigned d_code_row = (unsigned)a.I / 2, d_scale_row = (unsigned)a.I / 16;
    const unsigned d_slot_bytes = kFDownRows * (d_code_row + d_scale_row);
    const unsigned d_stage_bytes = max_slots * d_slot_bytes;

    unsigned char* gring = smem_raw;
    unsigned char* dring = gring + (size_t)kFusedGStages * g_stage_bytes;
    unsigned char* xs = dring + (size_t)kFusedDStages * d_stage_bytes;
    PageEntry* tabg = reinterpret_cast<PageEntry*>(xs + (size_t)nchunks_h * MATH::kStride);
    PageEntry* tabd = tabg + max_slots * 2 * a.P;
    uint64_t* gfull = reinterpret_cast<uint64_t*>(tabd + max_slots * a.P);
    uint64_t* gempty = gfull + kFusedGStages;
    uint64_t* dfull = gempty + kFusedGStages;
    uint64_t* dempty = dfull + kFusedDStages;
    unsigned* words = reinterpret_cast<unsigned*>(dempty + kFusedDStages);
    volatile unsigned* landed = words;
    volatile int* abort_flag = reinterpret_cast<int*>(words + kFusedGStages);
    float* wts = reinterpret_cast<float*>(words + kFusedGStages + 1);
    float* ybuf = wts + kMaxSlots;  // [parity][row][kMaxSlots]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();
    if (tid == 0) {
        for (int s = 0; s < kFusedGStages; ++s) {
            mbar_init(gfull + s, 1);
            mbar_init(gempty + s, kGroupWarps);
            landed[s] = 0;
        }
        for (int s = 0; s < kFusedDStages; ++s) mbar_init(dfull + s, 1);
        *abort_flag = 0;
    }
    // the activation vector does not come from the router: quantise it before waiting for the router
    if (warp < kFusedConsumerWarps) stage_activation<MATH>(xs, a.x, a.x_dtype, a.H, tid, kFusedConsumerWarps * 32);
    pdl_wait();  // expert ids, weights and the optional slot count are outputs of earlier kernels
    a.top_k = active_top_k(a);
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int dwarps = slots * kFDownWarpsPerSlot;

    int gd0, gd1;
    cta_share(a.H, gd0, gd1);
    if (slots == 0) {  // nothing selected (every CTA takes this branch): the layer output is zero
        if (!a.out_accumulate)
            for (int r = gd0 + tid; r < gd1; r += blockDim.x) a.out[r] = 0.f;
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < kFusedDStages; ++s) mbar_init(dempty + s, dwarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < slots * 2 * a.P; i += blockDim.x) {
        const int s = i / (2 * a.P), rem = i % (2 * a.P);
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[rem];
        else if (rem == 0) flag(a.status, kStatusBadExpert);
        tabg[i] = e;
    }
    for (int i = tid; i < slots * a.P; i += blockDim.x) {
        const int s = i / a.P, p = i - s * a.P;
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[kSegDown * a.P + p];
        tabd[i] = e;
    }
    for (int s = tid; s < slots; s += blockDim.x) wts[s] = s < a.top_k ? a.expert_weights[s] : a.shared_weight;
    __syncthreads();

    int gg0, gg1;
    cta_share(slots * a.I, gg0, gg1);

    if (warp == kFusedConsumerWarps) {
        // ── producer warp: gate/up tiles, then straight on to the down tiles ──
        bool ok = true;
        int ng = 0, nd = 0;
        {
            TileWalk walk(gg0, gg1, a.I, a.rpp_gu);
            Tile t;
            while (walk.next(t)) {
                const int st = ng % kFusedGStages;
                if (ng >= kFusedGStages) ok = mbar_wait(gempty + st, ((ng / kFusedGStages) - 1) & 1);
                if (!ok) break;
                const PageEntry eu = tabg[(t.slot * 2 + kSegUp) * a.P + t.page];
                const PageEntry eg = tabg[(t.slot * 2 + kSegGate) * a.P + t.page];
                unsigned char* sb = gring + (size_t)st * g_stage_bytes;
                const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
                const unsigned cb = t.nrows * g_code_row, sbz = t.nrows * g_scale_row;
                if (lane == 0) {
                    if (present) mbar_expect_tx(gfull + st, 2 * (cb + sbz));
                    else mbar_arrive(gfull + st);
                }
                __syncwarp();
                if (present && lane < 4) {
                    const PageEntry e = (lane & 1) ? eu : eg;  // lanes 0,2: gate; 1,3: up
                    const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                    if (lane < 2) bulk_load(sb + lane * kTileRows * g_code_row, base + (size_t)t.rin * g_code_row, cb, gfull + st);
                    else bulk_load(sb + 2 * kTileRows * g_code_row + (lane - 2) * kTileRows * g_scale_row,
                                   base + (size_t)e.row_count * g_code_row + (size_t)t.rin * g_scale_row, sbz, gfull + st);
                }
                ++ng;
            }
        }
        if (ok) {
            TileWalk walk(gd0, gd1, a.H, a.rpp_dn, kFDownRows);
            Tile t;
            while (walk.next(t)) {
                const int st = nd % kFusedDStages;
                if (nd >= kFusedDStages) ok = mbar_wait(dempty + st, ((nd / kFusedDStages) - 1) & 1);
                if (!ok) break;
                unsigned char* sb = dring + (size_t)st * d_stage_bytes;
                const int s = lane >> 1;
                PageEntry e{0, 0, 0, 0};
                if (s < slots) e = tabd[s * a.P + t.page];
                const bool mine = s < slots && e.ptr != 0 && t.rin + t.nrows <= e.row_count;
                const unsigned bytes = mine ? ((lane & 1) ? t.nrows * d_scale_row : t.nrows * d_code_row) : 0u;
                unsigned tx = bytes;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
                if (lane == 0) {
                    if (tx) mbar_expect_tx(dfull + st, tx);
                    else mbar_arrive(dfull + st);
                }
                __syncwarp();
                if (mine) {
                    const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                    if (lane & 1) bulk_load(sb + s * d_slot_bytes + kFDownRows * d_code_row, base + (size_t)e.row_count * d_code_row + (size_t)t.rin * d_scale_row, bytes, dfull + st);
                    else bulk_load(sb + s * d_slot_bytes, base + (size_t)t.rin * d_code_row, bytes, dfull + st);
                }
                ++nd;
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        if (lane == 0) {  // drain both rings
            for (int k = max(0, ng - kFusedGStages); k < ng; ++k)
                if (!mbar_wait(gfull + (k % kFusedGStages), (k / kFusedGStages) & 1)) flag(a.status, kStatusTimeout);
            for (int k = max(0, nd - kFusedDStages); k < nd; ++k)
                if (!mbar_wait(dfull + (k % kFusedDStages), (k / kFusedDStages) & 1)) flag(a.status, kStatusTimeout);
        }
        return;
    }

    // ── consumers, phase 1: gate/up ──
    bool alive = true;
    if (warp < kConsumerWarps) {
        const int group = warp / kGroupWarps, wi = warp % kGroupWarps;
        Ring ring{gfull, gempty, landed, kFusedGStages};
        const uint32_t stages_addr = smem_u32(gring);
        const uint32_t x_addr = smem_u32(xs) + lane * MATH::kStride;
        TileWalk walk(gg0, gg1, a.I, a.rpp_gu);
        Tile t;
        int n = 0;
        while (alive && walk.next(t)) {
            if (n % kGroups != group) { ++n; continue; }
            const int st = n % kFusedGStages;
            if (!ring.wait_full(n, wi == 0 && lane == 0)) {
                if (lane == 0) flag(a.status, kStatusTimeout);
                alive = false;
                break;
            }
            const int p0 = wi * kPairsPerWarp;
            if (p0 < t.nrows) {
                const PageEntry eu = tabg[(t.slot * 2 + kSegUp) * a.P + t.page];
                const PageEntry eg = tabg[(t.slot * 2 + kSegGate) * a.P + t.page];
                const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                if (present) {
                    const uint32_t sb = stages_addr + st * g_stage_bytes;
                    const uint32_t g_addr = sb + p0 * g_code_row + lane * 16;
                    const uint32_t u_addr = g_addr + kTileRows * g_code_row;
                    const uint32_t gs_addr = sb + 2 * kTileRows * g_code_row + p0 * g_scale_row + lane * 2;
                    const uint32_t us_addr = gs_addr + kTileRows * g_scale_row;
#pragma unroll
                    for (int i = 0; i < NCHG; ++i) {
                        const uint4 q[4] = {lds128(g_addr + i * 512), lds128(u_addr + i * 512),
                                            lds128(g_addr + g_code_row + i * 512), lds128(u_addr + g_code_row + i * 512)};
                        const float s4[4] = {scale_to_f32(lds16(gs_addr + i * 64)), scale_to_f32(lds16(us_addr + i * 64)),
                                             scale_to_f32(lds16(gs_addr + g_scale_row + i * 64)), scale_to_f32(lds16(us_addr + g_scale_row + i * 64))};
                        MATH::template chunk_s<4>(q, s4, x_addr + i * (32 * MATH::kStride), acc);
                    }
                } else if (lane == 0) {
                    flag(a.status, kStatusMissingPage);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = warp_sum(acc[k]);
                if (lane == 0) {
#pragma unroll
                    for (int k = 0; k < kPairsPerWarp; ++k) {
                        if (p0 + k < t.nrows) {
                            const float g16 = __half2float(__float2half_rn(acc[2 * k]));
                            const float u16 = __half2float(__float2half_rn(acc[2 * k + 1]));
                            a.act[(size_t)t.slot * a.I + t.row + p0 + k] = __float2half_rn(silu_mul_f32(g16, u16));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(gempty + st);
            ++n;
        }
    }
    if (!alive) *abort_flag = 1;

    // ── grid barrier: every CTA's activations are written ──
    asm volatile("bar.sync 1, %0;" ::"r"(kFusedConsumerWarps * 32) : "memory");
    if (tid == 0) {
        if (*abort_flag == 0 && !grid_barrier(gws, gridDim.x)) {
            flag(a.status, kStatusTimeout);
            *abort_flag = 1;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kFusedConsumerWarps * 32) : "memory");
    if (*abort_flag) return;
    if (warp >= dwarps) return;  // warps of unused slots

    // ── consumers, phase 2: down ── warp (s, h) keeps slot s's activation chunks in registers
    const int s = warp / kFDownWarpsPerSlot, h = warp % kFDownWarpsPerSlot;
    uint4 xv[NCHD][4];
    float sx[NCHD];
    int sq8[NCHD];
#pragma unroll
    for (int i = 0; i < NCHD; ++i)
        MATH::quantize_chunk(a.act + (size_t)s * a.I + (size_t)(lane + 32 * i) * 32, xv[i], sx[i], sq8[i]);

    const uint32_t dring_addr = smem_u32(dring);
    const uint32_t code_base = s * d_slot_bytes + lane * 16;
    const uint32_t scale_base = s * d_slot_bytes + kFDownRows * d_code_row + lane * 2;
    TileWalk walk(gd0, gd1, a.H, a.rpp_dn, kFDownRows);
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        const int st = n % kFusedDStages;
        if (!mbar_wait(dfull + st, (n / kFusedDStages) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        const PageEntry e = tabd[s * a.P + t.page];
        const bool present = e.ptr != 0 && t.rin + t.nrows <= e.row_count;
        float* yb = ybuf + (n & 1) * (kFDownRows * kMaxSlots);
        const uint32_t sb = dring_addr + st * d_stage_bytes;
#pragma unroll
        for (int r = h; r < kFDownRows; r += kFDownWarpsPerSlot) {
            float acc = 0.f;
            if (r < t.nrows && present) {
#pragma unroll
                for (int i = 0; i < NCHD; ++i) {
                    const uint4 q = lds128(sb + code_base + r * d_code_row + i * 512);
                    const float sc = scale_to_f32(lds16(sb + scale_base + r * d_scale_row + i * 64));
                    acc = MATH::chunk_r(q, sc, xv[i], sx[i], sq8[i], acc);
                }
            }
            const float y = warp_sum(acc);
            if (lane == 0) yb[r * kMaxSlots + s] = __half2float(__float2half_rn(y));
        }
        if (!present && h == 0 && lane == 0) flag(a.status, kStatusMissingPage);
        __syncwarp();
        if (lane == 0) mbar_arrive(dempty + st);
        asm volatile("bar.sync 2, %0;" ::"r"(dwarps * 32) : "memory");
        if (warp == 0 && lane < t.nrows) {
            float out = 0.f;
            for (int k = 0; k < slots; ++k) out = fmaf(wts[k], yb[lane * kMaxSlots + k], out);  // plan order
            const int r = t.row + lane;
            if (a.out_accumulate) a.out[r] += out;
            else a.out[r] = out;
        }
        ++n;
    }
}

int g_fused_mode = 2;  // 0 off, 1 cooperative launch, 2 cooperative + programmatic dependent launch

template <int NCHG, int NCHD>
static int launch_fused_t(const MoeLayerArgs& a, unsigned* gws, size_t smem, cudaStream_t st) {
    static int attr_err = [] {
        cudaError_t e = cudaFuncSetAttribute(moe_layer_fused_kernel<NCHG, NCHD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        return e == cudaSuccess ? 0 : (int)e;
    }();
    if (attr_err) return attr_err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count());
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_fused_mode == 2 && g_use_pdl) ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, moe_layer_fused_kernel<NCHG, NCHD>, a, gws);
}

// VIB3_ERR_UNSUPPORTED when the shape is outside what this kernel is specialised for.
int launch_layer_fused(const MoeLayerArgs& a, unsigned* gws, cudaStream_t st) {
    if (!g_fused_mode || !gws) return VIB3_ERR_UNSUPPORTED;
    if (a.H % 256 || a.I % 256) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int nch_g = (a.H / kGroupSize) % 32 == 0 ? a.H / kGroupSize / 32 : 0;
    const int nch_d = (a.I / kGroupSize) % 32 == 0 ? a.I / kGroupSize / 32 : 0;
    if (slots * kFDownWarpsPerSlot > kFusedConsumerWarps || slots > 16) return VIB3_ERR_UNSUPPORTED;
    const size_t g_stage = 2 * kTileRows * ((size_t)a.H / 2 + (size_t)a.H / 16);
    const size_t d_stage = (size_t)slots * kFDownRows * ((size_t)a.I / 2 + (size_t)a.I / 16);
    const size_t smem = kFusedGStages * g_stage + kFusedDStages * d_stage + (size_t)(a.H / kGroupSize) * MathQ16::kStride +
                        (size_t)slots * 3 * a.P * sizeof(PageEntry) + 2 * (kFusedGStages + kFusedDStages) * sizeof(uint64_t) +
                        (kFusedGStages + 2) * sizeof(unsigned) + kMaxSlots * sizeof(float) +
                        2 * kFDownRows * kMaxSlots * sizeof(float) + 256;
    if (smem > kSmemBudget) return VIB3_ERR_UNSUPPORTED;
    if (nch_g == 7 && nch_d == 2) return launch_fused_t<7, 2>(a, gws, smem, st);
    if (nch_g == 4 && nch_d == 2) return launch_fused_t<4, 2>(a, gws, smem, st);
    if (nch_g == 2 && nch_d == 2) return launch_fused_t<2, 2>(a, gws, smem, st);
    if (nch_g == 1 && nch_d == 2) return launch_fused_t<1, 2>(a, gws, smem, st);
    if (nch_g == 2 && nch_d == 1) return launch_fused_t<2, 1>(a, gws, smem, st);
    if (nch_g == 1 && nch_d == 1) return launch_fused_t<1, 1>(a, gws, smem, st);
    return VIB3_ERR_UNSUPPORTED;
}

}  // namespace vib3
