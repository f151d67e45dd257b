// Bulk-copy staged versions of the two MoE sublayer kernels.
//
// One persistent CTA per SM.  A producer thread streams row tiles of the page images into a ring
// of shared-memory stages with cp.async.bulk (the TMA unit's untiled copy; completion is counted
// on an mbarrier per stage), so the amount of weight data in flight is set by the ring (about
// 190 KB per SM) and not by registers.  Sixteen consumer warps in four groups take the stages in
// turn (the ring length is a multiple of the group count, so a stage always belongs to the same
// group); a warp owns one row (gate/up: one gate row and one up row) of a stage, reads codes and
// scales from shared memory with conflict-free 16-byte loads, and uses the same chunk arithmetic
// as the direct-load kernels, so both variants produce identical bits.
//
// Rows of a page are contiguous ([rows][K/2] codes, then [rows][K/16] scale bytes), so a tile of R
// rows is one contiguous run of codes and one of scales: 4 bulk copies per gate/up stage, 2 per
// slot per down stage.  cp.async.bulk needs 16-byte aligned addresses and sizes: K must be a
// multiple of 256 (then a row of scales is a multiple of 16 bytes) and page slots 16-byte aligned.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread sets
// VIB3_STATUS_TIMEOUT in the status word and leaves; the producer additionally drains the copies
// it has issued (bounded as well) before it returns.
#include "moe_common.cuh"

namespace vib3 {

constexpr int kConsumerWarps = 16;
constexpr int kGroups = 4;                       // consumer groups; group g takes tiles g, g+4, ...
constexpr int kTileRows = kConsumerWarps / kGroups;  // rows (row pairs) per stage: one per warp of a group
constexpr int kPipeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 8;
constexpr unsigned kSpinLimit = 1u << 22;
constexpr size_t kSmemBudget = 227 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned it = 0; it < kSpinLimit; ++it) {
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
// Untiled bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// A tile: up to kTileRows consecutive rows of one page of one slot.
struct Tile {
    int slot, page, rin, nrows, row;  // row = first row inside the slot's matrix
};

// Walk the CTA's share [g, g_end) of a row space made of `slots` matrices of `rows_per_slot`
// rows cut into pages of `rpp` rows.  Producer and consumers walk it identically.
struct TileWalk {
    int g, g_end, rows_per_slot, rpp;
    __device__ __forceinline__ bool next(Tile& t) {
        if (g >= g_end) return false;
        t.slot = g / rows_per_slot;
        t.row = g - t.slot * rows_per_slot;
        t.page = t.row / rpp;
        t.rin = t.row - t.page * rpp;
        int n = min(kTileRows, g_end - g);
        n = min(n, rpp - t.rin);
        n = min(n, rows_per_slot - t.row);
        t.nrows = n;
        g += n;
        return true;
    }
};

__device__ __forceinline__ void cta_share(int total, int& begin, int& end) {
    const long long b = (long long)total * blockIdx.x / gridDim.x;
    const long long e = (long long)total * (blockIdx.x + 1) / gridDim.x;
    begin = (int)b;
    end = (int)e;
}

// ── gate/up + SiLU, staged ─────────────────────────────────────────────────────────────────
// stage layout: [gate codes R*K/2][up codes R*K/2][gate scales R*K/16][up scales R*K/16]
template <class MATH>
__global__ void __launch_bounds__(kPipeThreads, 1) moe_gateup_pipe_kernel(MoeLayerArgs a, int nstages) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nchunks = a.H / kGroupSize;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t code_row = (size_t)a.H / 2, scale_row = (size_t)a.H / 16;
    const size_t stage_bytes = 2 * kTileRows * (code_row + scale_row);

    unsigned char* stages = smem_raw;
    typename MATH::XS* xs = reinterpret_cast<typename MATH::XS*>(stages + (size_t)nstages * stage_bytes);
    PageEntry* tab = reinterpret_cast<PageEntry*>(reinterpret_cast<unsigned char*>(xs) + (size_t)nchunks * MATH::kStride * sizeof(typename MATH::XS));
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + slots * 2 * a.P);
    uint64_t* empty = full + kMaxStages;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kTileRows);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < slots * 2 * a.P; i += blockDim.x) {
        const int s = i / (2 * a.P), rem = i % (2 * a.P);
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[rem];
        else if (rem == 0) flag(a.status, kStatusBadExpert);
        tab[i] = e;
    }
    __syncthreads();  // the page entries are all the producer needs

    int g0, g1;
    cta_share(slots * a.I, g0, g1);

    if (warp == kConsumerWarps) {
        // ── producer ──
        if (lane == 0) {
            TileWalk walk{g0, g1, a.I, a.rpp_gu};
            Tile t;
            int n = 0;
            bool ok = true;
            while (ok && walk.next(t)) {
                const int st = n % nstages;
                if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
                if (!ok) break;
                const PageEntry eu = tab[(t.slot * 2 + kSegUp) * a.P + t.page];
                const PageEntry eg = tab[(t.slot * 2 + kSegGate) * a.P + t.page];
                unsigned char* sb = stages + (size_t)st * stage_bytes;
                const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
                if (present) {
                    const unsigned cb = (unsigned)(t.nrows * code_row), sbz = (unsigned)(t.nrows * scale_row);
                    mbar_expect_tx(full + st, 2 * (cb + sbz));
                    const unsigned char* gp = reinterpret_cast<const unsigned char*>(eg.ptr);
                    const unsigned char* up = reinterpret_cast<const unsigned char*>(eu.ptr);
                    bulk_load(sb, gp + (size_t)t.rin * code_row, cb, full + st);
                    bulk_load(sb + kTileRows * code_row, up + (size_t)t.rin * code_row, cb, full + st);
                    bulk_load(sb + 2 * kTileRows * code_row, gp + (size_t)eg.row_count * code_row + (size_t)t.rin * scale_row, sbz, full + st);
                    bulk_load(sb + 2 * kTileRows * code_row + kTileRows * scale_row, up + (size_t)eu.row_count * code_row + (size_t)t.rin * scale_row, sbz, full + st);
                } else {
                    mbar_arrive(full + st);  // absent page: the stage completes empty, consumers write zeros
                }
                ++n;
            }
            if (!ok) flag(a.status, kStatusTimeout);
            // drain: every issued stage must have landed before the CTA's shared memory goes away
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        }
        return;
    }

    // ── consumers: quantise the activation vector while the first stages are in flight ──
    stage_activation<MATH>(xs, a.x, a.x_dtype, a.H, tid, kConsumerWarps * 32);
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32) : "memory");  // consumer warps only
    const int group = warp / kTileRows, wi = warp % kTileRows;
    TileWalk walk{g0, g1, a.I, a.rpp_gu};
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        if (n % kGroups != group) { ++n; continue; }
        const int st = n % nstages;
        if (!mbar_wait(full + st, (n / nstages) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        if (wi < t.nrows) {
            const PageEntry eu = tab[(t.slot * 2 + kSegUp) * a.P + t.page];
            const PageEntry eg = tab[(t.slot * 2 + kSegGate) * a.P + t.page];
            const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
            float acc[2] = {0.f, 0.f};  // [0] gate, [1] up
            if (present) {
                const unsigned char* sb = stages + (size_t)st * stage_bytes;
                const uint4* gcodes = reinterpret_cast<const uint4*>(sb + (size_t)wi * code_row);
                const uint4* ucodes = reinterpret_cast<const uint4*>(sb + (size_t)(kTileRows + wi) * code_row);
                const unsigned short* gsc = reinterpret_cast<const unsigned short*>(sb + 2 * kTileRows * code_row + (size_t)wi * scale_row);
                const unsigned short* usc = reinterpret_cast<const unsigned short*>(sb + 2 * kTileRows * code_row + (size_t)(kTileRows + wi) * scale_row);
#pragma unroll 2
                for (int c = lane; c < nchunks; c += 32) {
                    const uint4 q[2] = {gcodes[c], ucodes[c]};
                    const float s2[2] = {scale_to_f32(gsc[c]), scale_to_f32(usc[c])};
                    MATH::template chunk<2>(q, s2, xs + (size_t)c * MATH::kStride, acc);
                }
            } else if (lane == 0) {
                flag(a.status, kStatusMissingPage);
            }
            const float gsum = warp_sum(acc[0]);
            const float usum = warp_sum(acc[1]);
            if (lane == 0) {
                const float g16 = __half2float(__float2half_rn(gsum));
                const float u16 = __half2float(__float2half_rn(usum));
                a.act[(size_t)t.slot * a.I + t.row + wi] = __float2half_rn(silu_mul_f32(g16, u16));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + st);
        ++n;
    }
}

// ── down + routing weight + accumulate, staged ─────────────────────────────────────────────
// stage layout: per slot [codes R*I/2][scales R*I/16]
__global__ void __launch_bounds__(kPipeThreads, 1) moe_down_pipe_kernel(MoeLayerArgs a, int nstages) {
    using MATH = MathQ16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int nchunks = a.I / kGroupSize;
    const size_t code_row = (size_t)a.I / 2, scale_row = (size_t)a.I / 16;
    const size_t slot_bytes = kTileRows * (code_row + scale_row);
    const size_t stage_bytes = (size_t)slots * slot_bytes;

    unsigned char* stages = smem_raw;
    MATH::XS* acts = reinterpret_cast<MATH::XS*>(stages + (size_t)nstages * stage_bytes);
    PageEntry* tab = reinterpret_cast<PageEntry*>(reinterpret_cast<unsigned char*>(acts) + (size_t)slots * nchunks * MATH::kStride * sizeof(MATH::XS));
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + slots * a.P);
    uint64_t* empty = full + kMaxStages;
    float* wts = reinterpret_cast<float*>(empty + kMaxStages);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kTileRows);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < slots * a.P; i += blockDim.x) {
        const int s = i / a.P, p = i - s * a.P;
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[kSegDown * a.P + p];
        tab[i] = e;
    }
    for (int s = tid; s < slots; s += blockDim.x) wts[s] = s < a.top_k ? a.expert_weights[s] : a.shared_weight;
    __syncthreads();  // tab is needed by the producer before the activations are staged

    int g0, g1;
    cta_share(a.H, g0, g1);

    if (warp == kConsumerWarps) {
        // ── producer: the weights do not depend on the previous kernel, start streaming at once ──
        if (lane == 0) {
            TileWalk walk{g0, g1, a.H, a.rpp_dn};
            Tile t;
            int n = 0;
            bool ok = true;
            while (ok && walk.next(t)) {
                const int st = n % nstages;
                if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
                if (!ok) break;
                unsigned char* sb = stages + (size_t)st * stage_bytes;
                const unsigned cb = (unsigned)(t.nrows * code_row), sbz = (unsigned)(t.nrows * scale_row);
                unsigned tx = 0;
                for (int s = 0; s < slots; ++s) {
                    const PageEntry e = tab[s * a.P + t.page];
                    if (e.ptr != 0 && t.rin + t.nrows <= e.row_count) tx += cb + sbz;
                }
                if (tx) mbar_expect_tx(full + st, tx);
                else mbar_arrive(full + st);
                for (int s = 0; s < slots; ++s) {
                    const PageEntry e = tab[s * a.P + t.page];
                    if (e.ptr != 0 && t.rin + t.nrows <= e.row_count) {
                        const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                        bulk_load(sb + s * slot_bytes, base + (size_t)t.rin * code_row, cb, full + st);
                        bulk_load(sb + s * slot_bytes + kTileRows * code_row, base + (size_t)e.row_count * code_row + (size_t)t.rin * scale_row, sbz, full + st);
                    }
                }
                ++n;
            }
            if (!ok) flag(a.status, kStatusTimeout);
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        }
        return;
    }

    // consumers stage the activations of every slot (written by the gate/up kernel)
    {
        const int ctid = tid, cthreads = kConsumerWarps * 32;
        stage_activation<MATH>(acts, a.act, X_F16, slots * a.I, ctid, cthreads);
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");  // consumer warps only
    }

    const int group = warp / kTileRows, wi = warp % kTileRows;
    TileWalk walk{g0, g1, a.H, a.rpp_dn};
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        if (n % kGroups != group) { ++n; continue; }
        const int st = n % nstages;
        if (!mbar_wait(full + st, (n / nstages) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        if (wi < t.nrows) {
            const unsigned char* sb = stages + (size_t)st * stage_bytes;
            float out = 0.f;
            for (int s = 0; s < slots; ++s) {
                const PageEntry e = tab[s * a.P + t.page];
                float acc[1] = {0.f};
                if (e.ptr != 0 && t.rin + t.nrows <= e.row_count) {
                    const uint4* codes = reinterpret_cast<const uint4*>(sb + s * slot_bytes + (size_t)wi * code_row);
                    const unsigned short* sc = reinterpret_cast<const unsigned short*>(sb + s * slot_bytes + kTileRows * code_row + (size_t)wi * scale_row);
                    const MATH::XS* xs = acts + (size_t)s * nchunks * MATH::kStride;
#pragma unroll 2
                    for (int c = lane; c < nchunks; c += 32) {
                        const uint4 q[1] = {codes[c]};
                        const float s1[1] = {scale_to_f32(sc[c])};
                        MATH::template chunk<1>(q, s1, xs + (size_t)c * MATH::kStride, acc);
                    }
                } else if (lane == 0) {
                    flag(a.status, kStatusMissingPage);
                }
                const float y = warp_sum(acc[0]);
                out = fmaf(wts[s], __half2float(__float2half_rn(y)), out);
            }
            if (lane == 0) {
                const int r = t.row + wi;
                if (a.out_accumulate) a.out[r] += out;
                else a.out[r] = out;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + st);
        ++n;
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────────

static bool pipe_shape_ok(const MoeLayerArgs& a) {
    return a.H % 256 == 0 && a.I % 256 == 0;
}

// Number of ring stages: a multiple of kGroups, so that a stage is always consumed by the same
// group.  A group then never waits on a stage more than one phase ahead of what it has consumed
// itself, which the one-bit phase parity of an mbarrier wait requires.  0 = does not fit.
static int pick_stages(size_t fixed, size_t stage_bytes) {
    if (fixed >= kSmemBudget) return 0;
    int n = (int)((kSmemBudget - fixed) / stage_bytes);
    if (n > kMaxStages) n = kMaxStages;
    n -= n % kGroups;
    return n;
}

template <class MATH>
static int launch_gateup_pipe_t(const MoeLayerArgs& a, cudaStream_t st) {
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t stage_bytes = 2 * kTileRows * ((size_t)a.H / 2 + (size_t)a.H / 16);
    const size_t fixed = (size_t)(a.H / kGroupSize) * MATH::kStride * sizeof(typename MATH::XS) +
                         (size_t)slots * 2 * a.P * sizeof(PageEntry) + 2 * kMaxStages * sizeof(uint64_t) + 128;
    const int nstages = pick_stages(fixed, stage_bytes);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)nstages * stage_bytes;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(moe_gateup_pipe_kernel<MATH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int total = slots * a.I;
    const int grid = min(sm_count(), (total + kTileRows - 1) / kTileRows);
    moe_gateup_pipe_kernel<MATH><<<grid, kPipeThreads, smem, st>>>(a, nstages);
    return (int)cudaGetLastError();
}

int launch_gateup_pipelined(const MoeLayerArgs& a, cudaStream_t st) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    return launch_gateup_pipe_t<MathQ16>(a, st);
}

int launch_down_pipelined(const MoeLayerArgs& a, cudaStream_t st) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t stage_bytes = (size_t)slots * kTileRows * ((size_t)a.I / 2 + (size_t)a.I / 16);
    const size_t fixed = (size_t)slots * (a.I / kGroupSize) * MathQ16::kStride + (size_t)slots * a.P * sizeof(PageEntry) +
                         2 * kMaxStages * sizeof(uint64_t) + slots * sizeof(float) + 128;
    const int nstages = pick_stages(fixed, stage_bytes);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)nstages * stage_bytes;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(moe_down_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int grid = min(sm_count(), (a.H + kTileRows - 1) / kTileRows);
    moe_down_pipe_kernel<<<grid, kPipeThreads, smem, st>>>(a, nstages);
    return (int)cudaGetLastError();
}

}  // namespace vib3
