// Bulk-copy staged versions of the two MoE sublayer kernels.
//
// One persistent CTA per SM.  A producer thread streams row tiles of the page images into a ring
// of shared-memory stages with cp.async.bulk (the TMA unit's untiled copy; completion is counted
// on an mbarrier per stage), so the amount of weight data in flight is set by the ring (about
// 190 KB per SM) and not by registers.  Sixteen consumer warps in four groups take the stages in
// turn; a warp owns one row (gate/up: one gate row and one up row) of a stage, reads codes and
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
// rows cut into pages of `rpp` rows.  Producer and consumers walk it identically.  The position is
// kept incrementally (no division per tile).
struct TileWalk {
    int g, g_end, rows_per_slot, rpp;
    int slot, row, page, rin;
    __device__ __forceinline__ TileWalk(int g0, int g1, int rows_per_slot_, int rpp_)
        : g(g0), g_end(g1), rows_per_slot(rows_per_slot_), rpp(rpp_) {
        slot = g0 / rows_per_slot;
        row = g0 - slot * rows_per_slot;
        page = row / rpp;
        rin = row - page * rpp;
    }
    __device__ __forceinline__ bool next(Tile& t) {
        if (g >= g_end) return false;
        t.slot = slot; t.row = row; t.page = page; t.rin = rin;
        int n = min(kTileRows, g_end - g);
        n = min(n, rpp - rin);
        n = min(n, rows_per_slot - row);
        t.nrows = n;
        g += n; row += n; rin += n;
        if (row == rows_per_slot) { ++slot; row = 0; page = 0; rin = 0; }
        else if (rin == rpp) { ++page; rin = 0; }
        return true;
    }
};

__device__ __forceinline__ void cta_share(int total, int& begin, int& end) {
    const long long b = (long long)total * blockIdx.x / gridDim.x;
    const long long e = (long long)total * (blockIdx.x + 1) / gridDim.x;
    begin = (int)b;
    end = (int)e;
}

// Ring bookkeeping.  Tile n of a CTA uses stage n % nstages (use number u = n / nstages of that
// stage) and is consumed by group n % kGroups.  An mbarrier wait names its phase by one parity bit,
// so a waiter may be at most one phase ahead of the barrier.  Successive uses of a stage can belong
// to different groups; therefore the group that has seen use u land publishes landed[stage] = u + 1,
// and a group that wants use u first waits (bounded) until landed[stage] >= u.
struct Ring {
    uint64_t* full;
    uint64_t* empty;
    volatile unsigned* landed;
    int nstages;

    // consumer side: wait until tile n has landed.  One lane per warp may publish.
    __device__ __forceinline__ bool wait_full(int n, bool publish) {
        const int st = n % nstages;
        const unsigned u = (unsigned)(n / nstages);
        if (u > 0) {
            unsigned it = 0;
            while (landed[st] < u) {
                if (++it > kSpinLimit) return false;
            }
        }
        if (!mbar_wait(full + st, u & 1)) return false;
        if (publish) landed[st] = u + 1;
        return true;
    }
};

// ── gate/up + SiLU, staged ─────────────────────────────────────────────────────────────────
// stage layout: [gate codes R*K/2][up codes R*K/2][gate scales R*K/16][up scales R*K/16]
// NCH = chunks per lane when K/32 is a multiple of 32 (fully unrolled, constant offsets), 0 = any K.
template <int NCH>
__global__ void __launch_bounds__(kPipeThreads, 1) moe_gateup_pipe_kernel(MoeLayerArgs a, int nstages) {
    using MATH = MathQ16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nchunks = a.H / kGroupSize;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const unsigned code_row = (unsigned)a.H / 2, scale_row = (unsigned)a.H / 16;
    const unsigned stage_bytes = 2 * kTileRows * (code_row + scale_row);

    unsigned char* stages = smem_raw;
    unsigned char* xs = stages + (size_t)nstages * stage_bytes;
    PageEntry* tab = reinterpret_cast<PageEntry*>(xs + (size_t)nchunks * MATH::kStride);
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + slots * 2 * a.P);
    uint64_t* empty = full + kMaxStages;
    volatile unsigned* landed = reinterpret_cast<volatile unsigned*>(empty + kMaxStages);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kTileRows);
            landed[s] = 0;
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
        // ── producer warp: every lane walks the tiles; lane 0 arms the stage's barrier, lanes 0..3
        // each issue one of the tile's four copies, so a tile costs one lane's worth of latency ──
        TileWalk walk(g0, g1, a.I, a.rpp_gu);
        Tile t;
        int n = 0;
        bool ok = true;
        while (walk.next(t)) {
            const int st = n % nstages;
            if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
            if (!ok) break;
            const PageEntry eu = tab[(t.slot * 2 + kSegUp) * a.P + t.page];
            const PageEntry eg = tab[(t.slot * 2 + kSegGate) * a.P + t.page];
            unsigned char* sb = stages + (size_t)st * stage_bytes;
            const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
            const unsigned cb = t.nrows * code_row, sbz = t.nrows * scale_row;
            if (lane == 0) {
                if (present) mbar_expect_tx(full + st, 2 * (cb + sbz));
                else mbar_arrive(full + st);  // absent page: the stage completes empty, consumers write zeros
            }
            __syncwarp();
            if (present && lane < 4) {
                const PageEntry e = (lane & 1) ? eu : eg;            // lanes 0,2: gate; 1,3: up
                const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                if (lane < 2) bulk_load(sb + lane * kTileRows * code_row, base + (size_t)t.rin * code_row, cb, full + st);
                else bulk_load(sb + 2 * kTileRows * code_row + (lane - 2) * kTileRows * scale_row,
                               base + (size_t)e.row_count * code_row + (size_t)t.rin * scale_row, sbz, full + st);
            }
            ++n;
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        // drain: every issued stage must have landed before the CTA's shared memory goes away
        if (lane == 0)
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        return;
    }

    // ── consumers: quantise the activation vector while the first stages are in flight ──
    stage_activation<MATH>(xs, a.x, a.x_dtype, a.H, tid, kConsumerWarps * 32);
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32) : "memory");  // consumer warps only
    const int group = warp / kTileRows, wi = warp % kTileRows;
    Ring ring{full, empty, landed, nstages};
    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t x_addr = smem_u32(xs) + lane * MATH::kStride;
    TileWalk walk(g0, g1, a.I, a.rpp_gu);
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        if (n % kGroups != group) { ++n; continue; }
        const int st = n % nstages;
        if (!ring.wait_full(n, wi == 0 && lane == 0)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        if (wi < t.nrows) {
            const PageEntry eu = tab[(t.slot * 2 + kSegUp) * a.P + t.page];
            const PageEntry eg = tab[(t.slot * 2 + kSegGate) * a.P + t.page];
            const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
            float acc[2] = {0.f, 0.f};  // [0] gate, [1] up
            if (present) {
                const uint32_t sb = stages_addr + st * stage_bytes;
                const uint32_t g_addr = sb + wi * code_row + lane * 16;
                const uint32_t u_addr = g_addr + kTileRows * code_row;
                const uint32_t gs_addr = sb + 2 * kTileRows * code_row + wi * scale_row + lane * 2;
                const uint32_t us_addr = gs_addr + kTileRows * scale_row;
                if (NCH > 0) {
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const uint4 q[2] = {lds128(g_addr + i * 512), lds128(u_addr + i * 512)};
                        const float s2[2] = {scale_to_f32(lds16(gs_addr + i * 64)), scale_to_f32(lds16(us_addr + i * 64))};
                        MATH::template chunk_s<2>(q, s2, x_addr + i * (32 * MATH::kStride), acc);
                    }
                } else {
                    for (int c = lane; c < nchunks; c += 32) {
                        const int o = c - lane;
                        const uint4 q[2] = {lds128(g_addr + o * 16), lds128(u_addr + o * 16)};
                        const float s2[2] = {scale_to_f32(lds16(gs_addr + o * 2)), scale_to_f32(lds16(us_addr + o * 2))};
                        MATH::template chunk_s<2>(q, s2, x_addr + o * MATH::kStride, acc);
                    }
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
// stage layout: per slot [codes R*I/2][scales R*I/16].  A tile is R = 4 output rows x all slots.
// Its work units are (slot, pair of rows): the two rows share the slot's activation chunk loads.
// The units of a tile are dealt round-robin to the 4 warps of the group; per-unit results (already
// rounded to fp16 like the reference's down projection) meet in a small shared buffer, and after a
// group barrier warp w adds row w's contributions in plan order.
template <int NCH>
__global__ void __launch_bounds__(kPipeThreads, 1) moe_down_pipe_kernel(MoeLayerArgs a, int nstages) {
    using MATH = MathQ16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int nchunks = a.I / kGroupSize;
    const unsigned code_row = (unsigned)a.I / 2, scale_row = (unsigned)a.I / 16;
    const unsigned slot_bytes = kTileRows * (code_row + scale_row);
    const unsigned stage_bytes = slots * slot_bytes;

    unsigned char* stages = smem_raw;
    unsigned char* acts = stages + (size_t)nstages * stage_bytes;
    PageEntry* tab = reinterpret_cast<PageEntry*>(acts + (size_t)slots * nchunks * MATH::kStride);
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + slots * a.P);
    uint64_t* empty = full + kMaxStages;
    volatile unsigned* landed = reinterpret_cast<volatile unsigned*>(empty + kMaxStages);
    float* wts = const_cast<float*>(reinterpret_cast<volatile float*>(landed + kMaxStages));
    float* ybuf = wts + kMaxSlots;  // [group][parity][row][kMaxSlots]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kTileRows);
            landed[s] = 0;
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
        // ── producer warp: the weights do not depend on the previous kernel, so streaming starts at
        // once.  Lane k < 2 * slots issues copy k of a tile (slot k / 2: codes for even k, scales for
        // odd k); the byte total is summed across lanes for lane 0 to arm the barrier ──
        TileWalk walk(g0, g1, a.H, a.rpp_dn);
        Tile t;
        int n = 0;
        bool ok = true;
        while (walk.next(t)) {
            const int st = n % nstages;
            if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
            if (!ok) break;
            unsigned char* sb = stages + (size_t)st * stage_bytes;
            const int s = lane >> 1;
            PageEntry e{0, 0, 0, 0};
            if (s < slots) e = tab[s * a.P + t.page];
            const bool mine = s < slots && e.ptr != 0 && t.rin + t.nrows <= e.row_count;
            const unsigned bytes = mine ? ((lane & 1) ? t.nrows * scale_row : t.nrows * code_row) : 0u;
            unsigned tx = bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
            if (lane == 0) {
                if (tx) mbar_expect_tx(full + st, tx);
                else mbar_arrive(full + st);
            }
            __syncwarp();
            if (mine) {
                const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                if (lane & 1) bulk_load(sb + s * slot_bytes + kTileRows * code_row, base + (size_t)e.row_count * code_row + (size_t)t.rin * scale_row, bytes, full + st);
                else bulk_load(sb + s * slot_bytes, base + (size_t)t.rin * code_row, bytes, full + st);
            }
            ++n;
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        if (lane == 0)
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        return;
    }

    // consumers quantise the activations of every slot (written by the gate/up kernel)
    stage_activation<MATH>(acts, a.act, X_F16, slots * a.I, tid, kConsumerWarps * 32);
    asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32) : "memory");  // consumer warps only

    const int group = warp / kTileRows, wi = warp % kTileRows;
    Ring ring{full, empty, landed, nstages};
    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t acts_addr = smem_u32(acts) + lane * MATH::kStride;
    float* ygroup = ybuf + group * (2 * kTileRows * kMaxSlots);
    TileWalk walk(g0, g1, a.H, a.rpp_dn);
    Tile t;
    int n = 0, par = 0;
    while (walk.next(t)) {
        if (n % kGroups != group) { ++n; continue; }
        const int st = n % nstages;
        if (!ring.wait_full(n, wi == 0 && lane == 0)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        float* yb = ygroup + par * (kTileRows * kMaxSlots);
        const uint32_t sb = stages_addr + st * stage_bytes;
        for (int u = wi; u < slots * (kTileRows / 2); u += kTileRows) {
            const int s = u / (kTileRows / 2), r0 = 2 * (u % (kTileRows / 2));
            const PageEntry e = tab[s * a.P + t.page];
            float acc[2] = {0.f, 0.f};
            if (r0 < t.nrows) {
                if (e.ptr != 0 && t.rin + t.nrows <= e.row_count) {
                    const uint32_t c0 = sb + s * slot_bytes + r0 * code_row + lane * 16;
                    const uint32_t c1 = c0 + code_row;
                    const uint32_t s0 = sb + s * slot_bytes + kTileRows * code_row + r0 * scale_row + lane * 2;
                    const uint32_t s1 = s0 + scale_row;
                    const uint32_t xa = acts_addr + s * nchunks * MATH::kStride;
                    if (NCH > 0) {
#pragma unroll
                        for (int i = 0; i < NCH; ++i) {
                            const uint4 q[2] = {lds128(c0 + i * 512), lds128(c1 + i * 512)};
                            const float s2[2] = {scale_to_f32(lds16(s0 + i * 64)), scale_to_f32(lds16(s1 + i * 64))};
                            MATH::template chunk_s<2>(q, s2, xa + i * (32 * MATH::kStride), acc);
                        }
                    } else {
                        for (int c = lane; c < nchunks; c += 32) {
                            const int o = c - lane;
                            const uint4 q[2] = {lds128(c0 + o * 16), lds128(c1 + o * 16)};
                            const float s2[2] = {scale_to_f32(lds16(s0 + o * 2)), scale_to_f32(lds16(s1 + o * 2))};
                            MATH::template chunk_s<2>(q, s2, xa + o * MATH::kStride, acc);
                        }
                    }
                } else if (lane == 0) {
                    flag(a.status, kStatusMissingPage);
                }
            }
            const float y0 = warp_sum(acc[0]);
            const float y1 = warp_sum(acc[1]);
            if (lane == 0) {
                // fp16 rounding of the down projection (its output buffer is fp16 in the reference)
                yb[r0 * kMaxSlots + s] = __half2float(__float2half_rn(y0));
                yb[(r0 + 1) * kMaxSlots + s] = __half2float(__float2half_rn(y1));
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "r"(kTileRows * 32) : "memory");  // the group's 4 warps
        if (lane == 0) {
            if (wi < t.nrows) {
                float out = 0.f;
                for (int s = 0; s < slots; ++s) out = fmaf(wts[s], yb[wi * kMaxSlots + s], out);  // plan order
                const int r = t.row + wi;
                if (a.out_accumulate) a.out[r] += out;
                else a.out[r] = out;
            }
            mbar_arrive(empty + st);
        }
        par ^= 1;
        ++n;
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────────

static bool pipe_shape_ok(const MoeLayerArgs& a) {
    return a.H % 256 == 0 && a.I % 256 == 0;
}

// Number of ring stages that fit (at least kGroups so that every group can hold one), 0 = too few.
static int pick_stages(size_t fixed, size_t stage_bytes) {
    if (fixed >= kSmemBudget) return 0;
    int n = (int)((kSmemBudget - fixed) / stage_bytes);
    if (n > kMaxStages) n = kMaxStages;
    return n >= kGroups ? n : 0;
}

template <class K>
static int set_max_smem(K kernel) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int NCH>
static int launch_gateup_pipe_t(const MoeLayerArgs& a, cudaStream_t st, int nstages, size_t smem, int grid) {
    static int attr = set_max_smem(moe_gateup_pipe_kernel<NCH>);
    if (attr) return attr;
    moe_gateup_pipe_kernel<NCH><<<grid, kPipeThreads, smem, st>>>(a, nstages);
    return (int)cudaGetLastError();
}

int launch_gateup_pipelined(const MoeLayerArgs& a, cudaStream_t st) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const size_t stage_bytes = 2 * kTileRows * ((size_t)a.H / 2 + (size_t)a.H / 16);
    const size_t fixed = (size_t)(a.H / kGroupSize) * MathQ16::kStride + (size_t)slots * 2 * a.P * sizeof(PageEntry) +
                         2 * kMaxStages * sizeof(uint64_t) + kMaxStages * sizeof(unsigned) + 128;
    const int nstages = pick_stages(fixed, stage_bytes);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)nstages * stage_bytes;
    const int total = slots * a.I;
    const int grid = min(sm_count(), (total + kTileRows - 1) / kTileRows);
    const int nchunks = a.H / kGroupSize;
    const int nch = nchunks % 32 == 0 ? nchunks / 32 : 0;
    switch (nch) {
        case 1: return launch_gateup_pipe_t<1>(a, st, nstages, smem, grid);
        case 2: return launch_gateup_pipe_t<2>(a, st, nstages, smem, grid);
        case 4: return launch_gateup_pipe_t<4>(a, st, nstages, smem, grid);
        case 7: return launch_gateup_pipe_t<7>(a, st, nstages, smem, grid);
        case 8: return launch_gateup_pipe_t<8>(a, st, nstages, smem, grid);
        default: return launch_gateup_pipe_t<0>(a, st, nstages, smem, grid);
    }
}

template <int NCH>
static int launch_down_pipe_t(const MoeLayerArgs& a, cudaStream_t st, int nstages, size_t smem, int grid) {
    static int attr = set_max_smem(moe_down_pipe_kernel<NCH>);
    if (attr) return attr;
    moe_down_pipe_kernel<NCH><<<grid, kPipeThreads, smem, st>>>(a, nstages);
    return (int)cudaGetLastError();
}

int launch_down_pipelined(const MoeLayerArgs& a, cudaStream_t st) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    if (2 * slots > 32) return VIB3_ERR_UNSUPPORTED;  // one producer lane per copy of a tile
    const size_t stage_bytes = (size_t)slots * kTileRows * ((size_t)a.I / 2 + (size_t)a.I / 16);
    const size_t fixed = (size_t)slots * (a.I / kGroupSize) * MathQ16::kStride + (size_t)slots * a.P * sizeof(PageEntry) +
                         2 * kMaxStages * sizeof(uint64_t) + kMaxStages * sizeof(unsigned) + kMaxSlots * sizeof(float) +
                         (size_t)kGroups * 2 * kTileRows * kMaxSlots * sizeof(float) + 128;
    const int nstages = pick_stages(fixed, stage_bytes);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)nstages * stage_bytes;
    const int grid = min(sm_count(), (a.H + kTileRows - 1) / kTileRows);
    const int nchunks = a.I / kGroupSize;
    const int nch = nchunks % 32 == 0 ? nchunks / 32 : 0;
    switch (nch) {
        case 1: return launch_down_pipe_t<1>(a, st, nstages, smem, grid);
        case 2: return launch_down_pipe_t<2>(a, st, nstages, smem, grid);
        case 4: return launch_down_pipe_t<4>(a, st, nstages, smem, grid);
        case 8: return launch_down_pipe_t<8>(a, st, nstages, smem, grid);
        default: return launch_down_pipe_t<0>(a, st, nstages, smem, grid);
    }
}

}  // namespace vib3
