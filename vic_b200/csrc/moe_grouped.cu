// Grouped multi-token MoE sublayer: every DISTINCT expert that the tokens of a step select is read once.
//
// The reference has no such kernel — its prefill runs token by token through the batch-1 path
// (src/runtime/engine.rs:1837-1838), so an expert chosen by 40 tokens is read 40 times.  Here the
// (token, expert) pairs of the step are bucketed by expert on the device, and per expert the projections
// are real matrix products on the 5th-generation tensor cores:
//
//   D[128 weight rows x N tokens] += A[128 x 256] . B[N x 256]^T      per 256-column slab of K
//
//   A  the INT4 page tile.  cp.async.bulk.tensor (one 3-D tensor map over the whole page pool: byte in
//      row, row in page, pool slot) brings 128 B of codes per row and slab — and, once per tile, the rows' group
//      scales for all of K: the TMA unit pays per row segment, so 16-byte scale segments per slab would cost as
//      much as the codes — into shared
//      memory (128-byte swizzle, so that 32 lanes reading 32 rows hit 32 different bank groups); eight
//      warps turn the codes into fp16 weights (n - 8) * scale in registers and store them with tcgen05.st
//      into TENSOR MEMORY: the A operand never goes back through shared memory, whose bandwidth could
//      not carry 4x-expanded weights at the HBM rate.
//   B  the tokens of the expert: rows of a gathered fp16 activation matrix (pairs sorted by expert), loaded
//      by the same TMA unit as 128-byte-swizzled K-major tiles and read by the MMA through a shared-memory
//      descriptor.  Within every 8 columns the K order of both operands is (0,4,1,5,2,6,3,7): that is
//      the order in which one logic operation per two weights isolates the 4-bit codes, and a contraction
//      does not care about the order of K as long as both operands agree.
//   D  fp32 in tensor memory; tcgen05.ld brings it to registers for the epilogue (gate/up: SiLU product
//      rounded to fp16 as the batch-1 path does; down: fp16 per (pair, row), combined per token in plan
//      order by a last kernel, so that the result does not depend on scheduling).
//
// One elected thread issues the MMAs; completion is tracked with tcgen05.commit on mbarriers.  Every wait is
// bounded: a thread that gives up sets VIB3_STATUS_TIMEOUT and the CTA drains and frees its tensor memory.
// No cluster launch, no multicast: every CTA fetches its own tiles.
//
// The path stays HBM-bound by construction: at 128 tokens the step has 90 GFLOP of tensor work (64 us at
// peak) against up to 7 GB of distinct expert weights (1 ms of HBM time); the figure of merit is bytes per
// second over the distinct experts, the tensor pipe's utilisation is reported beside it.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <new>

#include "int4_math.cuh"
#include "launch_common.h"
#include "pipe_common.cuh"

namespace vib3 {

constexpr int kGrpConvWarps = 16;               // converting warps: two teams of 8; TMEM lane quarter = warp & 3
constexpr int kGrpMmaWarps = 4;                 // MMA-issuing warps: a thread issues one tcgen05.mma per ~100 cycles whatever its
                                                // size (measured), four issuers reach the tensor pipe's own rate
constexpr int kGrpFirstEpiWarp = 1 + kGrpMmaWarps;          // warp 0 TMA, 1..4 MMA, 5..8 epilogue, 9..24 converting
constexpr int kGrpFirstConvWarp = kGrpFirstEpiWarp + 4;
constexpr int kGrpXWarp = kGrpFirstConvWarp + kGrpConvWarps;   // issues the token tiles' copies
constexpr int kGrpThreads = (kGrpXWarp + 1) * 32;
constexpr int kGrpStages = 8;                   // weight ring
constexpr int kGrpSlabK = 256;                  // columns of K per pipeline step
constexpr int kGrpMaxN = 16;                    // tokens of one expert per accumulator (a "pass"); a slab is converted once for
                                                // up to TWO passes: the second token group goes to the other D buffer
constexpr int kGrpABufs = 3;                    // A-operand buffers in tensor memory: the converting warps run up to two slabs ahead
constexpr int kGrpXStages = kGrpABufs;          // token ring: stage i is released together with A buffer i (one commit frees both)
constexpr int kGrpRawBytes = 18 * 1024;         // a weight stage: codes 16 KB + scales 2 KB of 128 rows x 256 columns
constexpr int kGrpXGroupBytes = kGrpMaxN * kGrpSlabK * 2;   // 16 tokens x 256 columns fp16 = 8 KB
constexpr int kGrpXBytes = 2 * kGrpXGroupBytes;         // a token stage: the two token groups of a double pass
constexpr int kGrpTmemCols = 512;
constexpr int kGrpACols = kGrpSlabK / 2;        // 128 columns: 256 fp16 per row
constexpr int kGrpDCol0 = kGrpABufs * kGrpACols;   // the A buffers, then two D buffers of kGrpMmaWarps partial accumulators of kGrpMaxN columns
static_assert(kGrpDCol0 + 2 * kGrpMmaWarps * kGrpMaxN <= kGrpTmemCols, "tensor memory budget");
constexpr int kGrpMaxTokens = 128;
constexpr int kRouterMaxExpertsGrouped = 512;   // MAX_EXPERTS, src/core/types.rs:20

struct GroupedMaps {
    CUtensorMap gu_codes, gu_scales_full, gu_scales_last, dn_codes, dn_scales_full, dn_scales_last;
    CUtensorMap xg16, act16;
};

// Device-side description of the step, written by group_pairs_kernel.
struct GroupedWork {
    int n_active;            // distinct experts with at least one token (the shared expert counts as one)
    int n_pairs;
    int pad[2];
};

struct Unit;
// Trips over a unit's slabs: its passes are taken two at a time (each converted slab feeds both).
__host__ __device__ constexpr int grp_double_passes(int n_tok) { return (n_tok + 2 * kGrpMaxN - 1) / (2 * kGrpMaxN); }
struct GroupedArgs {
    const GroupedWork* work;
    __half* act;             // [pairs][I], K order permuted
    __half* y;               // [pairs][H]
    const Unit* units_gu;    // [n_active * tiles_gu]
    const Unit* units_dn;    // [n_active * tiles_dn]
    int tiles_gu, tiles_dn;
    int H, I;
    int* status;
};

// The waits of this kernel: mbarrier.try_wait with a suspend-time hint, so that a waiting warp sleeps in hardware
// until the barrier's phase completes (or the hint runs out) instead of polling.  Bounded: kGrpWaitTries tries of kGrpWaitHintNs each
// (about four seconds), then false.
constexpr unsigned kGrpWaitHintNs = 4000000u;
constexpr unsigned kGrpWaitTries = 1024u;
__device__ __forceinline__ bool mbar_wait_hint(uint64_t* bar, unsigned parity) {
    const uint32_t addr = smem_u32(bar);
    for (unsigned it = 0; it < kGrpWaitTries; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity), "r"(kGrpWaitHintNs) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 codes (one scale group, word j = columns 8j .. 8j+7) -> 16 half2 of (n - 8) * scale in the K order
// (0,4),(1,5),(2,6),(3,7) per word.  (n + 1024) and (16 n + 1024) are exact fp16 numbers made by one logic
// operation per pair; subtracting 1032, or multiplying by 1/16 and subtracting 72, is exact as well; the
// only rounding is the product with the scale.
__device__ __forceinline__ void dequant_chunk(const uint4& q, uint32_t scale2, uint32_t* out) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t w8 = w[j] >> 8;
        const uint32_t a0 = lop3_and_or(w[j], 0x000F000Fu, 0x64006400u);
        const uint32_t a1 = lop3_and_or(w[j], 0x00F000F0u, 0x64006400u);
        const uint32_t a2 = lop3_and_or(w8, 0x000F000Fu, 0x64006400u);
        const uint32_t a3 = lop3_and_or(w8, 0x00F000F0u, 0x64006400u);
        uint32_t r0, r1, r2, r3;
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r0) : "r"(a0), "r"(0x64086408u));                  // (n + 1024) - 1032
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r1) : "r"(a1), "r"(0x2C002C00u), "r"(0xD480D480u));  // / 16 - 72
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r2) : "r"(a2), "r"(0x64086408u));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r3) : "r"(a3), "r"(0x2C002C00u), "r"(0xD480D480u));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[4 * j + 0]) : "r"(r0), "r"(scale2));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[4 * j + 1]) : "r"(r1), "r"(scale2));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[4 * j + 2]) : "r"(r2), "r"(scale2));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[4 * j + 3]) : "r"(r3), "r"(scale2));
    }
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                 "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// Position of row r (column of the down projection) in the permuted K order.
__device__ __forceinline__ int perm8(int r) {
    const int i = r & 7;
    return (r & ~7) | (i < 4 ? 2 * i : 2 * (i - 4) + 1);
}

// One work unit: a 128-row A tile of one expert (gate/up: 64 gate rows and the same 64 up rows; down: 128 rows).
// The units of a step are listed by build_units_kernel; unit u = (active expert u / tiles, tile u % tiles).
struct __align__(16) Unit {
    int slot_a, slot_b;      // pool slots of the page(s); -1: page absent
    short row0;              // first row of the tile inside the page
    short rows;              // valid rows of the tile (gate/up: of each half)
    short scales_last;       // 1: the page is a last (short) page, its scales start earlier
    short pad;
    int mrow0;               // first row inside the matrix
    int n_tok, pair_off;     // the expert's tokens: count and first sorted pair
    int pad2;
};
static_assert(sizeof(Unit) == 32, "a unit is two 16-byte loads");

struct UnitWalk {
    const Unit* units;
    int n_units, u;
    Unit cur, nxt;
    bool have_next;
    __device__ __forceinline__ void load(Unit& t, int i) const {
        const uint4* p = reinterpret_cast<const uint4*>(units + i);
        const uint4 a = __ldg(p), b = __ldg(p + 1);
        uint4* q = reinterpret_cast<uint4*>(&t);
        q[0] = a;
        q[1] = b;
    }
    __device__ __forceinline__ UnitWalk(const Unit* units_, int n_units_) : units(units_), n_units(n_units_), u(blockIdx.x) {
        have_next = u < n_units;
        if (have_next) load(nxt, u);
    }
    // the next unit with work of this CTA (the one after it is requested at once, so its latency hides under this one)
    __device__ __forceinline__ bool next(Unit& t) {
        while (have_next) {
            cur = nxt;
            u += gridDim.x;
            have_next = u < n_units;
            if (have_next) load(nxt, u);
            if (cur.rows > 0 && cur.n_tok > 0) {
                t = cur;
                return true;
            }
        }
        return false;
    }
};

// DOWN = false: act[pair][perm(row)] = f16(silu(f16(Wg x)) * f16(Wu x)); DOWN = true: y[pair][row] = f16(Wd act).
//
// Warp roles: warp 0 issues the weights' TMA copies and the last warp the tokens'; warps 1..4 issue the MMAs (a quarter of a slab's K steps each, into a
// partial accumulator of their own); warps 5..8 run the epilogue; warps 9..24 convert codes into the A operand.
// Three rings decouple them: the weight ring (codes and scales of a slab; released as soon as the converting warps
// hold the slab in registers), the token ring (the slab's B tile; released by the MMAs' completion) and the A
// buffers in tensor memory (filled by the converting warps, released by the MMAs' completion).  A stage's life in
// the weight ring is then one memory latency plus one conversion, whatever the MMAs' lag.
template <bool DOWN>
__global__ void __launch_bounds__(kGrpThreads, 1) moe_grouped_kernel(const __grid_constant__ GroupedMaps maps, GroupedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* wring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* xring = wring + kGrpStages * kGrpRawBytes;
    float* exch = reinterpret_cast<float*>(xring + kGrpXStages * kGrpXBytes);                  // [64][kGrpMaxN + 1]
    uint64_t* full = reinterpret_cast<uint64_t*>(exch + 64 * (kGrpMaxN + 1));
    uint64_t* empty = full + kGrpStages;
    uint64_t* xfull = empty + kGrpStages;
    uint64_t* a_full = xfull + kGrpXStages;
    uint64_t* a_empty = a_full + kGrpABufs;
    uint64_t* d_full = a_empty + kGrpABufs;
    uint64_t* d_empty = d_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = DOWN ? a.I : a.H;
    const int nslab = K / kGrpSlabK;
    if (tid == 0) {
        for (int s = 0; s < kGrpStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kGrpConvWarps / 2);
        }
        for (int s = 0; s < kGrpXStages; ++s) {
            mbar_init(xfull + s, 1);
        }
        for (int s = 0; s < kGrpABufs; ++s) {
            mbar_init(a_full + s, kGrpConvWarps / 2);
            mbar_init(a_empty + s, kGrpMmaWarps);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(d_full + s, kGrpMmaWarps);
            mbar_init(d_empty + s, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kGrpTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();   // the work lists, the gathered tokens and (down) the intermediate are earlier kernels' outputs
    UnitWalk walk(DOWN ? a.units_dn : a.units_gu, a.work->n_active * (DOWN ? a.tiles_dn : a.tiles_gu));

    // Every role walks the same sequence: units blockIdx.x, + gridDim.x, ...; per unit ceil(n_tok / 16) passes, taken
    // two at a time (a converted slab feeds the MMAs of both token groups: an expert with 17 to 32 tokens is
    // converted once, the shared expert of 128 tokens four times instead of eight);
    // per pass nslab slabs.  `it` counts slabs (weight stage it % 8, token stage it % 8, A buffer it % 3), `pc`
    // passes (D buffer pc & 1).
    bool ok = true;
    if (warp == 0) {
        // ── TMA producer of the weight ring ──
        int it = 0;
        Unit t;
        while (ok && walk.next(t)) {
            const CUtensorMap* codes = DOWN ? &maps.dn_codes : &maps.gu_codes;
            const CUtensorMap* scales = DOWN ? (t.scales_last ? &maps.dn_scales_last : &maps.dn_scales_full)
                                             : (t.scales_last ? &maps.gu_scales_last : &maps.gu_scales_full);
            const int total = grp_double_passes(t.n_tok) * nslab;
            // One instruction for all issuing lanes (each lane's copy is a different box): the same copies issued
            // from one branch per lane cost four times as much of the warp's time.
            //   gate/up: lane 0/1 codes of gate/up, lane 2/3 their scales;   down: lane 0 codes, lane 1 scales
            const int nw = DOWN ? 2 : 4;
            const bool is_scale = lane >= nw / 2;
            const bool second = !DOWN && (lane & 1);   // the up matrix
            const CUtensorMap* m = is_scale ? scales : codes;
            const uint32_t dst_off = is_scale ? 16384 + (second ? 1024 : 0) : (second ? 8192 : 0);
            const int c2 = second ? t.slot_b : t.slot_a;
            for (int i = 0; i < total; ++i, ++it) {
                const int s = i % nslab;
                const int st = it % kGrpStages;
                if (it >= kGrpStages) ok = mbar_wait_hint(empty + st, ((it / kGrpStages) - 1) & 1);
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(full + st, kGrpRawBytes);
                __syncwarp();
                if (lane < nw) tma_load_3d(wring + (size_t)st * kGrpRawBytes + dst_off, m, is_scale ? s * 16 : s * 128, t.row0, c2, full + st);
                __syncwarp();
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        // drain: every issued copy must have landed before the CTA's shared memory goes away
        if (lane == 0)
            for (int k = max(0, it - kGrpStages); k < it; ++k)
                if (!mbar_wait_hint(full + (k % kGrpStages), (k / kGrpStages) & 1)) flag(a.status, kStatusTimeout);
    } else if (warp == kGrpXWarp) {
        // ── TMA producer of the token ring: one copy per slab (four K-major tiles of 64 columns) ──
        int it = 0;
        Unit t;
        const CUtensorMap* xmap = DOWN ? &maps.act16 : &maps.xg16;
        while (ok && walk.next(t)) {
            for (int p0 = 0; ok && p0 < t.n_tok; p0 += 2 * kGrpMaxN) {
                const int ng = t.n_tok - p0 > kGrpMaxN ? 2 : 1;   // token groups of this double pass
                for (int s = 0; s < nslab; ++s, ++it) {
                    const int xs = it % kGrpXStages;
                    if (it >= kGrpXStages) ok = mbar_wait_hint(a_empty + xs, ((it / kGrpXStages) - 1) & 1);
                    if (!ok) break;
                    if (lane == 0) {
                        mbar_expect_tx(xfull + xs, ng * kGrpXGroupBytes);
                        tma_load_3d(xring + (size_t)xs * kGrpXBytes, xmap, 0, t.pair_off + p0, s * (kGrpSlabK / 64), xfull + xs);
                        if (ng == 2)
                            tma_load_3d(xring + (size_t)xs * kGrpXBytes + kGrpXGroupBytes, xmap, 0, t.pair_off + p0 + kGrpMaxN,
                                        s * (kGrpSlabK / 64), xfull + xs);
                    }
                    __syncwarp();
                }
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        if (lane == 0)
            for (int k = max(0, it - kGrpXStages); k < it; ++k)
                if (!mbar_wait_hint(xfull + (k % kGrpXStages), (k / kGrpXStages) & 1)) flag(a.status, kStatusTimeout);
    } else if (warp <= kGrpMmaWarps) {
        // ── MMA issuers: warp w takes the K steps 4 (w - 1) .. 4 (w - 1) + 3 of every slab and accumulates them into
        // its own partial accumulator; the epilogue adds the four ──
        const int mw = warp - 1;
        int it = 0, pc = 0;
        Unit t;
        while (ok && walk.next(t)) {
            for (int p0 = 0; ok && p0 < t.n_tok; p0 += 2 * kGrpMaxN) {
                const uint32_t idesc = (1u << 4) | ((uint32_t)(kGrpMaxN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                // a double pass: token group g accumulates into D buffer (pc + g) & 1 — with two groups both buffers
                const int ng = t.n_tok - p0 > kGrpMaxN ? 2 : 1;
                for (int g = 0; ok && g < ng; ++g)
                    if (pc + g >= 2) ok = mbar_wait_hint(d_empty + ((pc + g) & 1), (((pc + g) >> 1) - 1) & 1);
                for (int s = 0; ok && s < nslab; ++s, ++it) {
                    const int xs = it % kGrpXStages, ab = it % kGrpABufs;
                    ok = mbar_wait_hint(xfull + xs, (it / kGrpXStages) & 1) && mbar_wait_hint(a_full + ab, (it / kGrpABufs) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            if (g >= ng) break;
                            const int db = (pc + g) & 1;
                            const uint32_t xaddr = smem_u32(xring + (size_t)xs * kGrpXBytes + g * kGrpXGroupBytes);
#pragma unroll
                            for (int kk = 0; kk < kGrpSlabK / 16 / kGrpMmaWarps; ++kk) {
                                const int k = mw * (kGrpSlabK / 16 / kGrpMmaWarps) + kk;
                                const uint32_t baddr = xaddr + (k >> 2) * kGrpMaxN * 128 + (k & 3) * 32;
                                const uint64_t bdesc = (uint64_t)((baddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                                       ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
                                const uint32_t acc = (s > 0 || kk > 0) ? 1u : 0u;
                                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                                             ::"r"(tmem + kGrpDCol0 + (db * kGrpMmaWarps + mw) * kGrpMaxN), "r"(tmem + ab * kGrpACols + 8 * k), "l"(bdesc),
                                             "r"(idesc), "r"(acc)
                                             : "memory");
                            }
                        }
                        umma_commit(a_empty + ab);
                        if (s == nslab - 1) {
                            umma_commit(d_full + (pc & 1));
                            if (ng == 2) umma_commit(d_full + ((pc + 1) & 1));
                        }
                    }
                    __syncwarp();
                }
                pc += ng;
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
    } else if (warp >= kGrpFirstConvWarp) {
        // ── converting warps: two teams of eight take alternate slabs, so that one team's waits (for the copy, for
        // the A buffer, for its stores into tensor memory) overlap the other team's arithmetic.  Within a team: row
        // m = 32 (warp % 4) + lane of the A tile, K half (128 columns) of the slab ──
        const int cw = warp - kGrpFirstConvWarp;
        const int q = warp & 3, team = cw >> 3, kh = (cw >> 2) & 1;
        const int m = 32 * q + lane;
        // where row m's codes and scales sit in a stage
        const int src_row = DOWN ? m : (m & 63);
        const uint32_t code_off = (DOWN ? 0u : (m >= 64 ? 8192u : 0u)) + (uint32_t)src_row * 128u;
        const uint32_t scale_off = 16384u + (DOWN ? 0u : (m >= 64 ? 1024u : 0u)) + (uint32_t)src_row * 16u + (uint32_t)kh * 8u;
        const int first_row = DOWN ? 32 * q : 32 * (q & 1);   // first row (of the matrix half) among this warp's 32
        const uint32_t sw = (uint32_t)(src_row & 7);
        int it = 0;
        Unit t;
        while (ok && walk.next(t)) {
            const int total = grp_double_passes(t.n_tok) * nslab;
            // a warp whose 32 rows all lie beyond the tile's last row has nothing to convert: its lanes of the
            // accumulator are never read
            const bool work = first_row < t.rows;
            for (int i = 0; ok && i < total; ++i, ++it) {
                if ((it & 1) != team) continue;
                const int st = it % kGrpStages, ab = it % kGrpABufs;
                ok = mbar_wait_hint(full + st, (it / kGrpStages) & 1);
                if (!ok) break;
                const uint32_t sb = smem_u32(wring + (size_t)st * kGrpRawBytes);
                const uint32_t cb = sb + code_off;
                const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + ab * kGrpACols + kh * 64;
                uint32_t h0[16], h1[16];
                uint32_t sc0 = 0, sc1 = 0;   // four group scales
                if (work) {
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(sc0), "=r"(sc1) : "r"(sb + scale_off));
                    const uint4 c0 = lds128(cb + (((uint32_t)(4 * kh) ^ sw) * 16u));
                    const uint4 c1 = lds128(cb + (((uint32_t)(4 * kh + 1) ^ sw) * 16u));
                    dequant_chunk(c0, __byte_perm(sc0, 0, 0x1010), h0);
                    dequant_chunk(c1, __byte_perm(sc0, 0, 0x3232), h1);
                }
                if (it >= kGrpABufs) ok = mbar_wait_hint(a_empty + ab, ((it / kGrpABufs) - 1) & 1);
                if (!ok) break;
                tc_fence_after();
                uint4 c2 = make_uint4(0, 0, 0, 0), c3 = c2;
                if (work) {
                    tmem_st16(taddr, h0);
                    tmem_st16(taddr + 16, h1);
                    c2 = lds128(cb + (((uint32_t)(4 * kh + 2) ^ sw) * 16u));
                    c3 = lds128(cb + (((uint32_t)(4 * kh + 3) ^ sw) * 16u));
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + st);   // the slab is in registers: the stage may be refilled
                if (work) {
                    dequant_chunk(c2, __byte_perm(sc1, 0, 0x1010), h0);
                    dequant_chunk(c3, __byte_perm(sc1, 0, 0x3232), h1);
                    tmem_st16(taddr + 32, h0);
                    tmem_st16(taddr + 48, h1);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full + ab);
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
    } else if (warp >= kGrpFirstEpiWarp) {
        // ── epilogue warps: TMEM lanes 32 (warp % 4) .. + 31 ──
        const int q = warp & 3;
        const int m = 32 * q + lane;
        int pc = 0;
        Unit t;
        while (ok && walk.next(t)) {
            for (int p0 = 0; ok && p0 < t.n_tok; p0 += kGrpMaxN, ++pc) {
                const int ntok = min(kGrpMaxN, t.n_tok - p0);
                const int db = pc & 1;
                ok = mbar_wait_hint(d_full + db, (pc >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + kGrpDCol0 + db * kGrpMmaWarps * kGrpMaxN;
                uint32_t d[16];
                {
                    // the four issuers' partial sums, added pairwise: (p0 + p1) + (p2 + p3)
                    uint32_t p[16], r[16];
                    tmem_ld16(taddr, d);
                    tmem_ld16(taddr + kGrpMaxN, p);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) d[j] = __float_as_uint(__uint_as_float(d[j]) + __uint_as_float(p[j]));
                    tmem_ld16(taddr + 2 * kGrpMaxN, r);
                    tmem_ld16(taddr + 3 * kGrpMaxN, p);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        d[j] = __float_as_uint(__uint_as_float(d[j]) + (__uint_as_float(r[j]) + __uint_as_float(p[j])));
                }
                // the accumulators are in registers: the MMAs of the pass after next may overwrite them
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_empty + db);
                if (DOWN) {
                    if (m < t.rows) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < ntok) a.y[(size_t)(t.pair_off + p0 + j) * a.H + t.mrow0 + m] = __float2half_rn(__uint_as_float(d[j]));
                    }
                } else {
                    // the up half hands its values to the gate half of the same rows
                    if (m >= 64) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) exch[(m - 64) * (kGrpMaxN + 1) + j] = __uint_as_float(d[j]);
                    }
                    asm volatile("bar.sync 3, 128;" ::: "memory");
                    if (m < 64 && m < t.rows) {
                        const int col = perm8(t.mrow0 + m);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (j < ntok) {
                                const float g16 = __half2float(__float2half_rn(__uint_as_float(d[j])));
                                const float u16 = __half2float(__float2half_rn(exch[m * (kGrpMaxN + 1) + j]));
                                a.act[(size_t)(t.pair_off + p0 + j) * a.I + col] = __float2half_rn(silu_mul_f32(g16, u16));
                            }
                        }
                    }
                    asm volatile("bar.sync 3, 128;" ::: "memory");
                }
            }
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
    }
    // Free the tensor memory once every role is done with it (a role that gave up has stopped touching it).
    tc_fence_before();
    __syncthreads();
    pdl_trigger();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGrpTmemCols) : "memory");
    }
}

// ── bucketing ────────────────────────────────────────────────────────────────────────────────
// One CTA.  Pairs (token, slot) -> sorted by expert (stable in token order); the shared expert, if any, is
// expert E with every token.  Also the list of active experts, most tokens first (ties: lower id), so that
// the experts with several passes start first.
struct GroupPairsArgs {
    const unsigned short* ids;   // [T] rows of top_k, stride in bytes
    int ids_stride;
    int T, top_k, E, has_shared;
    int expert_lo, expert_hi;    // only pairs whose expert lies in [lo, hi) are taken (an expert-parallel rank's share)
    GroupedWork* work;
    int* active;
    int* counts;     // [E + 1]
    int* offsets;    // [E + 2]
    int* pos;        // [T][top_k + 1]: sorted position of (token, slot); slot top_k = the shared expert
    unsigned short* pair_token;  // [pairs]
    int* status;
};

__global__ void __launch_bounds__(1024) group_pairs_kernel(GroupPairsArgs g) {
    constexpr int kWords = kGrpMaxTokens / 32;
    __shared__ __align__(16) int cnt[kRouterMaxExpertsGrouped + 4];
    __shared__ int off[kRouterMaxExpertsGrouped + 2];
    __shared__ unsigned mask[kRouterMaxExpertsGrouped][kWords];   // bit t of expert e: token t chose e
    __shared__ int warp_total[32];
    __shared__ int nact;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NE = g.E + 1;
    pdl_wait();
    for (int i = tid; i < g.E * kWords; i += blockDim.x) (&mask[0][0])[i] = 0;
    if (tid == 0) nact = 0;
    __syncthreads();
    const int total = g.T * g.top_k;
    for (int i = tid; i < total; i += blockDim.x) {
        const int t = i / g.top_k, s = i - t * g.top_k;
        const unsigned e = reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(g.ids) + (size_t)t * g.ids_stride)[s];
        if (e >= (unsigned)g.E) flag(g.status, kStatusBadExpert);
        else if ((int)e >= g.expert_lo && (int)e < g.expert_hi) atomicOr(&mask[e][t >> 5], 1u << (t & 31));
    }
    __syncthreads();
    // counts, then their exclusive prefix sum (one value per thread: warp scans, then a scan of the warps' totals)
    int c = 0;
    if (tid < g.E) {
#pragma unroll
        for (int w = 0; w < kWords; ++w) c += __popc(mask[tid][w]);
    } else if (tid == g.E) {
        c = g.has_shared ? g.T : 0;
    }
    for (int e = tid; e < kRouterMaxExpertsGrouped + 4; e += blockDim.x) cnt[e] = e == tid ? c : 0;
    int incl = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int v = warp_total[lane], iv = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, iv, d);
            if (lane >= d) iv += u;
        }
        warp_total[lane] = iv - v;
        if (lane == 31) g.work->n_pairs = iv;
    }
    __syncthreads();
    if (tid <= NE) off[tid] = warp_total[warp] + incl - c;   // (off[NE] = the total: the threads past NE hold zero counts)
    __syncthreads();
    if (tid < NE) {
        g.counts[tid] = c;
        g.offsets[tid] = off[tid];
        if (c > 0) {
            // position among the active experts, most tokens first (ties: lower id)
            int rank = 0;
            const int4* c4 = reinterpret_cast<const int4*>(cnt);
            for (int o4 = 0; o4 < (NE + 3) / 4; ++o4) {
                const int4 v = c4[o4];
                const int o = 4 * o4;
                rank += (v.x > c || (v.x == c && o < tid)) + (v.y > c || (v.y == c && o + 1 < tid)) + (v.z > c || (v.z == c && o + 2 < tid)) +
                        (v.w > c || (v.w == c && o + 3 < tid));
            }
            g.active[rank] = tid;
            atomicAdd(&nact, 1);
        }
    }
    // placement, stable in token order: a pair's position is its expert's offset plus the number of earlier tokens
    // that chose the expert
    for (int i = tid; i < total; i += blockDim.x) {
        const int t = i / g.top_k, s = i - t * g.top_k;
        const unsigned e = reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(g.ids) + (size_t)t * g.ids_stride)[s];
        int p = -1;   // a pair of another rank's expert
        if (e < (unsigned)g.E && (int)e >= g.expert_lo && (int)e < g.expert_hi) {
            p = off[e] + __popc(mask[e][t >> 5] & ((1u << (t & 31)) - 1u));
            for (int w = 0; w < (t >> 5); ++w) p += __popc(mask[e][w]);
            g.pair_token[p] = (unsigned short)t;
        }
        g.pos[t * (g.top_k + 1) + s] = p;
    }
    for (int t = tid; t < g.T; t += blockDim.x) {
        if (g.has_shared) g.pair_token[off[g.E] + t] = (unsigned short)t;
        g.pos[t * (g.top_k + 1) + g.top_k] = g.has_shared ? off[g.E] + t : -1;
    }
    __syncthreads();
    if (tid == 0) g.work->n_active = nact;
    pdl_trigger();
}

// The unit tables of the step: one thread per (active expert, tile).
struct BuildUnitsArgs {
    const PageEntry* page_table;
    const PageEntry* shared_pages;
    const unsigned char* pool_base;
    const GroupedWork* work;
    const int* active;
    const int* counts;
    const int* offsets;
    Unit* units_gu;
    Unit* units_dn;
    int tiles_gu, tiles_dn, tiles_per_page_gu, tiles_per_page_dn;
    int E, P, rpp_gu, rpp_dn;
    int* status;
};

__global__ void __launch_bounds__(256) build_units_kernel(BuildUnitsArgs b) {
    pdl_wait();
    const int per = b.tiles_gu + b.tiles_dn;
    const int total = b.work->n_active * per;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int ai = i / per, r = i - ai * per;
        const bool down = r >= b.tiles_gu;
        const int tile = down ? r - b.tiles_gu : r;
        const int tpp = down ? b.tiles_per_page_dn : b.tiles_per_page_gu;
        const int half_rows = down ? 128 : 64;
        const int page = tile / tpp, tp = tile - page * tpp;
        const int e = b.active[ai];
        const PageEntry* pg = e < b.E ? b.page_table + (size_t)e * 3 * b.P : b.shared_pages;
        const PageEntry ea = pg[(down ? kSegDown : kSegGate) * b.P + page];
        const PageEntry eb = down ? ea : pg[kSegUp * b.P + page];
        Unit u;
        const bool present = ea.ptr != 0 && eb.ptr != 0;
        if (!present) flag(b.status, kStatusMissingPage);
        u.slot_a = present ? (int)((ea.ptr - (unsigned long long)b.pool_base) >> 21) : -1;
        u.slot_b = present ? (int)((eb.ptr - (unsigned long long)b.pool_base) >> 21) : -1;
        u.row0 = (short)(tp * half_rows);
        u.rows = (short)(present ? max(0, min(half_rows, (int)ea.row_count - tp * half_rows)) : 0);
        u.scales_last = (short)(ea.row_count != (down ? b.rpp_dn : b.rpp_gu));
        u.pad = 0;
        u.mrow0 = ea.row_start + tp * half_rows;
        u.n_tok = b.counts[e];
        u.pair_off = b.offsets[e];
        u.pad2 = 0;
        (down ? b.units_dn : b.units_gu)[ai * (down ? b.tiles_dn : b.tiles_gu) + tile] = u;
    }
    pdl_trigger();
}

// xg[p][perm(k)] = fp16(x[token(p)][k]): the tokens gathered in pair order, K order permuted per 8 columns.
__global__ void __launch_bounds__(256) gather_tokens_kernel(const void* x, int x_dtype, int x_stride, const GroupedWork* work,
                                                            const unsigned short* pair_token, __half* xg, int H) {
    pdl_wait();
    const int n_pairs = work->n_pairs;
    const int items = H >> 3;
    for (int p = blockIdx.x; p < n_pairs; p += gridDim.x) {
        const unsigned char* row = reinterpret_cast<const unsigned char*>(x) + (size_t)pair_token[p] * x_stride;
        for (int i = threadIdx.x; i < items; i += blockDim.x) {
            float v[8];
            load_x8(row, x_dtype, i, v);
            const __half2 h0 = __floats2half2_rn(fminf(fmaxf(v[0], -65504.f), 65504.f), fminf(fmaxf(v[4], -65504.f), 65504.f));
            const __half2 h1 = __floats2half2_rn(fminf(fmaxf(v[1], -65504.f), 65504.f), fminf(fmaxf(v[5], -65504.f), 65504.f));
            const __half2 h2 = __floats2half2_rn(fminf(fmaxf(v[2], -65504.f), 65504.f), fminf(fmaxf(v[6], -65504.f), 65504.f));
            const __half2 h3 = __floats2half2_rn(fminf(fmaxf(v[3], -65504.f), 65504.f), fminf(fmaxf(v[7], -65504.f), 65504.f));
            uint4 o;
            o.x = *reinterpret_cast<const uint32_t*>(&h0);
            o.y = *reinterpret_cast<const uint32_t*>(&h1);
            o.z = *reinterpret_cast<const uint32_t*>(&h2);
            o.w = *reinterpret_cast<const uint32_t*>(&h3);
            reinterpret_cast<uint4*>(xg + (size_t)p * H)[i] = o;
        }
    }
    pdl_trigger();
}

// out[t][r] = sum over the token's slots in plan order of w * y[pair][r], then the shared expert (fp32 FMAs,
// cuda/src/kernels.cu:803-813).
__global__ void __launch_bounds__(256) combine_pairs_kernel(const __half* y, const int* pos, const float* weights, int w_stride,
                                                            int T, int top_k, int has_shared, float shared_weight, float* out,
                                                            int out_stride, int out_accumulate, int H) {
    __shared__ int sp[17];
    __shared__ float sw[17];
    pdl_wait();
    const int t = blockIdx.y;
    if ((int)threadIdx.x <= top_k) {
        const int s = threadIdx.x;
        const float* wrow = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(weights) + (size_t)t * w_stride);
        sp[s] = (s < top_k || has_shared) ? pos[t * (top_k + 1) + s] : -1;
        sw[s] = s < top_k ? wrow[s] : shared_weight;
    }
    __syncthreads();
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (r < H) {
        // all loads first, then the sum in plan order (the shared expert last)
        __half2 v[17];
#pragma unroll
        for (int s = 0; s < 17; ++s)
            if (s <= top_k && sp[s] >= 0) v[s] = *reinterpret_cast<const __half2*>(y + (size_t)sp[s] * H + r);
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int s = 0; s < 17; ++s)
            if (s <= top_k && sp[s] >= 0) {
                o0 = fmaf(sw[s], __low2float(v[s]), o0);
                o1 = fmaf(sw[s], __high2float(v[s]), o1);
            }
        float* o = out + (size_t)t * out_stride + r;
        if (out_accumulate) {
            o[0] += o0;
            o[1] += o1;
        } else {
            o[0] = o0;
            o[1] = o1;
        }
    }
    pdl_trigger();
}

}  // namespace vib3

using namespace vib3;

extern "C" int vib3_launch_moe_layer_int4_paged(const void* x, int x_dtype, const void* page_table, int num_experts,
                                                const void* shared_pages, const unsigned short* expert_ids,
                                                const float* expert_weights, int top_k, float shared_weight,
                                                void* act_scratch, float* out, int out_accumulate, int hidden_dim,
                                                int expert_hidden_dim, int pages_per_segment,
                                                int rows_per_page_gate_up, int rows_per_page_down, int group_size,
                                                int* status, void* stream);

// ── host side ────────────────────────────────────────────────────────────────────────────────

namespace {

struct GroupedHandle {
    GroupedMaps maps;
    unsigned char* pool_base;
    size_t capacity_pages;
    int H, I, rpp_gu, rpp_dn, max_tokens, top_k, E;
    // workspace carve-up (device pointers)
    GroupedWork* work;
    int *active, *counts, *offsets, *pos;
    unsigned short* pair_token;
    __half *xg, *act, *y;
    Unit *units_gu, *units_dn;
    int tiles_gu, tiles_dn, tiles_per_page_gu, tiles_per_page_dn;
    int max_pairs;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 3-D map over the pool: x = byte in a row (row_bytes), y = row in the page (rows), z = pool slot.
int make_pool_map(CUtensorMap* m, void* base, size_t row_bytes, int rows, size_t slots, int box_x, int box_y, bool swizzle) {
    const cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)rows, (cuuint64_t)slots};
    const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)(2u << 20)};
    const cuuint32_t box[3] = {(cuuint32_t)box_x, (cuuint32_t)box_y, 1};
    const cuuint32_t es[3] = {1, 1, 1};
    CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VIB3_ERR_STATE;
}

// fp16 rows [rows][cols] seen as x = column within a block of 64, y = row, z = block of 64 columns; a box is 64 columns x
// box_rows x 4 blocks, 128-byte swizzle: one copy brings a slab of 256 columns as four K-major operand tiles
// [box_rows][128 bytes].
int make_rows_map(CUtensorMap* m, void* base, int cols, int rows, int box_rows) {
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)(kGrpSlabK / 64)};
    const cuuint32_t es[3] = {1, 1, 1};
    CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VIB3_ERR_STATE;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Carve {
    size_t work, active, counts, offsets, pos, pair_token, units_gu, units_dn, xg, act, y, total;
    int tiles_gu, tiles_dn, tpp_gu, tpp_dn;
};

// tiles of a matrix of `rows` rows cut into pages of `rpp` rows, in tiles of `tile_rows`
int tiles_of(int rows, int rpp, int tile_rows, int* per_page) {
    *per_page = (rpp + tile_rows - 1) / tile_rows;
    return ((rows + rpp - 1) / rpp) * *per_page;
}

Carve carve(int max_tokens, int top_k, int E, int H, int I, int rpp_gu, int rpp_dn) {
    Carve c;
    const size_t pairs = (size_t)max_tokens * (top_k + 1);
    c.tiles_gu = tiles_of(I, rpp_gu, 64, &c.tpp_gu);
    c.tiles_dn = tiles_of(H, rpp_dn, 128, &c.tpp_dn);
    const size_t max_active = (size_t)(max_tokens * top_k < E ? max_tokens * top_k : E) + 1;
    size_t o = 0;
    c.work = o; o = align_up(o + sizeof(GroupedWork), 256);
    c.active = o; o = align_up(o + (E + 1) * sizeof(int), 256);
    c.counts = o; o = align_up(o + (E + 1) * sizeof(int), 256);
    c.offsets = o; o = align_up(o + (E + 2) * sizeof(int), 256);
    c.pos = o; o = align_up(o + pairs * sizeof(int), 256);
    c.pair_token = o; o = align_up(o + pairs * sizeof(unsigned short), 256);
    c.units_gu = o; o = align_up(o + max_active * c.tiles_gu * sizeof(Unit), 256);
    c.units_dn = o; o = align_up(o + max_active * c.tiles_dn * sizeof(Unit), 256);
    c.xg = o; o = align_up(o + pairs * (size_t)H * 2, 1024);
    c.act = o; o = align_up(o + pairs * (size_t)I * 2, 1024);
    c.y = o; o = align_up(o + pairs * (size_t)H * 2, 1024);
    c.total = o;
    return c;
}

template <class K, class... Args>
int launch_pdl(K kernel, dim3 grid, int threads, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, args...);
}

constexpr size_t kGrpSmem = 1024 + (size_t)kGrpStages * kGrpRawBytes + (size_t)kGrpXStages * kGrpXBytes +
                            64 * (kGrpMaxN + 1) * sizeof(float) + 48 * sizeof(uint64_t);

}  // namespace

extern "C" size_t vib3_moe_grouped_workspace_bytes(int max_tokens, int top_k, int num_experts, int hidden_dim, int expert_hidden_dim,
                                                   int rows_per_page_gate_up, int rows_per_page_down) {
    if (max_tokens <= 0 || top_k <= 0 || num_experts <= 0 || hidden_dim <= 0 || expert_hidden_dim <= 0 || rows_per_page_gate_up <= 0 ||
        rows_per_page_down <= 0)
        return 0;
    return carve(max_tokens, top_k, num_experts, hidden_dim, expert_hidden_dim, rows_per_page_gate_up, rows_per_page_down).total;
}

extern "C" int vib3_moe_grouped_prewarm(void* pool_base, size_t capacity_pages, int num_experts, int top_k, int hidden_dim,
                                        int expert_hidden_dim, int rows_per_page_gate_up, int rows_per_page_down,
                                        int last_page_rows_gate_up, int last_page_rows_down, int max_tokens, void* workspace,
                                        size_t workspace_bytes, void** handle_out) {
    if (!pool_base || !workspace || !handle_out) return VIB3_ERR_NULL;
    if (num_experts <= 0 || num_experts > kRouterMaxExpertsGrouped || top_k <= 0 || top_k > 16) return VIB3_ERR_COUNT;
    if (max_tokens <= 0 || max_tokens > kGrpMaxTokens) return VIB3_ERR_COUNT;
    if (hidden_dim % kGrpSlabK || expert_hidden_dim % kGrpSlabK) return VIB3_ERR_UNSUPPORTED;
    if (((uintptr_t)pool_base & 15) || ((uintptr_t)workspace & 1023)) return VIB3_ERR_ALIGN;
    if (rows_per_page_gate_up <= 0 || rows_per_page_down <= 0 || rows_per_page_gate_up > 32767 || rows_per_page_down > 32767) return VIB3_ERR_SHAPE;
    const Carve c = carve(max_tokens, top_k, num_experts, hidden_dim, expert_hidden_dim, rows_per_page_gate_up, rows_per_page_down);
    if (workspace_bytes < c.total) return VIB3_ERR_CAPACITY;
    if (!encode_fn()) return VIB3_ERR_UNSUPPORTED;
    GroupedHandle* h = new (std::nothrow) GroupedHandle();
    if (!h) return VIB3_ERR_STATE;
    unsigned char* pb = static_cast<unsigned char*>(pool_base);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    h->pool_base = pb; h->capacity_pages = capacity_pages;
    h->H = hidden_dim; h->I = expert_hidden_dim; h->rpp_gu = rows_per_page_gate_up; h->rpp_dn = rows_per_page_down;
    h->max_tokens = max_tokens; h->top_k = top_k; h->E = num_experts;
    h->work = reinterpret_cast<GroupedWork*>(ws + c.work);
    h->active = reinterpret_cast<int*>(ws + c.active);
    h->counts = reinterpret_cast<int*>(ws + c.counts);
    h->offsets = reinterpret_cast<int*>(ws + c.offsets);
    h->pos = reinterpret_cast<int*>(ws + c.pos);
    h->pair_token = reinterpret_cast<unsigned short*>(ws + c.pair_token);
    h->xg = reinterpret_cast<__half*>(ws + c.xg);
    h->act = reinterpret_cast<__half*>(ws + c.act);
    h->y = reinterpret_cast<__half*>(ws + c.y);
    h->units_gu = reinterpret_cast<Unit*>(ws + c.units_gu);
    h->units_dn = reinterpret_cast<Unit*>(ws + c.units_dn);
    h->tiles_gu = c.tiles_gu; h->tiles_dn = c.tiles_dn; h->tiles_per_page_gu = c.tpp_gu; h->tiles_per_page_dn = c.tpp_dn;
    h->max_pairs = max_tokens * (top_k + 1);
    const size_t gu_code_row = hidden_dim / 2, gu_scale_row = hidden_dim / 16;
    const size_t dn_code_row = expert_hidden_dim / 2, dn_scale_row = expert_hidden_dim / 16;
    int e = 0;
    e |= make_pool_map(&h->maps.gu_codes, pb, gu_code_row, rows_per_page_gate_up, capacity_pages, 128, 64, true);
    e |= make_pool_map(&h->maps.gu_scales_full, pb + (size_t)rows_per_page_gate_up * gu_code_row, gu_scale_row, rows_per_page_gate_up,
                       capacity_pages, 16, 64, false);
    e |= make_pool_map(&h->maps.gu_scales_last, pb + (size_t)last_page_rows_gate_up * gu_code_row, gu_scale_row, last_page_rows_gate_up,
                       capacity_pages, 16, 64, false);
    e |= make_pool_map(&h->maps.dn_codes, pb, dn_code_row, rows_per_page_down, capacity_pages, 128, 128, true);
    e |= make_pool_map(&h->maps.dn_scales_full, pb + (size_t)rows_per_page_down * dn_code_row, dn_scale_row, rows_per_page_down,
                       capacity_pages, 16, 128, false);
    e |= make_pool_map(&h->maps.dn_scales_last, pb + (size_t)last_page_rows_down * dn_code_row, dn_scale_row, last_page_rows_down,
                       capacity_pages, 16, 128, false);
    e |= make_rows_map(&h->maps.xg16, h->xg, hidden_dim, h->max_pairs, 16);
    e |= make_rows_map(&h->maps.act16, h->act, expert_hidden_dim, h->max_pairs, 16);
    if (e) {
        delete h;
        return VIB3_ERR_STATE;
    }
    cudaError_t ce = cudaFuncSetAttribute(moe_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGrpSmem);
    if (ce == cudaSuccess) ce = cudaFuncSetAttribute(moe_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGrpSmem);
    if (ce != cudaSuccess) {
        delete h;
        return (int)ce;
    }
    *handle_out = h;
    return VIB3_OK;
}

extern "C" void vib3_moe_grouped_destroy(void* handle) { delete static_cast<GroupedHandle*>(handle); }

extern "C" int vib3_launch_moe_grouped_int4(void* handle, const void* x, int x_dtype, int x_stride_bytes, int n_tokens,
                                            const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                            int weights_stride_bytes, const void* page_table, const void* shared_pages,
                                            float shared_weight, int pages_per_segment, int expert_lo, int expert_hi, float* out,
                                            int out_stride, int out_accumulate, int* status, void* stream) {
    GroupedHandle* h = static_cast<GroupedHandle*>(handle);
    if (!h || !x || !ids || !weights || !page_table || !out) return VIB3_ERR_NULL;
    if (n_tokens <= 0 || n_tokens > h->max_tokens) return VIB3_ERR_COUNT;
    if (expert_lo < 0 || expert_hi < expert_lo || expert_hi > h->E) return VIB3_ERR_COUNT;
    if (x_dtype < X_F32 || x_dtype > X_BF16) return VIB3_ERR_UNSUPPORTED;
    if (pages_per_segment <= 0 || pages_per_segment > kMaxPages) return VIB3_ERR_COUNT;
    if (pages_per_segment * h->tiles_per_page_gu < h->tiles_gu || pages_per_segment * h->tiles_per_page_dn < h->tiles_dn) return VIB3_ERR_SHAPE;
    if (((uintptr_t)x & 15) || (x_stride_bytes & 15) || (ids_stride_bytes & 1) || (weights_stride_bytes & 3) || ((uintptr_t)out & 7) ||
        (out_stride & 1) || out_stride < h->H)
        return VIB3_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const int has_shared = shared_pages ? 1 : 0;
    // One token with all of its experts here: the batch-1 kernels stream the nine experts faster than tensor-core
    // tiles that are fifteen sixteenths padding.
    if (n_tokens == 1 && expert_lo == 0 && expert_hi == h->E) {
        const int e = vib3_launch_moe_layer_int4_paged(x, x_dtype, page_table, h->E, shared_pages, ids, weights, h->top_k, shared_weight,
                                                       h->act, out, out_accumulate, h->H, h->I, pages_per_segment, h->rpp_gu, h->rpp_dn,
                                                       kGroupSize, status, stream);
        if (e != VIB3_ERR_UNSUPPORTED && e != VIB3_ERR_ALIGN) return e;
    }

    GroupPairsArgs g;
    g.ids = ids; g.ids_stride = ids_stride_bytes; g.T = n_tokens; g.top_k = h->top_k; g.E = h->E; g.has_shared = has_shared;
    g.expert_lo = expert_lo; g.expert_hi = expert_hi;
    g.work = h->work; g.active = h->active; g.counts = h->counts; g.offsets = h->offsets; g.pos = h->pos;
    g.pair_token = h->pair_token; g.status = status;
    int err = launch_pdl(group_pairs_kernel, dim3(1), 1024, 0, st, g);
    if (err) return err;
    err = launch_pdl(gather_tokens_kernel, dim3(min(h->max_pairs, 2 * sm_count())), 256, 0, st, x, x_dtype, x_stride_bytes,
                     (const GroupedWork*)h->work, (const unsigned short*)h->pair_token, h->xg, h->H);
    if (err) return err;

    BuildUnitsArgs bu;
    bu.page_table = (const PageEntry*)page_table; bu.shared_pages = (const PageEntry*)shared_pages; bu.pool_base = h->pool_base;
    bu.work = h->work; bu.active = h->active; bu.counts = h->counts; bu.offsets = h->offsets; bu.units_gu = h->units_gu;
    bu.units_dn = h->units_dn; bu.tiles_gu = h->tiles_gu; bu.tiles_dn = h->tiles_dn; bu.tiles_per_page_gu = h->tiles_per_page_gu;
    bu.tiles_per_page_dn = h->tiles_per_page_dn; bu.E = h->E; bu.P = pages_per_segment; bu.rpp_gu = h->rpp_gu; bu.rpp_dn = h->rpp_dn;
    bu.status = status;
    err = launch_pdl(build_units_kernel, dim3(64), 256, 0, st, bu);
    if (err) return err;

    GroupedArgs a;
    a.work = h->work; a.act = h->act; a.y = h->y; a.units_gu = h->units_gu; a.units_dn = h->units_dn;
    a.tiles_gu = h->tiles_gu; a.tiles_dn = h->tiles_dn; a.H = h->H; a.I = h->I; a.status = status;
    err = launch_pdl(moe_grouped_kernel<false>, dim3(sm_count()), kGrpThreads, kGrpSmem, st, h->maps, a);
    if (err) return err;
    err = launch_pdl(moe_grouped_kernel<true>, dim3(sm_count()), kGrpThreads, kGrpSmem, st, h->maps, a);
    if (err) return err;
    return launch_pdl(combine_pairs_kernel, dim3((h->H / 2 + 255) / 256, n_tokens), 256, 0, st, (const __half*)h->y, (const int*)h->pos, weights,
                      weights_stride_bytes, n_tokens, h->top_k, has_shared, shared_weight, out, out_stride, out_accumulate, h->H);
}
