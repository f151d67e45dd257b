// Building blocks of the bulk-copy staged kernels: mbarrier and cp.async.bulk wrappers (every wait
// bounded), the tile walk over a CTA's share of a paged row space, and the ring bookkeeping.
#pragma once
#include "moe_common.cuh"

namespace vib3 {

constexpr int kConsumerWarps = 16;
constexpr int kPairsPerWarp = 2;   // a consumer warp takes two row pairs (4 rows share each activation load)
// Row pairs per gate/up stage, by the kernel's NCH (32-column chunks per lane and row; 0 = any width).  A stage costs
// the producer warp a fixed time whatever its size (the walk, the barrier, issuing the copies: about 0.7 us), so
// short rows (hidden <= 4096) take eight pairs per stage and four warps consume it — measured on the Mixtral shape
// (hidden 4096): 35.7 -> 26.3 us for the launch; the Kimi shape keeps four (eight would leave its ring two stages).
constexpr int gateup_tile_rows(int nch) { return nch >= 1 && nch <= 4 ? 8 : 4; }
constexpr int gateup_nch(int hidden) { return (hidden / kGroupSize) % 32 == 0 ? (hidden / kGroupSize) / 32 : 0; }
constexpr int kPipeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 12;
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

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start
// while its predecessor in the stream is still running; it must execute pdl_wait() before it reads
// anything the predecessor wrote.  pdl_trigger() in the predecessor lets the successor's CTAs be
// scheduled as soon as SM resources free up.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A tile: up to tile_rows consecutive rows of one page of one slot.
struct Tile {
    int slot, page, rin, nrows, row;  // row = first row inside the slot's matrix
};

// Walk the CTA's share [g, g_end) of a row space made of `slots` matrices of `rows_per_slot`
// rows cut into pages of `rpp` rows.  Producer and consumers walk it identically.  The position is
// kept incrementally (no division per tile).
struct TileWalk {
    int g, g_end, rows_per_slot, rpp, tile_rows;
    int slot, row, page, rin;
    __device__ __forceinline__ TileWalk(int g0, int g1, int rows_per_slot_, int rpp_, int tile_rows_)
        : g(g0), g_end(g1), rows_per_slot(rows_per_slot_), rpp(rpp_), tile_rows(tile_rows_) {
        slot = g0 / rows_per_slot;
        row = g0 - slot * rows_per_slot;
        page = row / rpp;
        rin = row - page * rpp;
    }
    __device__ __forceinline__ bool next(Tile& t) {
        if (g >= g_end) return false;
        t.slot = slot; t.row = row; t.page = page; t.rin = rin;
        int n = min(tile_rows, g_end - g);
        n = min(n, rpp - rin);
        n = min(n, rows_per_slot - row);
        t.nrows = n;
        g += n; row += n; rin += n;
        if (row == rows_per_slot) { ++slot; row = 0; page = 0; rin = 0; }
        else if (rin == rpp) { ++page; rin = 0; }
        return true;
    }
};

// This CTA's contiguous share of `total` rows.  (32-bit arithmetic where the products fit — they do for every shape
// the staged kernels accept: a 64-bit division is a subroutine of some hundred instructions, and this runs, cold, on
// the path between the arrival of the routing and the first copy of the second pass.)
__device__ __forceinline__ void cta_share(int total, int& begin, int& end) {
    const unsigned g = gridDim.x, b = blockIdx.x;
    if ((unsigned)total <= 0xFFFFFFFFu / g) {
        begin = (int)((unsigned)total * b / g);
        end = (int)((unsigned)total * (b + 1) / g);
    } else {
        begin = (int)((long long)total * b / g);
        end = (int)((long long)total * (b + 1) / g);
    }
}

// Ring bookkeeping.  Tile n of a CTA uses stage n % nstages (use number u = n / nstages of that
// stage) and is consumed by group n % (number of groups).  An mbarrier wait names its phase by one parity bit,
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


}  // namespace vib3
