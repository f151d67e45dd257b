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
#include "pipe_common.cuh"
#include "router_core.cuh"

namespace vib3 {

// ── gate/up + SiLU, staged ─────────────────────────────────────────────────────────────────
// stage layout: [gate codes R*K/2][up codes R*K/2][gate scales R*K/16][up scales R*K/16]
// NCH = chunks per lane when K/32 is a multiple of 32 (fully unrolled, constant offsets), 0 = any K.
// At most 80 registers per thread: with more, a CTA of this kernel (17 warps) and a router CTA (8 warps
// of 48 registers) no longer fit in an SM's register file together, and the first pass cannot run beside
// the router (measured: 59 us per step instead of 56).
// ROUTED: the kernel also ROUTES the token.  Its CTAs first stream the router's weight rows through the same
// ring (one row per stage; CTA b takes rows [E b / G, E (b+1) / G)), one consumer warp per row forms the
// logit in the reference kernel's summation order (router_core.cuh) and stores it; the CTAs then meet at a
// counter in global memory (all of them are resident: one per SM), and in every CTA a pair of extra warps
// (a selecting warp and a helper) repeats the same scoring and selection over the E logits, so that every
// CTA knows the routing without another launch or a broadcast; CTA 0 also stores it for the kernels that
// follow.  While the counter fills and the selection runs, the ring already streams the shared expert
// (pass 0): the memory pipe never waits for the router.  Every wait is bounded.
constexpr int kRoutedThreads = kPipeThreads + 64;   // + selecting warp + helper warp

// slot_pages() with the routing taken from shared memory
__device__ __forceinline__ const PageEntry* routed_slot_pages(const MoeLayerArgs& a, const unsigned short* ids, int s) {
    if (s < a.top_k) {
        const unsigned e = ids[s];
        if (e >= (unsigned)a.num_experts) return nullptr;
        return a.page_table + (size_t)e * 3 * a.P;
    }
    return a.shared_pages;
}

struct RoutedSmem {
    TopKSmem topk;
    unsigned long long rows_done;      // one arrival per router row of this CTA
    unsigned long long routing_ready;  // the selecting warp arrives once the routing is in r_ids / r_w
    unsigned short r_ids[kRouterMaxTopK];
    float r_w[kRouterMaxTopK];
};

template <int NCH, bool ROUTED>
__global__ void __maxnreg__(ROUTED ? 104 : 80) moe_gateup_pipe_kernel(MoeLayerArgs a, RouterArgs r, int nstages) {
    using MATH = MathQ16;
    constexpr int kTileRows = gateup_tile_rows(NCH);         // row pairs per stage
    constexpr int kGroupWarps = kTileRows / kPairsPerWarp;   // warps that consume a stage
    constexpr int kGroups = kConsumerWarps / kGroupWarps;    // group g takes tiles g, g + kGroups, ...
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nchunks = a.H / kGroupSize;
    const int cap_k = a.top_k;                                  // routed slots the launch was sized for
    const int max_slots = cap_k + (a.shared_pages ? 1 : 0);     // shared-memory layout; the slots used may be fewer
    const unsigned code_row = (unsigned)a.H / 2, scale_row = (unsigned)a.H / 16;
    const unsigned stage_bytes = 2 * kTileRows * (code_row + scale_row);

    // A launch for a later window of a device-side pair list (slot_begin > 0) with nothing in its window has
    // no work.  The count was written by a kernel that had completed before the first launch of the chain
    // started, so it can be read without waiting; but the kernel may only END after its predecessor has:
    // a kernel that leaves before its dependency wait counts as complete, and the kernel after it would no
    // longer be ordered behind the predecessor.
    if (!ROUTED && a.slot_begin > 0 && a.num_active_dev && !a.shared_pages && *a.num_active_dev <= a.slot_begin) {
        pdl_wait();
        return;
    }
    // Grouped mode: the slots are (token, expert) pairs of several tokens.  A CTA's contiguous share of the
    // row space touches at most two slots, so it keeps two quantised activation vectors; which tokens they
    // belong to is known only after the wait.  The shared expert's token (shared_token) is an argument, so
    // pass 0 runs as in the single-token form — under whatever the pair list is still waiting for.
    const bool grouped = !ROUTED && a.slot_token != nullptr;
    const unsigned xbytes = (unsigned)nchunks * MATH::kStride;

    unsigned char* stages = smem_raw;
    unsigned char* xs = stages + (size_t)nstages * stage_bytes;
    PageEntry* tab = reinterpret_cast<PageEntry*>(xs + (size_t)(grouped ? 2 : 1) * xbytes);  // [max_slots][2][P], shared expert at cap_k
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + max_slots * 2 * a.P);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tab_ready = empty + kMaxStages;
    volatile unsigned* landed = reinterpret_cast<volatile unsigned*>(tab_ready + 1);
    // routed launches only: the token as given (later the ring of a near-tie recomputation), selection scratch
    unsigned char* xraw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(landed + kMaxStages) + 15) & ~(uintptr_t)15);
    const unsigned xraw_bytes = ROUTED ? max((unsigned)a.H * (a.x_dtype == X_F32 ? 4u : 2u), (unsigned)(kSeqRingFloats * sizeof(float))) : 0u;
    RoutedSmem& rs = *reinterpret_cast<RoutedSmem*>(xraw + ((xraw_bytes + 15) & ~15u));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int e0 = 0, e1 = 0;  // this CTA's router rows
    if (ROUTED) cta_share(r.E, e0, e1);
    const int nrows = e1 - e0;
    // A launch that does not route itself: the producer warp initialises the barriers and copies the shared expert's
    // table itself, and starts the first copies at once — the weights need neither the token nor the other warps;
    // the consumers meet it (and each other) at a named barrier once the token is staged.
    if (ROUTED ? tid == 0 : tid == kConsumerWarps * 32) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kGroupWarps);
            landed[s] = 0;
        }
        mbar_init(tab_ready, 1);
        if (ROUTED) {
            mbar_init(reinterpret_cast<uint64_t*>(&rs.rows_done), max(nrows, 1));
            mbar_init(reinterpret_cast<uint64_t*>(&rs.routing_ready), 1);
            topk_smem_init(rs.topk, 1);
            if (nrows == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&rs.rows_done));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Neither the activation vector nor the shared expert's pages come from the router: quantise the
    // vector and run the whole shared expert (pass 0) BEFORE the routing is known.  A launch that does not
    // route itself leaves enough shared memory free for a router CTA on the same SM, so its CTAs become
    // resident while the router is still running and the shared expert streams under the router's serial
    // tail.  Between the passes nobody waits for the whole CTA: the producer warp alone waits for the
    // routing, builds the routed slots' page table and goes on issuing copies while the consumers finish
    // pass 0.  A routed launch may follow the producer of its token with programmatic dependent launch:
    // everything that reads the token waits for that kernel first; the weights do not depend on it, so the
    // producer warp fills the ring meanwhile.
    if (ROUTED && warp != kConsumerWarps) pdl_wait();
    if (warp < kConsumerWarps && (!grouped || a.shared_pages))
        stage_activation<MATH>(xs, reinterpret_cast<const unsigned char*>(a.x) + (grouped ? (size_t)a.shared_token * a.x_stride : (size_t)0),
                               a.x_dtype, a.H, tid, kConsumerWarps * 32);
    if (ROUTED && warp < kConsumerWarps) {
        const int n16 = (a.H * (a.x_dtype == X_F32 ? 4 : 2)) >> 4;
        for (int i = tid; i < n16; i += kConsumerWarps * 32) reinterpret_cast<uint4*>(xraw)[i] = __ldg(reinterpret_cast<const uint4*>(a.x) + i);
    }
    if (ROUTED) {
        if (a.shared_pages)
            for (int i = tid; i < 2 * a.P; i += blockDim.x) tab[cap_k * 2 * a.P + i] = a.shared_pages[i];
        __syncthreads();
    } else if (warp == kConsumerWarps) {
        if (a.shared_pages)
            for (int i = lane; i < 2 * a.P; i += 32) tab[cap_k * 2 * a.P + i] = a.shared_pages[i];
        __syncwarp();
        asm volatile("bar.arrive 3, %0;" ::"r"(kPipeThreads) : "memory");
    } else {
        asm volatile("bar.sync 3, %0;" ::"r"(kPipeThreads) : "memory");
    }

    int n = 0;  // tiles of this CTA so far, over both passes (producer and consumers count alike)
    const int first_pass = a.shared_pages ? 0 : 1;

    if (warp == kConsumerWarps) {
        // ── producer warp: every lane walks the tiles; lane 0 arms the stage's barrier, lanes 0..3 each
        // issue one of the tile's four copies, so a tile costs one lane's worth of latency ──
        bool ok = true;
        if (ROUTED) {
            // the router's rows of this CTA, one row per stage (the launcher checked that they fit)
            const unsigned row_bytes = (unsigned)r.H * (r.w_dtype == W_F32 ? 4u : 2u);
            for (int i = 0; i < nrows; ++i, ++n) {
                if (lane == 0) {
                    mbar_expect_tx(full + n, row_bytes);
                    bulk_load(stages + (size_t)n * stage_bytes, reinterpret_cast<const unsigned char*>(r.W) + (size_t)(e0 + i) * row_bytes, row_bytes, full + n);
                }
            }
            __syncwarp();
        }
        for (int pass = first_pass; pass < 2 && ok; ++pass) {
            int g0, g1;
            if (pass == 0) {
                cta_share(a.I, g0, g1);
            } else {
                if (ROUTED) {
                    ok = mbar_wait(reinterpret_cast<uint64_t*>(&rs.routing_ready), 0);
                    if (!ok) break;
                } else {
                    pdl_wait();  // expert ids, weights and the optional slot count are outputs of earlier kernels
                    // Only now may the next kernel in the stream start: it reads the routing without waiting,
                    // and may overwrite nothing this kernel still reads.
                    pdl_trigger();
                }
                a.top_k = active_top_k(a);
                for (int i = lane; i < a.top_k * 2 * a.P; i += 32) {
                    const int s = i / (2 * a.P), rem = i % (2 * a.P);
                    const PageEntry* pg = ROUTED ? routed_slot_pages(a, rs.r_ids, s) : slot_pages(a, s);
                    PageEntry e{0, 0, 0, 0};
                    if (pg) e = pg[rem];
                    else if (rem == 0) flag(a.status, kStatusBadExpert);
                    tab[i] = e;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(tab_ready);  // release: the consumers acquire the table through this barrier
                cta_share(a.top_k * a.I, g0, g1);
            }
            TileWalk walk(g0, g1, a.I, a.rpp_gu, kTileRows);
            Tile t;
            while (walk.next(t)) {
                const int st = n % nstages;
                if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
                if (!ok) break;
                const int ts = (pass == 0 || t.slot >= a.top_k) ? cap_k : t.slot;  // the shared expert's entries sit at cap_k
                const PageEntry eu = tab[(ts * 2 + kSegUp) * a.P + t.page];
                const PageEntry eg = tab[(ts * 2 + kSegGate) * a.P + t.page];
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
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        // drain: every issued stage must have landed before the CTA's shared memory goes away
        if (lane == 0)
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        return;
    }

    Ring ring{full, empty, landed, nstages};
    if (ROUTED && warp > kConsumerWarps) {
        // ── selecting warp and helper warp ──
        const int gt = tid - (kConsumerWarps + 1) * 32;  // index in the group of 64
        bool ok = true;
        if (gt == 0) {
            ok = mbar_wait(reinterpret_cast<uint64_t*>(&rs.rows_done), 0);
            // arrive at the grid-wide counter (release this CTA's logits), then wait for everybody's
            unsigned int seen = 0;
            asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;" : "=r"(seen) : "l"(r.counter) : "memory");
            ++seen;
            for (unsigned it = 0; seen < gridDim.x && it < kRouterSpinLimit; ++it)
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(seen) : "l"(r.counter) : "memory");
            if (seen < gridDim.x) ok = false;
            if (!ok) flag(a.status, kStatusTimeout);
        }
        group_sync(64);
        router_finish(r, rs.topk, reinterpret_cast<float*>(xraw), gt, 64, r.mode != 0, blockIdx.x == 0, rs.r_ids, rs.r_w);
        if (gt == 0) {
            if (rs.topk.failed) flag(a.status, kStatusTimeout);
            __threadfence();  // CTA 0: ids and weights are in global memory before the next kernel may start
            mbar_arrive(reinterpret_cast<uint64_t*>(&rs.routing_ready));
            pdl_trigger();
            // the last CTA to leave the counter resets it for the next launch
            unsigned int left;
            asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;" : "=r"(left) : "l"(r.counter + 2) : "memory");
            if (left == gridDim.x - 1) {
                r.counter[0] = 0u;
                r.counter[2] = 0u;
            }
        }
        return;
    }

    // ── consumers ──
    const int group = warp / kGroupWarps, wi = warp % kGroupWarps;
    if (ROUTED) {
        // router rows: row i of this CTA sits in stage i and belongs to warp i % 16
        for (int i = 0; i < nrows; ++i) {
            if (i % kConsumerWarps != warp) continue;
            if (!ring.wait_full(i, lane == 0)) {
                if (lane == 0) flag(a.status, kStatusTimeout);
                return;
            }
            const unsigned char* wrow = stages + (size_t)i * stage_bytes;
            float logit = 0.f, absum = 0.f;
            if (r.w_dtype == W_F32) {
                if (r.x_dtype == X_F32) row_logit_smem<X_F32, W_F32>(wrow, xraw, r.H, lane, logit, absum);
                else if (r.x_dtype == X_F16) row_logit_smem<X_F16, W_F32>(wrow, xraw, r.H, lane, logit, absum);
                else row_logit_smem<X_BF16, W_F32>(wrow, xraw, r.H, lane, logit, absum);
            } else {
                if (r.x_dtype == X_F32) row_logit_smem<X_F32, W_F16>(wrow, xraw, r.H, lane, logit, absum);
                else if (r.x_dtype == X_F16) row_logit_smem<X_F16, W_F16>(wrow, xraw, r.H, lane, logit, absum);
                else row_logit_smem<X_BF16, W_F16>(wrow, xraw, r.H, lane, logit, absum);
            }
            __syncwarp();
            if (lane == 0) {
                const int e = e0 + i;
                if (r.logit_offset) logit = __fadd_rn(logit, r.logit_offset[e]);
                r.scores[e] = logit;
                if (r.exact_order) r.scores[r.E + e] = absum;
                if (r.mode != 0) r.scores[2 * r.E + e] = sigmoid_ref(logit);
                __threadfence();
                for (int k = 0; k < kGroupWarps; ++k) mbar_arrive(empty + i);   // the stage had one reader
                mbar_arrive(reinterpret_cast<uint64_t*>(&rs.rows_done));
            }
        }
        n = nrows;
    }
    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t x_base = smem_u32(xs) + lane * MATH::kStride;
    int slot_a = 0;  // grouped mode: the slot whose token's vector is in the first activation buffer
    for (int pass = first_pass; pass < 2; ++pass) {
        int g0, g1;
        if (pass == 0) {
            cta_share(a.I, g0, g1);
        } else {
            // The next kernel in the stream (the down kernel) reads the routing without waiting, so it may
            // start only when the router is known to have finished: after this thread's own wait.  By
            // then this thread has also finished the shared expert's rows (pass 0).  (A routed launch lets
            // it go from its selecting warp, once CTA 0 has stored the routing.)
            if (!ROUTED) {
                pdl_wait();
                pdl_trigger();
            }
            a.top_k = active_top_k(a);
            const bool ready = mbar_wait(tab_ready, 0);
            cta_share(a.top_k * a.I, g0, g1);
            if (grouped) {
                // pass 0 read the first activation buffer: every consumer warp must be through with it
                if (first_pass == 0) asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32) : "memory");
                // quantise the activation vectors of the (at most two) slots this CTA's rows belong to
                if (ready && g1 > g0) {
                    slot_a = g0 / a.I;
                    const int slot_b = (g1 - 1) / a.I;
                    const int tok_a = slot_a < a.top_k ? a.slot_token[slot_a] : a.shared_token;
                    stage_activation<MATH>(xs, reinterpret_cast<const unsigned char*>(a.x) + (size_t)tok_a * a.x_stride,
                                           a.x_dtype, a.H, tid, kConsumerWarps * 32);
                    if (slot_b != slot_a) {
                        const int tok_b = slot_b < a.top_k ? a.slot_token[slot_b] : a.shared_token;
                        stage_activation<MATH>(xs + xbytes, reinterpret_cast<const unsigned char*>(a.x) + (size_t)tok_b * a.x_stride,
                                               a.x_dtype, a.H, tid, kConsumerWarps * 32);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32) : "memory");  // consumer warps only
            }
            if (!ready) {  // (after the barrier: a named barrier counts threads, nobody may leave before it)
                if (lane == 0) flag(a.status, kStatusTimeout);
                return;
            }
        }
        TileWalk walk(g0, g1, a.I, a.rpp_gu, kTileRows);
        Tile t;
        while (walk.next(t)) {
            if (n % kGroups != group) { ++n; continue; }
            const int st = n % nstages;
            if (!ring.wait_full(n, wi == 0 && lane == 0)) {
                if (lane == 0) flag(a.status, kStatusTimeout);
                return;
            }
            const int p0 = wi * kPairsPerWarp;  // this warp's row pairs: p0 and p0 + 1 of the tile
            if (p0 < t.nrows) {
                const int ts = (pass == 0 || t.slot >= a.top_k) ? cap_k : t.slot;
                const PageEntry eu = tab[(ts * 2 + kSegUp) * a.P + t.page];
                const PageEntry eg = tab[(ts * 2 + kSegGate) * a.P + t.page];
                const bool present = eu.ptr != 0 && eg.ptr != 0 && t.rin + t.nrows <= eu.row_count && t.rin + t.nrows <= eg.row_count;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};  // gate p0, up p0, gate p0+1, up p0+1
                if (present) {
                    const uint32_t x_addr = x_base + ((grouped && t.slot != slot_a) ? xbytes : 0u);
                    const uint32_t sb = stages_addr + st * stage_bytes;
                    const uint32_t g_addr = sb + p0 * code_row + lane * 16;
                    const uint32_t u_addr = g_addr + kTileRows * code_row;
                    const uint32_t gs_addr = sb + 2 * kTileRows * code_row + p0 * scale_row + lane * 2;
                    const uint32_t us_addr = gs_addr + kTileRows * scale_row;
                    if (NCH > 0) {
#pragma unroll 1
                        for (int i = 0; i < NCH; ++i) {
                            const uint4 q[4] = {lds128(g_addr + i * 512), lds128(u_addr + i * 512),
                                                lds128(g_addr + code_row + i * 512), lds128(u_addr + code_row + i * 512)};
                            const float s4[4] = {scale_to_f32(lds16(gs_addr + i * 64)), scale_to_f32(lds16(us_addr + i * 64)),
                                                 scale_to_f32(lds16(gs_addr + scale_row + i * 64)), scale_to_f32(lds16(us_addr + scale_row + i * 64))};
                            MATH::template chunk_s<4>(q, s4, x_addr + i * (32 * MATH::kStride), acc);
                        }
                    } else {
                        for (int c = lane; c < nchunks; c += 32) {
                            const int o = c - lane;
                            const uint4 q[4] = {lds128(g_addr + o * 16), lds128(u_addr + o * 16),
                                                lds128(g_addr + code_row + o * 16), lds128(u_addr + code_row + o * 16)};
                            const float s4[4] = {scale_to_f32(lds16(gs_addr + o * 2)), scale_to_f32(lds16(us_addr + o * 2)),
                                                 scale_to_f32(lds16(gs_addr + scale_row + o * 2)), scale_to_f32(lds16(us_addr + scale_row + o * 2))};
                            MATH::template chunk_s<4>(q, s4, x_addr + o * MATH::kStride, acc);
                        }
                    }
                } else if (lane == 0) {
                    flag(a.status, kStatusMissingPage);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = warp_sum(acc[k]);
                if (lane == 0) {
                    // pass 0 writes the shared expert's rows at the front of the scratch buffer (act_slot order)
                    const int apos = (pass == 0 || t.slot >= a.top_k) ? 0 : t.slot + (a.shared_pages ? 1 : 0);
                    __half* dst = a.act + (size_t)apos * a.I + t.row + p0;
#pragma unroll
                    for (int k = 0; k < kPairsPerWarp; ++k) {
                        if (p0 + k < t.nrows) {
                            const float g16 = __half2float(__float2half_rn(acc[2 * k]));
                            const float u16 = __half2float(__float2half_rn(acc[2 * k + 1]));
                            dst[k] = __float2half_rn(silu_mul_f32(g16, u16));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);
            ++n;
        }
    }
}

// ── down + routing weight + accumulate, staged ─────────────────────────────────────────────
// Rows of the down matrices are short (I/2 bytes: 1 KB for I = 2048, two 16-byte chunks per lane),
// and every output row needs all experts.  Re-reading an expert's activation chunks from shared
// memory for every row would cost more shared-memory bandwidth than the codes themselves, so here
// the activations stay in REGISTERS: two warps per expert slot; each lane quantises the two
// activation chunks it is responsible for (the gate/up kernel's fp16 output) once, straight from
// global memory, and keeps them for the whole kernel.  All consumer warps work on the same tile
// (6 output rows x all slots; warp (slot, h) takes rows h, h+2, h+4), so every ring stage ahead of it
// is look-ahead.  Taller tiles mean larger bulk copies (6 KB of codes and 768 B of scales per slot):
// the copy engine's rate drops with copy size, and with 4-row tiles the ring itself, not the
// arithmetic, limited the kernel.  Per-row results y[row][slot] (rounded to fp16 as the reference's down projection)
// go to a small ring in shared memory; a separate combiner warp adds each row in plan order and
// writes the output.  The hand-over is by mbarriers (y-full: one arrival per consumer warp, y-empty:
// one arrival by the combiner), so consumer warps never wait for one another: they drift apart by
// up to the depth of the rings, and loads, integer math and shuffles of different warps overlap.
// stage layout: per slot [codes R*I/2][scales R*I/16], R = kDownRows.
// Two shapes (template parameters R = rows per tile, WPS = warps per slot): up to 9 slots R = 6, WPS = 2
// (measured on the Kimi shape with 9 slots: 4 rows 20.7 us, 5 rows 18.2 us, 6 rows 17.3-18.0 us, 8 rows
// 18.5 us); 10 to 17
// slots — the grouped launches of expert parallelism — R = 4, WPS = 1, so that two stages still fit.
// In grouped mode (MoeLayerArgs::slot_token) the slots are (token, expert) pairs in ascending token
// order and the combiner writes one output row per token.
constexpr int kDownYStages = 4;
constexpr int kDownTileRows = 6;      // rows of a tile in the fixed and (at most) in the run-time chosen shape
static_assert(kDownTileRows <= 32, "the combiner uses one lane per row of a tile");
constexpr int kDownMaxThreads = 640;  // 18 consumer warps for 9 slots + combiner + producer

// R = 0: tile height and warps per slot are chosen in the kernel from the number of ACTIVE slots (which
// may live in device memory): up to 9 slots 6 rows and 2 warps per slot, otherwise one warp per slot and
// 6 rows if two stages of that size fit, else 4 rows.  `ring` = bytes of the ring (R = 0) or its number
// of stages (R > 0).
template <int NCH, int R, int WPS>
__global__ void __launch_bounds__(kDownMaxThreads, 1) moe_down_pipe_kernel(MoeLayerArgs a, int ring) {
    constexpr bool kDyn = R == 0;
    constexpr int kRowsMax = kDyn ? kDownTileRows : R;
    constexpr int kDownRowsPerWarp = kDyn ? kDownTileRows : (R + (kDyn ? 1 : WPS) - 1) / (kDyn ? 1 : WPS);
    static_assert(kRowsMax <= kDownTileRows, "the host sizes the row ring for kDownTileRows rows");
    using MATH = MathQ16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int max_slots = a.top_k + (a.shared_pages ? 1 : 0);  // launch shape and shared-memory layout
    // The slot count may come from device memory; the kernel that wrote it had completed before the
    // gate/up kernel passed its dependency wait, like the expert ids (see below).
    // (An empty later window leaves only after its predecessor has completed, see the gate/up kernel.)
    if (a.slot_begin > 0 && a.num_active_dev && !a.shared_pages && a.out_accumulate && *a.num_active_dev <= a.slot_begin) {
        pdl_wait();
        return;
    }
    a.top_k = active_top_k(a);
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const unsigned code_row = (unsigned)a.I / 2, scale_row = (unsigned)a.I / 16;
    int rows_v = R, wps_v = WPS, nstages_v = ring;
    if (kDyn) {
        const unsigned row_bytes = code_row + scale_row;
        wps_v = slots <= 9 ? 2 : 1;
        rows_v = (slots <= 9 || 2u * slots * kDownTileRows * row_bytes <= (unsigned)ring) ? kDownTileRows : 4;
        nstages_v = min(kMaxStages, ring / max(1, (int)(slots * rows_v * row_bytes)));
    }
    const int kDownRows = rows_v, kDownWarpsPerSlot = wps_v, nstages = nstages_v;
    const int cwarps = slots * kDownWarpsPerSlot;       // consumer warps in use
    const int producer_warp = (int)(blockDim.x >> 5) - 1;
    const int combiner_warp = producer_warp - 1;
    const unsigned slot_bytes = kDownRows * (code_row + scale_row);
    const unsigned stage_bytes = (kDyn ? slots : max_slots) * slot_bytes;

    // fixed-size parts first, the ring (whose stage size may depend on the active slots) last
    PageEntry* tab = reinterpret_cast<PageEntry*>(smem_raw);
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + max_slots * a.P);
    uint64_t* empty = full + kMaxStages;
    uint64_t* yfull = empty + kMaxStages;
    uint64_t* yempty = yfull + kDownYStages;
    uint64_t* act_read = yempty + kDownYStages;  // one arrival per consumer warp once its activations are in registers
    float* wts = reinterpret_cast<float*>(act_read + 1);
    int* toks = reinterpret_cast<int*>(wts + kMaxSlots);  // grouped mode: token of each routed slot
    float* ybuf = reinterpret_cast<float*>(toks + kMaxSlots);  // [y stage][row][kMaxSlots]
    unsigned char* stages = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(ybuf + kDownYStages * kRowsMax * kMaxSlots) + 127) & ~(uintptr_t)127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The next kernel in the stream may overwrite the activation scratch before its own dependency
    // wait (the gate/up kernel does, for the shared expert).  It may therefore be let go only when every
    // consumer warp of this CTA has copied its chunks into registers: the warps arrive on `act_read` and
    // ONE thread, the combiner's first lane, issues the trigger for the CTA.
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, max(cwarps, 1));
        }
        for (int s = 0; s < kDownYStages; ++s) {
            mbar_init(yfull + s, max(cwarps, 1));
            mbar_init(yempty + s, 1);
        }
        mbar_init(act_read, max(cwarps, 1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Expert ids and routing weights were written by the router.  This kernel is launched only after
    // every thread of the gate/up kernel has passed its own wait for the router, so they are complete
    // and visible here without waiting.
    for (int i = tid; i < slots * a.P; i += blockDim.x) {
        const int s = i / a.P, p = i - s * a.P;
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[kSegDown * a.P + p];
        tab[i] = e;
    }
    for (int s = tid; s < slots; s += blockDim.x) {
        wts[s] = s < a.top_k ? __ldcg(a.expert_weights + s) : a.shared_weight;
        toks[s] = a.slot_token ? (s < a.top_k ? (int)a.slot_token[s] : a.shared_token) : 0;
    }
    __syncthreads();

    int g0, g1;
    cta_share(a.H, g0, g1);

    if (slots == 0) {  // nothing selected: the layer output is zero
        pdl_wait();  // (end only after the predecessor)
        if (!a.out_accumulate)
            for (int tk = 0; tk < (a.slot_token ? a.n_tokens : 1); ++tk)
                for (int r = g0 + tid; r < g1; r += blockDim.x) a.out[(size_t)tk * a.out_stride + r] = 0.f;
        return;
    }
    if (warp < combiner_warp && warp >= cwarps) return;  // warps of unused slots

    if (warp == producer_warp) {
        // ── producer warp: the weights do not depend on the previous kernel, so streaming starts at
        // once.  Lane k < 2 * slots issues copy k of a tile (slot k / 2: codes for even k, scales for
        // odd k); the byte total is summed across lanes for lane 0 to arm the barrier ──
        TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownRows);
        Tile t;
        int n = 0;
        bool ok = true;
        while (walk.next(t)) {
            const int st = n % nstages;
            if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
            if (!ok) break;
            unsigned char* sb = stages + (size_t)st * stage_bytes;
            // slots lane / 2 and (the 17th slot) 16 + lane / 2
            constexpr int kHalves = kDyn ? 2 : 1;  // a launch of fixed shape has at most 9 slots
            PageEntry e[kHalves];
            unsigned bytes[kHalves];
            unsigned tx = 0;
#pragma unroll
            for (int u = 0; u < kHalves; ++u) {
                bytes[u] = 0u;
                if (u == 1 && slots <= 16) break;  // (the same for every lane)
                const int s = u * 16 + (lane >> 1);
                e[u] = PageEntry{0, 0, 0, 0};
                if (s < slots) e[u] = tab[s * a.P + t.page];
                const bool mine = s < slots && e[u].ptr != 0 && t.rin + t.nrows <= e[u].row_count;
                bytes[u] = mine ? ((lane & 1) ? t.nrows * scale_row : t.nrows * code_row) : 0u;
                tx += bytes[u];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
            if (lane == 0) {
                if (tx) mbar_expect_tx(full + st, tx);
                else mbar_arrive(full + st);
            }
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kHalves; ++u) {
                if (bytes[u]) {
                    const int s = u * 16 + (lane >> 1);
                    const unsigned char* base = reinterpret_cast<const unsigned char*>(e[u].ptr);
                    if (lane & 1) bulk_load(sb + s * slot_bytes + kDownRows * code_row, base + (size_t)e[u].row_count * code_row + (size_t)t.rin * scale_row, bytes[u], full + st);
                    else bulk_load(sb + s * slot_bytes, base + (size_t)t.rin * code_row, bytes[u], full + st);
                }
            }
            ++n;
        }
        if (!ok && lane == 0) flag(a.status, kStatusTimeout);
        if (lane == 0)
            for (int k = max(0, n - nstages); k < n; ++k)
                if (!mbar_wait(full + (k % nstages), (k / nstages) & 1)) flag(a.status, kStatusTimeout);
        return;
    }

    if (warp == combiner_warp) {
        // ── combiner warp: lane r adds row r of each tile over the slots, in plan order ──
        if (lane == 0) {
            if (!mbar_wait(act_read, 0)) flag(a.status, kStatusTimeout);
            pdl_trigger();
        }
        __syncwarp();
        TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownRows);
        Tile t;
        int n = 0;
        while (walk.next(t)) {
            const int ys = n % kDownYStages;
            if (!mbar_wait(yfull + ys, (n / kDownYStages) & 1)) {
                if (lane == 0) flag(a.status, kStatusTimeout);
                return;
            }
            if (lane < t.nrows) {
                const float* yb = ybuf + ys * (kRowsMax * kMaxSlots) + lane * kMaxSlots;
                const int r = t.row + lane;
                if (a.slot_token == nullptr) {
                    float out = 0.f;
                    for (int k = 0; k < slots; ++k) out = fmaf(wts[k], yb[k], out);
                    if (a.out_accumulate) a.out[r] += out;
                    else a.out[r] = out;
                } else {
                    // one output row per token: its routed pairs in list order, then the shared expert
                    int k = 0;
                    for (int tk = 0; tk < a.n_tokens; ++tk) {
                        float out = 0.f;
                        while (k < a.top_k && toks[k] == tk) {
                            out = fmaf(wts[k], yb[k], out);
                            ++k;
                        }
                        if (a.shared_pages && tk == a.shared_token) out = fmaf(wts[a.top_k], yb[a.top_k], out);
                        float* o = a.out + (size_t)tk * a.out_stride + r;
                        if (a.out_accumulate) *o += out;
                        else *o = out;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(yempty + ys);
            ++n;
        }
        return;
    }

    // ── consumers: warp (s, h) keeps slot s's activation chunks in registers ──
    const int s = warp / kDownWarpsPerSlot, h = warp % kDownWarpsPerSlot;
    pdl_wait();  // the activations are the gate/up kernel's output
    uint4 xv[NCH][4];
    float sx[NCH];
    int sq8[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i)
        MATH::quantize_chunk(a.act + (size_t)act_slot(a, s) * a.I + (size_t)(lane + 32 * i) * 32, xv[i], sx[i], sq8[i]);
    // the scratch has been read: the sums below depend on every loaded value, so the loads have returned
#pragma unroll
    for (int i = 0; i < NCH; ++i) asm volatile("" ::"r"(sq8[i]));
    __syncwarp();
    if (lane == 0) mbar_arrive(act_read);

    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t code_base = s * slot_bytes + lane * 16;
    const uint32_t scale_base = s * slot_bytes + kDownRows * code_row + lane * 2;
    TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownRows);
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        const int st = n % nstages;
        if (!mbar_wait(full + st, (n / nstages) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        const PageEntry e = tab[s * a.P + t.page];
        const bool present = e.ptr != 0 && t.rin + t.nrows <= e.row_count;
        const uint32_t sb = stages_addr + st * stage_bytes;
        float y[kDownRowsPerWarp];
#pragma unroll
        for (int j = 0; j < kDownRowsPerWarp; ++j) {
            const int r = h + j * kDownWarpsPerSlot;
            float acc = 0.f;
            if (r < kDownRows && r < t.nrows && present) {
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const uint4 q = lds128(sb + code_base + r * code_row + i * 512);
                    const float sc = scale_to_f32(lds16(sb + scale_base + r * scale_row + i * 64));
                    acc = MATH::chunk_r(q, sc, xv[i], sx[i], sq8[i], acc);
                }
            }
            y[j] = acc;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + st);  // this warp has read everything it needs from the stage
#pragma unroll
        for (int j = 0; j < kDownRowsPerWarp; ++j)
            if (h + j * kDownWarpsPerSlot < kDownRows) y[j] = warp_sum(y[j]);
        if (!present && h == 0 && lane == 0) flag(a.status, kStatusMissingPage);
        const int ys = n % kDownYStages;
        if (n >= kDownYStages && !mbar_wait(yempty + ys, ((n / kDownYStages) - 1) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        if (lane == 0) {
            float* yb = ybuf + ys * (kRowsMax * kMaxSlots);
            // fp16 rounding of the down projection (its output buffer is fp16 in the reference)
#pragma unroll
            for (int j = 0; j < kDownRowsPerWarp; ++j)
                if (h + j * kDownWarpsPerSlot < kDownRows) yb[(h + j * kDownWarpsPerSlot) * kMaxSlots + s] = __half2float(__float2half_rn(y[j]));
            mbar_arrive(yfull + ys);
        }
        ++n;
    }
}

// ── down for wide experts: K split across warps ───────────────────────────────────────────────
// When an expert's activations do not fit in two chunks per lane (I > 2048; the Mixtral shape has I = 14336) the
// K range of a slot is split: warp (slot, ks) keeps chunks 64 ks + lane and 64 ks + 32 + lane of the slot's
// activations in registers and forms, for every row of a tile, the partial sum over its 2048 columns; the combiner
// adds a row's partials in ks order (fp32), rounds the row to fp16 as the reference's down projection does, and
// accumulates the slots in plan order.  (The partial sums change the fp32 association against the direct-load
// kernel, which runs one chain per lane over the whole row: results agree to rounding, not bit for bit.)
// slots * KS consumer warps (at most 16), one combiner, one producer.  Tiles of 4 rows x all slots.
// Not for grouped launches.
constexpr int kDownKsRows = 4;

__global__ void __launch_bounds__(kDownMaxThreads, 1) moe_down_ksplit_kernel(MoeLayerArgs a, int nstages, int KS) {
    using MATH = MathQ16;
    constexpr int NCH = 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int max_slots = a.top_k + (a.shared_pages ? 1 : 0);
    a.top_k = active_top_k(a);
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const unsigned code_row = (unsigned)a.I / 2, scale_row = (unsigned)a.I / 16;
    const int cwarps = slots * KS;
    const int producer_warp = (int)(blockDim.x >> 5) - 1;
    const int combiner_warp = producer_warp - 1;
    const unsigned slot_bytes = kDownKsRows * (code_row + scale_row);
    const unsigned stage_bytes = max_slots * slot_bytes;

    PageEntry* tab = reinterpret_cast<PageEntry*>(smem_raw);
    uint64_t* full = reinterpret_cast<uint64_t*>(tab + max_slots * a.P);
    uint64_t* empty = full + kMaxStages;
    uint64_t* yfull = empty + kMaxStages;
    uint64_t* yempty = yfull + kDownYStages;
    uint64_t* act_read = yempty + kDownYStages;
    float* wts = reinterpret_cast<float*>(act_read + 1);
    float* ybuf = wts + kMaxSlots;   // [y stage][row][kMaxSlots]: partial (slot, ks) at slot * KS + ks
    unsigned char* stages = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(ybuf + kDownYStages * kDownKsRows * kMaxSlots) + 127) & ~(uintptr_t)127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, max(cwarps, 1));
        }
        for (int s = 0; s < kDownYStages; ++s) {
            mbar_init(yfull + s, max(cwarps, 1));
            mbar_init(yempty + s, 1);
        }
        mbar_init(act_read, max(cwarps, 1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // (the routing is complete and visible: this kernel is launched only after every thread of the gate/up kernel has
    // passed its own wait for the router)
    for (int i = tid; i < slots * a.P; i += blockDim.x) {
        const int s = i / a.P, p = i - s * a.P;
        const PageEntry* pg = slot_pages(a, s);
        PageEntry e{0, 0, 0, 0};
        if (pg) e = pg[kSegDown * a.P + p];
        tab[i] = e;
    }
    for (int s = tid; s < slots; s += blockDim.x) wts[s] = s < a.top_k ? __ldcg(a.expert_weights + s) : a.shared_weight;
    __syncthreads();

    int g0, g1;
    cta_share(a.H, g0, g1);
    if (slots == 0) {
        pdl_wait();
        if (!a.out_accumulate)
            for (int r = g0 + tid; r < g1; r += blockDim.x) a.out[r] = 0.f;
        return;
    }
    if (warp < combiner_warp && warp >= cwarps) return;

    if (warp == producer_warp) {
        TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownKsRows);
        Tile t;
        int n = 0;
        bool ok = true;
        while (walk.next(t)) {
            const int st = n % nstages;
            if (n >= nstages) ok = mbar_wait(empty + st, ((n / nstages) - 1) & 1);
            if (!ok) break;
            unsigned char* sb = stages + (size_t)st * stage_bytes;
            // lane k < 2 * slots issues copy k of the tile (slot k / 2: codes for even k, scales for odd k)
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
            if (bytes) {
                const unsigned char* base = reinterpret_cast<const unsigned char*>(e.ptr);
                if (lane & 1) bulk_load(sb + s * slot_bytes + kDownKsRows * code_row, base + (size_t)e.row_count * code_row + (size_t)t.rin * scale_row, bytes, full + st);
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

    if (warp == combiner_warp) {
        if (lane == 0) {
            if (!mbar_wait(act_read, 0)) flag(a.status, kStatusTimeout);
            pdl_trigger();
        }
        __syncwarp();
        TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownKsRows);
        Tile t;
        int n = 0;
        while (walk.next(t)) {
            const int ys = n % kDownYStages;
            if (!mbar_wait(yfull + ys, (n / kDownYStages) & 1)) {
                if (lane == 0) flag(a.status, kStatusTimeout);
                return;
            }
            if (lane < t.nrows) {
                const float* yb = ybuf + ys * (kDownKsRows * kMaxSlots) + lane * kMaxSlots;
                float out = 0.f;
                for (int s = 0; s < slots; ++s) {
                    float y = 0.f;
                    for (int k = 0; k < KS; ++k) y += yb[s * KS + k];
                    out = fmaf(wts[s], __half2float(__float2half_rn(y)), out);
                }
                const int r = t.row + lane;
                if (a.out_accumulate) a.out[r] += out;
                else a.out[r] = out;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(yempty + ys);
            ++n;
        }
        return;
    }

    // ── consumers: warp (s, ks) ──
    const int s = warp / KS, ks = warp - s * KS;
    pdl_wait();  // the activations are the gate/up kernel's output
    uint4 xv[NCH][4];
    float sx[NCH];
    int sq8[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i)
        MATH::quantize_chunk(a.act + (size_t)act_slot(a, s) * a.I + (size_t)(64 * ks + lane + 32 * i) * 32, xv[i], sx[i], sq8[i]);
#pragma unroll
    for (int i = 0; i < NCH; ++i) asm volatile("" ::"r"(sq8[i]));
    __syncwarp();
    if (lane == 0) mbar_arrive(act_read);

    const uint32_t stages_addr = smem_u32(stages);
    const uint32_t code_base = s * slot_bytes + (64 * ks + lane) * 16;
    const uint32_t scale_base = s * slot_bytes + kDownKsRows * code_row + (64 * ks + lane) * 2;
    TileWalk walk(g0, g1, a.H, a.rpp_dn, kDownKsRows);
    Tile t;
    int n = 0;
    while (walk.next(t)) {
        const int st = n % nstages;
        if (!mbar_wait(full + st, (n / nstages) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        const PageEntry e = tab[s * a.P + t.page];
        const bool present = e.ptr != 0 && t.rin + t.nrows <= e.row_count;
        const uint32_t sb = stages_addr + st * stage_bytes;
        float y[kDownKsRows];
#pragma unroll
        for (int r = 0; r < kDownKsRows; ++r) {
            float acc = 0.f;
            if (r < t.nrows && present) {
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const uint4 q = lds128(sb + code_base + r * code_row + i * 512);
                    const float sc = scale_to_f32(lds16(sb + scale_base + r * scale_row + i * 64));
                    acc = MATH::chunk_r(q, sc, xv[i], sx[i], sq8[i], acc);
                }
            }
            y[r] = acc;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + st);
#pragma unroll
        for (int r = 0; r < kDownKsRows; ++r) y[r] = warp_sum(y[r]);
        if (!present && ks == 0 && lane == 0) flag(a.status, kStatusMissingPage);
        const int ys = n % kDownYStages;
        if (n >= kDownYStages && !mbar_wait(yempty + ys, ((n / kDownYStages) - 1) & 1)) {
            if (lane == 0) flag(a.status, kStatusTimeout);
            return;
        }
        if (lane == 0) {
            float* yb = ybuf + ys * (kDownKsRows * kMaxSlots);
#pragma unroll
            for (int r = 0; r < kDownKsRows; ++r) yb[r * kMaxSlots + warp] = y[r];
            mbar_arrive(yfull + ys);
        }
        ++n;
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────────

static bool pipe_shape_ok(const MoeLayerArgs& a) {
    return a.H % 256 == 0 && a.I % 256 == 0;
}

// Number of ring stages that fit, 0 = fewer than min_stages.
static int pick_stages(size_t fixed, size_t stage_bytes, int min_stages) {
    if (fixed >= kSmemBudget) return 0;
    int n = (int)((kSmemBudget - fixed) / stage_bytes);
    if (n > kMaxStages) n = kMaxStages;
    return n >= min_stages ? n : 0;
}

// Launch with the programmatic-stream-serialization attribute (g_use_pdl) or plainly.
template <class K, class... Args>
static int launch_pipe(K kernel, int grid, int threads, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <class K>
static int set_max_smem(K kernel) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int NCH, bool ROUTED>
static int launch_gateup_pipe_t(const MoeLayerArgs& a, const RouterArgs& r, cudaStream_t st, int nstages, size_t smem, int grid) {
    static int attr = set_max_smem(moe_gateup_pipe_kernel<NCH, ROUTED>);
    if (attr) return attr;
    return launch_pipe(moe_gateup_pipe_kernel<NCH, ROUTED>, grid, ROUTED ? kRoutedThreads : kPipeThreads, smem, st, a, r, nstages);
}

template <bool ROUTED>
static int launch_gateup_nch(const MoeLayerArgs& a, const RouterArgs& r, cudaStream_t st, int nstages, size_t smem, int grid) {
    const int nch = gateup_nch(a.H);
    switch (nch) {
        case 1: return launch_gateup_pipe_t<1, ROUTED>(a, r, st, nstages, smem, grid);
        case 2: return launch_gateup_pipe_t<2, ROUTED>(a, r, st, nstages, smem, grid);
        case 4: return launch_gateup_pipe_t<4, ROUTED>(a, r, st, nstages, smem, grid);
        case 7: return launch_gateup_pipe_t<7, ROUTED>(a, r, st, nstages, smem, grid);
        case 8: return launch_gateup_pipe_t<8, ROUTED>(a, r, st, nstages, smem, grid);
        default: return launch_gateup_pipe_t<0, ROUTED>(a, r, st, nstages, smem, grid);
    }
}

// router == nullptr: the routing (a.expert_ids / a.expert_weights) comes from an earlier kernel.
// Otherwise the kernel routes the token itself and CTA 0 stores the routing there; VIB3_ERR_UNSUPPORTED
// (nothing launched) when the router's rows do not fit the ring — the caller then launches the router separately.
int launch_gateup_pipelined(const MoeLayerArgs& a, cudaStream_t st, const RouterArgs* router) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    int nch = gateup_nch(a.H);
    if (nch != 1 && nch != 2 && nch != 4 && nch != 7 && nch != 8) nch = 0;   // the widths launch_gateup_nch instantiates
    const int tile_rows = gateup_tile_rows(nch);
    const size_t stage_bytes = 2 * tile_rows * ((size_t)a.H / 2 + (size_t)a.H / 16);
    size_t fixed = (size_t)(a.slot_token ? 2 : 1) * (a.H / kGroupSize) * MathQ16::kStride +
                   (size_t)slots * 2 * a.P * sizeof(PageEntry) +
                   (2 * kMaxStages + 1) * sizeof(uint64_t) + kMaxStages * sizeof(unsigned) + 128;
    const int total = slots * a.I;
    const int grid = min(sm_count(), (total + tile_rows - 1) / tile_rows);
    if (router) {
        const RouterArgs& r = *router;
        const size_t row_bytes = (size_t)r.H * (r.w_dtype == W_F32 ? 4 : 2);
        const size_t xraw = (size_t)a.H * (a.x_dtype == X_F32 ? 4 : 2);
        if (a.slot_token || a.num_active_dev || r.H != a.H || r.x != a.x || r.x_dtype != a.x_dtype) return VIB3_ERR_UNSUPPORTED;
        if (r.E > kRouterMaxExperts || r.H > kRouterXMax || r.H % 8 != 0 || row_bytes > stage_bytes) return VIB3_ERR_UNSUPPORTED;
        if (((uintptr_t)r.W & 15) || ((uintptr_t)r.x & 15)) return VIB3_ERR_UNSUPPORTED;
        fixed += ((xraw > kSeqRingFloats * sizeof(float) ? xraw : kSeqRingFloats * sizeof(float)) + 15) / 16 * 16 + sizeof(RoutedSmem) + 32;
        const int nstages = pick_stages(fixed, stage_bytes, 3);
        if (nstages == 0 || (r.E + grid - 1) / grid > nstages) return VIB3_ERR_UNSUPPORTED;
        return launch_gateup_nch<true>(a, r, st, nstages, fixed + (size_t)nstages * stage_bytes, grid);
    }
    // leave kRouterCtaSmem of the SM's shared memory to a router CTA, so that this kernel's CTAs become
    // resident while the router still runs (see the kernel's first pass)
    int nstages = pick_stages(fixed + kRouterCtaSmem, stage_bytes, 3);
    if (nstages == 0) nstages = pick_stages(fixed, stage_bytes, 3);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    return launch_gateup_nch<false>(a, RouterArgs{}, st, nstages, fixed + (size_t)nstages * stage_bytes, grid);
}

template <int NCH, int R, int WPS>
static int launch_down_pipe_t(const MoeLayerArgs& a, cudaStream_t st, int nstages, size_t smem, int grid, int threads) {
    static int attr = set_max_smem(moe_down_pipe_kernel<NCH, R, WPS>);
    if (attr) return attr;
    return launch_pipe(moe_down_pipe_kernel<NCH, R, WPS>, grid, threads, smem, st, a, nstages);
}

int launch_down_pipelined(const MoeLayerArgs& a, cudaStream_t st) {
    if (!pipe_shape_ok(a)) return VIB3_ERR_UNSUPPORTED;
    const int slots = a.top_k + (a.shared_pages ? 1 : 0);
    const int nchunks = a.I / kGroupSize;
    const size_t row_bytes = (size_t)a.I / 2 + (size_t)a.I / 16;
    // register-resident activations: at most two chunks per lane; wider experts split K across warps
    if (nchunks > 64) {
        const int KS = nchunks / 64;
        if (nchunks % 64 || a.slot_token || slots * KS > 16 || slots * KS > kMaxSlots) return VIB3_ERR_UNSUPPORTED;
        const size_t fixed_ks = (size_t)slots * a.P * sizeof(PageEntry) + (2 * (kMaxStages + kDownYStages) + 1) * sizeof(uint64_t) +
                                kMaxSlots * sizeof(float) + kDownYStages * kDownKsRows * kMaxSlots * sizeof(float) + 256;
        const size_t stage_ks = (size_t)slots * kDownKsRows * row_bytes;
        const int nst = pick_stages(fixed_ks, stage_ks, 2);
        if (nst == 0) return VIB3_ERR_UNSUPPORTED;
        static const int attr = set_max_smem(moe_down_ksplit_kernel);
        if (attr) return attr;
        const int grid_ks = min(sm_count(), (a.H + kDownKsRows - 1) / kDownKsRows);
        return launch_pipe(moe_down_ksplit_kernel, grid_ks, (slots * KS + 2) * 32, fixed_ks + (size_t)nst * stage_ks, st, a, nst, KS);
    }
    if (nchunks != 32 && nchunks != 64) return VIB3_ERR_UNSUPPORTED;
    const size_t fixed = (size_t)slots * a.P * sizeof(PageEntry) + (2 * (kMaxStages + kDownYStages) + 1) * sizeof(uint64_t) +
                         2 * kMaxSlots * sizeof(float) + kDownYStages * kDownTileRows * kMaxSlots * sizeof(float) + 256;
    if (slots > 9) {
        // Launch sized for up to 17 slots; how many are active is known only on the device, and the kernel
        // picks tile height, warps per slot and ring depth from that number.
        if (slots > kMaxSlots || fixed + 2 * (size_t)slots * 4 * row_bytes > kSmemBudget) return VIB3_ERR_UNSUPPORTED;
        const int ring = (int)(kSmemBudget - fixed);
        const int grid = min(sm_count(), (a.H + 3) / 4);
        return nchunks == 64 ? launch_down_pipe_t<2, 0, 0>(a, st, ring, kSmemBudget, grid, kDownMaxThreads)
                             : launch_down_pipe_t<1, 0, 0>(a, st, ring, kSmemBudget, grid, kDownMaxThreads);
    }
    constexpr int rows = kDownTileRows, wps = 2;
    const size_t stage_bytes = (size_t)slots * rows * row_bytes;
    const int nstages = pick_stages(fixed, stage_bytes, 2);
    if (nstages == 0) return VIB3_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)nstages * stage_bytes;
    const int grid = min(sm_count(), (a.H + rows - 1) / rows);
    const int threads = (slots * wps + 2) * 32;
    return nchunks == 64 ? launch_down_pipe_t<2, rows, wps>(a, st, nstages, smem, grid, threads)
                         : launch_down_pipe_t<1, rows, wps>(a, st, nstages, smem, grid, threads);
}

}  // namespace vib3
