// Router: logits GEMV, scoring (softmax / sigmoid), stable top-k, normalise and scale.
//
// Reference entry points kept with identical signatures:
//   vib3_launch_router_gemv       cuda/src/kernels.cu:1143  (x fp16, W fp16)
//   vib3_launch_router_gemv_f32   cuda/src/kernels.cu:1477  (x fp32, W fp16)
//   vib3_launch_router_topk       cuda/src/kernels.cu:4075  (GEMV + top-k, results stay on device)
// and one extended launcher, vib3_launch_router_topk_ex, that also accepts fp32 router weights
// and fp16/bf16 activations, any expert count up to 512 (the reference's bitonic kernel needs a
// power of two, kernels.cu:3899), and leaves ids and weights on the device in one call.
//
// Summation order of the logits: exactly the reference CUDA kernel's (kernels.cu:665-707) — 128
// chains per expert, chain t adds d = t, t+128, ... with fused multiply-add, a shfl_down tree
// per group of 32 chains, then (s0+s2)+(s1+s3) — so logits are bit-identical to the reference's on
// a GPU.  The work split is different: ONE warp per expert row, lane l owns the four chains
// 4l .. 4l+3, so that a lane's accesses are 16 bytes wide (fp32 weights) and a warp's cover 512
// contiguous bytes.  Two implementations of that split:
//   * rows-resident (the usual case: H a multiple of 8, aligned operands): a CTA brings three
//     expert rows into shared memory with one bulk copy each — requested before the kernel waits
//     for the producer of the token, so the weights travel under the previous kernel's tail — and
//     forms the logits of every token of the launch from there; a second launch (one CTA per token)
//     scores and selects.  The weights cross the memory system once per launch, not once per token.
//   * direct (any H, any alignment): rows read straight from global memory, 28 loads of a lane in
//     flight; the CTA that finishes last scores and selects.
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
// chain per expert (the CPU order) before the final selection (router_core.cuh).  This costs about
// 20 microseconds and happens for a few percent of tokens.
#include "pipe_common.cuh"
#include "router_core.cuh"

namespace vib3 {

constexpr int kRouterWarps = 3;         // expert rows per CTA, one warp each
constexpr int kRouterThreads = kRouterWarps * 32;
constexpr int kLoadGroups = 4;          // register groups of weight loads a lane keeps in flight ...
constexpr int kGroupLoads = 7;          // ... and 16-byte loads per group
constexpr int kInFlight = kLoadGroups * kGroupLoads;  // 28: half a 7168-wide fp32 row

// GEMV: one warp per expert row, kRouterWarps rows per CTA.  When `a.counter` is set, the CTA that
// finishes last also does the scoring and selection (one launch).  The direct path; see the rows-resident one below.
// XD >= 0: the vector path — H a multiple of 8 (fp32 x: of 4) and at most kRouterXMax, x and the rows of W
// 16-byte (fp16 W: 8-byte) aligned.  A lane first requests kInFlight weight items; the CTA then copies the
// activation vector as it is into shared memory with asynchronous 16-byte copies (no registers, nothing
// waits for anything until the barrier), and from then on a lane issues one new weight load per item it
// consumes.  XD < 0: any H, any alignment, x of the run-time dtype: the same chains with scalar loads.
template <int XD, int WD>
__global__ void __launch_bounds__(kRouterThreads) router_kernel(RouterArgs a) {
    __shared__ TopKSmem sm;
    __shared__ __align__(16) float xbuf[kRouterXMax];   // the activation vector; later the ring of a recomputation
    __shared__ int is_last;
    static_assert(kSeqRingFloats <= kRouterXMax, "the recomputation ring reuses the activation buffer");
    // let a dependent kernel (launched with programmatic stream serialization) begin its prologue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    router_args_of_token(a, blockIdx.y);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int expert = blockIdx.x * kRouterWarps + warp;
    const int row = min(expert, a.E - 1);  // every warp reaches the barrier below
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float aabs[4] = {0.f, 0.f, 0.f, 0.f};
    if (XD >= 0) {
        using WI = WItem<WD>;
        const void* wrow = reinterpret_cast<const unsigned char*>(a.W) + (size_t)row * a.H * (WD == W_F32 ? 4 : 2);
        const int n4 = a.H >> 2;                 // 4-column items of the row; lane l takes items l, l + 32, ...
        const int nj = (n4 - lane + 31) >> 5;    // this lane's items
        // Loads in flight are kept in kLoadGroups register groups that are consumed and refilled group by
        // group: a wait for one load also waits for every younger load that shares its scoreboard, so a
        // load must not share one with loads issued after it was due.
        typename WI::T w[kLoadGroups][kGroupLoads];
#pragma unroll
        for (int g = 0; g < kLoadGroups; ++g)
#pragma unroll
            for (int i = 0; i < kGroupLoads; ++i)
                if (g * kGroupLoads + i < nj) w[g][i] = WI::load(wrow, lane + 32 * (g * kGroupLoads + i));
        unsigned char* xraw = reinterpret_cast<unsigned char*>(xbuf);
        {
            const int n16 = (a.H * (XD == X_F32 ? 4 : 2)) >> 4;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xraw);
            const unsigned char* src = reinterpret_cast<const unsigned char*>(a.x);
            for (int i = tid; i < n16; i += kRouterThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * i), "l"(src + 16 * (size_t)i) : "memory");
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        for (int j0 = 0; j0 < nj; j0 += kInFlight) {
#pragma unroll
            for (int g = 0; g < kLoadGroups; ++g) {
#pragma unroll
                for (int i = 0; i < kGroupLoads; ++i) {
                    const int j = j0 + g * kGroupLoads + i;
                    if (j < nj) {
                        const float4 wv = WI::cvt(w[g][i]);
                        const float4 xv = x_item<XD < 0 ? 0 : XD>(xraw, lane + 32 * j);
                        acc[0] = fmaf(xv.x, wv.x, acc[0]);
                        acc[1] = fmaf(xv.y, wv.y, acc[1]);
                        acc[2] = fmaf(xv.z, wv.z, acc[2]);
                        acc[3] = fmaf(xv.w, wv.w, acc[3]);
                        aabs[0] += fabsf(xv.x * wv.x);
                        aabs[1] += fabsf(xv.y * wv.y);
                        aabs[2] += fabsf(xv.z * wv.z);
                        aabs[3] += fabsf(xv.w * wv.w);
                    }
                }
#pragma unroll
                for (int i = 0; i < kGroupLoads; ++i) {
                    const int jn = j0 + g * kGroupLoads + i + kInFlight;
                    if (jn < nj) w[g][i] = WI::load(wrow, lane + 32 * jn);
                }
            }
        }
    } else {
        const bool staged = a.H <= kRouterXMax;
        if (staged)
            for (int d = tid; d < a.H; d += kRouterThreads) xbuf[d] = load_x_as_f32(a.x, a.x_dtype, d);
        __syncthreads();
        const size_t base = (size_t)row * a.H;
        for (int d0 = 4 * lane; d0 < a.H; d0 += 128) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int d = d0 + c;
                if (d < a.H) {
                    const float wv = load_w(a.W, WD, base + d);
                    const float xv = staged ? xbuf[d] : load_x_as_f32(a.x, a.x_dtype, d);
                    acc[c] = fmaf(xv, wv, acc[c]);
                    aabs[c] += fabsf(xv * wv);
                }
            }
        }
    }
    float logit = chain_tree(acc);
    const float absum = warp_total((aabs[0] + aabs[1]) + (aabs[2] + aabs[3]));
    if (lane == 0 && expert < a.E) {
        if (a.logit_offset) logit = __fadd_rn(logit, a.logit_offset[expert]);
        a.scores[expert] = logit;
        if (a.exact_order) a.scores[a.E + expert] = absum;
        // single launch, sigmoid scoring: the double-precision exponential runs here, in parallel over
        // the CTAs, instead of in the last CTA's serial tail
        if (a.counter != nullptr && a.mode != 0) a.scores[2 * a.E + expert] = sigmoid_ref(logit);
    }
    if (a.counter == nullptr) return;
    __syncthreads();
    if (tid == 0) {
        // release this CTA's logits and acquire everybody else's in one operation
        unsigned int ticket;
        asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(a.counter) : "memory");
        is_last = ticket == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    if (tid == 0) topk_smem_init(sm, kRouterWarps - 1);
    __syncthreads();
    router_finish(a, sm, xbuf, tid, kRouterThreads, a.mode != 0, true, nullptr, nullptr);
    if (tid == 0) *a.counter = 0u;  // ready for the next launch
}

__global__ void __launch_bounds__(kRouterThreads) router_topk_kernel(RouterArgs a) {
    __shared__ TopKSmem sm;
    __shared__ __align__(16) float ring[kSeqRingFloats];
    if (threadIdx.x == 0) topk_smem_init(sm, kRouterWarps - 1);
    __syncthreads();
    router_finish(a, sm, ring, threadIdx.x, kRouterThreads, false, true, nullptr, nullptr);
}

// ── rows-resident router ─────────────────────────────────────────────────────────────────────
// The vector path of the router as two launches that follow one another by programmatic dependent launch.
//
// router_rows_kernel: a CTA takes kRowsPerCta expert rows.  Its first thread requests the rows with one bulk
// copy each into shared memory BEFORE the kernel waits for its predecessor (the router's weights are constants:
// the copies run under the tail of the kernel that produces the token), so every byte of a row is in flight at
// once and a logit costs one memory round trip.  The tokens' vectors are staged with asynchronous 16-byte
// copies, tok_chunk tokens at a time in two buffers; warp (row, slot) forms the logit of its row for token
// slot of the chunk, in the reference kernel's order (row_logit_smem).  With several tokens the rows stay in
// shared memory: the router's weights cross the memory system once per launch, not once per token.
// The kernel needs most of an SM's shared memory, so it does not share an SM with the expert kernel; it is
// short, and the expert kernel's CTAs start as its CTAs leave.
//
// router_select_kernel: one CTA per token scores, selects and writes ids and weights (router_finish).  It lets
// its own dependents start at once — the expert kernel streams the shared expert meanwhile — and then waits
// for the logits.
//
// A wait that runs out sets workspace word 3 (when a workspace is given) and leaves.
constexpr int kRowsPerCta = 3;
constexpr int kTokSlots = 4;            // tokens of a chunk worked on side by side
constexpr int kRowsThreads = kRowsPerCta * kTokSlots * 32;

template <int XD, int WD>
__global__ void __launch_bounds__(kRowsThreads) router_rows_kernel(RouterArgs a, int n_tokens, int tok_chunk) {
    extern __shared__ __align__(128) unsigned char rsm[];
    const unsigned row_bytes = (unsigned)a.H * (WD == W_F32 ? 4u : 2u);
    const unsigned xbytes = (unsigned)a.H * (XD == X_F32 ? 4u : 2u);
    unsigned char* rows = rsm;
    unsigned char* xb = rows + kRowsPerCta * row_bytes;                             // [2][tok_chunk][xbytes]
    uint64_t* full = reinterpret_cast<uint64_t*>(xb + 2u * tok_chunk * xbytes);     // one barrier per row
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int e0 = blockIdx.x * kRowsPerCta;
    const int nrows = min(kRowsPerCta, a.E - e0);
    if (tid == 0) {
        if (!a.hold_dependents) pdl_trigger();
        for (int r = 0; r < nrows; ++r) mbar_init(full + r, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int r = 0; r < nrows; ++r) {
            mbar_expect_tx(full + r, row_bytes);
            bulk_load(rows + (size_t)r * row_bytes, reinterpret_cast<const unsigned char*>(a.W) + (size_t)(e0 + r) * row_bytes, row_bytes, full + r);
        }
    }
    __syncthreads();
    pdl_wait();   // the tokens are the predecessor's output
    // A predecessor that let this kernel start early is still writing the tokens until here, and the expert kernel
    // two launches on reads them before its own wait: then the chain behind this kernel starts only now.
    if (a.hold_dependents && tid == 0) pdl_trigger();
    const int nchunks = (n_tokens + tok_chunk - 1) / tok_chunk;
    const int n16 = (int)(xbytes >> 4);
    auto stage = [&](int c) {
        const int t0 = c * tok_chunk, nt = min(tok_chunk, n_tokens - t0);
        const uint32_t dst = smem_u32(xb + (size_t)(c & 1) * tok_chunk * xbytes);
        for (int i = tid; i < nt * n16; i += kRowsThreads) {
            const int tk = i / n16, j = i - tk * n16;
            const unsigned char* src = reinterpret_cast<const unsigned char*>(a.x) + (size_t)(t0 + tk) * a.x_stride + 16 * (size_t)j;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + tk * xbytes + 16 * j), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0);
    const int ri = warp / kTokSlots, ts = warp % kTokSlots;
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
            stage(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int t = c * tok_chunk + ts;
        if (ri < nrows && ts < tok_chunk && t < n_tokens) {
            if (mbar_wait(full + ri, 0)) {
                float logit, absum;
                row_logit_smem<XD, WD>(rows + (size_t)ri * row_bytes, xb + ((size_t)(c & 1) * tok_chunk + ts) * xbytes, a.H, lane, logit, absum);
                if (lane == 0) {
                    const int e = e0 + ri;
                    float* sc = a.scores + (size_t)t * a.scores_stride;
                    if (a.logit_offset) logit = __fadd_rn(logit, a.logit_offset[e]);
                    sc[e] = logit;
                    if (a.exact_order) sc[a.E + e] = absum;
                    // single launch, sigmoid scoring: the double-precision exponential runs here, in parallel
                    if (a.counter != nullptr && a.mode != 0) sc[2 * a.E + e] = sigmoid_ref(logit);
                }
            } else if (lane == 0 && a.counter) {
                a.counter[(size_t)t * a.counter_stride + 3] = 1u;
            }
        }
        __syncthreads();   // the buffer is staged again two chunks later
    }
}

__global__ void __launch_bounds__(kRouterThreads) router_select_kernel(RouterArgs a) {
    __shared__ TopKSmem sm;
    __shared__ __align__(16) float ring[kSeqRingFloats];
    if (threadIdx.x == 0) {
        pdl_trigger();
        topk_smem_init(sm, kRouterWarps - 1);
    }
    router_args_of_token(a, blockIdx.x);
    pdl_wait();   // the logits are the rows kernel's output
    __syncthreads();
    router_finish(a, sm, ring, threadIdx.x, kRouterThreads, a.mode != 0, true, nullptr, nullptr);
}

template <class K, class... Args>
static int launch_router_pdl(K kernel, dim3 grid, int threads, size_t smem, cudaStream_t st, Args... args) {
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

// The rows-resident pair of launches; VIB3_ERR_UNSUPPORTED when the rows and two token buffers do not fit.
template <int XD, int WD>
static int launch_rows_t(const RouterArgs& a, cudaStream_t st, int n_tokens) {
    const size_t row_bytes = (size_t)a.H * (WD == W_F32 ? 4 : 2), xbytes = (size_t)a.H * (XD == X_F32 ? 4 : 2);
    int tok_chunk = n_tokens < kTokSlots ? n_tokens : kTokSlots;
    while (tok_chunk > 1 && kRowsPerCta * row_bytes + 2 * tok_chunk * xbytes + 64 > kSmemBudget) --tok_chunk;
    const size_t smem = kRowsPerCta * row_bytes + 2 * tok_chunk * xbytes + 64;
    if (smem > kSmemBudget) return VIB3_ERR_UNSUPPORTED;
    static const cudaError_t attr = cudaFuncSetAttribute(router_rows_kernel<XD, WD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    if (attr != cudaSuccess) return (int)attr;
    const dim3 grid((a.E + kRowsPerCta - 1) / kRowsPerCta);
    if (int e = launch_router_pdl(router_rows_kernel<XD, WD>, grid, kRowsThreads, smem, st, a, n_tokens, tok_chunk)) return e;
    if (a.counter == nullptr) return VIB3_OK;   // logits only
    return launch_router_pdl(router_select_kernel, dim3(n_tokens), kRouterThreads, 0, st, a);
}

template <int XD, int WD>
static int launch_router_t(const RouterArgs& a, cudaStream_t st, int n_tokens) {
    if (XD >= 0) {
        const int e = launch_rows_t<XD < 0 ? 0 : XD, WD>(a, st, n_tokens);
        if (e != VIB3_ERR_UNSUPPORTED) return e;
    }
    // The largest shared-memory carve-out: the gate/up kernel that follows sizes itself to fit beside one
    // router CTA on an SM, which only works if both want the same SM configuration.
    static const cudaError_t carve = cudaFuncSetAttribute(router_kernel<XD, WD>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                          (int)cudaSharedmemCarveoutMaxShared);
    (void)carve;
    const dim3 grid((a.E + kRouterWarps - 1) / kRouterWarps, n_tokens);
    router_kernel<XD, WD><<<grid, kRouterThreads, 0, st>>>(a);
    return (int)cudaGetLastError();
}

template <int WD>
static int launch_router_w(const RouterArgs& a, cudaStream_t st, int n_tokens) {
    const uintptr_t walign = WD == W_F32 ? 15 : 7;
    const bool vec = a.H % (a.x_dtype == X_F32 ? 4 : 8) == 0 && a.H <= kRouterXMax && ((uintptr_t)a.x & 15) == 0 &&
                     (a.x_stride & 15) == 0 && ((uintptr_t)a.W & walign) == 0;
    if (!vec) return launch_router_t<-1, WD>(a, st, n_tokens);
    if (a.x_dtype == X_F32) return launch_router_t<X_F32, WD>(a, st, n_tokens);
    if (a.x_dtype == X_F16) return launch_router_t<X_F16, WD>(a, st, n_tokens);
    return launch_router_t<X_BF16, WD>(a, st, n_tokens);
}

static int launch_router(const RouterArgs& a, cudaStream_t st, int n_tokens = 1) {
    if (a.w_dtype == W_F32) return launch_router_w<W_F32>(a, st, n_tokens);
    if (a.w_dtype == W_F16) return launch_router_w<W_F16>(a, st, n_tokens);
    return VIB3_ERR_UNSUPPORTED;
}

static int check_router(const RouterArgs& a) {
    if (!a.x || !a.W || !a.scores) return VIB3_ERR_NULL;
    if (a.H <= 0 || a.E <= 0) return VIB3_ERR_SHAPE;
    if (a.x_dtype < X_F32 || a.x_dtype > X_BF16) return VIB3_ERR_UNSUPPORTED;
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
    router_topk_kernel<<<1, kRouterThreads, 0, st>>>(a);
    return (int)cudaGetLastError();
}

namespace vib3 {
int launch_router_args(const RouterArgs& a, cudaStream_t st) { return launch_router(a, st); }
}  // namespace vib3

// Fill and validate the arguments of the single-launch router (shared with the expert kernel that routes
// in its own prologue).
namespace vib3 {
int make_router_args(const void* x, int x_dtype, const void* W, int w_dtype, float* scores_buf, const float* bias,
                     const float* logit_offset, unsigned short* out_ids, float* out_weights, int hidden_dim, int num_experts,
                     int top_k, int scoring_mode, float scaling_factor, int normalize, int exact_order,
                     unsigned int* workspace, RouterArgs& a) {
    a = RouterArgs{};
    a.x = x; a.x_dtype = x_dtype; a.W = W; a.w_dtype = w_dtype; a.scores = scores_buf; a.bias = bias;
    a.logit_offset = logit_offset;
    a.out_ids = out_ids; a.out_weights = out_weights; a.counter = workspace; a.H = hidden_dim; a.E = num_experts;
    a.top_k = top_k; a.mode = scoring_mode; a.scaling = scaling_factor; a.normalize = normalize;
    a.exact_order = exact_order & 1; a.hold_dependents = (exact_order >> 1) & 1;
    if (w_dtype != W_F16 && w_dtype != W_F32) return VIB3_ERR_UNSUPPORTED;
    if (int e = check_router(a)) return e;
    if (int e = check_topk(a)) return e;
    if (!workspace) return VIB3_ERR_NULL;
    return VIB3_OK;
}
}  // namespace vib3

// Extended launcher: one call (two launches chained by programmatic dependent launch; one on the direct path).  scores_buf holds 3E floats ([0, E) receives the logits, the rest is scratch);
// workspace is four 32-bit words, zero before the first call: [0] is an arrival counter that every
// call leaves at zero, [1] counts the near-tie recomputations done so far (diagnostics), [2] is used by
// vib3_launch_moe_layer_routed_int4_paged, [3] is spare.
extern "C" int vib3_launch_router_topk_ex(const void* x, int x_dtype, const void* W, int w_dtype, float* scores_buf,
                                          const float* bias, const float* logit_offset, unsigned short* out_ids,
                                          float* out_weights,
                                          int hidden_dim, int num_experts, int top_k, int scoring_mode,
                                          float scaling_factor, int normalize, int exact_order,
                                          unsigned int* workspace, void* stream) {
    RouterArgs a;
    if (int e = make_router_args(x, x_dtype, W, w_dtype, scores_buf, bias, logit_offset, out_ids, out_weights, hidden_dim,
                                 num_experts, top_k, scoring_mode, scaling_factor, normalize, exact_order, workspace, a)) return e;
    return launch_router(a, (cudaStream_t)stream);
}

// The extended launcher for n_tokens tokens in one call: token t reads x + t * x_stride_bytes
// and writes scores_buf + t * scores_stride (3E floats each), out_ids + t * ids_stride, out_weights + t *
// weights_stride, and uses the four workspace words at workspace + 4 t.  The router's weights are read once
// per call (rows-resident path; the direct path reads them from L2 for every token after the first).
extern "C" int vib3_launch_router_topk_batch(const void* x, int x_dtype, int x_stride_bytes, int n_tokens, const void* W, int w_dtype,
                                             float* scores_buf, int scores_stride, const float* bias, const float* logit_offset,
                                             unsigned short* out_ids, int ids_stride, float* out_weights, int weights_stride,
                                             int hidden_dim, int num_experts, int top_k, int scoring_mode, float scaling_factor,
                                             int normalize, int exact_order, unsigned int* workspace, void* stream) {
    RouterArgs a;
    if (int e = make_router_args(x, x_dtype, W, w_dtype, scores_buf, bias, logit_offset, out_ids, out_weights, hidden_dim,
                                 num_experts, top_k, scoring_mode, scaling_factor, normalize, exact_order, workspace, a)) return e;
    if (n_tokens <= 0 || n_tokens > 65535) return VIB3_ERR_COUNT;
    if (x_stride_bytes <= 0 || scores_stride < 3 * num_experts || ids_stride < top_k || weights_stride < top_k) return VIB3_ERR_SHAPE;
    a.x_stride = x_stride_bytes; a.scores_stride = scores_stride; a.ids_stride = ids_stride; a.weights_stride = weights_stride;
    a.counter_stride = 4;
    return launch_router(a, (cudaStream_t)stream, n_tokens);
}
