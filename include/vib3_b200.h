/*
 * C ABI of libvib3_cuda.so — the B200 (sm_100a) implementation of the vib3 INT4 MoE decode path.
 *
 * Conventions (the reference's, src/compute/cuda_ffi.rs:143-1066, cuda/src/kernels.cu:1040):
 *   - every launcher returns int: 0 launched; > 0 the cudaError_t of the launch; < 0 refused
 *     before any launch (VIB3_ERR_*);
 *   - the last argument of a launcher is a cudaStream_t passed as void* (NULL = default stream);
 *   - launchers never synchronise, never allocate and keep no state; all pointers are device
 *     pointers owned by the caller unless stated otherwise.
 *
 * INT4 page layout (src/compute/kernels.rs:94-98): `rows` rows of ceil(K/2) code bytes (low
 * nibble = even column, weight = (nibble - 8) * scale), then `rows` rows of ceil(K/group)
 * fp16 scales.
 */
#ifndef VIB3_B200_H
#define VIB3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VIB3_OK 0
#define VIB3_ERR_UNSUPPORTED (-1)
#define VIB3_ERR_COUNT (-2)
#define VIB3_ERR_NULL (-3)
#define VIB3_ERR_ALIGN (-4)
#define VIB3_ERR_SHAPE (-5)
#define VIB3_ERR_RANGE (-6)
#define VIB3_ERR_STATE (-7)
#define VIB3_ERR_CAPACITY (-8)

/* activation dtypes (x_dtype) and router-weight dtypes (w_dtype) */
#define VIB3_X_F32 0
#define VIB3_X_F16 1
#define VIB3_X_BF16 2
#define VIB3_W_F16 0
#define VIB3_W_F32 1

/* bits of the device status word written by the paged kernels */
#define VIB3_STATUS_MISSING_PAGE 1
#define VIB3_STATUS_BAD_EXPERT 2
#define VIB3_STATUS_TIMEOUT 4       /* a bounded wait inside a kernel gave up */

/* ── Entry points with the reference's signatures ───────────────────────────────────────── */

/* replaces cuda/src/kernels.cu:1043 (declared at src/compute/cuda_ffi.rs, INT4 partial matmul, fp16 x) */
int vib3_launch_partial_matmul_int4(const void* x_f16, const void* w_packed, const void* scales, void* y_f16,
                                    int K, int M_slice, int group_size, void* stream);
/* replaces cuda/src/kernels.cu:1202 (fp32 x) */
int vib3_launch_partial_matmul_int4_f32(const void* x_f32, const void* w_packed, const void* scales, void* y_f16,
                                        int K, int M_slice, int group_size, void* stream);
/* replaces cuda/src/kernels.cu:1278 (src/compute/cuda_ffi.rs:344-355): y = f16(silu(Wg x) * (Wu x)) */
int vib3_launch_fused_swiglu_int4_f32(const void* x_f32, const void* up_w, const void* up_s, const void* gate_w,
                                      const void* gate_s, void* y_f16, int K, int M_slice, int group_size,
                                      void* stream);
/* replaces cuda/src/kernels.cu:1069: y = f16(silu(first) * second) */
int vib3_launch_silu_mul(const void* silu_operand_f16, const void* mul_operand_f16, void* y_f16, int dim,
                         void* stream);
/* replace cuda/src/kernels.cu:1108, :1120, :2513: out += w * y */
int vib3_launch_weighted_accumulate(void* out_f16, const void* y_f16, float w, int dim, void* stream);
int vib3_launch_weighted_accumulate_f32(void* out_f32, const void* y_f16, float w, int dim, void* stream);
int vib3_launch_weighted_accumulate_f32_f32(void* out_f32, const void* y_f32, float w, int dim, void* stream);
/* replaces cuda/src/kernels.cu:1132: acc += layer_out */
int vib3_launch_residual_add_f32_f32(void* acc_f32, const void* layer_out_f32, int dim, void* stream);
/* replaces cuda/src/kernels.cu:1178: output = input * inv_rms(input) * weight (fp32 in and out, fp16 weight) */
int vib3_launch_rms_norm_f32(const void* input_f32, void* output_f32, const void* weight_f16, int hidden_dim, float eps,
                             void* stream);
/* replace cuda/src/kernels.cu:1143 and :1477: logits[e] = W[e,:] . x, W fp16 [E,H] */
int vib3_launch_router_gemv(const void* x_f16, const void* W_f16, float* scores, int hidden_dim, int num_experts,
                            void* stream);
int vib3_launch_router_gemv_f32(const void* x_f32, const void* W_f16, float* scores, int hidden_dim,
                                int num_experts, void* stream);
/* replaces cuda/src/kernels.cu:4075: GEMV + scoring + top-k, ids u16[top_k] and weights f32[top_k]
 * stay on the device.  scoring_mode 0 = softmax, 1 = sigmoid (bias used for selection only).
 * Unlike the reference's kernel, num_experts need not be a power of two (<= 512). */
int vib3_launch_router_topk(const void* x_f32, const void* W_f16, float* scores_buf, const float* bias_or_null,
                            unsigned short* out_ids, float* out_weights, int hidden_dim, int num_experts,
                            int top_k, int scoring_mode, float scaling_factor, void* stream);

/* ── Entry points added for the fused, paged path ───────────────────────────────────────── */

/* Router in one call, results left on the device (no counterpart signature in the reference; semantics of
 * run_router_with_scoring_and_bias, src/compute/kernels.rs:2307-2440).  x_dtype VIB3_X_*,
 * w_dtype VIB3_W_*.  bias: added to the score for selection only (the reference's correction bias);
 * logit_offset: added to the logit before scoring.  scores_buf: 3 * num_experts floats; the first
 * num_experts receive the logits, the rest is scratch.
 * exact_order != 0 makes the selected indices equal to those of the reference's CPU router
 * (sequential fp32 summation) even for near-tied experts; bit 1 of exact_order (value 2) is for a producer of x
 * that lets its dependents start before it has finished (vib3_launch_residual_rms_norm with bit 1 of `center`): the
 * router's first kernel then holds back the launches behind it until x is complete — the expert kernels read x
 * before their own dependency wait.  workspace: four uint32, zero before
 * the first call; [0] is left zero by every call, [1] counts near-tie recomputations, [2] is used by
 * vib3_launch_moe_layer_routed_int4_paged, [3] is set if a bounded wait in the kernels ran out; calls
 * sharing a workspace must not overlap.  The launches carry the programmatic-dependent-launch attribute:
 * the router's weights are requested while the preceding kernel of the stream is still finishing. */
int vib3_launch_router_topk_ex(const void* x, int x_dtype, const void* W, int w_dtype, float* scores_buf,
                               const float* bias_or_null, const float* logit_offset_or_null,
                               unsigned short* out_ids, float* out_weights,
                               int hidden_dim, int num_experts, int top_k, int scoring_mode, float scaling_factor,
                               int normalize, int exact_order, unsigned int* workspace, void* stream);

/* vib3_launch_router_topk_ex for n_tokens tokens in one call (no counterpart in the reference, whose
 * prefill routes token by token): token t reads x + t * x_stride_bytes and writes scores_buf + t *
 * scores_stride (floats, >= 3 * num_experts), out_ids + t * ids_stride, out_weights + t * weights_stride
 * (entries, >= top_k); workspace: 4 * n_tokens uint32, zero before the first call (word 3 of a token's four is
 * set if a bounded wait in the kernels ran out).  The router's weights are read once per call. */
int vib3_launch_router_topk_batch(const void* x, int x_dtype, int x_stride_bytes, int n_tokens, const void* W,
                                  int w_dtype, float* scores_buf, int scores_stride, const float* bias_or_null,
                                  const float* logit_offset_or_null, unsigned short* out_ids, int ids_stride,
                                  float* out_weights, int weights_stride, int hidden_dim, int num_experts, int top_k,
                                  int scoring_mode, float scaling_factor, int normalize, int exact_order,
                                  unsigned int* workspace, void* stream);

/* Device page-table entry, one per (expert, segment, page): the device form of ResolvedPage
 * (src/runtime/query_planner.rs:36-42).  ptr == 0 marks an absent page. */
typedef struct vib3_page_entry {
    uint64_t ptr;
    uint16_t row_start;
    uint16_t row_count;
    uint32_t reserved;
} vib3_page_entry;

/* Whole MoE sublayer for one token in two launches (gate/up + SiLU, then down + weighted
 * accumulate); replaces the per-page sequence of src/runtime/engine.rs:6094-6107, :6215-6223,
 * :6290-6296 and the role of vib3_launch_moe_experts_fused_gpu (cuda/src/kernels.cu:5868) for
 * INT4 weights with several pages per segment.
 *   page_table   [num_experts][3][pages_per_segment] entries, segment 0 up, 1 gate, 2 down
 *   shared_pages [3][pages_per_segment] entries of the shared expert, or NULL
 *   expert_ids / expert_weights   [top_k] on the device (router output)
 *   x            [hidden_dim] activations, 16-byte aligned
 *   act_scratch  (top_k + 1) * expert_hidden_dim fp16 values, 16-byte aligned
 *   out          [hidden_dim] fp32; overwritten, or added to when out_accumulate != 0
 *   status       device int that receives VIB3_STATUS_* bits, or NULL */
int vib3_launch_moe_layer_int4_paged(const void* x, int x_dtype, const void* page_table, int num_experts,
                                     const void* shared_pages, const unsigned short* expert_ids,
                                     const float* expert_weights, int top_k, float shared_weight,
                                     void* act_scratch, float* out, int out_accumulate, int hidden_dim,
                                     int expert_hidden_dim, int pages_per_segment, int rows_per_page_gate_up,
                                     int rows_per_page_down, int group_size, int* status, void* stream);

/* Router and experts of one token in one call; the routing (ids_out u16[top_k], weights_out f32[top_k],
 * device) is an OUTPUT, written for the caller and for the kernels that follow.  Replaces
 * run_router_gpu_topk_nosync (src/compute/kernels.rs:1890-1953) followed by the per-page expert sequence
 * (src/runtime/engine.rs:6094-6107, :6215-6223, :6290-6296).  Where the shapes allow (hidden and expert
 * dimensions multiples of 256, a router row no larger than a ring stage) the gate/up kernel streams the
 * router's rows through its own ring and selects in its prologue — two launches for the layer and no idle
 * memory pipe while the router's serial tail runs; otherwise the router is launched first.  Router
 * arguments as for vib3_launch_router_topk_ex (workspace: four uint32, zero before the first call; [0]
 * and [2] are left zero), layer arguments as for vib3_launch_moe_layer_int4_paged.  The launch may
 * follow the kernel that produces x with programmatic dependent launch. */
int vib3_launch_moe_layer_routed_int4_paged(const void* x, int x_dtype, const void* router_w, int w_dtype,
                                            float* scores_buf, const float* bias_or_null,
                                            const float* logit_offset_or_null, unsigned short* ids_out,
                                            float* weights_out, int num_experts, int top_k, int scoring_mode,
                                            float scaling_factor, int normalize, int exact_order,
                                            unsigned int* workspace, const void* page_table,
                                            const void* shared_pages, float shared_weight, void* act_scratch,
                                            float* out, int out_accumulate, int hidden_dim, int expert_hidden_dim,
                                            int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down,
                                            int group_size, int* status, void* stream);

/* The two halves of vib3_launch_moe_layer_int4_paged as separate launches, same arguments: the
 * first writes act_scratch (out is not touched), the second reads it and writes out. */
int vib3_launch_moe_gate_up_int4_paged(const void* x, int x_dtype, const void* page_table, int num_experts,
                                       const void* shared_pages, const unsigned short* expert_ids,
                                       const float* expert_weights, int top_k, float shared_weight,
                                       void* act_scratch, float* out, int out_accumulate, int hidden_dim,
                                       int expert_hidden_dim, int pages_per_segment, int rows_per_page_gate_up,
                                       int rows_per_page_down, int group_size, int* status, void* stream);
int vib3_launch_moe_down_int4_paged(const void* x, int x_dtype, const void* page_table, int num_experts,
                                    const void* shared_pages, const unsigned short* expert_ids,
                                    const float* expert_weights, int top_k, float shared_weight, void* act_scratch,
                                    float* out, int out_accumulate, int hidden_dim, int expert_hidden_dim,
                                    int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down,
                                    int group_size, int* status, void* stream);

/* vib3_launch_moe_layer_int4_paged with a device-side slot count: only the first
 * min(top_k, *num_active_dev) entries of expert_ids / expert_weights are used (0 is allowed: with no
 * shared expert the output is zero).  For expert parallelism, where the number of a token's experts
 * that live on this GPU is known only on the device. */
int vib3_launch_moe_layer_int4_paged_var(const void* x, int x_dtype, const void* page_table, int num_experts,
                                         const void* shared_pages, const unsigned short* expert_ids,
                                         const float* expert_weights, int top_k, float shared_weight,
                                         void* act_scratch, float* out, int out_accumulate, int hidden_dim,
                                         int expert_hidden_dim, int pages_per_segment, int rows_per_page_gate_up,
                                         int rows_per_page_down, int group_size, int* status, void* stream,
                                         const int* num_active_dev);
/* One token through one MoE sublayer from and to HOST memory: copies the token in, launches the router
 * and the two expert kernels and waits for the stream — the only entry point here that copies or
 * synchronises (the reference's engine does the same around its launches, src/runtime/engine.rs:
 * 5052-5360).  x_host: ordinary or pinned host memory.  If out_dev is null, out_host must be
 * device-addressable (pinned) memory and the last kernel stores the result into it directly;
 * otherwise the kernels write out_dev and a device-to-host copy follows.  x_dev: device scratch for
 * the token.  Other arguments as for vib3_launch_router_topk_ex / vib3_launch_moe_layer_int4_paged. */
int vib3_moe_layer_step_host(const void* x_host, int x_dtype, void* x_dev, const void* router_w, int w_dtype,
                             float* scores_buf, const float* bias_or_null, unsigned short* ids_dev, float* weights_dev,
                             int num_experts, int top_k, int scoring_mode, float scaling_factor, int normalize,
                             int exact_order, unsigned int* workspace, const void* page_table,
                             const void* shared_pages, float shared_weight, void* act_scratch, float* out_dev_or_null,
                             float* out_host, int hidden_dim, int expert_hidden_dim, int pages_per_segment,
                             int rows_per_page_gate_up, int rows_per_page_down, int group_size, int* status,
                             void* stream);
/* vib3_moe_layer_step_host bound to one layer as a CUDA graph: create once (allocates pinned staging memory and
 * the graph: at start-up, outside any stream capture, on a non-default stream; the role of
 * vib3_moe_prewarm_gpu_bufs, cuda/src/kernels.cu:6507), then per token vib3_moe_step_run(handle, x_host, stream):
 * host-to-host copy of the token into the staging buffer, one graph launch (copy in, router, gate/up, down storing
 * into out_host_pinned), stream synchronisation.  Arguments as for vib3_moe_layer_step_host; out_host_pinned must
 * be pinned (device-addressable) host memory and receives every token's result. */
int vib3_moe_step_create(int x_dtype, void* x_dev, const void* router_w, int w_dtype, float* scores_buf,
                         const float* bias_or_null, unsigned short* ids_dev, float* weights_dev, int num_experts, int top_k,
                         int scoring_mode, float scaling_factor, int normalize, int exact_order, unsigned int* workspace,
                         const void* page_table, const void* shared_pages, float shared_weight, void* act_scratch,
                         float* out_host_pinned, int hidden_dim, int expert_hidden_dim, int pages_per_segment,
                         int rows_per_page_gate_up, int rows_per_page_down, int group_size, int* status, void* stream,
                         void** handle_out);
int vib3_moe_step_run(void* handle, const void* x_host, void* stream);
void vib3_moe_step_destroy(void* handle);

/* Grouped form for expert parallelism: one launch pair for the (token, expert) pairs of SEVERAL tokens
 * that this GPU owns.  pair_experts / pair_weights / pair_tokens: device lists in ascending token order
 * (as vib3_launch_select_local_pairs writes them), *num_pairs_dev their length; this launch takes the
 * pairs [pair_begin, pair_begin + pair_capacity) of them (pair_capacity <= 16; launches with
 * pair_begin > 0 normally pass out_accumulate = 1 and no shared expert).  x: n_tokens activation vectors
 * x_stride_bytes apart (16-byte multiples); out: n_tokens fp32 rows out_stride floats apart, every
 * token's row is written (zero where the token has no pair here).  The shared expert, if given, belongs
 * to token shared_token; its vector is read, and its rows of act_scratch are written, BEFORE the launch
 * waits for its predecessor in the stream (so that it runs under whatever still produces the pair lists): that
 * vector must come from an older launch than the predecessor.  act_scratch: (pair_capacity + 1) * expert_hidden_dim fp16 values.  Only for
 * shapes the staged kernels take (hidden and expert dimensions multiples of 256, expert dimension 1024
 * or 2048); VIB3_ERR_UNSUPPORTED otherwise. */
int vib3_launch_moe_layer_int4_paged_grouped(const void* x, int x_dtype, int x_stride_bytes, int n_tokens,
                                             const void* page_table, int num_experts, const void* shared_pages,
                                             int shared_token, const unsigned short* pair_experts,
                                             const float* pair_weights, const unsigned short* pair_tokens,
                                             int pair_capacity, int pair_begin, const int* num_pairs_dev,
                                             float shared_weight, void* act_scratch, float* out, int out_stride,
                                             int out_accumulate, int hidden_dim, int expert_hidden_dim,
                                             int pages_per_segment, int rows_per_page_gate_up, int rows_per_page_down,
                                             int group_size, int* status, void* stream);
/* The (token, expert, weight) triples, token-major, whose expert lies in [expert_lo, expert_hi).
 * ids / weights: n_tokens rows of top_k entries, row strides in bytes.  The lists hold `capacity`
 * entries; *count_out receives the number found even if larger. */
int vib3_launch_select_local_pairs(const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                   int weights_stride_bytes, int n_tokens, int top_k, int expert_lo, int expert_hi,
                                   unsigned short* pair_experts, float* pair_weights, unsigned short* pair_tokens,
                                   int capacity, int* count_out, void* stream);
/* out[c] = sum over r of in[r * row_stride + c], rows added in order (fp32; 16-byte aligned pointers,
 * row_stride a multiple of 4): combines the partial sums an expert-parallel rank has received. */
int vib3_launch_sum_rows_f32(const float* in, int rows, int cols, int row_stride, float* out, void* stream);
/* ── Expert-parallel exchange over peer memory (one process per GPU, same node) ──────────────────────
 * No counterpart in the reference (single GPU).  vib3_peer_alloc: a zero-filled device allocation that other
 * processes can map, and its 64-byte inter-process handle; vib3_peer_open maps a peer's allocation from its
 * handle (the handles travel between the processes by any host transport); vib3_peer_close / vib3_peer_free
 * undo them.  Only plain peer loads and stores are used on these buffers. */
int vib3_peer_alloc(size_t bytes, void** ptr_out, unsigned char* handle_out_64);
int vib3_peer_open(const unsigned char* handle_64, void** ptr_out);
int vib3_peer_close(void* ptr);
int vib3_peer_free(void* ptr);
/* Store `bytes` bytes (may be 0: a bare signal) from src + d * src_stride_bytes into dst_table[d] + rank *
 * dst_stride_bytes for every destination d < world, then make them visible system-wide and store the step number
 * (*step_counter + step_offset) into flag_table[d][rank].  dst_table / flag_table: device arrays of `world` pointers, entry
 * r = rank r's buffer (the caller's own allocation for r == rank).  16-byte aligned pointers and strides. */
int vib3_launch_peer_publish(const void* src, size_t src_stride_bytes, int bytes, void* const* dst_table,
                             size_t dst_stride_bytes, unsigned int* const* flag_table, const unsigned int* step_counter,
                             int step_offset, int rank, int world, void* stream);
/* The same for rows of fp32 values with a second addend: destination d receives src[d] + add_src[d] if
 * *add_count > add_threshold, else src[d] (rows src_stride_bytes apart in both; bytes a multiple of 16).  For the partial
 * rows of an expert-parallel step whose launch windows beyond the first ran beside the first one into a buffer of their
 * own: they hold pairs only when the rank's pair count exceeds the first window. */
int vib3_launch_peer_publish_rows(const float* src, const float* add_src, size_t src_stride_bytes, int bytes,
                                  const int* add_count, int add_threshold, void* const* dst_table, size_t dst_stride_bytes,
                                  unsigned int* const* flag_table, const unsigned int* step_counter, int step_offset,
                                  int rank, int world, void* stream);
/* Wait (bounded: about two seconds, then VIB3_STATUS_TIMEOUT in *status) until each of flags[0 .. world) has
 * reached *step_counter + 1; advance != 0 then stores that step into *step_counter.  Kernels launched after this
 * one read what the peers stored before their flags. */
int vib3_launch_peer_wait(const unsigned int* flags, unsigned int* step_counter, int world, int advance, int* status,
                          void* stream);
/* vib3_launch_peer_wait (advancing) for the `world` token messages, then vib3_launch_select_local_pairs over them, as
 * one launch; and the wait for the partial rows of the current step (flags reach *step_counter, which the message
 * wait advanced) followed by vib3_launch_sum_rows_f32, as one launch. */
int vib3_launch_peer_select_pairs(const unsigned int* flags, unsigned int* step_counter, int world, int* status,
                                  const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                  int weights_stride_bytes, int top_k, int expert_lo, int expert_hi,
                                  unsigned short* pair_experts, float* pair_weights, unsigned short* pair_tokens,
                                  int capacity, int* count_out, void* stream);
int vib3_launch_peer_sum_rows(const unsigned int* flags, const unsigned int* step_counter, int world, int* status,
                              const float* in, int rows, int cols, int row_stride, float* out, void* stream);
/* Keep, in order, the (expert, weight) pairs with expert_lo <= expert < expert_hi; *count_out = how
 * many.  ids_out / weights_out have top_k entries (unused ones are filled with expert_lo / 0). */
int vib3_launch_select_local_experts(const unsigned short* ids, const float* weights, int top_k, int expert_lo,
                                     int expert_hi, unsigned short* ids_out, float* weights_out, int* count_out,
                                     void* stream);

/* Same work as vib3_launch_moe_layer_int4_paged, for callers that cannot supply act_scratch because
 * they may not allocate device memory (all VRAM already given to a page pool, allocation forbidden
 * after warm-up, no allocator in the binding).  This entry point has no counterpart in the
 * reference.  The intermediate lives in a 544 KiB array inside the library image, held by every GPU
 * the library is loaded on.  Limit: (top_k + 1 if shared_pages) * expert_hidden_dim <= 278,528, else
 * VIB3_ERR_CAPACITY and nothing is launched.  The first call on a device loads the array onto that
 * device (lazy module loading: 544 KiB are reserved then, and the call fails with the runtime's
 * out-of-memory code if they are not free) and resolves its address: issue it before any stream
 * capture and before free VRAM is handed to a pool.  All calls on a device share the array; calls whose
 * kernels may overlap on the GPU race on it.  Nothing is allocated or freed by this entry point. */
int vib3_launch_moe_layer_int4_paged_noalloc(const void* x, int x_dtype, const void* page_table, int num_experts,
                                             const void* shared_pages, const unsigned short* expert_ids,
                                             const float* expert_weights, int top_k, float shared_weight,
                                             float* out, int out_accumulate, int hidden_dim,
                                             int expert_hidden_dim, int pages_per_segment,
                                             int rows_per_page_gate_up, int rows_per_page_down, int group_size,
                                             int* status, void* stream);

/* The steps either side of the MoE sublayer in the reference's layer loop — residual_add_f32_f32
 * (cuda/src/kernels.cu:1132, called at src/runtime/engine.rs:5302) and the next rms_norm_f32 (:1178, called at
 * engine.rs:5072) — as one launch over n_tokens rows: hidden[t] += delta[t] + delta2[t] (either may be NULL;
 * delta2 is fp32 with a stride in floats: e.g. the previous MoE sublayer's output summed over expert-parallel ranks),
 * x_out[t] = cast(hidden[t] * inv_rms(hidden[t]) * weight) (weight_f16 NULL: no weight).  Dtypes VIB3_X_*;
 * strides of delta and x_out in bytes, of hidden in floats.  center != 0 (no counterpart in the reference) removes
 * the row's mean before normalising: for stacks of synthetic layers whose uniformly drawn INT4 codes have mean -0.5
 * (a common term that feeds itself through the residual stream).  Bit 1 of `center` (value 2): the launch is a
 * programmatic dependent of its predecessor in any case (the norm weights are requested before the wait); with this
 * bit it also lets the NEXT launch of the stream start at once.  That launch must wait for its predecessor before it
 * touches hidden or x_out, and must keep later launches that read them from starting: the router launches do both
 * when bit 1 of their exact_order argument is set; use the pair together.  With out_accumulate = 1 in the MoE
 * launch that follows, a layer is this launch plus the MoE launches. */
int vib3_launch_residual_rms_norm(float* hidden, int hidden_stride, const void* delta_or_null, int delta_dtype,
                                  int delta_stride_bytes, const float* delta2_or_null, int delta2_stride,
                                  const void* weight_f16_or_null, float eps, int center, void* x_out, int x_dtype,
                                  int x_stride_bytes, int hidden_dim, int n_tokens, void* stream);

/* ── Grouped multi-token layer (every distinct expert read once; tcgen05 tensor-core tiles) ── */
/* No counterpart in the reference, whose prefill runs the batch-1 path token by token
 * (src/runtime/engine.rs:1837-1838); the nearest precedent is its fused NVFP4 expert launch
 * (cuda/src/kernels.cu:5357-5612, :5868).  Bytes of device scratch vib3_moe_grouped_prewarm needs. */
size_t vib3_moe_grouped_workspace_bytes(int max_tokens, int top_k, int num_experts, int hidden_dim,
                                        int expert_hidden_dim, int rows_per_page_gate_up, int rows_per_page_down);
/* Builds the TMA tensor maps of the grouped kernels over a page pool (pool_base: start of the pool's
 * single allocation, 16-byte aligned, capacity_pages slots of 2 MiB) and over the caller's scratch
 * (workspace, 1024-byte aligned, at least vib3_moe_grouped_workspace_bytes).  hidden_dim and
 * expert_hidden_dim must be multiples of 256.  last_page_rows_*: rows of the last (ragged) page of a
 * gate/up and of a down matrix.  The handle owns host memory only; nothing is allocated on the device
 * (the role of vib3_moe_prewarm_gpu_bufs, cuda/src/kernels.cu:6507).  Like it, call it before any
 * stream capture. */
int vib3_moe_grouped_prewarm(void* pool_base, size_t capacity_pages, int num_experts, int top_k, int hidden_dim,
                             int expert_hidden_dim, int rows_per_page_gate_up, int rows_per_page_down,
                             int last_page_rows_gate_up, int last_page_rows_down, int max_tokens, void* workspace,
                             size_t workspace_bytes, void** handle_out);
void vib3_moe_grouped_destroy(void* handle);
/* One MoE sublayer for n_tokens (<= max_tokens <= 128) tokens: ids / weights are the tokens' routing
 * (rows of top_k entries, strides in bytes, device), x the activations (rows x_stride_bytes apart), out
 * [n_tokens] fp32 rows out_stride floats apart (overwritten, or added to).  Only the pairs whose expert lies
 * in [expert_lo, expert_hi) are computed (0 and num_experts: all; an expert-parallel rank passes its own range
 * and sums the ranks' outputs afterwards), and the shared expert only if shared_pages is given.  Six launches (bucketing, token
 * gather, work-unit tables, gate/up, down, per-token combine in plan order), no host synchronisation.  The pages of the
 * page tables must lie in the pool given to vib3_moe_grouped_prewarm. */
int vib3_launch_moe_grouped_int4(void* handle, const void* x, int x_dtype, int x_stride_bytes, int n_tokens,
                                 const unsigned short* ids, int ids_stride_bytes, const float* weights,
                                 int weights_stride_bytes, const void* page_table, const void* shared_pages,
                                 float shared_weight, int pages_per_segment, int expert_lo, int expert_hi, float* out,
                                 int out_stride, int out_accumulate, int* status, void* stream);

/* Library options.  key 0: use the bulk-copy staged MoE kernels where the shape allows (default 1);
 * 0 forces the direct-load kernels.  key 1: launch the staged kernels with programmatic dependent
 * launch so that their prologue overlaps the previous kernel's tail (default 1).  key 2:
 * vib3_launch_moe_layer_routed_int4_paged routes inside the gate/up kernel (default 0: the router is a
 * launch of its own, which measures faster on the Kimi shape).  The switches are
 * atomics: a launch running concurrently on another thread sees the old or the new value.  Returns
 * the previous value, or VIB3_ERR_UNSUPPORTED for an unknown key. */
int vib3_config_set(int key, int value);

/* ── Host side: VRAM page pool and query planner (C view of the C++ classes) ────────────── */
/* Mirrors PageBufferManager's T1 pool + resident snapshot (src/storage/buffer_manager.rs:206-288,
 * :622-761, :883-899) and QueryPlanner::plan_layer (src/runtime/query_planner.rs:158-272). */

typedef struct vib3_pool vib3_pool;

/* Pool of `capacity_pages` slots of 2 MiB.  device_base == NULL: the pool allocates its slots
 * with one cudaMalloc; otherwise it adopts caller-owned device memory of capacity_pages * 2 MiB.
 * Slots are handed out in a pseudo-random order derived from slot_seed (0 = sequential). */
vib3_pool* vib3_pool_create(void* device_base, size_t capacity_pages, uint64_t slot_seed);
void vib3_pool_destroy(vib3_pool* pool);
/* Place a page: picks a free slot, copies nbytes from host memory when host_data != NULL
 * (otherwise the caller fills the slot itself), records the catalog row range.  Returns the
 * slot index, or VIB3_ERR_*. */
long long vib3_pool_load_page(vib3_pool* pool, uint16_t layer, uint16_t expert, uint16_t segment,
                              uint16_t page_idx, uint16_t row_start, uint16_t row_count, const void* host_data,
                              size_t nbytes);
void* vib3_pool_slot_ptr(const vib3_pool* pool, long long slot);
/* Freeze the page table into the resident snapshot; lookups are only allowed afterwards. */
int vib3_pool_freeze(vib3_pool* pool);
/* get_page_resident: VIB3_OK and the handle fields, or VIB3_ERR_RANGE when the page is absent. */
int vib3_pool_get_page_resident(const vib3_pool* pool, uint64_t page_key, void** device_ptr, uint16_t* row_start,
                                uint16_t* row_count, uint32_t* size);
size_t vib3_pool_resident_pages(const vib3_pool* pool);
/* Build (once per layer, cached) the device page table [num_experts][3][pages_per_segment] and
 * return its device pointer; shared = 1 builds the [3][pages] block of the shared expert
 * (expert id 0xFFFF, segments 14/15/16 = up/gate/down, src/storage/convert.rs:2014-2032). */
int vib3_pool_device_page_table(vib3_pool* pool, uint16_t layer, int num_experts, int pages_per_segment,
                                int shared, void** device_table);
uint64_t vib3_page_key(uint16_t layer, uint16_t expert, uint16_t segment, uint16_t page_idx);

/* plan_layer on the resident snapshot: for each (expert, weight) the pages of segments 0,1,2 in
 * catalog order.  Writes up to max_pages resolved pages and returns their number, or
 * VIB3_ERR_RANGE if a page is missing (Error::PageNotFound). */
typedef struct vib3_resolved_page {
    uint64_t key;
    void* device_ptr;
    uint16_t expert_id;
    uint16_t segment;
    uint16_t row_start;
    uint16_t row_count;
} vib3_resolved_page;
int vib3_planner_plan_layer(const vib3_pool* pool, uint16_t layer, const uint16_t* expert_ids, int num_active,
                            int pages_per_segment, vib3_resolved_page* out_pages, int max_pages);

/* ── `.vib3` container: INT4 quantiser, page-split writer, reader (host only) ───────────── */
/* Mirrors quantize_weights_to_int4 (src/compute/kernels.rs:3778-3831), add_pages_from_data
 * (src/storage/convert.rs:1841-1901), Vib3Writer::finalize and Vib3File::open
 * (src/storage/format.rs:842-1090, :241-339) for uncompressed INT4 pages. */
/* bytes of a quantised [rows, cols] matrix: rows * ceil(cols / 2) codes + rows * ceil(cols / 32) 16-bit scales */
size_t vib3_int4_matrix_bytes(int rows, int cols);
/* group-32 quantisation: scale = max|w| / 7 (1 for an all-zero group), q = clamp(round(w / scale) + 8, 0, 15), low
 * nibble = even column.  scale_format 0: bf16 (what the reference's quantiser writes), 1: fp16 (what its CUDA
 * kernels and this library's kernels decode). */
int vib3_quantize_int4(const float* w, int rows, int cols, int scale_format, uint8_t* out);
typedef struct vib3_writer vib3_writer;
vib3_writer* vib3_writer_create(const char* path, const char* metadata_json, uint32_t num_layers, uint32_t num_experts,
                                uint32_t num_active_experts, uint32_t hidden_dim, uint32_t expert_hidden_dim);
/* cuts a quantised matrix into 2 MiB pages (rows_per_page = 2 MiB / bytes_per_row) and queues them; returns the
 * number of pages */
int vib3_writer_add_int4_matrix(vib3_writer* w, uint16_t layer, uint16_t expert, uint16_t segment, int rows, int cols,
                                const uint8_t* int4_data);
/* sorts the catalog by (layer, expert, segment, page), builds the expert index and writes the file */
int vib3_writer_finalize(vib3_writer* w);
void vib3_writer_destroy(vib3_writer* w);
typedef struct vib3_file vib3_file;
typedef struct vib3_file_page {
    uint16_t layer, expert, segment, page_idx;
    uint16_t row_start, row_count, col_count, compression;
    uint64_t file_offset;
    uint32_t raw_size;
} vib3_file_page;
/* NULL on failure with *error_out = VIB3_ERR_SHAPE (too small), _UNSUPPORTED (magic / version), _RANGE (a section or
 * page beyond the end of the file), _STATE (cannot open) */
vib3_file* vib3_file_open(const char* path, int* error_out);
void vib3_file_close(vib3_file* f);
int vib3_file_page_count(const vib3_file* f);
int vib3_file_summary(const vib3_file* f, uint32_t* num_layers, uint32_t* num_experts, uint32_t* num_active_experts,
                      uint32_t* hidden_dim, uint32_t* expert_hidden_dim, uint32_t* expert_dtype,
                      uint64_t* page_data_offset);
int vib3_file_page_info(const vib3_file* f, int index, vib3_file_page* out);
int vib3_file_read_page(vib3_file* f, int index, void* dst, size_t dst_bytes);
/* every page of layers [layer_lo, layer_hi) and experts [expert_lo, expert_hi) (plus the shared expert) into the
 * pool — PageBufferManager::preload_all (src/storage/buffer_manager.rs:1226-1254); returns the pages loaded */
long long vib3_file_load_into_pool(vib3_file* f, vib3_pool* pool, int layer_lo, int layer_hi, int expert_lo, int expert_hi);

const char* vib3_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* VIB3_B200_H */
