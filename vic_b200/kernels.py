"""Launch wrappers with the names, argument meaning and error behaviour of the reference's Rust
launchers (src/compute/kernels.rs), over the C ABI of libvib3_cuda.so.

Pointers are raw device addresses (ints) or CUDA tensors; ``stream`` is a raw cudaStream_t (int)
and defaults to torch's current stream.  A non-zero launcher return raises Vib3Error, as the
reference maps it to Error::Cuda (kernels.rs:145-150).  There is no CPU path here: the
reference's ``CudaStream::cpu_only()`` fallbacks are restated only in the test oracle."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .core_types import INT4_GROUP_SIZE, SCORING_SIGMOID, SCORING_SOFTMAX, W_F16, W_F32, X_BF16, X_F16, X_F32
from .lib import check, lib


def _ptr(t) -> int:
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    if not t.is_cuda and not t.is_pinned():
        raise ValueError("device tensor (or pinned, device-addressable host tensor) expected")
    return t.data_ptr()


def _stream(stream: Optional[int]) -> int:
    return torch.cuda.current_stream().cuda_stream if stream is None else stream


def x_dtype_code(t: torch.Tensor) -> int:
    return {torch.float32: X_F32, torch.float16: X_F16, torch.bfloat16: X_BF16}[t.dtype]


def partial_matmul(input, weight_page, output, k: int, m_slice: int, stream: Optional[int] = None) -> None:
    """kernels.rs:25-152, INT4 arm: y_f16[m_slice] = W_page . x_f16; the scales pointer is derived
    from the page pointer exactly as kernels.rs:94-98 does."""
    page = _ptr(weight_page)
    scales = page + ((k + 1) // 2) * m_slice
    check("partial_matmul_int4", lib().vib3_launch_partial_matmul_int4(
        _ptr(input), page, scales, _ptr(output), k, m_slice, INT4_GROUP_SIZE, _stream(stream)))


def partial_matmul_f32(input, weight_page, output, k: int, m_slice: int, stream: Optional[int] = None) -> None:
    """kernels.rs:375-455, INT4 arm: fp32 input, fp16 output."""
    page = _ptr(weight_page)
    scales = page + ((k + 1) // 2) * m_slice
    check("partial_matmul_int4_f32", lib().vib3_launch_partial_matmul_int4_f32(
        _ptr(input), page, scales, _ptr(output), k, m_slice, INT4_GROUP_SIZE, _stream(stream)))


def silu_mul(silu_operand, mul_operand, output, dim: int, stream: Optional[int] = None) -> None:
    check("silu_mul", lib().vib3_launch_silu_mul(_ptr(silu_operand), _ptr(mul_operand), _ptr(output), dim, _stream(stream)))


def partial_swiglu_f32(input, up_page, gate_page, output, hidden_dim: int, m_slice: int,
                       swiglu_temps: Optional[Tuple] = None, stream: Optional[int] = None) -> None:
    """kernels.rs:459-600, INT4 arm.  With temps: the reference's decomposition (two fp32-input
    matmuls rounded to fp16, then silu_mul, kernels.rs:493-541).  Without: the fused kernel
    (cuda_ffi.rs:344-355), one rounding."""
    if swiglu_temps is not None:
        up_tmp, gate_tmp = swiglu_temps
        partial_matmul_f32(input, up_page, up_tmp, hidden_dim, m_slice, stream)
        partial_matmul_f32(input, gate_page, gate_tmp, hidden_dim, m_slice, stream)
        silu_mul(gate_tmp, up_tmp, output, m_slice, stream)
        return
    up, gate = _ptr(up_page), _ptr(gate_page)
    off = ((hidden_dim + 1) // 2) * m_slice
    check("fused_swiglu_int4_f32", lib().vib3_launch_fused_swiglu_int4_f32(
        _ptr(input), up, up + off, gate, gate + off, _ptr(output), hidden_dim, m_slice, INT4_GROUP_SIZE, _stream(stream)))


def weighted_accumulate(output, expert_output, weight: float, dim: int, stream: Optional[int] = None) -> None:
    check("weighted_accumulate", lib().vib3_launch_weighted_accumulate(_ptr(output), _ptr(expert_output), weight, dim, _stream(stream)))


def weighted_accumulate_f32(output, expert_output, weight: float, dim: int, stream: Optional[int] = None) -> None:
    check("weighted_accumulate_f32", lib().vib3_launch_weighted_accumulate_f32(_ptr(output), _ptr(expert_output), weight, dim, _stream(stream)))


def weighted_accumulate_f32_f32(output, expert_output, weight: float, dim: int, stream: Optional[int] = None) -> None:
    check("weighted_accumulate_f32_f32", lib().vib3_launch_weighted_accumulate_f32_f32(_ptr(output), _ptr(expert_output), weight, dim, _stream(stream)))


def residual_add_f32_f32(accumulator, layer_output, dim: int, stream: Optional[int] = None) -> None:
    check("residual_add_f32_f32", lib().vib3_launch_residual_add_f32_f32(_ptr(accumulator), _ptr(layer_output), dim, _stream(stream)))


def rms_norm_f32(input_f32, output_f32, weight_f16, hidden_dim: int, eps: float, stream: Optional[int] = None) -> None:
    """kernels.rs:2560-2603 (GPU arm): fp32 in, fp32 out, fp16 weight."""
    check("rms_norm_f32", lib().vib3_launch_rms_norm_f32(_ptr(input_f32), _ptr(output_f32), _ptr(weight_f16), hidden_dim, eps,
                                                        _stream(stream)))


EXACT_HOLD = 2   # added to a router launch's exact_order: the producer of x lets its dependents start early


def residual_rms_norm(hidden: torch.Tensor, delta, weight_f16, eps: float, x_out: torch.Tensor, stream: Optional[int] = None,
                      delta2=None, center: bool = False, early_dependents: bool = False) -> None:
    """hidden [T, H] fp32 += delta [T, H] + delta2 [T, H] fp32 (either may be None); x_out [T, H] = cast(rms_norm(hidden) *
    weight): one launch.  ``early_dependents``: the next launch of the stream may start while this one runs; it must
    be a router launch with ``EXACT_HOLD`` added to its exact_order argument (see include/vib3_b200.h)."""
    T, H = hidden.shape
    check("residual_rms_norm", lib().vib3_launch_residual_rms_norm(
        _ptr(hidden), hidden.stride(0), _ptr(delta), x_dtype_code(delta) if delta is not None else 0,
        delta.stride(0) * delta.element_size() if delta is not None else 0, _ptr(delta2),
        delta2.stride(0) if delta2 is not None else 0, _ptr(weight_f16), eps, int(center) | (2 if early_dependents else 0), _ptr(x_out),
        x_dtype_code(x_out), x_out.stride(0) * x_out.element_size(), H, T, _stream(stream)))


def router_gemv_f32(hidden_state, router_weights_f16, scores, hidden_dim: int, num_experts: int,
                    stream: Optional[int] = None) -> None:
    check("router_gemv_f32", lib().vib3_launch_router_gemv_f32(_ptr(hidden_state), _ptr(router_weights_f16), _ptr(scores),
                                                              hidden_dim, num_experts, _stream(stream)))


def router_gemv(hidden_state_f16, router_weights_f16, scores, hidden_dim: int, num_experts: int,
                stream: Optional[int] = None) -> None:
    check("router_gemv", lib().vib3_launch_router_gemv(_ptr(hidden_state_f16), _ptr(router_weights_f16), _ptr(scores),
                                                      hidden_dim, num_experts, _stream(stream)))


def run_router_gpu_topk_nosync(hidden_state_f32, router_weights_f16, scores_buf, bias, out_ids, out_weights,
                               hidden_dim: int, num_experts: int, top_k: int, scoring_mode: int,
                               scaling_factor: float, stream: Optional[int] = None) -> None:
    """kernels.rs:1890-1953: results stay on the device."""
    check("router_topk", lib().vib3_launch_router_topk(
        _ptr(hidden_state_f32), _ptr(router_weights_f16), _ptr(scores_buf), _ptr(bias), _ptr(out_ids), _ptr(out_weights),
        hidden_dim, num_experts, top_k, scoring_mode, scaling_factor, _stream(stream)))


def run_router_gpu_topk(hidden_state_f32, router_weights_f16, scores_buf, bias, out_ids, out_weights, hidden_dim: int,
                        num_experts: int, top_k: int, scoring_mode: int, scaling_factor: float,
                        stream: Optional[int] = None):
    """kernels.rs:1811-1873: launch, synchronise, two small D2H copies -> [(expert, weight)]."""
    run_router_gpu_topk_nosync(hidden_state_f32, router_weights_f16, scores_buf, bias, out_ids, out_weights, hidden_dim,
                               num_experts, top_k, scoring_mode, scaling_factor, stream)
    torch.cuda.current_stream().synchronize()
    ids = out_ids[:top_k].cpu().view(torch.int16).numpy().view("uint16")
    ws = out_weights[:top_k].cpu().numpy()
    return [(int(i), float(w)) for i, w in zip(ids, ws)]


def router_topk_ex(x: torch.Tensor, W: torch.Tensor, scores_buf, bias, out_ids, out_weights, top_k: int,
                   scoring_mode: int, scaling_factor: float, normalize: bool, exact_order: bool, workspace,
                   stream: Optional[int] = None, logit_offset=None) -> None:
    """Single-launch router for fp16/bf16/fp32 activations and fp16/fp32 weights."""
    E, H = W.shape
    w_dtype = {torch.float16: W_F16, torch.float32: W_F32}[W.dtype]
    check("router_topk_ex", lib().vib3_launch_router_topk_ex(
        _ptr(x), x_dtype_code(x), _ptr(W), w_dtype, _ptr(scores_buf), _ptr(bias), _ptr(logit_offset), _ptr(out_ids),
        _ptr(out_weights), H, E,
        top_k, scoring_mode, scaling_factor, int(normalize), int(exact_order), _ptr(workspace), _stream(stream)))


def router_topk_batch(xs: torch.Tensor, W: torch.Tensor, scores_buf: torch.Tensor, bias, logit_offset, out_ids: torch.Tensor,
                      out_weights: torch.Tensor, top_k: int, scoring_mode: int, scaling_factor: float, normalize: bool,
                      exact_order: bool, workspace: torch.Tensor, stream: Optional[int] = None) -> None:
    """The router for T tokens in ONE call (the weights are read once): xs [T, H]; scores_buf [T, 3E] fp32,
    out_ids [T, >= top_k] int16, out_weights [T, >= top_k] fp32, workspace [T, 4] int32 (zero before the first call)."""
    E, H = W.shape
    T = xs.shape[0]
    w_dtype = {torch.float16: W_F16, torch.float32: W_F32}[W.dtype]
    check("router_topk_batch", lib().vib3_launch_router_topk_batch(
        _ptr(xs), x_dtype_code(xs), xs.stride(0) * xs.element_size(), T, _ptr(W), w_dtype, _ptr(scores_buf),
        scores_buf.stride(0), _ptr(bias), _ptr(logit_offset), _ptr(out_ids), out_ids.stride(0), _ptr(out_weights),
        out_weights.stride(0), H, E, top_k, scoring_mode, scaling_factor, int(normalize), int(exact_order), _ptr(workspace),
        _stream(stream)))


def moe_layer_int4_paged(x: torch.Tensor, page_table: int, num_experts: int, shared_pages: int, expert_ids,
                         expert_weights, top_k: int, shared_weight: float, act_scratch, out, out_accumulate: bool,
                         hidden_dim: int, expert_hidden_dim: int, pages_per_segment: int, rows_per_page_gate_up: int,
                         rows_per_page_down: int, status=None, stream: Optional[int] = None, phase: int = 3) -> None:
    """phase 3: both launches; 1: gate/up + SiLU only; 2: down + accumulate only."""
    fn = {3: lib().vib3_launch_moe_layer_int4_paged, 1: lib().vib3_launch_moe_gate_up_int4_paged,
          2: lib().vib3_launch_moe_down_int4_paged}[phase]
    check("moe_layer_int4_paged", fn(
        _ptr(x), x_dtype_code(x), page_table, num_experts, shared_pages or 0, _ptr(expert_ids), _ptr(expert_weights), top_k,
        shared_weight, _ptr(act_scratch), _ptr(out), int(out_accumulate), hidden_dim, expert_hidden_dim,
        pages_per_segment, rows_per_page_gate_up, rows_per_page_down, INT4_GROUP_SIZE, _ptr(status), _stream(stream)))


def moe_layer_routed_int4_paged(x: torch.Tensor, router_w: torch.Tensor, scores_buf, bias, logit_offset, ids_out, weights_out,
                                top_k: int, scoring_mode: int, scaling_factor: float, normalize: bool, exact_order: bool,
                                workspace, page_table: int, num_experts: int, shared_pages: int, shared_weight: float,
                                act_scratch, out, out_accumulate: bool, hidden_dim: int, expert_hidden_dim: int,
                                pages_per_segment: int, rows_per_page_gate_up: int, rows_per_page_down: int, status=None,
                                stream: Optional[int] = None) -> None:
    """Router and experts of one token; the routing (ids_out, weights_out) is an output.  Two launches where
    the gate/up kernel can route the token in its own prologue, three otherwise."""
    w_dtype = {torch.float16: W_F16, torch.float32: W_F32}[router_w.dtype]
    check("moe_layer_routed_int4_paged", lib().vib3_launch_moe_layer_routed_int4_paged(
        _ptr(x), x_dtype_code(x), _ptr(router_w), w_dtype, _ptr(scores_buf), _ptr(bias), _ptr(logit_offset), _ptr(ids_out),
        _ptr(weights_out), num_experts, top_k, scoring_mode, scaling_factor, int(normalize), int(exact_order), _ptr(workspace),
        page_table, shared_pages or 0, shared_weight, _ptr(act_scratch), _ptr(out), int(out_accumulate), hidden_dim,
        expert_hidden_dim, pages_per_segment, rows_per_page_gate_up, rows_per_page_down, INT4_GROUP_SIZE, _ptr(status),
        _stream(stream)))


def moe_layer_int4_paged_var(x: torch.Tensor, page_table: int, num_experts: int, shared_pages: int, expert_ids,
                             expert_weights, top_k: int, shared_weight: float, act_scratch, out, out_accumulate: bool,
                             hidden_dim: int, expert_hidden_dim: int, pages_per_segment: int,
                             rows_per_page_gate_up: int, rows_per_page_down: int, num_active_dev, status=None,
                             stream: Optional[int] = None) -> None:
    """The fused sublayer over the first min(top_k, *num_active_dev) routed slots (device-side count)."""
    check("moe_layer_int4_paged_var", lib().vib3_launch_moe_layer_int4_paged_var(
        _ptr(x), x_dtype_code(x), page_table, num_experts, shared_pages or 0, _ptr(expert_ids), _ptr(expert_weights), top_k,
        shared_weight, _ptr(act_scratch), _ptr(out), int(out_accumulate), hidden_dim, expert_hidden_dim,
        pages_per_segment, rows_per_page_gate_up, rows_per_page_down, INT4_GROUP_SIZE, _ptr(status), _stream(stream),
        _ptr(num_active_dev)))


def moe_layer_int4_paged_grouped(x, x_dtype: int, x_stride_bytes: int, n_tokens: int, page_table: int, num_experts: int,
                                 shared_pages: int, shared_token: int, pair_experts, pair_weights, pair_tokens,
                                 pair_capacity: int, pair_begin: int, num_pairs_dev, shared_weight: float, act_scratch, out,
                                 out_stride: int, out_accumulate: bool, hidden_dim: int, expert_hidden_dim: int,
                                 pages_per_segment: int, rows_per_page_gate_up: int, rows_per_page_down: int, status=None,
                                 stream: Optional[int] = None) -> None:
    """One launch pair over the (token, expert) pairs of several tokens (expert parallelism)."""
    check("moe_layer_int4_paged_grouped", lib().vib3_launch_moe_layer_int4_paged_grouped(
        _ptr(x), x_dtype, x_stride_bytes, n_tokens, page_table, num_experts, shared_pages or 0, shared_token,
        _ptr(pair_experts), _ptr(pair_weights), _ptr(pair_tokens), pair_capacity, pair_begin, _ptr(num_pairs_dev),
        shared_weight, _ptr(act_scratch), _ptr(out), out_stride, int(out_accumulate), hidden_dim, expert_hidden_dim,
        pages_per_segment, rows_per_page_gate_up, rows_per_page_down, INT4_GROUP_SIZE, _ptr(status), _stream(stream)))


def select_local_pairs(ids, ids_stride_bytes: int, weights, weights_stride_bytes: int, n_tokens: int, top_k: int,
                       expert_lo: int, expert_hi: int, pair_experts, pair_weights, pair_tokens, capacity: int, count_out,
                       stream: Optional[int] = None) -> None:
    check("select_local_pairs", lib().vib3_launch_select_local_pairs(
        _ptr(ids), ids_stride_bytes, _ptr(weights), weights_stride_bytes, n_tokens, top_k, expert_lo, expert_hi,
        _ptr(pair_experts), _ptr(pair_weights), _ptr(pair_tokens), capacity, _ptr(count_out), _stream(stream)))


def moe_layer_step_host(x_host: torch.Tensor, x_dev: torch.Tensor, router_w: torch.Tensor, scores_buf, bias, ids_dev, weights_dev,
                        num_experts: int, top_k: int, scoring_mode: int, scaling_factor: float, normalize: bool,
                        exact_order: bool, workspace, page_table: int, shared_pages: int, shared_weight: float, act_scratch,
                        out_dev, out_host: torch.Tensor, hidden_dim: int, expert_hidden_dim: int, pages_per_segment: int,
                        rows_per_page_gate_up: int, rows_per_page_down: int, status=None, stream: Optional[int] = None) -> None:
    """One token from and to host memory through one C call (copy in, router, experts, synchronise)."""
    w_dtype = {torch.float16: W_F16, torch.float32: W_F32}[router_w.dtype]
    if x_host.is_cuda or out_host.is_cuda:
        raise ValueError("host tensors expected")
    if out_dev is None and not out_host.is_pinned():
        raise ValueError("out_host must be pinned when no device output buffer is given")
    check("moe_layer_step_host", lib().vib3_moe_layer_step_host(
        x_host.data_ptr(), x_dtype_code(x_host), _ptr(x_dev), _ptr(router_w), w_dtype, _ptr(scores_buf), _ptr(bias), _ptr(ids_dev),
        _ptr(weights_dev), num_experts, top_k, scoring_mode, scaling_factor, int(normalize), int(exact_order), _ptr(workspace),
        page_table, shared_pages or 0, shared_weight, _ptr(act_scratch), _ptr(out_dev), out_host.data_ptr(), hidden_dim,
        expert_hidden_dim, pages_per_segment, rows_per_page_gate_up, rows_per_page_down, INT4_GROUP_SIZE, _ptr(status),
        _stream(stream)))


def sum_rows_f32(rows_in: torch.Tensor, out: torch.Tensor, stream: Optional[int] = None) -> None:
    """out[c] = sum_r rows_in[r, c], rows added in order."""
    check("sum_rows_f32", lib().vib3_launch_sum_rows_f32(_ptr(rows_in), rows_in.shape[0], rows_in.shape[1], rows_in.stride(0),
                                                         _ptr(out), _stream(stream)))


def peer_publish(src: torch.Tensor, src_stride_bytes: int, nbytes: int, dst_table: torch.Tensor, dst_stride_bytes: int,
                 flag_table: torch.Tensor, step_counter: torch.Tensor, step_offset: int, rank: int, world: int,
                 stream: Optional[int] = None) -> None:
    """Store nbytes from src (+ d * src_stride_bytes) into every rank d's buffer at slot `rank`, then the flag
    (*step_counter + step_offset)."""
    check("peer_publish", lib().vib3_launch_peer_publish(_ptr(src), src_stride_bytes, nbytes, _ptr(dst_table), dst_stride_bytes,
                                                         _ptr(flag_table), _ptr(step_counter), step_offset, rank, world, _stream(stream)))


def peer_publish_rows(src: torch.Tensor, add_src: torch.Tensor, row_bytes: int, add_count: torch.Tensor, add_threshold: int,
                      dst_table: torch.Tensor, dst_stride_bytes: int, flag_table: torch.Tensor, step_counter: torch.Tensor,
                      step_offset: int, rank: int, world: int, stream: Optional[int] = None) -> None:
    """peer_publish of fp32 rows: rank d receives src[d] + (add_src[d] if *add_count > add_threshold)."""
    check("peer_publish_rows", lib().vib3_launch_peer_publish_rows(
        _ptr(src), _ptr(add_src), src.stride(0) * 4, row_bytes, _ptr(add_count), add_threshold, _ptr(dst_table), dst_stride_bytes,
        _ptr(flag_table), _ptr(step_counter), step_offset, rank, world, _stream(stream)))


def peer_wait(flags: torch.Tensor, step_counter: torch.Tensor, world: int, advance: bool, status, stream: Optional[int] = None) -> None:
    """Wait (bounded) until every peer's flag has reached the next step; advance the step counter."""
    check("peer_wait", lib().vib3_launch_peer_wait(_ptr(flags), _ptr(step_counter), world, int(advance), _ptr(status), _stream(stream)))


def peer_select_pairs(flags, step_counter, world: int, status, ids, ids_stride_bytes: int, weights, weights_stride_bytes: int,
                      top_k: int, expert_lo: int, expert_hi: int, pair_experts, pair_weights, pair_tokens, capacity: int, count_out,
                      stream: Optional[int] = None) -> None:
    """peer_wait for the messages (advancing the step) and select_local_pairs over them in one launch."""
    check("peer_select_pairs", lib().vib3_launch_peer_select_pairs(
        _ptr(flags), _ptr(step_counter), world, _ptr(status), _ptr(ids), ids_stride_bytes, _ptr(weights), weights_stride_bytes, top_k,
        expert_lo, expert_hi, _ptr(pair_experts), _ptr(pair_weights), _ptr(pair_tokens), capacity, _ptr(count_out), _stream(stream)))


def peer_sum_rows(flags, step_counter, world: int, status, rows_in: torch.Tensor, out: torch.Tensor, stream: Optional[int] = None) -> None:
    """Wait for the partial rows of the current step, then out[c] = sum_r rows_in[r, c] in row order: one launch."""
    check("peer_sum_rows", lib().vib3_launch_peer_sum_rows(_ptr(flags), _ptr(step_counter), world, _ptr(status), _ptr(rows_in),
                                                           rows_in.shape[0], rows_in.shape[1], rows_in.stride(0), _ptr(out), _stream(stream)))


def select_local_experts(ids, weights, top_k: int, expert_lo: int, expert_hi: int, ids_out, weights_out, count_out,
                         stream: Optional[int] = None) -> None:
    check("select_local_experts", lib().vib3_launch_select_local_experts(
        _ptr(ids), _ptr(weights), top_k, expert_lo, expert_hi, _ptr(ids_out), _ptr(weights_out), _ptr(count_out),
        _stream(stream)))


__all__ = [n for n in dir() if not n.startswith("_")] + ["SCORING_SOFTMAX", "SCORING_SIGMOID"]
