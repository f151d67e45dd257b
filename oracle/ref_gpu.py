"""The reference's own CUDA kernels (oracle/_ref/libvib3_ref.so, compiled unmodified by the Makefile
beside this file) driven in the reference engine's per-page order.  TEST AND BASELINE INFRASTRUCTURE
ONLY: the parity tests use it as a second checker, bench.py's baseline leg times it; the product
package never imports it."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libvib3_ref.so")


def load_ref_lib():
    """ctypes handle of the reference's kernels with their argument types, or None when not built."""
    if not os.path.exists(REF_LIB_PATH):
        return None
    lib = ctypes.CDLL(REF_LIB_PATH)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    sigs = {
        "vib3_launch_partial_matmul_int4": [vp, vp, vp, vp, i, i, i, vp],
        "vib3_launch_partial_matmul_int4_f32": [vp, vp, vp, vp, i, i, i, vp],
        "vib3_launch_fused_swiglu_int4_f32": [vp, vp, vp, vp, vp, vp, i, i, i, vp],
        "vib3_launch_silu_mul": [vp, vp, vp, i, vp],
        "vib3_launch_weighted_accumulate_f32": [vp, vp, f, i, vp],
        "vib3_launch_router_gemv_f32": [vp, vp, vp, i, i, vp],
        "vib3_launch_router_topk": [vp, vp, vp, vp, vp, vp, i, i, i, i, f, vp],
    }
    for n, a in sigs.items():
        fn = getattr(lib, n)
        fn.restype = i
        fn.argtypes = a
    return lib


class RefSublayerBuffers:
    """The temporaries of the engine's expert loop (src/runtime/engine.rs:1005-1011)."""

    def __init__(self, H: int, I: int, dev):
        import torch
        self.up_tmp = torch.zeros(I, dtype=torch.float16, device=dev)
        self.gate_tmp = torch.zeros(I, dtype=torch.float16, device=dev)
        self.expert_out = torch.zeros(I, dtype=torch.float16, device=dev)
        self.down_out = torch.zeros(H, dtype=torch.float16, device=dev)
        self.layer_out = torch.zeros(H, dtype=torch.float32, device=dev)


def ref_moe_sublayer(ref, model, layer, x_f32, activation, planner, bufs=None):
    """The reference engine's INT4 call sequence (engine.rs:6094-6107, :6215-6223, :6290-6296) on the
    reference's own kernels: returns layer_out_f32 (torch, device) and the launch count."""
    import torch
    from vic_b200.core_types import EXPERT_SHARED
    sh = model.shape
    H, I = sh.hidden, sh.intermediate
    b = bufs or RefSublayerBuffers(H, I, x_f32.device)
    st = torch.cuda.current_stream().cuda_stream
    entries = list(activation) + ([(EXPERT_SHARED, 1.0)] if sh.shared_experts else [])
    plan = planner.plan_layer(layer, entries)
    b.layer_out.zero_()
    launches = 1
    for ep in plan.experts:
        segs = sorted(set(p.id.segment for p in ep.pages))
        ups = [p for p in ep.pages if p.id.segment == segs[0]]
        gates = [p for p in ep.pages if p.id.segment == segs[1]]
        downs = [p for p in ep.pages if p.id.segment == segs[2]]
        b.expert_out.zero_()
        for up, gate in zip(ups, gates):
            m = up.row_count
            off = (H // 2) * m
            assert ref.vib3_launch_partial_matmul_int4_f32(x_f32.data_ptr(), up.device_ptr, up.device_ptr + off, b.up_tmp.data_ptr(), H, m, 32, st) == 0
            assert ref.vib3_launch_partial_matmul_int4_f32(x_f32.data_ptr(), gate.device_ptr, gate.device_ptr + off, b.gate_tmp.data_ptr(), H, m, 32, st) == 0
            assert ref.vib3_launch_silu_mul(b.gate_tmp.data_ptr(), b.up_tmp.data_ptr(), b.expert_out.data_ptr() + 2 * up.row_start, m, st) == 0
            launches += 3
        b.down_out.zero_()
        for dp in downs:
            m = dp.row_count
            off = (I // 2) * m
            assert ref.vib3_launch_partial_matmul_int4(b.expert_out.data_ptr(), dp.device_ptr, dp.device_ptr + off, b.down_out.data_ptr() + 2 * dp.row_start, I, m, 32, st) == 0
            launches += 1
        assert ref.vib3_launch_weighted_accumulate_f32(b.layer_out.data_ptr(), b.down_out.data_ptr(), ep.weight, H, st) == 0
        launches += 3  # two buffer clears and the accumulate
    return b.layer_out, launches


def time_reference_gpu_layer(model, xs_f32, router_w_f16, iters: int = 12):
    """One Kimi- or Mixtral-shape layer-token the way the reference engine runs INT4 experts on a GPU:
    router GEMV kernel, stream synchronisation and a copy of the logits to the host (its selection
    kernel needs a power-of-two expert count, cuda/src/kernels.cu:3899, so selection runs on the host
    as in its CPU router), page plan, then the per-page launches.  CUDA events around `iters` tokens.
    Returns {"us_per_layer", "launches"} or None when the reference library is not built."""
    import torch
    from oracle import oracle as O
    from vic_b200.buffer_manager import QueryPlanner
    ref = load_ref_lib()
    if ref is None:
        return None
    sh = model.shape
    dev = xs_f32.device
    planner = QueryPlanner(model.pool, sh.pages_per_segment)
    bufs = RefSublayerBuffers(sh.hidden, sh.intermediate, dev)
    scores = torch.zeros(sh.num_experts, dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream()

    def token(i):
        layer = i % model.n_layers
        x = xs_f32[i % xs_f32.shape[0]]
        assert ref.vib3_launch_router_gemv_f32(x.data_ptr(), router_w_f16[layer].data_ptr(), scores.data_ptr(), sh.hidden,
                                               sh.num_experts, st.cuda_stream) == 0
        st.synchronize()
        ids, ws = O.router_select(scores.cpu().numpy(), sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        _, n = ref_moe_sublayer(ref, model, layer, x, list(zip(ids.tolist(), ws.tolist())), planner, bufs)
        return n + 1

    launches = token(0)
    token(1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        token(2 + i)
    e1.record()
    torch.cuda.synchronize()
    return {"us_per_layer": e0.elapsed_time(e1) * 1e3 / iters, "launches": launches}
