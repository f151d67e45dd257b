"""Shared helpers for the parity tests: tolerances of the target specification and the bridge
from a device page pool to the oracle's page structures."""
from __future__ import annotations

import numpy as np

MAX_ABS_TOL = 2e-2   # layer outputs: max-abs
REL_L2_TOL = 1e-3    # layer outputs: relative L2


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    d = np.linalg.norm(a - b)
    n = np.linalg.norm(b)
    return float(d / n) if n > 0 else float(d)


def max_abs(a, b) -> float:
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)))) if np.size(a) else 0.0


def assert_close(got, want, what="", max_abs_tol=MAX_ABS_TOL, rel_l2_tol=REL_L2_TOL):
    ma, rl = max_abs(got, want), rel_l2(got, want)
    assert ma <= max_abs_tol and rl <= rel_l2_tol, f"{what}: max-abs {ma:.3e} (tol {max_abs_tol}), rel-L2 {rl:.3e} (tol {rel_l2_tol})"
    return ma, rl


def oracle_experts(O, model, layer, activation):
    """Build the oracle's expert list (host copies of the pages) for [(expert, weight)] plus the
    shared expert, from the pool's resident snapshot."""
    from vic_b200.core_types import (EXPERT_SHARED, SEG_DOWN, SEG_GATE, SEG_SHARED_DOWN, SEG_SHARED_GATE, SEG_SHARED_UP,
                                     SEG_UP, PageId)
    sh = model.shape
    entries = list(activation) + ([(EXPERT_SHARED, 1.0)] if sh.shared_experts else [])
    out = []
    for e, w in entries:
        segs = (SEG_SHARED_UP, SEG_SHARED_GATE, SEG_SHARED_DOWN) if e == EXPERT_SHARED else (SEG_UP, SEG_GATE, SEG_DOWN)
        lists = []
        for seg, geom in zip(segs, (sh.gate_up, sh.gate_up, sh.down)):
            pages = []
            for p in range(geom.num_pages):
                h = model.pool.get_page_resident(PageId(layer, int(e), seg, p))
                assert h is not None
                pages.append(O.OraclePage(model.pool.page_bytes_host(h), h.row_start, h.row_count))
            lists.append(pages)
        out.append(O.OracleExpert(float(w), lists[0], lists[1], lists[2]))
    return out


def load_ref_lib():
    """The reference's own CUDA kernels compiled unmodified (oracle/Makefile, target `ref`), or None."""
    import ctypes
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libvib3_ref.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
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


def ref_moe_sublayer(ref, model, layer, x_f32, activation, planner):
    """The reference engine's INT4 call sequence (engine.rs:6094-6107, :6215-6223, :6290-6296) on the
    reference's own kernels: returns layer_out_f32 (torch, device) and the launch count."""
    import torch
    from vic_b200.core_types import EXPERT_SHARED
    sh = model.shape
    H, I = sh.hidden, sh.intermediate
    dev = x_f32.device
    st = torch.cuda.current_stream().cuda_stream
    up_tmp = torch.zeros(I, dtype=torch.float16, device=dev)
    gate_tmp = torch.zeros(I, dtype=torch.float16, device=dev)
    expert_out = torch.zeros(I, dtype=torch.float16, device=dev)
    down_out = torch.zeros(H, dtype=torch.float16, device=dev)
    layer_out = torch.zeros(H, dtype=torch.float32, device=dev)
    entries = list(activation) + ([(EXPERT_SHARED, 1.0)] if sh.shared_experts else [])
    plan = planner.plan_layer(layer, entries)
    launches = 0
    for ep in plan.experts:
        segs = sorted(set(p.id.segment for p in ep.pages))
        ups = [p for p in ep.pages if p.id.segment == segs[0]]
        gates = [p for p in ep.pages if p.id.segment == segs[1]]
        downs = [p for p in ep.pages if p.id.segment == segs[2]]
        expert_out.zero_()
        for up, gate in zip(ups, gates):
            m = up.row_count
            off = (H // 2) * m
            assert ref.vib3_launch_partial_matmul_int4_f32(x_f32.data_ptr(), up.device_ptr, up.device_ptr + off, up_tmp.data_ptr(), H, m, 32, st) == 0
            assert ref.vib3_launch_partial_matmul_int4_f32(x_f32.data_ptr(), gate.device_ptr, gate.device_ptr + off, gate_tmp.data_ptr(), H, m, 32, st) == 0
            assert ref.vib3_launch_silu_mul(gate_tmp.data_ptr(), up_tmp.data_ptr(), expert_out.data_ptr() + 2 * up.row_start, m, st) == 0
            launches += 3
        down_out.zero_()
        for dp in downs:
            m = dp.row_count
            off = (I // 2) * m
            assert ref.vib3_launch_partial_matmul_int4(expert_out.data_ptr(), dp.device_ptr, dp.device_ptr + off, down_out.data_ptr() + 2 * dp.row_start, I, m, 32, st) == 0
            launches += 1
        assert ref.vib3_launch_weighted_accumulate_f32(layer_out.data_ptr(), down_out.data_ptr(), ep.weight, H, st) == 0
        launches += 1
    return layer_out, launches
