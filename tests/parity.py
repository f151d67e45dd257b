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


from oracle.ref_gpu import load_ref_lib, ref_moe_sublayer  # noqa: E402,F401  (the reference's own CUDA kernels, checker only)
