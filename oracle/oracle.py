"""numpy front end of the CPU oracle (``vib3_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` import
this module; the product package never does.  Every function is a thin wrapper over one C
function, which cites the reference lines it restates, plus two layer-level compositions that
follow the reference engine's call order (src/runtime/engine.rs:6002-6110, :6164-6226,
:6278-6297).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libvib3_oracle.so")

SCALE_BF16 = 0  # what the reference's CPU kernels decode
SCALE_FP16 = 1  # what the reference's CUDA kernels decode
ORDER_SEQUENTIAL = 0  # reference CPU router: one f32 chain per expert
ORDER_GPU128 = 1  # reference CUDA router GEMV: 128 interleaved fma chains + shuffle tree
MODE_SOFTMAX = 0
MODE_SIGMOID = 1
GROUP_SIZE = 32  # INT4_GROUP_SIZE, src/compute/kernels.rs:3737
PAGE_SIZE = 2 * 1024 * 1024  # src/core/types.rs:14


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "vib3_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libvib3_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.vo_f16_to_f32.restype = ctypes.c_float
        _lib.vo_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.vo_f32_to_f16.restype = ctypes.c_uint16
        _lib.vo_f32_to_f16.argtypes = [ctypes.c_float]
        _lib.vo_bf16_to_f32.restype = ctypes.c_float
        _lib.vo_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.vo_f32_to_bf16.restype = ctypes.c_uint16
        _lib.vo_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.vo_page_key.restype = ctypes.c_uint64
        _lib.vo_page_key.argtypes = [ctypes.c_uint16] * 4
        _lib.vo_router_select.restype = ctypes.c_int
        _lib.vo_router.restype = ctypes.c_int
        _lib.vo_set_num_threads.restype = ctypes.c_int
        _lib.vo_set_num_threads.argtypes = [ctypes.c_int]
        _lib.vo_build_flags.restype = ctypes.c_char_p
    return _lib


def set_num_threads(n: int = 0) -> int:
    """Use n OpenMP threads for the row loops (0: leave as is); returns the count in force."""
    return int(lib().vo_set_num_threads(int(n)))


def build_flags() -> str:
    return lib().vo_build_flags().decode()


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _f(v: float) -> ctypes.c_float:
    return ctypes.c_float(float(v))


# ── INT4 kernels ───────────────────────────────────────────────────────────────────────────

def matmul_int4_rows_f32(x_f32, page_u8, K: int, M: int, group_size: int = GROUP_SIZE,
                         scale_format: int = SCALE_FP16) -> np.ndarray:
    """Raw f32 row sums of one page (row loop of cpu_matmul_int4_grouped, no output rounding)."""
    x = _c(x_f32, np.float32)
    page = _c(page_u8, np.uint8)
    assert x.size >= K and page.size >= page_bytes(K, M, group_size)
    y = np.empty(M, np.float32)
    lib().vo_matmul_int4_rows_f32(_p(x), _p(page), _p(y), K, M, group_size, scale_format)
    return y


def matmul_int4(x_f16, page_u8, K: int, M: int, group_size: int = GROUP_SIZE,
                scale_format: int = SCALE_BF16) -> np.ndarray:
    """``partial_matmul(.., DType::INT4)`` on the CPU stream: f16 in, f16 out."""
    x = _c(x_f16, np.float16)
    page = _c(page_u8, np.uint8)
    y = np.empty(M, np.float16)
    lib().vo_matmul_int4(_p(x), _p(page), _p(y), K, M, group_size, scale_format)
    return y


def swiglu_int4(x_f16, up_page, gate_page, H: int, M: int, group_size: int = GROUP_SIZE,
                scale_format: int = SCALE_BF16) -> np.ndarray:
    """``partial_swiglu(.., DType::INT4)`` on the CPU stream: f16 in, f16 out."""
    x = _c(x_f16, np.float16)
    y = np.empty(M, np.float16)
    lib().vo_swiglu_int4(_p(x), _p(_c(up_page, np.uint8)), _p(_c(gate_page, np.uint8)), _p(y), H, M,
                         group_size, scale_format)
    return y


def swiglu_int4_f32in(x_f32, up_page, gate_page, H: int, M: int, group_size: int = GROUP_SIZE,
                      scale_format: int = SCALE_FP16) -> np.ndarray:
    x = _c(x_f32, np.float32)
    y = np.empty(M, np.float16)
    lib().vo_swiglu_int4_f32in(_p(x), _p(_c(up_page, np.uint8)), _p(_c(gate_page, np.uint8)), _p(y), H, M,
                               group_size, scale_format)
    return y


def silu_mul(a_f16, b_f16) -> np.ndarray:
    a = _c(a_f16, np.float16)
    b = _c(b_f16, np.float16)
    y = np.empty(a.size, np.float16)
    lib().vo_silu_mul(_p(a), _p(b), _p(y), a.size)
    return y


def weighted_accumulate(out_f16: np.ndarray, y_f16, w: float) -> None:
    assert out_f16.dtype == np.float16 and out_f16.flags.c_contiguous
    y = _c(y_f16, np.float16)
    lib().vo_weighted_accumulate(_p(out_f16), _p(y), _f(w), out_f16.size)


def weighted_accumulate_f32(out_f32: np.ndarray, y_f16, w: float) -> None:
    assert out_f32.dtype == np.float32 and out_f32.flags.c_contiguous
    y = _c(y_f16, np.float16)
    lib().vo_weighted_accumulate_f32(_p(out_f32), _p(y), _f(w), out_f32.size)


def weighted_accumulate_f32_f32(out_f32: np.ndarray, y_f32, w: float) -> None:
    assert out_f32.dtype == np.float32 and out_f32.flags.c_contiguous
    y = _c(y_f32, np.float32)
    lib().vo_weighted_accumulate_f32_f32(_p(out_f32), _p(y), _f(w), out_f32.size)


def residual_add_f32_f32(acc_f32: np.ndarray, layer_out_f32) -> None:
    assert acc_f32.dtype == np.float32 and acc_f32.flags.c_contiguous
    lib().vo_residual_add_f32_f32(_p(acc_f32), _p(_c(layer_out_f32, np.float32)), acc_f32.size)


def rms_norm_f32(x_f32, w_f32=None, eps: float = 1e-6) -> np.ndarray:
    x = _c(x_f32, np.float32)
    w = None if w_f32 is None else _c(w_f32, np.float32)
    y = np.empty_like(x)
    lib().vo_rms_norm_f32(_p(x), _p(w), _p(y), x.size, _f(eps))
    return y


# ── Router ─────────────────────────────────────────────────────────────────────────────────

def router_logits(x_f32, W, order: int = ORDER_SEQUENTIAL) -> np.ndarray:
    """Raw logits; W is [E,H] float16 (the reference's format) or float32."""
    x = _c(x_f32, np.float32)
    assert W.dtype in (np.float16, np.float32) and W.ndim == 2 and W.flags.c_contiguous
    E, H = W.shape
    logits = np.empty(E, np.float32)
    lib().vo_router_logits(_p(x), _p(W), int(W.dtype == np.float32), E, H, order, _p(logits))
    return logits


def router_select(logits, top_k: int, mode: int, scaling_factor: float = 1.0, normalize: bool = True,
                  bias=None) -> Tuple[np.ndarray, np.ndarray]:
    lg = _c(logits, np.float32)
    b = None if bias is None else _c(bias, np.float32)
    k = min(top_k, lg.size)
    ids = np.empty(k, np.uint16)
    w = np.empty(k, np.float32)
    n = lib().vo_router_select(_p(lg), lg.size, top_k, mode, _f(scaling_factor), int(normalize), _p(b),
                               _p(ids), _p(w))
    assert n == k
    return ids, w


def router(x_f32, W, top_k: int, mode: int, scaling_factor: float = 1.0, normalize: bool = True,
           bias=None, order: int = ORDER_SEQUENTIAL, logit_offset=None) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """``run_router_with_scoring_and_bias``: returns (ids u16[k], weights f32[k], logits f32[E]).
    ``logit_offset`` (not in the reference: the synthetic expert-load skew of the multi-token
    benchmark config) is added to the logits with one fp32 addition before scoring."""
    logits = router_logits(x_f32, W, order)
    if logit_offset is not None:
        logits = (logits + np.asarray(logit_offset, np.float32)).astype(np.float32)
    ids, w = router_select(logits, top_k, mode, scaling_factor, normalize, bias)
    return ids, w, logits


# ── Quantiser, page geometry ───────────────────────────────────────────────────────────────

def page_bytes(K: int, M: int, group_size: int = GROUP_SIZE) -> int:
    return M * ((K + 1) // 2) + M * ((K + group_size - 1) // group_size) * 2


def quantize_int4(w_f32, group_size: int = GROUP_SIZE, scale_format: int = SCALE_BF16) -> np.ndarray:
    w = _c(w_f32, np.float32)
    rows, cols = w.shape
    out = np.empty(page_bytes(cols, rows, group_size), np.uint8)
    lib().vo_quantize_int4(_p(w), rows, cols, group_size, scale_format, _p(out))
    return out


def dequantize_int4(data_u8, rows: int, cols: int, group_size: int = GROUP_SIZE,
                    scale_format: int = SCALE_BF16) -> np.ndarray:
    data = _c(data_u8, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().vo_dequantize_int4(_p(data), rows, cols, group_size, scale_format, _p(out))
    return out


def int4_page_geometry(rows: int, cols: int, group_size: int = GROUP_SIZE,
                       page_size: int = PAGE_SIZE) -> Tuple[int, int, int]:
    """(bytes_per_row, rows_per_page, num_pages)."""
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().vo_int4_page_geometry(rows, cols, group_size, page_size, ctypes.byref(a), ctypes.byref(b),
                                ctypes.byref(c))
    return a.value, b.value, c.value


def page_key(layer: int, expert: int, segment: int, page_idx: int) -> int:
    return int(lib().vo_page_key(layer, expert, segment, page_idx))


def split_int4_pages(matrix_u8, rows: int, cols: int, group_size: int = GROUP_SIZE,
                     page_size: int = PAGE_SIZE) -> List[Tuple[np.ndarray, int, int]]:
    """Cut a quantised matrix into page images: list of (bytes, row_start, row_count)."""
    m = _c(matrix_u8, np.uint8)
    _, _, npages = int4_page_geometry(rows, cols, group_size, page_size)
    out = np.empty(m.size, np.uint8)
    rs = np.empty(npages, np.int32)
    rc = np.empty(npages, np.int32)
    lib().vo_split_int4_pages(_p(m), rows, cols, group_size, page_size, _p(out), _p(rs), _p(rc))
    pages, o = [], 0
    for p in range(npages):
        n = page_bytes(cols, int(rc[p]), group_size)
        pages.append((out[o:o + n].copy(), int(rs[p]), int(rc[p])))
        o += n
    return pages


# ── Layer-level compositions in the reference engine's call order ──────────────────────────

@dataclass
class OraclePage:
    """One resolved page of a plan: host bytes plus the catalog's row range."""
    data: np.ndarray
    row_start: int
    row_count: int


@dataclass
class OracleExpert:
    """One entry of a layer plan: routing weight and the pages of segments 0 (up), 1 (gate),
    2 (down) in page order (src/core/types.rs:204)."""
    weight: float
    up: Sequence[OraclePage]
    gate: Sequence[OraclePage]
    down: Sequence[OraclePage]


def expert_forward_gpu_order(x_f32, ex: OracleExpert, H: int, I: int, scale_format: int = SCALE_FP16):
    """One expert in the order the reference engine drives its CUDA launchers for INT4
    (engine.rs:6094-6107 → kernels.rs:493-541; engine.rs:6215-6223): per (up, gate) page pair
    two f32-input matmuls rounded to f16, then silu(gate)*up rounded to f16; per down page an
    f16-input matmul rounded to f16.  Row sums use the CPU row kernel's sequential order.
    Returns (act_f16[I], down_f16[H])."""
    x = _c(x_f32, np.float32)
    act = np.zeros(I, np.float16)
    for up, gate in zip(ex.up, ex.gate):
        assert up.row_start == gate.row_start and up.row_count == gate.row_count
        u = matmul_int4_rows_f32(x, up.data, H, up.row_count, GROUP_SIZE, scale_format).astype(np.float16)
        g = matmul_int4_rows_f32(x, gate.data, H, gate.row_count, GROUP_SIZE, scale_format).astype(np.float16)
        act[up.row_start:up.row_start + up.row_count] = silu_mul(g, u)
    down = np.zeros(H, np.float16)
    act32 = act.astype(np.float32)
    for pg in ex.down:
        d = matmul_int4_rows_f32(act32, pg.data, I, pg.row_count, GROUP_SIZE, scale_format)
        down[pg.row_start:pg.row_start + pg.row_count] = d.astype(np.float16)
    return act, down


def expert_forward_cpu_order(x_f16, ex: OracleExpert, H: int, I: int, scale_format: int = SCALE_BF16):
    """One expert through the reference's CPU entry points: ``partial_swiglu`` (up and gate kept
    in f32, one f16 rounding) then ``partial_matmul``.  Returns (act_f16[I], down_f16[H])."""
    act = np.zeros(I, np.float16)
    for up, gate in zip(ex.up, ex.gate):
        act[up.row_start:up.row_start + up.row_count] = swiglu_int4(
            x_f16, up.data, gate.data, H, up.row_count, GROUP_SIZE, scale_format)
    down = np.zeros(H, np.float16)
    for pg in ex.down:
        down[pg.row_start:pg.row_start + pg.row_count] = matmul_int4(
            act, pg.data, I, pg.row_count, GROUP_SIZE, scale_format)
    return act, down


def moe_layer(x_f32, experts: Sequence[OracleExpert], H: int, I: int, scale_format: int = SCALE_FP16,
              order: str = "gpu") -> np.ndarray:
    """MoE sublayer output in f32: zeroed accumulator, then ``out += weight * down_f16`` expert by
    expert in plan order (engine.rs:5200, :6290-6296); a shared expert is one more entry with
    weight 1.0 at the end (engine.rs:6442-6451)."""
    out = np.zeros(H, np.float32)
    for ex in experts:
        if order == "gpu":
            _, down = expert_forward_gpu_order(x_f32, ex, H, I, scale_format)
        else:
            _, down = expert_forward_cpu_order(np.asarray(x_f32, np.float32).astype(np.float16), ex, H, I,
                                               scale_format)
        weighted_accumulate_f32(out, down, ex.weight)
    return out
