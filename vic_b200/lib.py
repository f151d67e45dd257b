"""ctypes loader of libvib3_cuda.so.  The library is the product: if it is missing it is built
with nvcc; if that fails the import fails — there is no CPU or PyTorch fallback."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_lib = None

ERR_NAMES = {
    -1: "unsupported", -2: "count out of range", -3: "null pointer", -4: "misaligned pointer",
    -5: "bad shape", -6: "row range / page missing", -7: "wrong state", -8: "larger than the built-in buffer",
}


class Vib3Error(RuntimeError):
    """Mirror of the reference's Error::Cuda(String) raised by its launch wrappers
    (src/compute/kernels.rs:145-150) for any non-zero launcher return."""

    def __init__(self, what: str, code: int):
        self.code = code
        kind = ERR_NAMES.get(code, f"cudaError {code}" if code > 0 else "refused")
        super().__init__(f"{what} failed (err={code}: {kind})")


class PageEntry(C.Structure):
    _fields_ = [("ptr", C.c_uint64), ("row_start", C.c_uint16), ("row_count", C.c_uint16), ("reserved", C.c_uint32)]


class ResolvedPage(C.Structure):
    _fields_ = [("key", C.c_uint64), ("device_ptr", C.c_void_p), ("expert_id", C.c_uint16), ("segment", C.c_uint16),
                ("row_start", C.c_uint16), ("row_count", C.c_uint16)]


_vp, _i, _f = C.c_void_p, C.c_int, C.c_float

# every symbol include/vib3_b200.h declares, with its argument types
SIGNATURES = {
    "vib3_launch_partial_matmul_int4": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "vib3_launch_partial_matmul_int4_f32": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "vib3_launch_fused_swiglu_int4_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "vib3_launch_silu_mul": (_i, [_vp, _vp, _vp, _i, _vp]),
    "vib3_launch_weighted_accumulate": (_i, [_vp, _vp, _f, _i, _vp]),
    "vib3_launch_weighted_accumulate_f32": (_i, [_vp, _vp, _f, _i, _vp]),
    "vib3_launch_weighted_accumulate_f32_f32": (_i, [_vp, _vp, _f, _i, _vp]),
    "vib3_launch_residual_add_f32_f32": (_i, [_vp, _vp, _i, _vp]),
    "vib3_launch_router_gemv": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "vib3_launch_router_gemv_f32": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "vib3_launch_router_topk": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "vib3_launch_router_topk_ex": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp, _vp]),
    "vib3_launch_moe_layer_int4_paged": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _i, _i, _i,
                                              _i, _i, _vp, _vp]),
    "vib3_launch_moe_gate_up_int4_paged": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _i, _i, _i,
                                                _i, _i, _vp, _vp]),
    "vib3_launch_moe_down_int4_paged": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _i, _i, _i,
                                             _i, _i, _vp, _vp]),
    "vib3_launch_moe_layer_routed_int4_paged": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp, _vp,
                                                     _vp, _f, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "vib3_launch_moe_layer_int4_paged_noalloc": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _i, _i, _i, _i,
                                                      _i, _vp, _vp]),
    "vib3_launch_moe_layer_int4_paged_var": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _f, _vp, _vp, _i, _i, _i, _i, _i,
                                                  _i, _i, _vp, _vp, _vp]),
    "vib3_launch_moe_layer_int4_paged_grouped": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _f, _vp,
                                                      _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "vib3_launch_select_local_pairs": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "vib3_moe_layer_step_host": (_i, [_vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _f, _vp,
                                      _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "vib3_moe_step_create": (_i, [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _f, _vp, _vp, _i, _i,
                                  _i, _i, _i, _i, _vp, _vp, C.POINTER(_vp)]),
    "vib3_moe_step_run": (_i, [_vp, _vp, _vp]),
    "vib3_moe_step_destroy": (None, [_vp]),
    "vib3_launch_sum_rows_f32": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "vib3_peer_alloc": (_i, [C.c_size_t, C.POINTER(_vp), _vp]),
    "vib3_peer_open": (_i, [_vp, C.POINTER(_vp)]),
    "vib3_peer_close": (_i, [_vp]),
    "vib3_peer_free": (_i, [_vp]),
    "vib3_launch_peer_publish": (_i, [_vp, C.c_size_t, _i, _vp, C.c_size_t, _vp, _vp, _i, _i, _i, _vp]),
    "vib3_launch_peer_publish_rows": (_i, [_vp, _vp, C.c_size_t, _i, _vp, _i, _vp, C.c_size_t, _vp, _vp, _i, _i, _i, _vp]),
    "vib3_launch_peer_select_pairs": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "vib3_launch_peer_sum_rows": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "vib3_launch_peer_wait": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "vib3_launch_select_local_experts": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "vib3_moe_grouped_workspace_bytes": (C.c_size_t, [_i, _i, _i, _i, _i, _i, _i]),
    "vib3_moe_grouped_prewarm": (_i, [_vp, C.c_size_t, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, C.c_size_t, C.POINTER(_vp)]),
    "vib3_moe_grouped_destroy": (None, [_vp]),
    "vib3_launch_moe_grouped_int4": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _f, _i, _i, _i, _vp, _i, _i, _vp, _vp]),
    "vib3_launch_router_topk_batch": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _i,
                                           _i, _vp, _vp]),
    "vib3_launch_rms_norm_f32": (_i, [_vp, _vp, _vp, _i, _f, _vp]),
    "vib3_launch_residual_rms_norm": (_i, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _f, _i, _vp, _i, _i, _i, _i, _vp]),
    "vib3_config_set": (_i, [_i, _i]),
    "vib3_pool_create": (_vp, [_vp, C.c_size_t, C.c_uint64]),
    "vib3_pool_destroy": (None, [_vp]),
    "vib3_pool_load_page": (C.c_longlong, [_vp, C.c_uint16, C.c_uint16, C.c_uint16, C.c_uint16, C.c_uint16,
                                           C.c_uint16, _vp, C.c_size_t]),
    "vib3_pool_slot_ptr": (_vp, [_vp, C.c_longlong]),
    "vib3_pool_freeze": (_i, [_vp]),
    "vib3_pool_get_page_resident": (_i, [_vp, C.c_uint64, C.POINTER(_vp), C.POINTER(C.c_uint16),
                                         C.POINTER(C.c_uint16), C.POINTER(C.c_uint32)]),
    "vib3_pool_resident_pages": (C.c_size_t, [_vp]),
    "vib3_pool_device_page_table": (_i, [_vp, C.c_uint16, _i, _i, _i, C.POINTER(_vp)]),
    "vib3_page_key": (C.c_uint64, [C.c_uint16] * 4),
    "vib3_planner_plan_layer": (_i, [_vp, C.c_uint16, _vp, _i, _i, _vp, _i]),
    "vib3_int4_matrix_bytes": (C.c_size_t, [_i, _i]),
    "vib3_quantize_int4": (_i, [_vp, _i, _i, _i, _vp]),
    "vib3_writer_create": (_vp, [C.c_char_p, C.c_char_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "vib3_writer_add_int4_matrix": (_i, [_vp, C.c_uint16, C.c_uint16, C.c_uint16, _i, _i, _vp]),
    "vib3_writer_finalize": (_i, [_vp]),
    "vib3_writer_destroy": (None, [_vp]),
    "vib3_file_open": (_vp, [C.c_char_p, C.POINTER(_i)]),
    "vib3_file_close": (None, [_vp]),
    "vib3_file_page_count": (_i, [_vp]),
    "vib3_file_summary": (_i, [_vp] + [C.POINTER(C.c_uint32)] * 6 + [C.POINTER(C.c_uint64)]),
    "vib3_file_page_info": (_i, [_vp, _i, _vp]),
    "vib3_file_read_page": (_i, [_vp, _i, _vp, C.c_size_t]),
    "vib3_file_load_into_pool": (C.c_longlong, [_vp, _vp, _i, _i, _i, _i]),
    "vib3_b200_version": (C.c_char_p, []),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path):
            path = _build.build()
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(what: str, code: int) -> None:
    if code != 0:
        raise Vib3Error(what, int(code))
