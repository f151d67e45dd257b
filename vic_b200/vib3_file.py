"""Python view of the `.vib3` container code (csrc/host/vib3_file.cpp): INT4 quantiser, page-split writer and
reader — the counterparts of quantize_weights_to_int4 (src/compute/kernels.rs:3778-3831), add_pages_from_data
(src/storage/convert.rs:1841-1901), Vib3Writer / Vib3File (src/storage/format.rs)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from .core_types import EXPERT_SHARED, SEG_DOWN, SEG_GATE, SEG_SHARED_DOWN, SEG_SHARED_GATE, SEG_SHARED_UP, SEG_UP, MoeShape
from .lib import Vib3Error, check, lib

SCALE_BF16, SCALE_FP16 = 0, 1


class _FilePage(C.Structure):
    _fields_ = [("layer", C.c_uint16), ("expert", C.c_uint16), ("segment", C.c_uint16), ("page_idx", C.c_uint16),
                ("row_start", C.c_uint16), ("row_count", C.c_uint16), ("col_count", C.c_uint16), ("compression", C.c_uint16),
                ("file_offset", C.c_uint64), ("raw_size", C.c_uint32)]


def quantize_int4(w: np.ndarray, scale_format: int = SCALE_FP16) -> np.ndarray:
    """fp32 [rows, cols] -> packed buffer [rows * ceil(cols/2) codes][rows * ceil(cols/32) scales]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    out = np.zeros(lib().vib3_int4_matrix_bytes(rows, cols), dtype=np.uint8)
    check("quantize_int4", lib().vib3_quantize_int4(w.ctypes.data, rows, cols, scale_format, out.ctypes.data))
    return out


@dataclass
class FilePage:
    layer: int
    expert: int
    segment: int
    page_idx: int
    row_start: int
    row_count: int
    col_count: int
    compression: int
    file_offset: int
    raw_size: int


class Vib3Writer:
    def __init__(self, path: str, shape: MoeShape, num_layers: int, metadata_json: str = "{}"):
        self._h = lib().vib3_writer_create(path.encode(), metadata_json.encode(), num_layers, shape.num_experts, shape.top_k,
                                           shape.hidden, shape.intermediate)
        if not self._h:
            raise Vib3Error("vib3_writer_create", -7)
        self.shape = shape

    def add_int4_matrix(self, layer: int, expert: int, segment: int, rows: int, cols: int, data: np.ndarray) -> int:
        data = np.ascontiguousarray(data, dtype=np.uint8)
        assert data.size == lib().vib3_int4_matrix_bytes(rows, cols)
        n = lib().vib3_writer_add_int4_matrix(self._h, layer, expert, segment, rows, cols, data.ctypes.data)
        if n < 0:
            raise Vib3Error("vib3_writer_add_int4_matrix", n)
        return n

    def add_expert(self, layer: int, expert: int, up: np.ndarray, gate: np.ndarray, down: np.ndarray,
                   scale_format: int = SCALE_FP16) -> int:
        """fp32 up / gate [I, H] and down [H, I] of one expert (expert = EXPERT_SHARED for the shared one): quantise
        and queue its pages under the reference's segment ids."""
        segs = (SEG_SHARED_UP, SEG_SHARED_GATE, SEG_SHARED_DOWN) if expert == EXPERT_SHARED else (SEG_UP, SEG_GATE, SEG_DOWN)
        n = 0
        for seg, w in zip(segs, (up, gate, down)):
            n += self.add_int4_matrix(layer, expert, seg, w.shape[0], w.shape[1], quantize_int4(w, scale_format))
        return n

    def finalize(self) -> None:
        check("vib3_writer_finalize", lib().vib3_writer_finalize(self._h))
        self.close()

    def close(self) -> None:
        if self._h:
            lib().vib3_writer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Vib3File:
    def __init__(self, path: str):
        err = C.c_int(0)
        self._h = lib().vib3_file_open(path.encode(), C.byref(err))
        if not self._h:
            raise Vib3Error(f"vib3_file_open({path})", err.value)

    def close(self) -> None:
        if self._h:
            lib().vib3_file_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def summary(self) -> dict:
        v = [C.c_uint32() for _ in range(6)]
        off = C.c_uint64()
        check("vib3_file_summary", lib().vib3_file_summary(self._h, *[C.byref(x) for x in v], C.byref(off)))
        keys = ("num_layers", "num_experts", "num_active_experts", "hidden_dim", "expert_hidden_dim", "expert_dtype")
        d = {k: x.value for k, x in zip(keys, v)}
        d["page_data_offset"] = off.value
        return d

    def pages(self) -> List[FilePage]:
        out = []
        for i in range(lib().vib3_file_page_count(self._h)):
            p = _FilePage()
            check("vib3_file_page_info", lib().vib3_file_page_info(self._h, i, C.byref(p)))
            out.append(FilePage(*[getattr(p, f) for f, _ in _FilePage._fields_]))
        return out

    def read_page(self, index: int, raw_size: int) -> np.ndarray:
        buf = np.zeros(raw_size, dtype=np.uint8)
        check("vib3_file_read_page", lib().vib3_file_read_page(self._h, index, buf.ctypes.data, buf.size))
        return buf

    def load_into_pool(self, pool, layers=(0, 65536), experts=(0, 65535)) -> int:
        """Every page of the given layer and expert ranges (and the shared expert) into a PageBufferManager."""
        n = lib().vib3_file_load_into_pool(self._h, pool._h, layers[0], layers[1], experts[0], experts[1])
        if n < 0:
            raise Vib3Error("vib3_file_load_into_pool", int(n))
        return int(n)
