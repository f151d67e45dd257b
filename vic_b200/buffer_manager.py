"""Python view of the C++ VRAM page pool and query planner (csrc/host/page_pool.*), the
counterparts of PageBufferManager (src/storage/buffer_manager.rs) and QueryPlanner
(src/runtime/query_planner.rs) for VRAM-resident INT4 expert pages."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .core_types import PAGE_SIZE, PageId
from .lib import ResolvedPage as _CResolvedPage
from .lib import Vib3Error, lib


@dataclass
class PageHandle:
    """buffer_manager.rs PageHandle plus the catalog row range."""
    device_ptr: int
    size: int
    row_start: int
    row_count: int


@dataclass
class ResolvedPage:
    """query_planner.rs:36-42"""
    id: PageId
    device_ptr: int
    row_start: int
    row_count: int


@dataclass
class ExpertPlan:
    """query_planner.rs:28-34"""
    expert_id: int
    weight: float
    pages: List[ResolvedPage]
    fully_resident: bool = True


@dataclass
class LayerPlan:
    """query_planner.rs:21-26"""
    layer: int
    experts: List[ExpertPlan]
    all_resident: bool = True


class PageBufferManager:
    """T1 (VRAM) pool of 2 MiB slots with a frozen resident snapshot.

    ``storage`` is a uint8 tensor of capacity_pages * 2 MiB that backs the slots.  On a CUDA device
    this is the VRAM pool; a CPU tensor gives a host-memory pool for tests of the host logic
    (placement, snapshot, planner), which never touch the GPU."""

    def __init__(self, capacity_pages: int, device: Optional[torch.device] = None, slot_seed: int = 0,
                 storage: Optional[torch.Tensor] = None):
        self.capacity_pages = capacity_pages
        if storage is None:
            dev = device if device is not None else torch.device("cuda")
            storage = torch.empty(capacity_pages * PAGE_SIZE + 256, dtype=torch.uint8, device=dev)
        off = (-storage.data_ptr()) % 256
        self.storage = storage[off:off + capacity_pages * PAGE_SIZE]
        self._raw = storage
        self._h = lib().vib3_pool_create(self.storage.data_ptr(), capacity_pages, slot_seed)
        if not self._h:
            raise Vib3Error("vib3_pool_create", -7)

    def close(self) -> None:
        if self._h:
            lib().vib3_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def base_ptr(self) -> int:
        return self.storage.data_ptr()

    def slot_view(self, slot: int, nbytes: int = PAGE_SIZE) -> torch.Tensor:
        return self.storage[slot * PAGE_SIZE: slot * PAGE_SIZE + nbytes]

    def load_page(self, pid: PageId, row_start: int, row_count: int, data=None, nbytes: Optional[int] = None) -> int:
        """Place a page and return its slot.  ``data``: host bytes (numpy uint8) copied into the slot;
        None: the slot is reserved and the caller fills ``slot_view(slot)`` itself."""
        if data is not None:
            arr = np.ascontiguousarray(data, dtype=np.uint8)
            nbytes = arr.size
            if self.storage.is_cuda:
                ptr = arr.ctypes.data_as(C.c_void_p)
            else:
                ptr = None  # host-memory pool: copy below without the CUDA runtime
        else:
            arr, ptr = None, None
            assert nbytes is not None
        slot = lib().vib3_pool_load_page(self._h, pid.layer, pid.expert, pid.segment, pid.page_idx, row_start,
                                         row_count, ptr, nbytes)
        if slot < 0:
            raise Vib3Error("vib3_pool_load_page", int(slot))
        if arr is not None and not self.storage.is_cuda:
            self.slot_view(slot, nbytes).copy_(torch.from_numpy(arr))
        return int(slot)

    def freeze(self) -> None:
        rc = lib().vib3_pool_freeze(self._h)
        if rc:
            raise Vib3Error("vib3_pool_freeze", rc)

    def resident_pages(self) -> int:
        return int(lib().vib3_pool_resident_pages(self._h))

    def get_page_resident(self, pid: PageId) -> Optional[PageHandle]:
        ptr, rs, rc, sz = C.c_void_p(), C.c_uint16(), C.c_uint16(), C.c_uint32()
        code = lib().vib3_pool_get_page_resident(self._h, pid.key(), C.byref(ptr), C.byref(rs), C.byref(rc), C.byref(sz))
        if code == -6:
            return None
        if code:
            raise Vib3Error("vib3_pool_get_page_resident", code)
        return PageHandle(ptr.value, sz.value, rs.value, rc.value)

    def device_page_table(self, layer: int, num_experts: int, pages_per_segment: int, shared: bool = False) -> int:
        out = C.c_void_p()
        code = lib().vib3_pool_device_page_table(self._h, layer, num_experts, pages_per_segment, int(shared), C.byref(out))
        if code:
            raise Vib3Error("vib3_pool_device_page_table", code)
        return out.value

    def page_bytes_host(self, handle: PageHandle) -> np.ndarray:
        """Copy a resident page back to the host (for the oracle in tests)."""
        off = handle.device_ptr - self.base_ptr
        return self.storage[off:off + handle.size].cpu().numpy()


class QueryPlanner:
    """plan_layer over the resident snapshot (query_planner.rs:158-272)."""

    def __init__(self, pool: PageBufferManager, pages_per_segment: int):
        self.pool = pool
        self.pages_per_segment = pages_per_segment

    def plan_layer(self, layer: int, activation: Sequence) -> LayerPlan:
        """``activation``: sequence of (expert_id, weight), as ExpertActivation.experts.  Raises
        Vib3Error (the reference's Error::PageNotFound) when a page of an active expert is absent."""
        cap = 3 * self.pages_per_segment
        buf = (_CResolvedPage * cap)()
        experts: List[ExpertPlan] = []
        for e, w in activation:
            eid = np.asarray([int(e)], dtype=np.uint16)
            n = lib().vib3_planner_plan_layer(self.pool._h, layer, eid.ctypes.data_as(C.c_void_p), 1,
                                              self.pages_per_segment, C.cast(buf, C.c_void_p), cap)
            if n < 0:
                raise Vib3Error("plan_layer (PageNotFound)" if n == -6 else "plan_layer", n)
            pages = []
            for i in range(n):
                k = buf[i].key
                pid = PageId((k >> 48) & 0xFFFF, (k >> 32) & 0xFFFF, (k >> 16) & 0xFFFF, k & 0xFFFF)
                pages.append(ResolvedPage(pid, buf[i].device_ptr or 0, buf[i].row_start, buf[i].row_count))
            experts.append(ExpertPlan(int(e), float(w), pages))
        return LayerPlan(layer, experts)
