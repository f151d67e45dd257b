"""Seeded synthetic weights in the reference's on-device format: INT4 codes uniform in [-8, 7]
(stored as nibble = code + 8), group-32 fp16 scales |N(0, 0.02)| / 7, cut into 2 MiB pages with
the converter's rule (src/storage/convert.rs:1841-1901) and placed in a VRAM page pool.

Scales are rounded to 8 significant bits inside fp16's normal range, so the same real number is
exact in fp16 (what the CUDA kernels decode) and in bf16 (what the reference's CPU kernels
decode)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .buffer_manager import PageBufferManager
from .core_types import (EXPERT_SHARED, PAGE_SIZE, SEG_DOWN, SEG_GATE, SEG_SHARED_DOWN, SEG_SHARED_GATE, SEG_SHARED_UP,
                         SEG_UP, Int4Geometry, MoeShape, PageId)


def synth_scales(shape, gen: torch.Generator, device) -> torch.Tensor:
    s = torch.randn(shape, generator=gen, device=device, dtype=torch.float32).abs_().mul_(0.02 / 7.0)
    s.clamp_(min=2.0 ** -13)
    return s.to(torch.bfloat16).to(torch.float16)


def fill_random_codes(pool: PageBufferManager, gen: torch.Generator, chunk_bytes: int = 1 << 30) -> None:
    """Uniform random bytes over the whole pool: every nibble uniform in 0..15."""
    st = pool.storage
    for o in range(0, st.numel(), chunk_bytes):
        st[o:o + chunk_bytes].random_(0, 256, generator=gen)


@dataclass
class PlacedPage:
    pid: PageId
    slot: int
    row_start: int
    row_count: int
    cols: int
    nbytes: int


@dataclass
class SyntheticMoe:
    """A set of layers of one MoE shape resident in a page pool, plus router weights."""
    shape: MoeShape
    n_layers: int
    pool: PageBufferManager
    router_w: torch.Tensor                      # [n_layers, E, H]
    pages: List[PlacedPage] = field(default_factory=list)
    experts_present: Optional[List[int]] = None  # None = all

    def page_table(self, layer: int) -> int:
        return self.pool.device_page_table(layer, self.shape.num_experts, self.shape.pages_per_segment)

    def shared_table(self, layer: int) -> int:
        if not self.shape.shared_experts:
            return 0
        return self.pool.device_page_table(layer, self.shape.num_experts, self.shape.pages_per_segment, shared=True)


def _segments(shape: MoeShape, expert: int) -> List[Tuple[int, Int4Geometry]]:
    if expert == EXPERT_SHARED:
        return [(SEG_SHARED_UP, shape.gate_up), (SEG_SHARED_GATE, shape.gate_up), (SEG_SHARED_DOWN, shape.down)]
    return [(SEG_UP, shape.gate_up), (SEG_GATE, shape.gate_up), (SEG_DOWN, shape.down)]


def pages_needed(shape: MoeShape, n_layers: int, n_experts: Optional[int] = None) -> int:
    ne = shape.num_experts if n_experts is None else n_experts
    return n_layers * (ne + shape.shared_experts) * shape.pages_per_expert


def build_synthetic_moe(shape: MoeShape, n_layers: int, device, seed: int, slot_seed: int = 0,
                        experts: Optional[Iterable[int]] = None, router_dtype=torch.float32,
                        spare_pages: int = 0, per_page_content: bool = False) -> SyntheticMoe:
    """Place every page of ``n_layers`` layers (all experts, or only ``experts``) into a fresh pool in a
    seeded random slot order, fill codes and scales from a seeded generator, freeze the pool.

    ``per_page_content``: derive every page's bytes from (seed, page id) alone, so that a pool holding
    only a subset of the experts (one expert-parallel rank's shard) holds exactly the same bytes for
    them as the pool holding all experts, and the router weights are the same too.  Slower to build;
    meant for parity tests."""
    device = torch.device(device)
    elist = list(range(shape.num_experts)) if experts is None else sorted(set(int(e) for e in experts))
    n_pages = n_layers * (len(elist) + shape.shared_experts) * shape.pages_per_expert + spare_pages
    pool = PageBufferManager(n_pages, device=device, slot_seed=slot_seed,
                             storage=None if device.type == "cuda" else torch.empty(n_pages * PAGE_SIZE + 256, dtype=torch.uint8))
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    placed: List[PlacedPage] = []
    for layer in range(n_layers):
        for e in elist + ([EXPERT_SHARED] if shape.shared_experts else []):
            for seg, geom in _segments(shape, e):
                for p in range(geom.num_pages):
                    r0, rc = geom.page_rows(p)
                    nbytes = rc * geom.bytes_per_row
                    slot = pool.load_page(PageId(layer, e, seg, p), r0, rc, None, nbytes)
                    placed.append(PlacedPage(PageId(layer, e, seg, p), slot, r0, rc, geom.cols, nbytes))
    if per_page_content:
        pg_gen = torch.Generator(device=device)
        for pg in placed:
            pg_gen.manual_seed((seed * 0x9E3779B1 + pg.pid.key() * 0x85EBCA6B) % (2 ** 63))
            view = pool.slot_view(pg.slot, pg.nbytes)
            ncode = pg.row_count * ((pg.cols + 1) // 2)
            view[:ncode].random_(0, 256, generator=pg_gen)
            sc = synth_scales((pg.nbytes - ncode) // 2, pg_gen, device)
            view[ncode:].copy_(sc.view(torch.uint8))
        pool.freeze()
        gen.manual_seed(seed)
        router_w = (torch.randn(n_layers, shape.num_experts, shape.hidden, generator=gen, device=device,
                                dtype=torch.float32) * 0.02).to(router_dtype)
        return SyntheticMoe(shape, n_layers, pool, router_w, placed, None if experts is None else elist)
    fill_random_codes(pool, gen)
    # scales: one vectorised write per page geometry
    pool2d = pool.storage.view(n_pages, PAGE_SIZE)
    classes: Dict[Tuple[int, int], List[int]] = {}
    for pg in placed:
        classes.setdefault((pg.row_count, pg.cols), []).append(pg.slot)
    for (rc, cols), slots in sorted(classes.items()):
        off = rc * ((cols + 1) // 2)
        n_sc = rc * ((cols + 31) // 32)
        for i in range(0, len(slots), 512):
            idx = torch.tensor(slots[i:i + 512], device=device, dtype=torch.long)
            sc = synth_scales((len(idx), n_sc), gen, device)
            pool2d.narrow(1, off, 2 * n_sc).index_copy_(0, idx, sc.view(torch.uint8).view(len(idx), 2 * n_sc))
    pool.freeze()
    router_w = (torch.randn(n_layers, shape.num_experts, shape.hidden, generator=gen, device=device,
                            dtype=torch.float32) * 0.02).to(router_dtype)
    return SyntheticMoe(shape, n_layers, pool, router_w, placed, None if experts is None else elist)


def synth_activation(shape: MoeShape, gen: torch.Generator, device, dtype=torch.bfloat16, n: int = 1) -> torch.Tensor:
    """Token activations ~ N(0, 1) in the configured dtype, [n, H]."""
    return torch.randn(n, shape.hidden, generator=gen, device=device, dtype=torch.float32).to(dtype)
