"""Constants and page identifiers of the reference's core types (src/core/types.rs)."""
from __future__ import annotations

from dataclasses import dataclass

PAGE_SIZE = 2 * 1024 * 1024      # types.rs:14
MAX_EXPERTS = 512                # types.rs:20
MAX_ACTIVE_EXPERTS = 16          # types.rs:26
INT4_GROUP_SIZE = 32             # src/compute/kernels.rs:3737
EXPERT_SHARED = 0xFFFF           # types.rs:170
SEG_UP, SEG_GATE, SEG_DOWN = 0, 1, 2          # types.rs:204
SEG_SHARED_UP, SEG_SHARED_GATE, SEG_SHARED_DOWN = 14, 15, 16  # src/storage/convert.rs:2014-2032

X_F32, X_F16, X_BF16 = 0, 1, 2
W_F16, W_F32 = 0, 1
SCORING_SOFTMAX, SCORING_SIGMOID = 0, 1


@dataclass(frozen=True)
class PageId:
    """types.rs:199-265"""
    layer: int
    expert: int
    segment: int
    page_idx: int

    def key(self) -> int:
        return (self.layer << 48) | (self.expert << 32) | (self.segment << 16) | self.page_idx

    @staticmethod
    def shared(layer: int, segment: int, page_idx: int) -> "PageId":
        return PageId(layer, EXPERT_SHARED, segment, page_idx)


@dataclass(frozen=True)
class Int4Geometry:
    """Page geometry of one INT4 matrix [rows, cols] (src/storage/convert.rs:1807-1812, :1854-1860)."""
    rows: int
    cols: int

    @property
    def packed_k(self) -> int:
        return (self.cols + 1) // 2

    @property
    def num_groups(self) -> int:
        return (self.cols + INT4_GROUP_SIZE - 1) // INT4_GROUP_SIZE

    @property
    def bytes_per_row(self) -> int:
        return self.packed_k + self.num_groups * 2

    @property
    def rows_per_page(self) -> int:
        return max(PAGE_SIZE // self.bytes_per_row, 1)

    @property
    def num_pages(self) -> int:
        return -(-self.rows // self.rows_per_page)

    def page_rows(self, page_idx: int):
        r0 = page_idx * self.rows_per_page
        return r0, min(self.rows_per_page, self.rows - r0)

    def page_bytes(self, page_idx: int) -> int:
        return self.page_rows(page_idx)[1] * self.bytes_per_row

    @property
    def matrix_bytes(self) -> int:
        return self.rows * self.bytes_per_row


@dataclass(frozen=True)
class MoeShape:
    """One MoE layer's sizes."""
    name: str
    hidden: int
    intermediate: int
    num_experts: int
    top_k: int
    shared_experts: int
    scoring: int
    scaling_factor: float
    normalize: bool

    @property
    def gate_up(self) -> Int4Geometry:
        return Int4Geometry(self.intermediate, self.hidden)

    @property
    def down(self) -> Int4Geometry:
        return Int4Geometry(self.hidden, self.intermediate)

    @property
    def pages_per_segment(self) -> int:
        return max(self.gate_up.num_pages, self.down.num_pages)

    @property
    def pages_per_expert(self) -> int:
        return 2 * self.gate_up.num_pages + self.down.num_pages

    @property
    def expert_bytes(self) -> int:
        return 2 * self.gate_up.matrix_bytes + self.down.matrix_bytes


# Mixtral-8x7B-shape layer: softmax over the top-2
MIXTRAL = MoeShape("mixtral-8x7b", 4096, 14336, 8, 2, 0, SCORING_SOFTMAX, 1.0, True)
# Kimi-K2.5-shape layer (types.rs:30-68): sigmoid scoring, top-8 renormalised, x2.827, one shared expert
KIMI = MoeShape("kimi-k2.5", 7168, 2048, 384, 8, 1, SCORING_SIGMOID, 2.827, True)
