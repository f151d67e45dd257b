"""No-GPU checks: the shared library loads and exports every symbol the header declares; the host
side (page pool, resident snapshot, planner) behaves like the reference's on host memory."""
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from vic_b200 import lib as L
    hdr = open(os.path.join(ROOT, "include", "vib3_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)   # declarations only, not the prose
    declared = set(re.findall(r"\b(vib3_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"vib3_page_entry", "vib3_resolved_page"}
    assert len(declared) >= 24
    handle = L.lib()
    for name in sorted(declared):
        assert hasattr(handle, name), name
    assert set(L.SIGNATURES) == declared
    assert b"sm_100a" in handle.vib3_b200_version()


def test_page_entry_layouts():
    import ctypes
    from vic_b200.lib import PageEntry, ResolvedPage
    assert ctypes.sizeof(PageEntry) == 16 and PageEntry.row_start.offset == 8 and PageEntry.row_count.offset == 10
    assert ctypes.sizeof(ResolvedPage) == 24


def _tiny():
    from vic_b200.core_types import SCORING_SOFTMAX, MoeShape
    return MoeShape("tiny", 64, 96, 4, 2, 1, SCORING_SOFTMAX, 1.0, True)


def test_pool_placement_snapshot_and_planner_on_host_memory(oracle):
    from vic_b200.buffer_manager import QueryPlanner
    from vic_b200.core_types import EXPERT_SHARED, PAGE_SIZE, PageId
    from vic_b200.lib import Vib3Error
    from vic_b200.synth import build_synthetic_moe
    sh = _tiny()
    m = build_synthetic_moe(sh, 2, "cpu", seed=1, slot_seed=7)
    assert m.pool.resident_pages() == 2 * 5 * 3 == len(m.pages)
    slots = [p.slot for p in m.pages]
    assert sorted(slots) == list(range(30)) and slots != sorted(slots)      # a permutation, scattered
    # the same seed gives the same placement; sequential when slot_seed == 0
    m2 = build_synthetic_moe(sh, 2, "cpu", seed=1, slot_seed=7)
    assert [p.slot for p in m2.pages] == slots
    assert torch.equal(m.pool.storage, m2.pool.storage)
    m3 = build_synthetic_moe(sh, 2, "cpu", seed=1, slot_seed=0)
    assert [p.slot for p in m3.pages] == list(range(30))
    h = m.pool.get_page_resident(PageId(1, 2, 0, 0))
    assert h is not None and h.row_start == 0 and h.row_count == 96 and h.size == 96 * (32 + 4)
    assert (h.device_ptr - m.pool.base_ptr) % PAGE_SIZE == 0
    assert m.pool.get_page_resident(PageId(1, 2, 0, 1)) is None and m.pool.get_page_resident(PageId(2, 0, 0, 0)) is None
    plan = QueryPlanner(m.pool, sh.pages_per_segment).plan_layer(1, [(2, 0.5), (0, 0.25), (EXPERT_SHARED, 1.0)])
    assert [(e.expert_id, e.weight, len(e.pages)) for e in plan.experts] == [(2, 0.5, 3), (0, 0.25, 3), (0xFFFF, 1.0, 3)]
    assert [p.id.segment for p in plan.experts[0].pages] == [0, 1, 2]        # catalog order
    assert [p.id.segment for p in plan.experts[2].pages] == [14, 15, 16]
    assert plan.experts[0].pages[0].device_ptr == h.device_ptr
    with pytest.raises(Vib3Error):
        QueryPlanner(m.pool, sh.pages_per_segment).plan_layer(1, [(9, 1.0)])  # Error::PageNotFound
    # a frozen pool accepts no more pages
    with pytest.raises(Vib3Error):
        m.pool.load_page(PageId(0, 3, 5, 0), 0, 1, None, 16)


def test_pool_full_duplicate_and_unfrozen_lookup():
    from vic_b200.buffer_manager import PageBufferManager, QueryPlanner
    from vic_b200.core_types import PAGE_SIZE, PageId
    from vic_b200.lib import Vib3Error
    pool = PageBufferManager(2, storage=torch.empty(2 * PAGE_SIZE + 256, dtype=torch.uint8))
    data = np.arange(64, dtype=np.uint8)
    s0 = pool.load_page(PageId(0, 0, 0, 0), 0, 4, data)
    assert np.array_equal(pool.slot_view(s0, 64).numpy(), data)
    with pytest.raises(Vib3Error):
        pool.load_page(PageId(0, 0, 0, 0), 0, 4, data)                  # already resident
    with pytest.raises(Vib3Error):
        pool.get_page_resident(PageId(0, 0, 0, 0))                      # snapshot not frozen yet
    pool.load_page(PageId(0, 0, 0, 2), 8, 4, data)
    with pytest.raises(Vib3Error):
        pool.load_page(PageId(0, 0, 0, 3), 12, 4, data)                 # TierFull
    pool.freeze()
    with pytest.raises(Vib3Error):
        QueryPlanner(pool, 4).plan_layer(0, [(0, 1.0)])                 # page 1 of segment 0 is missing


def test_synthetic_pages_match_the_converter_split(oracle):
    """Pages placed by the generator have the converter's geometry and decode with both scale encodings."""
    from vic_b200.core_types import PageId
    from vic_b200.synth import build_synthetic_moe
    sh = _tiny()
    m = build_synthetic_moe(sh, 1, "cpu", seed=2, slot_seed=3)
    h = m.pool.get_page_resident(PageId(0, 1, 1, 0))
    page = m.pool.page_bytes_host(h)
    K, M = sh.hidden, h.row_count
    sc = page[M * K // 2:].view(np.float16).astype(np.float32)
    assert np.all(sc >= 2.0 ** -13) and np.all(sc < 0.03)
    # exactly representable in bf16 as well: 8 significant bits
    assert np.array_equal(torch.from_numpy(sc).to(torch.bfloat16).float().numpy(), sc)
    x = np.random.default_rng(0).standard_normal(K).astype(np.float32)
    y16 = oracle.matmul_int4_rows_f32(x, page, K, M, 32, oracle.SCALE_FP16)
    page_bf = page.copy()
    page_bf[M * K // 2:] = torch.from_numpy(sc).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint8)
    ybf = oracle.matmul_int4_rows_f32(x, page_bf, K, M, 32, oracle.SCALE_BF16)
    assert np.array_equal(y16, ybf)
    codes = page[:M * K // 2]
    assert codes.min() == 0 and codes.max() == 255


def test_oracle_layer_orders_agree(oracle):
    """The engine-order chain (fp16 after each projection) and the CPU-kernel chain (one rounding) differ
    only by fp16 rounding noise."""
    from tests.parity import oracle_experts, rel_l2
    from vic_b200.synth import build_synthetic_moe
    sh = _tiny()
    m = build_synthetic_moe(sh, 1, "cpu", seed=5, slot_seed=1)
    x = np.random.default_rng(1).standard_normal(sh.hidden).astype(np.float16).astype(np.float32)
    ex = oracle_experts(oracle, m, 0, [(1, 0.6), (3, 0.4)])
    a = oracle.moe_layer(x, ex, sh.hidden, sh.intermediate, oracle.SCALE_FP16, "gpu")
    b = oracle.moe_layer(x, ex, sh.hidden, sh.intermediate, oracle.SCALE_FP16, "cpu")
    assert rel_l2(a, b) < 2e-3 and np.all(np.isfinite(a))
