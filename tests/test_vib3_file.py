"""The `.vib3` container code on the host: product-side quantiser against the oracle's restatement of
quantize_weights_to_int4, the page split against the oracle's add_pages_from_data, the file layout (header, catalog
order, alignment) as the reference's reader expects it, and a round trip writer -> file -> reader -> page pool."""
import os
import struct

import numpy as np
import pytest
import torch


def _shape():
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    # gate/up 4000 x 1024: 3640 + 360 rows; down 1024 x 4000: 932 + 92 rows — ragged last pages in both
    return MoeShape("file-mid", 1024, 4000, 3, 2, 1, SCORING_SIGMOID, 2.0, True)


@pytest.mark.parametrize("rows,cols", [(5, 64), (7, 100), (3, 33), (64, 1024)])
@pytest.mark.parametrize("fmt", [0, 1])
def test_quantiser_equals_the_oracle(oracle, rows, cols, fmt):
    from vic_b200.vib3_file import quantize_int4
    rng = np.random.default_rng(rows * 1000 + cols)
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    w[0, :min(32, cols)] = 0.0                      # an all-zero group: scale 1
    w[1, 0] = 0.35                                  # exact halves: round half away from zero
    got = quantize_int4(w, fmt)
    want = oracle.quantize_int4(w, 32, oracle.SCALE_BF16 if fmt == 0 else oracle.SCALE_FP16)
    assert np.array_equal(got, want)
    # and back: dequantised weights are within half a step of the originals
    back = oracle.dequantize_int4(got, rows, cols, 32, oracle.SCALE_BF16 if fmt == 0 else oracle.SCALE_FP16)
    assert np.max(np.abs(back - w)) <= np.abs(w).max() / 7 * 0.51 + 1e-6


def test_writer_reader_round_trip_and_layout(tmp_path, oracle):
    from vic_b200.buffer_manager import PageBufferManager, QueryPlanner
    from vic_b200.core_types import EXPERT_SHARED, PAGE_SIZE, PageId
    from vic_b200.lib import Vib3Error
    from vic_b200.vib3_file import Vib3File, Vib3Writer, quantize_int4
    sh = _shape()
    rng = np.random.default_rng(5)
    path = str(tmp_path / "model.vib3")
    w = Vib3Writer(path, sh, 2, '{"name": "file-mid"}')
    mats = {}
    n_pages = 0
    for layer in (1, 0):                       # out of order on purpose: the catalog is sorted at finalize
        for e in (2, EXPERT_SHARED, 0, 1):
            up = (rng.standard_normal((sh.intermediate, sh.hidden)) * 0.02).astype(np.float32)
            gate = (rng.standard_normal((sh.intermediate, sh.hidden)) * 0.02).astype(np.float32)
            down = (rng.standard_normal((sh.hidden, sh.intermediate)) * 0.02).astype(np.float32)
            mats[(layer, e)] = (up, gate, down)
            n_pages += w.add_expert(layer, e, up, gate, down)
    w.finalize()
    assert n_pages == 2 * 4 * sh.pages_per_expert

    raw = open(path, "rb").read()
    magic, version = struct.unpack_from("<QI", raw, 0)
    assert magic == 0x3342495600000001 and version == 1           # format.rs:39-40
    f = Vib3File(path)
    s = f.summary()
    assert (s["num_layers"], s["num_experts"], s["num_active_experts"], s["hidden_dim"], s["expert_hidden_dim"], s["expert_dtype"]) == \
        (2, sh.num_experts, sh.top_k, sh.hidden, sh.intermediate, 5)
    assert s["page_data_offset"] % PAGE_SIZE == 0
    pages = f.pages()
    assert len(pages) == n_pages
    keys = [(p.layer, p.expert, p.segment, p.page_idx) for p in pages]
    assert keys == sorted(keys)                                    # catalog order (format.rs:881-892)
    assert all(p.file_offset % 4096 == 0 and p.compression == 0 for p in pages)
    # page contents: the oracle's page split of the oracle's quantisation of the same matrix
    for idx, p in enumerate(pages):
        segs = {0: 0, 1: 1, 2: 2, 14: 0, 15: 1, 16: 2}
        m = mats[(p.layer, p.expert)][segs[p.segment]]
        want_pages = oracle.split_int4_pages(oracle.quantize_int4(m, 32, oracle.SCALE_FP16), m.shape[0], m.shape[1])
        data, r0, rc = want_pages[p.page_idx]
        assert (p.row_start, p.row_count, p.col_count, p.raw_size) == (r0, rc, m.shape[1], data.size)
        if idx % 5 == 0:
            assert np.array_equal(f.read_page(idx, p.raw_size), data)

    # into a (host-memory) pool: layer 1 only, experts 0..1 and the shared expert
    cap = 3 * sh.pages_per_expert
    pool = PageBufferManager(cap, storage=torch.empty(cap * PAGE_SIZE + 256, dtype=torch.uint8))
    assert f.load_into_pool(pool, layers=(1, 2), experts=(0, 2)) == cap
    pool.freeze()
    assert pool.resident_pages() == cap
    assert pool.get_page_resident(PageId(1, 2, 0, 0)) is None and pool.get_page_resident(PageId(0, 0, 0, 0)) is None
    plan = QueryPlanner(pool, sh.pages_per_segment).plan_layer(1, [(1, 0.5), (EXPERT_SHARED, 1.0)])
    assert [len(ep.pages) for ep in plan.experts] == [sh.pages_per_expert] * 2
    h = pool.get_page_resident(PageId(1, 1, 2, 1))
    m = mats[(1, 1)][2]
    want = oracle.split_int4_pages(oracle.quantize_int4(m, 32, oracle.SCALE_FP16), m.shape[0], m.shape[1])[1][0]
    assert np.array_equal(pool.page_bytes_host(h), want)
    f.close()

    # a damaged file is refused with the reader's checks (format.rs:249-268)
    bad = str(tmp_path / "bad.vib3")
    open(bad, "wb").write(b"\0" * 100)
    with pytest.raises(Vib3Error):
        Vib3File(bad)
    open(bad, "wb").write(b"\1" + raw[1:4096])
    with pytest.raises(Vib3Error):
        Vib3File(bad)
    open(bad, "wb").write(raw[:len(raw) // 2])          # pages beyond the end of the file
    with pytest.raises(Vib3Error):
        Vib3File(bad)
