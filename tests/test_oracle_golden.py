"""The CPU oracle against every known-answer vector the reference's own tests hold for this path
(tests/integration_test.rs), plus self-consistency of its building blocks.  No GPU."""
import numpy as np
import pytest


def test_int4_lut_matmul_basic(oracle):
    # tests/integration_test.rs:1709-1785: K=4, M=2, scale 1.0 written as BF16 0x3f80
    buf = np.array([0x89, 0x88, 0x98, 0x88, 0x80, 0x3F, 0x80, 0x3F], np.uint8)
    y = oracle.matmul_int4(np.array([1, 2, 3, 4], np.float16), buf, 4, 2, 32, oracle.SCALE_BF16)
    assert abs(float(y[0]) - 1.0) < 0.1 and abs(float(y[1]) - 2.0) < 0.1
    assert y.tolist() == [1.0, 2.0]
    # same numbers with the scale re-encoded as FP16 0x3C00 for the CUDA-side convention
    buf16 = np.array([0x89, 0x88, 0x98, 0x88, 0x00, 0x3C, 0x00, 0x3C], np.uint8)
    assert oracle.matmul_int4(np.array([1, 2, 3, 4], np.float16), buf16, 4, 2, 32, oracle.SCALE_FP16).tolist() == [1.0, 2.0]


def test_int4_lut_matmul_with_scale(oracle):
    # tests/integration_test.rs:1788-1831: K=2, M=1, code 0xAA, scale 0.5 (BF16 0x3f00) -> 10
    buf = np.array([0xAA, 0x00, 0x3F], np.uint8)
    y = oracle.matmul_int4(np.array([3, 7], np.float16), buf, 2, 1, 32, oracle.SCALE_BF16)
    assert abs(float(y[0]) - 10.0) < 0.5 and float(y[0]) == 10.0
    buf16 = np.array([0xAA, 0x00, 0x38], np.uint8)
    assert float(oracle.matmul_int4(np.array([3, 7], np.float16), buf16, 2, 1, 32, oracle.SCALE_FP16)[0]) == 10.0


def test_weighted_accumulate(oracle):
    # tests/integration_test.rs:420-451
    out = np.array([1, 2, 3, 4], np.float16)
    oracle.weighted_accumulate(out, np.array([10, 20, 30, 40], np.float16), 0.5)
    assert abs(float(out[0]) - 6.0) < 0.1 and abs(float(out[1]) - 12.0) < 0.1
    assert out.tolist() == [6.0, 12.0, 18.0, 24.0]
    out32 = np.array([1, 2, 3, 4], np.float32)
    oracle.weighted_accumulate_f32(out32, np.array([10, 20, 30, 40], np.float16), 0.5)
    assert out32.tolist() == [6.0, 12.0, 18.0, 24.0]


def test_run_router_softmax_sums_to_one(oracle):
    # tests/integration_test.rs:454-485: 4 experts, top-2, weights sum to ~1
    H, E = 8, 4
    x = (np.arange(H) * 0.1).astype(np.float16).astype(np.float32)
    W = np.zeros((E, H), np.float16)
    for e in range(E):
        W[e, e * 2] = 1.0
    ids, w, _ = oracle.router(x, W, 2, oracle.MODE_SOFTMAX)
    assert len(ids) == 2 and abs(float(w.sum()) - 1.0) < 0.01
    assert ids.tolist() == [3, 2]  # logits 0, .2, .4, .6


def test_quantize_int4_roundtrip(oracle):
    # tests/integration_test.rs:2300-2374: the same 32x128 gradient matrix and ramp input;
    # quantise -> partial_matmul vs f32 matmul, max relative error per row < 0.5
    rows, cols = 32, 128
    r = np.arange(rows, dtype=np.float32)[:, None]
    c = np.arange(cols, dtype=np.float32)[None, :]
    w = ((r - 16.0) * (c - 64.0)) / np.float32(16.0 * 64.0) * np.float32(0.5)
    x32 = (np.arange(cols, dtype=np.float32) / np.float32(cols)) - np.float32(0.5)
    ref = np.zeros(rows, np.float32)
    for i in range(rows):
        acc = np.float32(0)
        for j in range(cols):
            acc = np.float32(acc + x32[j] * w[i, j])
        ref[i] = acc
    q = oracle.quantize_int4(w.astype(np.float32), 32, oracle.SCALE_BF16)
    assert q.size == rows * cols // 2 + rows * (cols // 32) * 2   # test_quantize_weights_to_int4_basic
    y = oracle.matmul_int4(x32.astype(np.float16), q, cols, rows, 32, oracle.SCALE_BF16).astype(np.float32)
    rel = np.abs(y - ref) / (np.abs(ref) + 1e-6)
    assert float(rel.max()) < 0.5
    # dequantise inverts the page format to within half a quantisation step (+ bf16 scale rounding)
    d = oracle.dequantize_int4(q, rows, cols, 32, oracle.SCALE_BF16)
    step = np.abs(w).reshape(rows, cols // 32, 32).max(axis=2, keepdims=True) / 7
    assert np.all(np.abs(d.reshape(rows, cols // 32, 32) - w.reshape(rows, cols // 32, 32)) <= step * 0.52 + 1e-7)


def test_scale_fallback(oracle):
    # kernels.rs:2791-2795: non-finite or non-positive scale -> 1/8
    buf = np.array([0x99, 0x00, 0x00], np.uint8)  # codes (+1,+1), scale bits 0 -> 0.0 -> fallback
    y = oracle.matmul_int4(np.array([1, 1], np.float16), buf, 2, 1, 32, oracle.SCALE_BF16)
    assert float(y[0]) == 0.25


def test_half_conversions_match_numpy(oracle):
    L = oracle.lib()
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([L.vo_f16_to_f32(int(h)) for h in allh[::7]], np.float32)
    r = ref[::7]
    assert np.all((r.view(np.uint32) == got.view(np.uint32)) | (np.isnan(r) & np.isnan(got)))
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000)).astype(np.float32)
    mids = ((ref[:-1].astype(np.float64) + ref[1:].astype(np.float64)) / 2)[::5].astype(np.float32)
    xs = np.concatenate([xs, mids[np.isfinite(mids)]])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([L.vo_f32_to_f16(float(v)) for v in xs], np.uint16)
    assert np.array_equal(want, got16)
    # bf16 round trip
    import torch
    t = torch.from_numpy(xs[:5000].copy())
    want_bf = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got_bf = np.array([L.vo_f32_to_bf16(float(v)) for v in xs[:5000]], np.uint16)
    assert np.array_equal(want_bf, got_bf)


def test_page_geometry_matches_converter_rule(oracle):
    # convert.rs:1807-1812, :1854-1860 -> the Kimi and Mixtral geometries
    assert oracle.int4_page_geometry(2048, 7168) == (4032, 520, 4)
    assert oracle.int4_page_geometry(7168, 2048) == (1152, 1820, 4)
    assert oracle.int4_page_geometry(14336, 4096) == (2304, 910, 16)
    assert oracle.int4_page_geometry(4096, 14336) == (8064, 260, 16)
    from vic_b200.core_types import KIMI, MIXTRAL
    assert (KIMI.gate_up.rows_per_page, KIMI.down.rows_per_page) == (520, 1820)
    assert (MIXTRAL.gate_up.rows_per_page, MIXTRAL.down.rows_per_page) == (910, 260)
    assert KIMI.expert_bytes == 24772608 and MIXTRAL.expert_bytes == 99090432
    assert KIMI.gate_up.page_rows(3) == (1560, 488) and KIMI.down.page_rows(3) == (5460, 1708)


def test_page_key(oracle):
    # types.rs:259-264
    assert oracle.page_key(1, 2, 3, 4) == (1 << 48) | (2 << 32) | (3 << 16) | 4
    from vic_b200.core_types import PageId
    assert PageId(60, 383, 2, 3).key() == oracle.page_key(60, 383, 2, 3)
    assert PageId.shared(5, 14, 1).key() == oracle.page_key(5, 0xFFFF, 14, 1)


def test_split_pages_then_paged_matmul_equals_whole(oracle):
    rng = np.random.default_rng(3)
    rows, cols = 150, 96
    w = rng.standard_normal((rows, cols)).astype(np.float32) * 0.02
    q = oracle.quantize_int4(w, 32, oracle.SCALE_FP16)
    x = rng.standard_normal(cols).astype(np.float32)
    whole = oracle.matmul_int4_rows_f32(x, q, cols, rows, 32, oracle.SCALE_FP16)
    pages = oracle.split_int4_pages(q, rows, cols, 32, page_size=54 * 40)  # 40 rows per page
    assert [p[2] for p in pages] == [40, 40, 40, 30]
    parts = np.concatenate([oracle.matmul_int4_rows_f32(x, d, cols, rc, 32, oracle.SCALE_FP16) for d, _, rc in pages])
    assert np.array_equal(whole, parts)


def test_router_sigmoid_semantics(oracle):
    # kernels.rs:2388-2436: bias moves selection only; weights from the unbiased sigmoid,
    # normalised then scaled; ties keep the lower index
    H, E = 16, 6
    x = np.ones(H, np.float32)
    W = np.zeros((E, H), np.float32)
    for e, v in enumerate([0.1, 0.3, 0.3, -0.2, 0.05, 0.0]):
        W[e, 0] = v
    ids, w, logits = oracle.router(x, W, 3, oracle.MODE_SIGMOID, 2.5, True)
    assert ids.tolist() == [1, 2, 0]
    assert abs(float(w.sum()) - 2.5) < 1e-5
    bias = np.array([0, 0, 0, 10, 0, 0], np.float32)
    ids_b, w_b, _ = oracle.router(x, W, 3, oracle.MODE_SIGMOID, 2.5, True, bias)
    assert ids_b.tolist() == [3, 1, 2]
    sig = 1 / (1 + np.exp(-logits.astype(np.float64)))
    want = sig[[3, 1, 2]] / sig[[3, 1, 2]].sum() * 2.5
    assert np.allclose(w_b, want, rtol=1e-6)
    ids_n, w_n, _ = oracle.router(x, W, 2, oracle.MODE_SIGMOID, 1.0, False)
    assert np.allclose(w_n, sig[[1, 2]], rtol=1e-6)


def test_router_orders_agree_to_rounding(oracle):
    rng = np.random.default_rng(5)
    H, E = 7168, 384
    W = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    worst = 0.0
    for t in range(24):
        x = (rng.standard_normal(H) * rng.uniform(0.3, 3.0)).astype(np.float32)
        if t % 2:
            x = (x.view(np.uint32) & 0xFFFF0000).view(np.float32)   # bf16-representable token
        a = oracle.router_logits(x, W, oracle.ORDER_SEQUENTIAL)
        b = oracle.router_logits(x, W, oracle.ORDER_GPU128)
        if t == 0:
            exact = W.astype(np.float64) @ x.astype(np.float64)
            tol = 2e-6 * np.abs(W * x).sum(axis=1).max()
            assert np.max(np.abs(a - exact)) < tol and np.max(np.abs(b - exact)) < tol
        # the bound the GPU router uses to detect near-ties must dominate the real difference
        absum = np.abs(W * x).sum(axis=1)
        eps = 8 * 2.0 ** -24 * (np.sqrt(H) * np.abs(b) + absum)
        worst = max(worst, float(np.max(np.abs(a - b) / eps)))
    assert worst < 0.25, worst   # 9,216 expert-token samples: a 4x margin
