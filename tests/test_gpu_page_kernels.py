"""Per-page entry points (the reference's launcher signatures) against the CPU oracle and, where
built, against the reference's own CUDA kernels.  All calls go through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

from tests.parity import assert_close, load_ref_lib, rel_l2

pytestmark = pytest.mark.gpu


def _page(rng, K, M, group=32):
    """Random page image: codes uniform, scales |N(0,.02)|/7 exact in fp16 and bf16."""
    packed_k = (K + 1) // 2
    groups = (K + group - 1) // group
    codes = rng.integers(0, 256, size=M * packed_k, dtype=np.uint8)
    s = np.maximum(np.abs(rng.standard_normal(M * groups)) * 0.02 / 7, 2.0 ** -13).astype(np.float32)
    s = torch.from_numpy(s).to(torch.bfloat16).to(torch.float16).numpy()
    return np.concatenate([codes, s.view(np.uint8)])


def _dev(a, cuda_dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev)


def test_known_answers_through_the_abi(cuda_dev, oracle):
    from vic_b200 import kernels
    # tests/integration_test.rs:1709-1785 with the scale re-encoded as fp16 1.0
    buf = _dev(np.array([0x89, 0x88, 0x98, 0x88, 0x00, 0x3C, 0x00, 0x3C], np.uint8), cuda_dev)
    x = torch.tensor([1, 2, 3, 4], dtype=torch.float16, device=cuda_dev)
    y = torch.zeros(2, dtype=torch.float16, device=cuda_dev)
    kernels.partial_matmul(x, buf, y, 4, 2)
    assert y.cpu().tolist() == [1.0, 2.0]
    y.zero_()
    kernels.partial_matmul_f32(x.float(), buf, y, 4, 2)
    assert y.cpu().tolist() == [1.0, 2.0]
    # tests/integration_test.rs:1788-1831, scale 0.5
    buf = _dev(np.array([0xAA, 0x00, 0x38], np.uint8), cuda_dev)  # scales at an odd address
    x = torch.tensor([3, 7], dtype=torch.float16, device=cuda_dev)
    y = torch.zeros(1, dtype=torch.float16, device=cuda_dev)
    kernels.partial_matmul(x, buf, y, 2, 1)
    assert y.cpu().tolist() == [10.0]
    # tests/integration_test.rs:420-451
    out = torch.tensor([1, 2, 3, 4], dtype=torch.float16, device=cuda_dev)
    kernels.weighted_accumulate(out, torch.tensor([10, 20, 30, 40], dtype=torch.float16, device=cuda_dev), 0.5, 4)
    assert out.cpu().tolist() == [6.0, 12.0, 18.0, 24.0]


SHAPES = [(32, 1), (64, 3), (96, 5), (1024, 37), (7168, 520), (7168, 488), (2048, 1820), (2048, 1708), (4096, 910),
          (14336, 196)]


@pytest.mark.parametrize("K,M", SHAPES)
def test_partial_matmul_vs_oracle(cuda_dev, oracle, K, M):
    from vic_b200 import kernels
    rng = np.random.default_rng(K * 131 + M)
    page = _page(rng, K, M)
    x16 = rng.standard_normal(K).astype(np.float16)
    want = oracle.matmul_int4_rows_f32(x16.astype(np.float32), page, K, M, 32, oracle.SCALE_FP16)
    dpage, y = _dev(page, cuda_dev), torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    kernels.partial_matmul(_dev(x16, cuda_dev), dpage, y, K, M)
    got = y.cpu().numpy().astype(np.float32)
    # fp16 outputs: with a handful of rows a single 1-ulp difference (2^-11) dominates the norm
    tol = 4e-4 if M >= 32 else 1e-3
    assert_close(got, want, f"partial_matmul K={K} M={M}", rel_l2_tol=tol)
    # fp32 input entry point
    x32 = rng.standard_normal(K).astype(np.float32)
    want32 = oracle.matmul_int4_rows_f32(x32, page, K, M, 32, oracle.SCALE_FP16)
    kernels.partial_matmul_f32(_dev(x32, cuda_dev), dpage, y, K, M)
    assert_close(y.cpu().numpy().astype(np.float32), want32, f"partial_matmul_f32 K={K} M={M}", rel_l2_tol=tol)
    # f64 truth: the GPU result must not be further from it than fp16 output rounding explains
    w = oracle.dequantize_int4(page, M, K, 32, oracle.SCALE_FP16).astype(np.float64)
    truth = w @ x32.astype(np.float64)
    assert rel_l2(y.cpu().numpy().astype(np.float64), truth) < tol


@pytest.mark.parametrize("K,M", [(32, 2), (96, 7), (7168, 520), (7168, 488), (4096, 686)])
def test_swiglu_vs_oracle(cuda_dev, oracle, K, M):
    from vic_b200 import kernels
    rng = np.random.default_rng(K * 7 + M)
    up, gate = _page(rng, K, M), _page(rng, K, M)
    x32 = rng.standard_normal(K).astype(np.float32)
    dx, dup, dgate = _dev(x32, cuda_dev), _dev(up, cuda_dev), _dev(gate, cuda_dev)
    y = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    # fused: one rounding, the CPU kernel's semantics (kernels.rs:3040-3042)
    kernels.partial_swiglu_f32(dx, dup, dgate, y, K, M)
    want = oracle.swiglu_int4_f32in(x32, up, gate, K, M, 32, oracle.SCALE_FP16).astype(np.float32)
    assert_close(y.cpu().numpy().astype(np.float32), want, "fused swiglu", rel_l2_tol=5e-4)
    # decomposed with temps: the reference GPU path's rounding points (kernels.rs:493-541)
    t1 = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    t2 = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    kernels.partial_swiglu_f32(dx, dup, dgate, y, K, M, swiglu_temps=(t1, t2))
    u = oracle.matmul_int4_rows_f32(x32, up, K, M, 32, oracle.SCALE_FP16).astype(np.float16)
    g = oracle.matmul_int4_rows_f32(x32, gate, K, M, 32, oracle.SCALE_FP16).astype(np.float16)
    assert_close(y.cpu().numpy().astype(np.float32), oracle.silu_mul(g, u).astype(np.float32), "decomposed swiglu",
                 rel_l2_tol=1e-3)


@pytest.mark.parametrize("K,M,group", [(2, 1, 32), (4, 2, 128), (33, 3, 32), (130, 9, 128), (70, 4, 16)])
def test_general_path_odd_shapes(cuda_dev, oracle, K, M, group):
    from vic_b200.lib import lib
    rng = np.random.default_rng(K + M)
    page = _page(rng, K, M, group)
    x16 = rng.standard_normal(K).astype(np.float16)
    want = oracle.matmul_int4_rows_f32(x16.astype(np.float32), page, K, M, group, oracle.SCALE_FP16)
    dpage, dx = _dev(page, cuda_dev), _dev(x16, cuda_dev)
    y = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    scales = dpage.data_ptr() + ((K + 1) // 2) * M
    rc = lib().vib3_launch_partial_matmul_int4(dx.data_ptr(), dpage.data_ptr(), scales, y.data_ptr(), K, M, group, None)
    assert rc == 0
    assert_close(y.cpu().numpy().astype(np.float32), want, "general path", rel_l2_tol=1e-3)


def test_elementwise_entry_points(cuda_dev, oracle):
    from vic_b200 import kernels
    rng = np.random.default_rng(11)
    n = 7168
    a = rng.standard_normal(n).astype(np.float16)
    b = rng.standard_normal(n).astype(np.float16)
    y = torch.zeros(n, dtype=torch.float16, device=cuda_dev)
    kernels.silu_mul(_dev(a, cuda_dev), _dev(b, cuda_dev), y, n)
    got, want = y.cpu().numpy(), oracle.silu_mul(a, b)
    ulp_off = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
    assert ulp_off.max() <= 1 and (ulp_off > 0).mean() < 0.01
    out32 = rng.standard_normal(n).astype(np.float32)
    d = _dev(out32, cuda_dev)
    kernels.weighted_accumulate_f32(d, _dev(a, cuda_dev), 0.37, n)
    want32 = out32.copy()
    oracle.weighted_accumulate_f32(want32, a, 0.37)
    assert np.allclose(d.cpu().numpy(), want32, rtol=0, atol=2e-7 * 4)
    y32 = rng.standard_normal(n).astype(np.float32)
    kernels.weighted_accumulate_f32_f32(d, _dev(y32, cuda_dev), -1.5, n)
    oracle.weighted_accumulate_f32_f32(want32, y32, -1.5)
    assert np.allclose(d.cpu().numpy(), want32, rtol=0, atol=1e-6)
    kernels.residual_add_f32_f32(d, _dev(y32, cuda_dev), n)
    oracle.residual_add_f32_f32(want32, y32)
    assert np.allclose(d.cpu().numpy(), want32, rtol=0, atol=1e-6)


def test_refusals_do_not_launch(cuda_dev):
    from vic_b200.lib import lib
    L = lib()
    t = torch.zeros(64, dtype=torch.float16, device=cuda_dev)
    p = t.data_ptr()
    assert L.vib3_launch_partial_matmul_int4(None, p, p, p, 32, 1, 32, None) == -3
    assert L.vib3_launch_partial_matmul_int4(p, p, p, None, 32, 1, 32, None) == -3
    assert L.vib3_launch_partial_matmul_int4(p, p, p, p, 0, 1, 32, None) == -5
    assert L.vib3_launch_partial_matmul_int4(p, p, p, p, 32, -1, 32, None) == -5
    assert L.vib3_launch_partial_matmul_int4(p, p, p, p, 32, 0, 32, None) == 0      # empty slice: nothing to do
    assert L.vib3_launch_partial_matmul_int4(p, p, p, p + 1, 32, 1, 32, None) == -4
    assert L.vib3_launch_silu_mul(None, p, p, 4, None) == -3
    assert L.vib3_launch_weighted_accumulate_f32(p, p, 1.0, -1, None) == -5
    assert L.vib3_launch_weighted_accumulate_f32(p, p, 1.0, 0, None) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("K,M", [(7168, 520), (2048, 1708), (4096, 910)])
def test_against_reference_cuda_kernels(cuda_dev, K, M):
    """Same page, same input, the reference's unmodified kernels on the same GPU."""
    ref = load_ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libvib3_ref.so not built")
    from vic_b200 import kernels
    rng = np.random.default_rng(K + 3 * M)
    page = _page(rng, K, M)
    x32 = rng.standard_normal(K).astype(np.float32)
    dpage, dx = _dev(page, cuda_dev), _dev(x32, cuda_dev)
    ours = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    theirs = torch.zeros(M, dtype=torch.float16, device=cuda_dev)
    kernels.partial_matmul_f32(dx, dpage, ours, K, M)
    st = torch.cuda.current_stream().cuda_stream
    assert ref.vib3_launch_partial_matmul_int4_f32(dx.data_ptr(), dpage.data_ptr(), dpage.data_ptr() + (K // 2) * M,
                                                   theirs.data_ptr(), K, M, 32, st) == 0
    torch.cuda.synchronize()
    a, b = ours.cpu().numpy(), theirs.cpu().numpy()
    assert_close(a.astype(np.float32), b.astype(np.float32), "vs reference kernel", rel_l2_tol=4e-4)
    ulp = np.abs(a.view(np.int16).astype(np.int32) - b.view(np.int16).astype(np.int32))
    assert ulp.max() <= 2
    x16 = x32.astype(np.float16)
    dx16 = _dev(x16, cuda_dev)
    kernels.partial_matmul(dx16, dpage, ours, K, M)
    assert ref.vib3_launch_partial_matmul_int4(dx16.data_ptr(), dpage.data_ptr(), dpage.data_ptr() + (K // 2) * M,
                                               theirs.data_ptr(), K, M, 32, st) == 0
    torch.cuda.synchronize()
    assert_close(ours.cpu().numpy().astype(np.float32), theirs.cpu().numpy().astype(np.float32), "vs reference kernel f16",
                 rel_l2_tol=4e-4)


@pytest.mark.parametrize("H,T", [(7168, 3), (4096, 1), (200, 2)])
def test_rms_norm_entry_points(cuda_dev, oracle, H, T):
    """vib3_launch_rms_norm_f32 (reference signature) and the fused residual-add + norm launch against the CPU
    restatement of rms_norm (sequential sum of squares there, a tree here: a few ulps) and, where it is built,
    the reference's own kernel."""
    from vic_b200 import kernels
    from tests.parity import load_ref_lib
    g = torch.Generator(device="cpu").manual_seed(H + T)
    h = torch.randn(T, H, generator=g) * 2.0
    delta = (torch.randn(T, H, generator=g) * 0.3).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.float16)
    eps = 1e-6
    hd, dd, wd = h.to(cuda_dev), delta.to(cuda_dev), w.to(cuda_dev)
    out = torch.zeros(H, dtype=torch.float32, device=cuda_dev)
    kernels.rms_norm_f32(hd[0], out, wd, H, eps)
    want = oracle.rms_norm_f32(h[0].numpy(), w.float().numpy(), eps)
    assert np.allclose(out.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    ref = load_ref_lib()
    if ref is not None and hasattr(ref, "vib3_launch_rms_norm_f32"):
        import ctypes
        fn = ref.vib3_launch_rms_norm_f32
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
        theirs = torch.zeros(H, dtype=torch.float32, device=cuda_dev)
        assert fn(hd[0].data_ptr(), theirs.data_ptr(), wd.data_ptr(), H, eps, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert np.allclose(out.cpu().numpy(), theirs.cpu().numpy(), rtol=2e-6, atol=1e-7)   # its build uses approximate sqrt / reciprocal
    # fused: hidden += delta; x = bf16(norm(hidden) * w), all T rows in one launch
    hid = hd.clone()
    x = torch.zeros(T, H, dtype=torch.bfloat16, device=cuda_dev)
    kernels.residual_rms_norm(hid, dd, wd, eps, x)
    torch.cuda.synchronize()
    h2 = (h + delta.float())
    assert torch.equal(hid.cpu(), h2)
    for t in range(T):
        want = oracle.rms_norm_f32(h2[t].numpy(), w.float().numpy(), eps)
        got = x[t].float().cpu().numpy()
        assert np.allclose(got, torch.from_numpy(want).to(torch.bfloat16).float().numpy(), rtol=1e-2, atol=1e-6)
        assert np.mean(got == torch.from_numpy(want).to(torch.bfloat16).float().numpy()) > 0.99
    # no delta, no weight, fp32 out
    x32 = torch.zeros(T, H, dtype=torch.float32, device=cuda_dev)
    kernels.residual_rms_norm(hid, None, None, eps, x32)
    want = oracle.rms_norm_f32(h2[0].numpy(), None, eps)
    assert np.allclose(x32[0].cpu().numpy(), want, rtol=1e-6, atol=1e-7)


def test_rms_norm_centering_and_second_delta(cuda_dev, oracle):
    from vic_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(12)
    T, H = 4, 1024
    h = torch.randn(T, H, generator=g) + 3.0
    d1 = (torch.randn(T, H, generator=g) * 0.2).to(torch.float16)
    d2 = torch.randn(T, H, generator=g) * 0.1
    hid = h.to(cuda_dev)
    x = torch.zeros(T, H, dtype=torch.float32, device=cuda_dev)
    kernels.residual_rms_norm(hid, d1.to(cuda_dev), None, 1e-6, x, delta2=d2.to(cuda_dev), center=True)
    torch.cuda.synchronize()
    h2 = h + d1.float() + d2
    assert torch.allclose(hid.cpu(), h2, rtol=0, atol=1e-6)
    for t in range(T):
        c = (h2[t] - h2[t].mean()).numpy()
        want = oracle.rms_norm_f32(c, None, 1e-6)
        assert np.allclose(x[t].cpu().numpy(), want, rtol=1e-5, atol=1e-6)
        assert abs(float(x[t].mean())) < 1e-5
