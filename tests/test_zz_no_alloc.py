"""vib3_launch_moe_layer_int4_paged_noalloc — the fused MoE sublayer for callers that may not
allocate device memory (a host whose page pool owns all free VRAM, a serving loop that bans
cudaMalloc after warm-up, a binding without an allocator).  The intermediate sits in an array inside
the library instead of a caller buffer, so its results must equal those of the entry point that takes
a scratch buffer, call after call.  Runs last (file name) so that a failure here cannot hide others."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(dec, layer, x, out):
    from vic_b200.core_types import INT4_GROUP_SIZE
    from vic_b200.kernels import x_dtype_code
    from vic_b200.lib import lib
    sh = dec.model.shape
    return lib().vib3_launch_moe_layer_int4_paged_noalloc(
        x.data_ptr(), x_dtype_code(x), dec.tables[layer], sh.num_experts, dec.shared_tables[layer] or None,
        dec.ids.data_ptr(), dec.weights.data_ptr(), sh.top_k, 1.0, out.data_ptr(), 0, sh.hidden, sh.intermediate,
        sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page, INT4_GROUP_SIZE,
        dec.status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_noalloc_entry_point_matches_scratch_entry_point_twice_in_a_row(cuda_dev):
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    # multiples of 256 so that the bulk-copy staged kernels run; 4 * 2048 values of intermediate
    sh = MoeShape("noalloc", 1024, 2048, 6, 3, 1, SCORING_SIGMOID, 2.5, True)
    model = build_synthetic_moe(sh, 1, cuda_dev, seed=21, slot_seed=5)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, 2)
    out_a = torch.zeros(sh.hidden, dtype=torch.float32, device=cuda_dev)
    out_b = torch.full((sh.hidden,), 7.0, dtype=torch.float32, device=cuda_dev)
    for t in range(2):                      # two calls in a row: the array keeps the last call's contents
        dec.route(0, xs[t])
        dec.experts(0, xs[t], out=out_a)    # existing entry point, caller-owned scratch
        rc = _call_noalloc(dec, 0, xs[t], out_b)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        assert torch.isfinite(out_b).all()
        # same kernels, same arithmetic: the tolerance of the layer tests (max-abs 2e-2, rel-L2 1e-3)
        # is met with room to spare — the outputs are in fact identical
        a, b = out_a.cpu().numpy(), out_b.cpu().numpy()
        assert np.max(np.abs(a - b)) <= 2e-2 and np.linalg.norm(a - b) <= 1e-3 * np.linalg.norm(a)
        assert torch.equal(out_a, out_b)
    assert not torch.equal(out_a, torch.zeros_like(out_a))


def test_noalloc_rejects_oversized_request_without_launching(cuda_dev):
    from vic_b200.lib import lib
    t = torch.zeros(4096, dtype=torch.float32, device=cuda_dev)
    p = t.data_ptr()
    # 17 slots * 32768 > 278,528 values
    rc = lib().vib3_launch_moe_layer_int4_paged_noalloc(p, 2, p, 8, p, p, p, 16, 1.0, p, 0, 256, 32768, 1, 32768, 256, 32, None, None)
    assert rc == -8
    rc = lib().vib3_launch_moe_layer_int4_paged_noalloc(p, 2, p, 8, None, p, p, -1, 1.0, p, 0, 256, 512, 1, 512, 256, 32, None, None)
    assert rc == -2      # the code vib3_launch_moe_layer_int4_paged gives for a negative count
    # the limit itself: 17 slots of 16384 values are exactly the array (accepted as far as the capacity check
    # goes: the call is then refused for its null output, -3, before anything is launched); one value more is not
    rc = lib().vib3_launch_moe_layer_int4_paged_noalloc(p, 2, p, 8, p, p, p, 16, 1.0, None, 0, 256, 16384, 1, 16384, 256, 32, None, None)
    assert rc == -3
    rc = lib().vib3_launch_moe_layer_int4_paged_noalloc(p, 2, p, 8, None, p, p, 1, 1.0, p, 0, 256, 278529, 1, 278529, 256, 32, None, None)
    assert rc == -8
    torch.cuda.synchronize()


def test_noalloc_without_shared_expert(cuda_dev):
    """No shared expert: the slots are the routed experts alone (a different layout of the built-in array)."""
    from vic_b200.core_types import SCORING_SOFTMAX, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    sh = MoeShape("noalloc-noshared", 512, 1024, 8, 2, 0, SCORING_SOFTMAX, 1.0, True)
    model = build_synthetic_moe(sh, 1, cuda_dev, seed=22, slot_seed=6)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(4)
    xs = synth_activation(sh, g, cuda_dev, torch.float16, 2)
    out_a = torch.zeros(sh.hidden, dtype=torch.float32, device=cuda_dev)
    out_b = torch.full((sh.hidden,), -3.0, dtype=torch.float32, device=cuda_dev)
    for t in range(2):
        dec.route(0, xs[t])
        dec.experts(0, xs[t], out=out_a)
        assert _call_noalloc(dec, 0, xs[t], out_b) == 0
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        a, b = out_a.cpu().numpy(), out_b.cpu().numpy()
        assert np.max(np.abs(a - b)) <= 2e-2 and np.linalg.norm(a - b) <= 1e-3 * np.linalg.norm(a)
        assert torch.equal(out_a, out_b)
