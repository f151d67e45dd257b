"""The grouped multi-token layer (every distinct expert read once, tensor-core tiles) against the batch-1 path
token by token and against the per-token CPU oracle: 1/8/32/128 tokens, expert load skewed by a per-expert
Zipf(s = 1.1) logit offset so that some experts receive no token and a few receive most."""
import numpy as np
import pytest
import torch

from tests.parity import assert_close, oracle_experts

pytestmark = pytest.mark.gpu

_cache = {}


def _model(name, dev):
    from vic_b200.core_types import KIMI, SCORING_SIGMOID, MoeShape
    from vic_b200.synth import build_synthetic_moe
    if name not in _cache:
        _cache.clear()
        torch.cuda.empty_cache()
        shapes = {"kimi": KIMI,
                  # ragged last pages in both projections, 12 experts, no expert dimension equal to the hidden one
                  "mid": MoeShape("grp-mid", 1024, 2304, 12, 3, 1, SCORING_SIGMOID, 2.5, True),
                  "noshared": MoeShape("grp-noshared", 512, 1024, 8, 2, 0, SCORING_SIGMOID, 1.0, True)}
        _cache[name] = build_synthetic_moe(shapes[name], 1, dev, seed=1234 + 3, slot_seed=17)
    return _cache[name]


@pytest.mark.parametrize("name,T,xdt,checked", [
    ("mid", 5, torch.bfloat16, 5), ("mid", 37, torch.float16, 4), ("noshared", 9, torch.float32, 3),
    ("kimi", 1, torch.bfloat16, 1), ("kimi", 8, torch.bfloat16, 3), ("kimi", 32, torch.bfloat16, 3), ("kimi", 128, torch.bfloat16, 4)])
def test_grouped_equals_per_token_path_and_oracle(cuda_dev, oracle, name, T, xdt, checked):
    from vic_b200.grouped import GroupedDecoder, zipf_logit_offset
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model(name, cuda_dev)
    sh = model.shape
    gd = GroupedDecoder(model, max_tokens=max(T, 16))
    dec = MoeDecoder(model)
    off = zipf_logit_offset(sh.num_experts, 7)
    off_d = torch.from_numpy(off).to(cuda_dev)
    g = torch.Generator(device=cuda_dev).manual_seed(1234 + T)
    xs = synth_activation(sh, g, cuda_dev, xdt, T)
    out = gd.forward(0, xs, logit_offset=off_d).clone()
    torch.cuda.synchronize()
    assert int(gd.status.item()) == 0
    ids = gd.ids[:T, :sh.top_k].cpu().numpy().view(np.uint16)
    ws = gd.weights[:T, :sh.top_k].cpu().numpy()
    out_n = out.cpu().numpy()
    assert np.all(np.isfinite(out_n))
    # the batched router routes every token exactly as the batch-1 router does
    want = torch.zeros_like(out)
    for t in range(T):
        dec.forward_layer(0, xs[t], out=want[t], logit_offset=off_d)
        torch.cuda.synchronize()
        i1, w1 = dec.routing()
        assert np.array_equal(ids[t], i1), (t, ids[t], i1)
        assert np.array_equal(ws[t], w1)
    assert int(dec.status.item()) == 0
    want_n = want.cpu().numpy()
    for t in range(T):
        assert_close(out_n[t], want_n[t], f"{name} T={T} token {t} vs batch-1 path")
    distinct = len(set(ids.reshape(-1).tolist())) + sh.shared_experts
    assert int(gd.n_distinct.item()) == distinct
    if name == "kimi" and T == 128:
        counts = np.bincount(ids.reshape(-1), minlength=sh.num_experts)
        assert (counts == 0).sum() > 50 and counts.max() > 64     # idle experts, and one that needs two passes
    xs_n = xs.float().cpu().numpy()
    for t in np.linspace(0, T - 1, checked).astype(int):
        exp = oracle.moe_layer(xs_n[t], oracle_experts(oracle, model, 0, list(zip(ids[t].tolist(), ws[t].tolist()))), sh.hidden,
                               sh.intermediate, oracle.SCALE_FP16, "gpu")
        assert_close(out_n[t], exp, f"{name} T={T} token {t} vs oracle")


def test_grouped_accumulates_and_refuses_bad_arguments(cuda_dev):
    from vic_b200.grouped import GroupedDecoder
    from vic_b200.lib import lib
    from vic_b200.synth import synth_activation
    model = _model("mid", cuda_dev)
    sh = model.shape
    gd = GroupedDecoder(model, max_tokens=16)
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, 6)
    base = gd.forward(0, xs).clone()
    resid = torch.randn(6, sh.hidden, device=cuda_dev)
    want = resid + base
    gd.route(0, xs)
    gd.experts(0, xs, out=resid, accumulate=True)
    torch.cuda.synchronize()
    assert torch.allclose(resid, want, rtol=0, atol=1e-5)
    # more tokens than the handle was built for, a null output: refused before any launch
    p = xs.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    E = sh.num_experts
    assert lib().vib3_launch_moe_grouped_int4(gd._h, p, 2, 2 * sh.hidden, 17, p, 32, p, 64, p, None, 1.0, 4, 0, E, p, sh.hidden, 0, None, st) == -2
    assert lib().vib3_launch_moe_grouped_int4(gd._h, p, 2, 2 * sh.hidden, 4, p, 32, p, 64, p, None, 1.0, 4, 0, E, None, sh.hidden, 0, None, st) == -3
    assert lib().vib3_launch_moe_grouped_int4(gd._h, p, 2, 2 * sh.hidden, 4, p, 32, p, 64, p, None, 1.0, 4, 3, E + 1, p, sh.hidden, 0, None, st) == -2
    # expert ranges: the outputs of disjoint ranges (the shared expert in one of them) add up to the whole
    whole = gd.forward(0, xs).clone()
    part = torch.zeros_like(whole)
    gd.experts(0, xs, out=part, expert_range=(0, 5), shared=True)
    gd.experts(0, xs, out=part, accumulate=True, expert_range=(5, E), shared=False)
    torch.cuda.synchronize()
    assert int(gd.status.item()) == 0
    assert torch.allclose(part, whole, rtol=0, atol=2e-5)
    assert lib().vib3_moe_grouped_workspace_bytes(0, 8, 384, 7168, 2048, 520, 1820) == 0
