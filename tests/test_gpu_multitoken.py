"""Multi-token decode (BASELINE config 3: 1/8/32/128 tokens, expert load skewed by a per-expert
Zipf(s = 1.1) logit offset so that some experts receive no token).  The reference has no grouped
kernel: its prefill runs token by token through the batch-1 path, which is the oracle here."""
import numpy as np
import pytest
import torch

from tests.parity import assert_close, oracle_experts

pytestmark = pytest.mark.gpu

_model_cache = {}


def _kimi(dev):
    from vic_b200.core_types import KIMI
    from vic_b200.synth import build_synthetic_moe
    if "m" not in _model_cache:
        _model_cache["m"] = build_synthetic_moe(KIMI, 1, dev, seed=1234 + 3, slot_seed=17)
    return _model_cache["m"]


def zipf_offset(num_experts, seed, s=1.1):
    rank = np.random.default_rng(seed).permutation(num_experts) + 1
    return (-s * np.log(rank)).astype(np.float32)


@pytest.mark.parametrize("T,checked", [(1, 1), (8, 8), (32, 6), (128, 6)])
def test_multi_token_vs_per_token_oracle(cuda_dev, oracle, T, checked):
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _kimi(cuda_dev)
    sh = model.shape
    dec = MoeDecoder(model)
    off = zipf_offset(sh.num_experts, 7)
    off_d = torch.from_numpy(off).to(cuda_dev)
    g = torch.Generator(device=cuda_dev).manual_seed(1234 + T)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, T)
    ids_d = torch.zeros(T, 16, dtype=torch.int16, device=cuda_dev)
    ws_d = torch.zeros(T, 16, dtype=torch.float32, device=cuda_dev)
    outs = dec.forward_tokens(0, xs, logit_offset=off_d, routing_out=(ids_d, ws_d))
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    outs_n = outs.cpu().numpy()
    assert np.all(np.isfinite(outs_n))
    ids_n = ids_d[:, :sh.top_k].cpu().numpy().view(np.uint16)
    ws_n = ws_d[:, :sh.top_k].cpu().numpy()
    W = model.router_w[0].cpu().numpy()
    xs_n = xs.float().cpu().numpy()
    # routing of every token: indices bit-exact against the CPU router with the same logit offset
    for t in range(T):
        oi, ow, _ = oracle.router(xs_n[t], W, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, None,
                                  oracle.ORDER_SEQUENTIAL, logit_offset=off)
        assert np.array_equal(ids_n[t], oi), (t, ids_n[t], oi)
        assert np.allclose(ws_n[t], ow, rtol=1e-4)
    # the skew concentrates the load: at 128 tokens some experts get none, a few get many
    if T == 128:
        counts = np.bincount(ids_n.reshape(-1), minlength=sh.num_experts)
        assert (counts == 0).sum() > 50 and counts.max() >= 16
    # layer outputs of a sample of tokens against the per-token oracle chain
    for t in np.linspace(0, T - 1, checked).astype(int):
        want = oracle.moe_layer(xs_n[t], oracle_experts(oracle, model, 0, list(zip(ids_n[t].tolist(), ws_n[t].tolist()))),
                                sh.hidden, sh.intermediate, oracle.SCALE_FP16, "gpu")
        assert_close(outs_n[t], want, f"T={T} token {t}")
