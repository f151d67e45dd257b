"""Real weights into the page pool: seeded fp32 expert matrices -> product-side quantiser -> `.vib3` page-split writer
-> reader -> VRAM pool -> fused layer (batch-1 and grouped), against the oracle's quantiser, page split and layer."""
import numpy as np
import pytest
import torch

from tests.parity import assert_close

pytestmark = pytest.mark.gpu


def test_quantised_file_round_trip_feeds_the_fused_layer(cuda_dev, oracle, tmp_path):
    from vic_b200.buffer_manager import PageBufferManager
    from vic_b200.core_types import EXPERT_SHARED, SCORING_SIGMOID, MoeShape
    from vic_b200.grouped import GroupedDecoder
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import SyntheticMoe
    from vic_b200.vib3_file import Vib3File, Vib3Writer
    sh = MoeShape("file-gpu", 1024, 2304, 6, 2, 1, SCORING_SIGMOID, 2.0, True)   # ragged last pages, staged kernels
    rng = np.random.default_rng(9)
    path = str(tmp_path / "m.vib3")
    wr = Vib3Writer(path, sh, 1)
    mats = {}
    for e in list(range(sh.num_experts)) + [EXPERT_SHARED]:
        mats[e] = tuple((rng.standard_normal(s) * 0.03).astype(np.float32)
                        for s in ((sh.intermediate, sh.hidden), (sh.intermediate, sh.hidden), (sh.hidden, sh.intermediate)))
        wr.add_expert(0, e, *mats[e])
    wr.finalize()
    f = Vib3File(path)
    cap = (sh.num_experts + 1) * sh.pages_per_expert
    pool = PageBufferManager(cap, device=cuda_dev, slot_seed=5)
    assert f.load_into_pool(pool) == cap
    pool.freeze()
    g = torch.Generator(device=cuda_dev).manual_seed(2)
    router_w = torch.randn(1, sh.num_experts, sh.hidden, generator=g, device=cuda_dev) * 0.02
    model = SyntheticMoe(sh, 1, pool, router_w)
    dec = MoeDecoder(model)
    gd = GroupedDecoder(model, max_tokens=16)
    xs = torch.randn(5, sh.hidden, generator=g, device=cuda_dev).to(torch.bfloat16)
    grouped = gd.forward(0, xs).clone()
    torch.cuda.synchronize()
    assert int(gd.status.item()) == 0

    def oracle_expert(e, w):
        lists = []
        for m in mats[e]:
            q = oracle.quantize_int4(m, 32, oracle.SCALE_FP16)
            lists.append([oracle.OraclePage(d, r0, rc) for d, r0, rc in oracle.split_int4_pages(q, m.shape[0], m.shape[1])])
        return oracle.OracleExpert(float(w), lists[0], lists[1], lists[2])
    W = router_w[0].cpu().numpy()
    for t in range(5):
        out = dec.forward_layer(0, xs[t]).cpu().numpy()
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        ids, ws = dec.routing()
        x32 = xs[t].float().cpu().numpy()
        oi, ow, _ = oracle.router(x32, W, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        assert np.array_equal(ids, oi)
        experts = [oracle_expert(int(e), w) for e, w in zip(oi.tolist(), ow.tolist())] + [oracle_expert(EXPERT_SHARED, 1.0)]
        want = oracle.moe_layer(x32, experts, sh.hidden, sh.intermediate, oracle.SCALE_FP16, "gpu")
        assert_close(out, want, f"token {t} batch-1")
        assert_close(grouped[t].cpu().numpy(), want, f"token {t} grouped")
    f.close()
