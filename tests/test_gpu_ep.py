"""Expert parallelism on real GPUs (needs >= 2; skipped otherwise): every rank's token through
ExpertParallelDecoder must equal the single-GPU fused layer on the full model within tolerance, with
identical top-k on every rank."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _shape():
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    # staged kernels run (multiples of 256); 8 experts over 2 ranks
    return MoeShape("ep-mid", 1024, 2048, 8, 3, 1, SCORING_SIGMOID, 2.5, True)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from vic_b200 import ep
        from vic_b200.moe import MoeDecoder
        from vic_b200.synth import build_synthetic_moe
        sh = _shape()
        mine = ep.build_rank_model(sh, 2, dev, 11, rank, world, per_page_content=True)
        full = build_synthetic_moe(sh, 2, dev, seed=11, slot_seed=3, per_page_content=True)
        epd = ep.ExpertParallelDecoder(mine, rank, world)
        ref = MoeDecoder(full)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        # every rank runs every step's collectives whatever it observes; verdicts are reported at the end
        worst, problems = 0.0, []
        for step in range(6):
            x = torch.randn(sh.hidden, generator=g, device=dev).to(torch.bfloat16)
            layer = step % 2
            out = epd.step(layer, x).clone()
            ids_ep = epd.routing()[0].tolist()
            want = ref.forward_layer(layer, x).clone()
            torch.cuda.synchronize()
            if ids_ep != ref.routing()[0].tolist():
                problems.append(f"step {step}: routing differs")
            if int(ref.status.item()) != 0 or int(epd.dec.status.item()) != 0:
                problems.append(f"step {step}: status word set")
            a, b = out.cpu().numpy(), want.cpu().numpy()
            worst = max(worst, float(np.linalg.norm(a - b) / np.linalg.norm(b)))
            if np.max(np.abs(a - b)) > 2e-2:
                problems.append(f"step {step}: max-abs {np.max(np.abs(a - b)):.3e}")
        ret[rank] = (worst, problems)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_equals_single_gpu():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        worst, problems = ret[r]
        assert not problems, (r, problems)
        assert worst <= 1e-3, (r, worst)   # relative L2 of the layer output
