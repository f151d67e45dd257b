"""Expert parallelism on CPU ranks (gloo, world size 2): placement, the per-step message, the gather
and the cross-rank combine of vic_b200/ep.py, with the CPU oracle standing in for the GPU kernels.
The summed result of the ranks must equal the single-rank layer output for every rank's token."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _shape():
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    return MoeShape("ep-tiny", 64, 96, 8, 3, 1, SCORING_SIGMOID, 2.0, True)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from tests.parity import oracle_experts
        from vic_b200 import ep
        from vic_b200.core_types import EXPERT_SHARED, MAX_ACTIVE_EXPERTS
        from vic_b200.synth import build_synthetic_moe
        sh = _shape()
        H = sh.hidden
        full = build_synthetic_moe(sh, 1, "cpu", seed=11, slot_seed=3, per_page_content=True)
        mine = ep.build_rank_model(sh, 1, "cpu", 11, rank, world, per_page_content=True)
        assert sorted(set(p.pid.expert for p in mine.pages) - {EXPERT_SHARED}) == ep.local_experts(rank, sh.num_experts, world)
        assert torch.equal(full.router_w, mine.router_w)
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(H, generator=g).to(torch.bfloat16)
        W = full.router_w[0].numpy()
        ids, ws, _ = O.router(x.float().numpy(), W, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        ids_t = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.int16)
        ws_t = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.float32)
        ids_t[:sh.top_k] = torch.from_numpy(ids.astype(np.int16))
        ws_t[:sh.top_k] = torch.from_numpy(ws)
        ids_off, w_off, nbytes = ep.message_layout(H)
        assert nbytes % 16 == 0 and ids_off == 2 * H and w_off == ids_off + 2 * MAX_ACTIVE_EXPERTS
        send = torch.zeros(nbytes, dtype=torch.uint8)
        recv = torch.zeros(world, nbytes, dtype=torch.uint8)
        ep.pack_message(send, x, ids_t, ws_t)
        ep.gather_messages(send, recv, world)
        xs, gids, gws = ep.unpack_messages(recv, H)
        assert torch.equal(xs[rank], x) and torch.equal(gids[rank], ids_t) and torch.equal(gws[rank], ws_t)
        # every rank computes, for every token, the contribution of ITS experts (CPU oracle as the kernel)
        partial = torch.zeros(world, H, dtype=torch.float32)
        for t in range(world):
            act = [(int(e), float(w)) for e, w in zip(gids[t, :sh.top_k].tolist(), gws[t, :sh.top_k].tolist())
                   if ep.expert_owner(int(e), sh.num_experts, world) == rank]
            experts = oracle_experts(O, mine, 0, act) if t == rank else oracle_experts(O, mine, 0, act)[:len(act)]
            partial[t] = torch.from_numpy(O.moe_layer(xs[t].float().numpy(), experts, H, sh.intermediate, O.SCALE_FP16, "gpu"))
        out = torch.zeros(H, dtype=torch.float32)
        ep.combine_partials(out, partial, rank, world)
        want = O.moe_layer(x.float().numpy(), oracle_experts(O, full, 0, list(zip(ids.tolist(), ws.tolist()))), H,
                           sh.intermediate, O.SCALE_FP16, "gpu")
        err = float(np.max(np.abs(out.numpy() - want)))
        ret[rank] = (err, float(np.max(np.abs(want))))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_flow_on_two_cpu_ranks(oracle):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        err, mag = ret[r]
        assert mag > 0 and err <= 1e-5 * max(mag, 1.0), (r, err, mag)


def test_placement():
    from vic_b200.ep import expert_owner, local_experts
    for world in (1, 2, 4, 8):
        owners = [expert_owner(e, 384, world) for e in range(384)]
        assert owners == sorted(owners) and set(owners) == set(range(world))
        assert all(len(local_experts(r, 384, world)) == 384 // world for r in range(world))
    assert local_experts(1, 8, 2) == [4, 5, 6, 7]


def test_stack_placement_rules_and_imbalance_bound():
    """Host logic of the expert-parallel stack: every layer's shared expert has exactly one owner and the owners
    take turns; expert ranges tile [0, E) without overlap; the Monte-Carlo imbalance bound reproduces the
    figures the scaling targets were derived from (8 GPUs, uniform routing: about 3.1x at batch 1, 6.6x at batch 32)."""
    from vic_b200 import ep
    for world in (1, 2, 4, 8):
        owners = [ep.shared_expert_owner(l, world) for l in range(61)]
        assert all(0 <= o < world for o in owners) and len(set(owners)) == world
        cover = []
        for r in range(world):
            lo, hi = ep.expert_range(r, 384, world)
            assert list(range(lo, hi)) == ep.local_experts(r, 384, world)
            cover += list(range(lo, hi))
        assert cover == list(range(384))
    b1 = ep.imbalance_bound(384, 8, 8, 1, trials=1500)
    b32 = ep.imbalance_bound(384, 8, 8, 32, trials=300)
    assert 2.8 < b1["speedup_bound"] < 3.4 and abs(b1["distinct_experts"] - 8) < 1e-9
    assert 6.2 < b32["speedup_bound"] < 7.0 and 180 < b32["distinct_experts"] < 195
    assert ep.imbalance_bound(384, 8, 1, 4, trials=10)["speedup_bound"] == 1.0


def test_peer_exchange_buffer_layout():
    """The parts of a rank's peer-exchange buffer are aligned for 16-byte stores and do not overlap, at every world size."""
    from vic_b200 import ep
    from vic_b200.core_types import KIMI
    _, _, msg = ep.message_layout(KIMI.hidden)
    assert msg % 16 == 0
    for world in (2, 3, 4, 8):
        recv, rows, f1, f2, total = ep.peer_layout(KIMI.hidden, msg, world)
        parts = [(recv, world * msg), (rows, world * KIMI.hidden * 4), (f1, world * 4), (f2, world * 4)]
        for off, size in parts:
            assert off % 256 == 0
        for (a, sa), (b, _) in zip(parts, parts[1:]):
            assert a + sa <= b
        assert parts[-1][0] + parts[-1][1] <= total
