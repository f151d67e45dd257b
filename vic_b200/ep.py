"""Expert-parallel MoE decode over G GPUs of one node (one process per GPU, torch.distributed).

Placement: routed expert e lives on rank e // (E / G); every rank keeps the router weights and the
shared expert.  Each rank decodes its own token stream (batch 1 per rank: G tokens per step, weak
scaling), which is how a data-parallel attention stage feeds an expert-parallel MoE stage:

  1. every rank routes its own token (router weights are replicated, so the top-k is the one a
     single GPU would compute: bit-exact by construction); the router writes ids and weights straight
     into the rank's message, next to the token;
  2. all_gather of the messages (token activation, expert ids, routing weights): 14.4 KB per rank;
  3. each rank lists, on the device, the (token, expert, weight) pairs of the step whose expert it owns
     (token-major, order preserved) and runs ONE grouped launch pair of the expert kernels over them — on
     average top_k pairs per rank, i.e. the work of a single-GPU token — plus the shared expert for its
     own token; the kernels read the tokens in place from the gathered messages.  A launch takes up
     to 16 pairs; further launches for pairs 16.., 32.. follow unconditionally (the count lives on the
     device) and return at once when there is nothing for them;
  4. reduce_scatter of the per-token partial sums [G, H] fp32: each rank receives the full layer
     output of its own token.

Peer data always lands in local HBM (NCCL receive buffers) before a kernel reads it.  The only
difference from the single-GPU result is the fp32 association of the cross-rank sum.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .core_types import KIMI, MAX_ACTIVE_EXPERTS, MoeShape


def expert_owner(expert: int, num_experts: int, world: int) -> int:
    """Rank that holds a routed expert: contiguous blocks of E / G experts."""
    per = (num_experts + world - 1) // world
    return min(expert // per, world - 1)


def local_experts(rank: int, num_experts: int, world: int) -> List[int]:
    return [e for e in range(num_experts) if expert_owner(e, num_experts, world) == rank]


PAIRS_PER_LAUNCH = 16   # capacity of one grouped launch (kernel limit)


def message_layout(hidden: int) -> Tuple[int, int, int]:
    """Byte offsets of (expert ids u16[16], routing weights f32[16]) after the bf16 token, and the message
    size: [token bf16 x H][ids][weights], a multiple of 16 bytes so that every token starts aligned."""
    ids_off = hidden * 2
    w_off = ids_off + MAX_ACTIVE_EXPERTS * 2
    size = w_off + MAX_ACTIVE_EXPERTS * 4
    return ids_off, w_off, (size + 15) // 16 * 16


def message_views(buf: torch.Tensor, hidden: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Views into a message buffer ([bytes] or [G, bytes] uint8): token bf16 [.., H], ids int16 [.., 16],
    weights fp32 [.., 16].  The router writes through the last two; the kernels read the first in place."""
    ids_off, w_off, _ = message_layout(hidden)
    x = buf[..., :ids_off].view(torch.bfloat16)
    ids = buf[..., ids_off:w_off].view(torch.int16)
    ws = buf[..., w_off:w_off + MAX_ACTIVE_EXPERTS * 4].view(torch.float32)
    return x, ids, ws


def pack_message(buf: torch.Tensor, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Fill one rank's message from separate tensors (the GPU path lets the router write ids and weights
    in place and only copies the token)."""
    mx, mi, mw = message_views(buf, x.numel())
    mx.copy_(x)
    mi.copy_(ids)
    mw.copy_(weights)


def unpack_messages(recv: torch.Tensor, hidden: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[G, bytes] gathered messages -> (tokens [G, H] bf16, ids [G, 16] int16, weights [G, 16] fp32) views."""
    return message_views(recv, hidden)


def gather_messages(send: torch.Tensor, recv: torch.Tensor, world: int, group=None, scratch: Optional[torch.Tensor] = None) -> None:
    """Every rank's message to every rank.  With `scratch` ([G, bytes]) the exchange is one all-to-all of
    point-to-point transfers (one hop whatever G is) instead of the ring all-gather (G-1 hops)."""
    if world == 1:
        recv[0].copy_(send)
    elif scratch is not None:
        scratch.copy_(send.expand(world, -1))
        dist.all_to_all_single(recv.view(-1), scratch.view(-1), group=group)
    else:
        dist.all_gather_into_tensor(recv.view(-1), send, group=group)


def combine_partials(out: torch.Tensor, partial: torch.Tensor, rank: int, world: int, group=None,
                     scratch: Optional[torch.Tensor] = None) -> None:
    """Sum the per-token partial layer outputs [G, H] over ranks; rank r keeps row r.  With `scratch`
    ([G, H] fp32, device) row t of every rank goes to rank t in one all-to-all and the rank adds the G rows
    it received in rank order; otherwise NCCL's ring reduce-scatter does both."""
    if world == 1:
        out.copy_(partial[0])
    elif dist.get_backend(group) != "nccl":  # gloo (CPU tests) has no reduce_scatter
        tmp = partial.clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        out.copy_(tmp[rank])
    elif scratch is not None:
        from . import kernels
        dist.all_to_all_single(scratch.view(-1), partial.view(-1), group=group)
        kernels.sum_rows_f32(scratch, out)
    else:
        dist.reduce_scatter_tensor(out, partial.view(-1), op=dist.ReduceOp.SUM, group=group)


class ExpertParallelDecoder:
    """One rank's share of an expert-parallel MoE layer stack."""

    def __init__(self, model, rank: int, world: int, group=None):
        from .moe import MoeDecoder
        self.model, self.rank, self.world, self.group = model, rank, world, group
        self.dec = MoeDecoder(model, exact_order=True)
        sh = model.shape
        dev = model.router_w.device
        self.ids_off, self.w_off, self.msg_bytes = message_layout(sh.hidden)
        self.send = torch.zeros(self.msg_bytes, dtype=torch.uint8, device=dev)
        self.recv = torch.zeros(world, self.msg_bytes, dtype=torch.uint8, device=dev)
        self.send_x, self.send_ids, self.send_w = message_views(self.send, sh.hidden)
        self.recv_x, self.recv_ids, self.recv_w = message_views(self.recv, sh.hidden)
        self.partial = torch.zeros(world, sh.hidden, dtype=torch.float32, device=dev)
        self.out = torch.zeros(sh.hidden, dtype=torch.float32, device=dev)
        # "a2a": both exchanges as one-hop all-to-alls (plus a row sum); "ring": NCCL all-gather / reduce-scatter
        # measured: two ranks ring 11 + 11 us, a2a 14 + 14 us; eight ranks ring 21 + 19 us, a2a 16 + 17 us
        self.collectives = os.environ.get("VIB3_EP_COLLECTIVES", "a2a" if world >= 8 else "ring")
        self.send_rep = torch.zeros(world, self.msg_bytes, dtype=torch.uint8, device=dev) if self.collectives == "a2a" else None
        self.partial_in = torch.zeros(world, sh.hidden, dtype=torch.float32, device=dev) if self.collectives == "a2a" else None
        cap = world * sh.top_k
        self.pair_e = torch.zeros(cap, dtype=torch.int16, device=dev)
        self.pair_w = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.pair_t = torch.zeros(cap, dtype=torch.int16, device=dev)
        self.n_pairs = torch.zeros(1, dtype=torch.int32, device=dev)
        self.act = torch.zeros((PAIRS_PER_LAUNCH + 1) * sh.intermediate, dtype=torch.float16, device=dev)
        mine = local_experts(rank, sh.num_experts, world)
        self.expert_lo, self.expert_hi = (mine[0], mine[-1] + 1) if mine else (0, 0)
        self.grouped_launches = (cap + PAIRS_PER_LAUNCH - 1) // PAIRS_PER_LAUNCH
        # router, pair selection, (gate/up, down) per grouped launch, the row sum of the all-to-all form
        self.launches_per_step = 2 + 2 * self.grouped_launches + (1 if self.collectives == "a2a" else 0)

    def step(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        """x: this rank's token [H] bf16.  Returns this rank's token's layer output [H] fp32."""
        self.route(layer, x)
        self.gather()
        self.experts(layer)
        return self.combine()

    def route(self, layer: int, x: torch.Tensor) -> None:
        from . import kernels
        sh, dec = self.model.shape, self.dec
        self.send_x.copy_(x)
        # the router writes the expert ids and routing weights into the message
        kernels.router_topk_ex(self.send_x, self.model.router_w[layer], dec.scores, None, self.send_ids, self.send_w,
                               sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, dec.exact_order, dec.workspace)

    def gather(self) -> None:
        gather_messages(self.send, self.recv, self.world, self.group, self.send_rep)

    def experts(self, layer: int) -> None:
        from . import kernels
        from .core_types import X_BF16
        sh, dec = self.model.shape, self.dec
        H = sh.hidden
        kernels.select_local_pairs(self.recv_ids, self.msg_bytes, self.recv_w, self.msg_bytes, self.world, sh.top_k,
                                   self.expert_lo, self.expert_hi, self.pair_e, self.pair_w, self.pair_t,
                                   self.pair_e.numel(), self.n_pairs)
        for j in range(self.grouped_launches):
            kernels.moe_layer_int4_paged_grouped(
                self.recv_x, X_BF16, self.msg_bytes, self.world, dec.tables[layer], sh.num_experts,
                dec.shared_tables[layer] if j == 0 else 0, self.rank, self.pair_e, self.pair_w, self.pair_t,
                PAIRS_PER_LAUNCH, j * PAIRS_PER_LAUNCH, self.n_pairs, 1.0, self.act, self.partial, H, j > 0, H,
                sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page, dec.status)

    def combine(self) -> torch.Tensor:
        combine_partials(self.out, self.partial, self.rank, self.world, self.group, self.partial_in)
        return self.out

    def routing(self):
        """This rank's token's routing of the last step (host copies)."""
        k = self.model.shape.top_k
        return (self.send_ids[:k].cpu().view(torch.int16).numpy().view("uint16"), self.send_w[:k].cpu().numpy())


def build_rank_model(shape: MoeShape, n_layers: int, device, seed: int, rank: int, world: int, per_page_content=False):
    from .synth import build_synthetic_moe
    return build_synthetic_moe(shape, n_layers, device, seed=seed, slot_seed=99 + rank,
                               experts=local_experts(rank, shape.num_experts, world), per_page_content=per_page_content)


def bench_main(args) -> None:
    """bench.py --gpus N (N > 1), launched by torch.distributed.run: one rank per GPU."""
    import bench as B
    from .synth import synth_activation
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    sh = KIMI
    layers = B.PHYS_LAYERS
    model = build_rank_model(sh, layers, dev, B.SEED, rank, world)
    ep = ExpertParallelDecoder(model, rank, world)
    gen = torch.Generator(device=dev).manual_seed(B.SEED + 1000 * rank)
    xs = synth_activation(sh, gen, dev, torch.bfloat16, B.N_TOKENS)
    K, W = args.steps, args.warmup

    def step(i):
        ep.step(i % layers, xs[i % B.N_TOKENS])

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    # The step (kernels + NCCL collectives) is captured into a CUDA graph so that the 2G+1 launches
    # per step are not bound by the host; if capture is refused the loop runs eagerly.
    chunk = min(K, 32)
    graph, mode = None, "eager"
    if os.environ.get("VIB3_EP_NO_GRAPH") != "1":
        try:
            stream = torch.cuda.Stream(device=dev)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(chunk):
                        step(i)
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
            graph, mode = g, "cuda-graph"
        except Exception as exc:  # noqa: BLE001
            graph, mode = None, f"eager (graph capture refused: {type(exc).__name__})"
            torch.cuda.synchronize()
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        graph = None
    dist.barrier()
    sampler = B.ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    if graph is not None:
        for _ in range(K // chunk):
            graph.replay()
        for i in range(K % chunk):
            step(i)
    else:
        for i in range(K):
            step(i)
    e1.record()
    torch.cuda.synchronize()
    ms_local = e0.elapsed_time(e1)
    dist.barrier()
    clocks = sampler.stop() if sampler else None

    # e2e: token from pinned host memory in, layer output back to the host, every step
    x_host = [xs[i].cpu().pin_memory() for i in range(B.N_TOKENS)]
    out_host = torch.zeros(sh.hidden, dtype=torch.float32).pin_memory()
    x_dev = torch.zeros(sh.hidden, dtype=torch.bfloat16, device=dev)

    def e2e_step(i):
        x_dev.copy_(x_host[i % B.N_TOKENS], non_blocking=True)
        out_host.copy_(ep.step(i % layers, x_dev), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for i in range(min(W, 4)):
        e2e_step(i)
    dist.barrier()
    e0.record()
    for i in range(K):
        e2e_step(i)
    e1.record()
    torch.cuda.synchronize()
    e2e_local = e0.elapsed_time(e1)

    # where the step's time goes: each phase alone, 16 times back to back in a CUDA graph of its own
    # (CUDA events on this rank; every rank replays the same graphs, so the collectives match up)
    phases = {}
    if graph is not None:
        def time_phase(fn, reps=16):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                gp = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gp, stream=side):
                    for i in range(reps):
                        fn(i)
                gp.replay()
                side.synchronize()
                dist.barrier()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(side)
                for _ in range(4):
                    gp.replay()
                a1.record(side)
                side.synchronize()
            return a0.elapsed_time(a1) * 1e3 / (4 * reps)
        phases["route"] = time_phase(lambda i: ep.route(i % layers, xs[i % B.N_TOKENS]))
        phases["all_gather"] = time_phase(lambda i: ep.gather())
        phases["experts"] = time_phase(lambda i: ep.experts(i % layers))
        phases["reduce_scatter"] = time_phase(lambda i: ep.combine())
    dist.barrier()

    t = torch.tensor([ms_local, e2e_local], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        b_gu, b_dn, b_r = B.algorithmic_bytes(sh)
        line = {
            "metric": B.METRIC, "value": world * K / (ms * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights, 16-bit fixed-point activations, int32/fp32 accumulate", "data": "synthetic",
            "config": {"workload": "C1 kimi-k2.5-shape MoE layer, batch-1 decode per rank, experts sharded expert-parallel",
                       "hidden": sh.hidden, "experts": sh.num_experts, "experts_per_gpu": sh.num_experts // world,
                       "top_k": sh.top_k, "shared_experts": 1, "intermediate": sh.intermediate, "tokens_per_step": world,
                       "physical_layers": layers, "launch_mode": mode, "l2_policy": "inputs larger than L2: layers and tokens rotate",
                       "parallelism": f"ep{world}: exchange of (token, routing) + exchange and sum of partial sums, NCCL ({ep.collectives})"},
            "e2e": {"value": world * K / (e2e_ms * 1e-3), "unit": B.UNIT, "h2d_bytes_per_step": world * sh.hidden * 2,
                    "d2h_bytes_per_step": world * sh.hidden * 4, "ms_per_step": e2e_ms / K},
            "gpu_launches": K * ep.launches_per_step * world,
            "phase_us_rank0": {k: round(v, 1) for k, v in phases.items()},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": world * (b_gu + b_dn + b_r) / (ms * 1e-3 / K) / 1e9,
                         "peak": world * B.measured_peaks()[0], "unit": "GB/s",
                         "frac": (b_gu + b_dn + b_r) / (ms * 1e-3 / K) / 1e9 / B.measured_peaks()[0],
                         "traffic": None, "note": "whole step over all ranks (per-kernel roofline is reported at N=1)"},
        }
        print(json.dumps(line))
    # leave without tearing the communicator down under a live CUDA graph that holds its kernels
    graph = None
    torch.cuda.synchronize()
    import sys
    sys.stdout.flush()
    os._exit(0)
