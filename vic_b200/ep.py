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

The two exchanges come in three forms (ExpertParallelDecoder(collectives=...)): "peer" — the default on GPUs — stores
the message / the partial rows straight into the peers' buffers over NVLink and follows them with a flag
(csrc/ep_peer.cu); "ring" and "a2a" use NCCL.
Peer data always lands in local HBM before a kernel reads it.  The only difference from the single-GPU result is
the fp32 association of the cross-rank sum.
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


class _DevMem:
    """A device allocation owned by somebody else, as an object torch can wrap (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def peer_layout(hidden: int, msg_bytes: int, world: int) -> Tuple[int, int, int, int, int]:
    """Byte offsets (messages, partial rows, message flags, row flags) and total size of a rank's exchange buffer:
    [G messages][G rows of H fp32][G flags][G flags], every part 256-byte aligned."""
    def up(v):
        return (v + 255) // 256 * 256
    recv_off = 0
    rows_off = up(world * msg_bytes)
    flags1_off = rows_off + up(world * hidden * 4)
    flags2_off = flags1_off + up(world * 4)
    return recv_off, rows_off, flags1_off, flags2_off, flags2_off + up(world * 4)


class PeerExchange:
    """The two exchanges of a decode step over peer memory instead of NCCL (csrc/ep_peer.cu): every rank maps every
    other rank's exchange buffer; a message or a partial row is stored straight into the peers' buffers and followed
    by a flag.  Layout of a rank's buffer: [G messages][G rows of H fp32: row r = rank r's partial sum of this
    rank's token][G flags of the messages][G flags of the rows]."""

    def __init__(self, hidden: int, msg_bytes: int, rank: int, world: int, device, group=None):
        import ctypes as C
        from .lib import check, lib
        self.rank, self.world, self.group = rank, world, group
        self.msg_bytes, self.hidden = msg_bytes, hidden
        self.recv_off, self.rows_off, self.flags1_off, self.flags2_off, self.nbytes = peer_layout(hidden, msg_bytes, world)
        handle = (C.c_ubyte * 64)()
        ptr = C.c_void_p()
        check("peer_alloc", lib().vib3_peer_alloc(self.nbytes, C.byref(ptr), handle))
        self._own = ptr.value
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.bases: List[int] = []
        self._opened: List[int] = []
        for r in range(world):
            if r == rank:
                self.bases.append(self._own)
                continue
            q = C.c_void_p()
            check("peer_open", lib().vib3_peer_open((C.c_ubyte * 64).from_buffer_copy(handles[r]), C.byref(q)))
            self.bases.append(q.value)
            self._opened.append(q.value)
        mem = torch.as_tensor(_DevMem(self._own, self.nbytes), device=device)
        self.recv = mem[self.recv_off:self.recv_off + world * msg_bytes].view(world, msg_bytes)
        self.rows = mem[self.rows_off:self.rows_off + world * hidden * 4].view(torch.float32).view(world, hidden)
        self.flags1 = mem[self.flags1_off:self.flags1_off + world * 4].view(torch.int32)
        self.flags2 = mem[self.flags2_off:self.flags2_off + world * 4].view(torch.int32)

        def table(off):
            return torch.tensor([b + off for b in self.bases], dtype=torch.int64, device=device)
        self.recv_table, self.rows_table = table(self.recv_off), table(self.rows_off)
        self.flags1_table, self.flags2_table = table(self.flags1_off), table(self.flags2_off)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)   # the step both exchanges are at
        torch.cuda.synchronize(device)
        dist.barrier(group=group)   # every rank has mapped every buffer before anybody stores into one

    def publish_message(self, send: torch.Tensor) -> None:
        """This rank's message into slot `rank` of every rank's buffer, flagged with the NEXT step."""
        from . import kernels
        kernels.peer_publish(send, 0, self.msg_bytes, self.recv_table, self.msg_bytes, self.flags1_table, self.counter, 1,
                             self.rank, self.world)

    def wait_select_pairs(self, status, ids, weights, top_k, lo, hi, pair_e, pair_w, pair_t, n_pairs) -> None:
        """Wait for every rank's message of the next step (the step counter advances), then list this rank's pairs."""
        from . import kernels
        kernels.peer_select_pairs(self.flags1, self.counter, self.world, status, ids, self.msg_bytes, weights, self.msg_bytes, top_k,
                                  lo, hi, pair_e, pair_w, pair_t, pair_e.numel(), n_pairs)

    def publish_rows(self, partial: torch.Tensor, overflow: Optional[torch.Tensor] = None, n_pairs: Optional[torch.Tensor] = None,
                     first_window: int = 0) -> None:
        """Row t of `partial` ([G, H] fp32) goes to rank t's row `rank`, flagged with the current step.  ``overflow``:
        a second [G, H] buffer that is added when ``*n_pairs > first_window`` (the later launch windows' sums)."""
        from . import kernels
        if overflow is None:
            kernels.peer_publish(partial, self.hidden * 4, self.hidden * 4, self.rows_table, self.hidden * 4, self.flags2_table,
                                 self.counter, 0, self.rank, self.world)
        else:
            kernels.peer_publish_rows(partial, overflow, self.hidden * 4, n_pairs, first_window, self.rows_table, self.hidden * 4,
                                      self.flags2_table, self.counter, 0, self.rank, self.world)

    def wait_sum_rows(self, status, out: torch.Tensor) -> None:
        """Wait for every rank's partial row of the current step, then add the rows in rank order."""
        from . import kernels
        kernels.peer_sum_rows(self.flags2, self.counter, self.world, status, self.rows, out)

    def close(self) -> None:
        from .lib import lib
        if self._own is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # nobody unmaps or frees while a peer may still store
        for q in self._opened:
            lib().vib3_peer_close(q)
        dist.barrier(group=self.group)
        lib().vib3_peer_free(self._own)
        self._own, self._opened = None, []


class ExpertParallelDecoder:
    """One rank's share of an expert-parallel MoE layer stack."""

    def __init__(self, model, rank: int, world: int, group=None, collectives: Optional[str] = None):
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
        # "peer": stores into the peers' buffers over NVLink, followed by flags (PeerExchange); "a2a": both exchanges
        # as NCCL one-hop all-to-alls (plus a row sum); "ring": NCCL all-gather / reduce-scatter
        # measured: two ranks ring 11 + 11 us, a2a 14 + 14 us; eight ranks ring 21 + 19 us, a2a 16 + 17 us
        on_gpus = world > 1 and dev.type == "cuda" and dist.is_initialized() and dist.get_backend(group) == "nccl"
        self.collectives = collectives or ("peer" if on_gpus else "ring")
        self.peer = None
        if self.collectives == "peer":
            self.peer = PeerExchange(sh.hidden, self.msg_bytes, rank, world, dev, group)
            self.recv = self.peer.recv
            self.recv_x, self.recv_ids, self.recv_w = message_views(self.recv, sh.hidden)
        self.send_rep = torch.zeros(world, self.msg_bytes, dtype=torch.uint8, device=dev) if self.collectives == "a2a" else None
        self.partial_in = torch.zeros(world, sh.hidden, dtype=torch.float32, device=dev) if self.collectives == "a2a" else None
        cap = world * sh.top_k
        self.pair_e = torch.zeros(cap, dtype=torch.int16, device=dev)
        self.pair_w = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.pair_t = torch.zeros(cap, dtype=torch.int16, device=dev)
        self.n_pairs = torch.zeros(1, dtype=torch.int32, device=dev)
        self.act = torch.zeros((PAIRS_PER_LAUNCH + 1) * sh.intermediate, dtype=torch.float16, device=dev)
        # Peer form with more than one launch window: the windows beyond the first — empty in all but a few steps
        # in a thousand, but their launches still cost a dependency hop each — run on a second stream beside
        # the first window, with scratch and partial sums of their own; the row exchange adds the two.
        self.side = None
        mine = local_experts(rank, sh.num_experts, world)
        self.expert_lo, self.expert_hi = (mine[0], mine[-1] + 1) if mine else (0, 0)
        self.grouped_launches = (cap + PAIRS_PER_LAUNCH - 1) // PAIRS_PER_LAUNCH
        # router, pair selection, (gate/up, down) per grouped launch, the row sum of the all-to-all form
        self.launches_per_step = 2 + 2 * self.grouped_launches + (1 if self.collectives == "a2a" else 0)
        if self.peer is not None:   # router (2), publish, wait + pair selection, grouped pairs, publish, wait + row sum
            self.launches_per_step = 2 + 1 + 1 + 2 * self.grouped_launches + 1 + 1
            if self.grouped_launches > 1 and dev.type == "cuda":
                self.side = torch.cuda.Stream(device=dev)
                self.act2 = torch.zeros_like(self.act)
                self.partial2 = torch.zeros_like(self.partial)

    def step(self, layer: int, x: torch.Tensor, logit_offset: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: this rank's token [H] bf16.  Returns this rank's token's layer output [H] fp32."""
        self.route(layer, x, logit_offset)
        self.gather()
        self.experts(layer)
        return self.combine()

    def route(self, layer: int, x: torch.Tensor, logit_offset: Optional[torch.Tensor] = None) -> None:
        from . import kernels
        sh, dec = self.model.shape, self.dec
        self.send_x.copy_(x)
        # the router writes the expert ids and routing weights into the message
        kernels.router_topk_ex(self.send_x, self.model.router_w[layer], dec.scores, None, self.send_ids, self.send_w,
                               sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, dec.exact_order, dec.workspace,
                               logit_offset=logit_offset)

    def gather(self) -> None:
        if self.peer is not None:
            self.peer.publish_message(self.send)   # stores only: the wait is the first thing experts() does
            return
        gather_messages(self.send, self.recv, self.world, self.group, self.send_rep)

    def experts(self, layer: int) -> None:
        from . import kernels
        from .core_types import X_BF16
        sh, dec = self.model.shape, self.dec
        H = sh.hidden
        if self.peer is not None:
            self.peer.wait_select_pairs(dec.status, self.recv_ids, self.recv_w, sh.top_k, self.expert_lo, self.expert_hi,
                                        self.pair_e, self.pair_w, self.pair_t, self.n_pairs)
        else:
            kernels.select_local_pairs(self.recv_ids, self.msg_bytes, self.recv_w, self.msg_bytes, self.world, sh.top_k,
                                       self.expert_lo, self.expert_hi, self.pair_e, self.pair_w, self.pair_t,
                                       self.pair_e.numel(), self.n_pairs)
        def window(j, act, out, accumulate):
            kernels.moe_layer_int4_paged_grouped(
                self.recv_x, X_BF16, self.msg_bytes, self.world, dec.tables[layer], sh.num_experts,
                dec.shared_tables[layer] if j == 0 else 0, self.rank, self.pair_e, self.pair_w, self.pair_t,
                PAIRS_PER_LAUNCH, j * PAIRS_PER_LAUNCH, self.n_pairs, 1.0, act, out, H, accumulate, H,
                sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page, dec.status)
        if self.side is not None:
            main = torch.cuda.current_stream()
            self.side.wait_stream(main)            # after the pair list
            with torch.cuda.stream(self.side):
                for j in range(1, self.grouped_launches):
                    window(j, self.act2, self.partial2, j > 1)
            window(0, self.act, self.partial, False)
            main.wait_stream(self.side)
            return
        for j in range(self.grouped_launches):
            window(j, self.act, self.partial, j > 0)

    def combine(self) -> torch.Tensor:
        if self.peer is not None:
            if self.side is not None:
                self.peer.publish_rows(self.partial, self.partial2, self.n_pairs, PAIRS_PER_LAUNCH)
            else:
                self.peer.publish_rows(self.partial)
            self.peer.wait_sum_rows(self.dec.status, self.out)
            return self.out
        combine_partials(self.out, self.partial, self.rank, self.world, self.group, self.partial_in)
        return self.out

    def close(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def routing(self):
        """This rank's token's routing of the last step (host copies)."""
        k = self.model.shape.top_k
        return (self.send_ids[:k].cpu().view(torch.int16).numpy().view("uint16"), self.send_w[:k].cpu().numpy())


def shared_expert_owner(layer: int, world: int) -> int:
    """The rank that computes the shared expert of a layer when the hidden state is replicated (stack mode):
    layers take turns, so that no rank repeats another's bytes."""
    return layer % world


def expert_range(rank: int, num_experts: int, world: int) -> Tuple[int, int]:
    mine = local_experts(rank, num_experts, world)
    return (mine[0], mine[-1] + 1) if mine else (0, 0)


class ExpertParallelStack:
    """The n_layers-deep MoE stack, expert-parallel, for ONE batch of tokens that every rank holds (the hidden
    state is replicated; a data-parallel attention stage would all-gather its tokens first).  Per layer: fused
    residual-add + RMS-norm launch (the attention block's stand-in is a seeded bf16 tensor added to the hidden
    state; the previous layer's MoE output, summed over ranks, is added by the same launch), the router (replicated:
    identical top-k on every rank by construction), the rank's own experts — batch 1 through the batch-1 kernels over
    the token's local experts, larger batches through the grouped tensor-core kernels restricted to the rank's
    expert range — the shared expert on rank layer mod G, and an all-reduce of the partial outputs.
    Physical layers are reused in rotation (layer l -> l mod L)."""

    def __init__(self, model, rank: int, world: int, n_layers: int, batch: int, seed: int = 77, group=None):
        from .moe import MoeDecoder
        self.model, self.rank, self.world, self.n_layers, self.T, self.group = model, rank, world, n_layers, batch, group
        sh = model.shape
        dev = model.router_w.device
        g = torch.Generator(device=dev).manual_seed(seed)           # the same tensors on every rank
        self.attn = (torch.randn(n_layers, batch, sh.hidden, generator=g, device=dev) * 0.3).to(torch.bfloat16)
        self.norm_w = (1.0 + 0.1 * torch.randn(n_layers, sh.hidden, generator=g, device=dev)).to(torch.float16)
        self.h0 = torch.randn(batch, sh.hidden, generator=g, device=dev)
        self.h = torch.zeros(batch, sh.hidden, dtype=torch.float32, device=dev)
        self.x = torch.zeros(batch, sh.hidden, dtype=torch.bfloat16, device=dev)
        self.partial = torch.zeros(batch, sh.hidden, dtype=torch.float32, device=dev)
        self.lo, self.hi = expert_range(rank, sh.num_experts, world)
        self.dec = MoeDecoder(model, exact_order=True)
        self.gd = None
        if batch > 1:
            from .grouped import GroupedDecoder
            self.gd = GroupedDecoder(model, max_tokens=batch)
        self.ids_loc = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.int16, device=dev)
        self.w_loc = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.float32, device=dev)
        self.n_loc = torch.zeros(1, dtype=torch.int32, device=dev)
        self.launches_per_layer = (4 if batch == 1 else 8) + (1 if world > 1 else 0)

    def layer(self, l: int, prev: Optional[torch.Tensor]) -> torch.Tensor:
        from . import kernels as K
        sh, dec = self.model.shape, self.dec
        phys = l % self.model.n_layers
        own_shared = shared_expert_owner(l, self.world) == self.rank
        K.residual_rms_norm(self.h, self.attn[l], self.norm_w[l], 1e-6, self.x, delta2=prev, center=True, early_dependents=True)
        if self.T == 1:
            dec.route(phys, self.x[0], hold=True)
            K.select_local_experts(dec.ids, dec.weights, sh.top_k, self.lo, self.hi, self.ids_loc, self.w_loc, self.n_loc)
            K.moe_layer_int4_paged_var(self.x[0], dec.tables[phys], sh.num_experts, dec.shared_tables[phys] if own_shared else 0,
                                       self.ids_loc, self.w_loc, sh.top_k, 1.0, dec.act, self.partial[0], False, sh.hidden,
                                       sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page,
                                       self.n_loc, dec.status)
        else:
            self.gd.route(phys, self.x, hold=True)
            self.gd.experts(phys, self.x, out=self.partial, expert_range=(self.lo, self.hi), shared=own_shared)
        if self.world > 1:
            dist.all_reduce(self.partial, op=dist.ReduceOp.SUM, group=self.group)
        return self.partial

    def step(self, i: int = 0) -> torch.Tensor:
        """One batch through the whole stack; returns the final hidden state [T, H] fp32 (replicated)."""
        from . import kernels as K
        self.h.copy_(self.h0)
        prev = None
        for l in range(self.n_layers):
            prev = self.layer(l, prev)
        self.h.add_(prev)
        return self.h

    def status(self) -> int:
        return int(self.dec.status.item()) | (int(self.gd.status.item()) if self.gd is not None else 0)


def imbalance_bound(num_experts: int, top_k: int, world: int, tokens: int, trials: int = 2000, seed: int = 1) -> dict:
    """Monte-Carlo bound on expert-parallel speed-up from load imbalance alone (uniform routing): a step waits for
    the rank with the most DISTINCT experts to read, so speed-up <= distinct experts of the step / that maximum."""
    import numpy as np
    rng = np.random.default_rng(seed)
    per = (num_experts + world - 1) // world
    tot, worst = 0.0, 0.0
    for _ in range(trials):
        picks = np.concatenate([rng.choice(num_experts, top_k, replace=False) for _ in range(tokens)])
        distinct = np.unique(picks)
        owners = np.minimum(distinct // per, world - 1)
        tot += len(distinct)
        worst += np.bincount(owners, minlength=world).max()
    return {"tokens": tokens, "distinct_experts": tot / trials, "busiest_rank_experts": worst / trials,
            "speedup_bound": tot / worst, "efficiency_bound": tot / worst / world}


def build_rank_model(shape: MoeShape, n_layers: int, device, seed: int, rank: int, world: int, per_page_content=False):
    from .synth import build_synthetic_moe
    return build_synthetic_moe(shape, n_layers, device, seed=seed, slot_seed=99 + rank,
                               experts=local_experts(rank, shape.num_experts, world), per_page_content=per_page_content)


def parity_check(rank: int, world: int, dev, steps: int = 6, group=None) -> dict:
    """Every rank decodes its own tokens through ExpertParallelDecoder on a small model and compares with the
    single-GPU fused layer on the FULL model (same bytes: pages are derived from (seed, page id)).  top_k = 12 and
    16 experts per rank, so that a step has up to 12 * world pairs; on odd steps a logit offset pulls every token to
    rank 0's experts: rank 0 then owns ALL pairs (several launch windows) and the other ranks none (empty windows
    ahead of the collective).  Collective: every rank calls this together.  Returns the worst figures over ranks."""
    from .core_types import SCORING_SIGMOID
    from .moe import MoeDecoder
    from .synth import build_synthetic_moe
    sh = MoeShape("ep-parity", 1024, 2048, 16 * world, 12, 1, SCORING_SIGMOID, 2.5, True)
    mine = build_rank_model(sh, 2, dev, 11, rank, world, per_page_content=True)
    full = build_synthetic_moe(sh, 2, dev, seed=11, slot_seed=3, per_page_content=True)
    epd = ExpertParallelDecoder(mine, rank, world, group)
    ref = MoeDecoder(full)
    off = torch.zeros(sh.num_experts, dtype=torch.float32, device=dev)
    off[:16] = 8.0
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    worst_abs, worst_rel, topk_equal, status, max_pairs = 0.0, 0.0, 1, 0, 0
    for step in range(steps):
        x = torch.randn(sh.hidden, generator=g, device=dev).to(torch.bfloat16)
        o = off if step % 2 else None
        layer = step % 2
        out = epd.step(layer, x, o).clone()
        ids_ep = epd.routing()[0].tolist()
        want = ref.forward_layer(layer, x, logit_offset=o).clone()
        torch.cuda.synchronize()
        if ids_ep != ref.routing()[0].tolist():
            topk_equal = 0
        status |= int(ref.status.item()) | int(epd.dec.status.item())
        max_pairs = max(max_pairs, int(epd.n_pairs.item()))
        worst_abs = max(worst_abs, float((out - want).abs().max()))
        worst_rel = max(worst_rel, float((out - want).norm() / want.norm()))
    t = torch.tensor([worst_abs, worst_rel, float(1 - topk_equal), float(status), float(max_pairs)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    res = {"max_abs": float(t[0]), "rel_l2": float(t[1]), "topk_equal": bool(t[2] == 0), "status": int(t[3]),
           "max_local_pairs": int(t[4]), "steps": steps, "collectives": epd.collectives,
           "ok": bool(t[0] <= 2e-2 and t[1] <= 1e-3 and t[2] == 0 and t[3] == 0)}
    epd.close()
    del epd, ref, mine, full
    torch.cuda.empty_cache()
    return res


def stack_parity_check(rank: int, world: int, dev, batch: int, n_layers: int = 5, group=None) -> dict:
    """ExpertParallelStack on the ranks' shards against the same stack on one GPU with the full model."""
    from .core_types import SCORING_SIGMOID
    from .synth import build_synthetic_moe
    sh = MoeShape("ep-stack-parity", 1024, 2048, 8 * world, 4, 1, SCORING_SIGMOID, 2.5, True)
    mine = build_rank_model(sh, 2, dev, 13, rank, world, per_page_content=True)
    full = build_synthetic_moe(sh, 2, dev, seed=13, slot_seed=3, per_page_content=True)
    a = ExpertParallelStack(mine, rank, world, n_layers, batch, group=group)
    b = ExpertParallelStack(full, 0, 1, n_layers, batch)
    ha = a.step().clone()
    hb = b.step().clone()
    torch.cuda.synchronize()
    t = torch.tensor([float((ha - hb).abs().max()), float((ha - hb).norm() / hb.norm()), float(a.status() | b.status())],
                     dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    res = {"batch": batch, "layers": n_layers, "max_abs": float(t[0]), "rel_l2": float(t[1]), "status": int(t[2]),
           "ok": bool(t[1] <= 2e-3 and t[2] == 0)}
    del a, b, mine, full
    torch.cuda.empty_cache()
    return res


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

    def timed_graph(fn, chunk, min_steps, min_ms):
        """(ms per step as the max over ranks, steps timed): one CUDA graph of `chunk` steps (kernels and NCCL
        collectives), replayed as often as every rank needs for min_steps steps and min_ms milliseconds."""
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for i in range(3):
                fn(i)
            stream.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(chunk):
                    fn(i)
            g.replay()
            stream.synchronize()
            replays = max(1, -(-min_steps // chunk))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for attempt in range(2):
                dist.barrier()
                stream.synchronize()
                e0.record(stream)
                for _ in range(replays):
                    g.replay()
                e1.record(stream)
                stream.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t[0])
                if ms >= min_ms:
                    break
                replays = int(replays * min_ms / max(ms, 1e-3) * 1.1) + 1   # (the same on every rank: ms is the maximum)
            del g
        torch.cuda.current_stream().wait_stream(stream)
        return ms / (replays * chunk), replays * chunk

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    sampler = B.ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    chunk = max(1, min(K, 32))
    ms_step, timed_steps = timed_graph(step, chunk, max(K, B.MIN_TIMED_STEPS), B.MIN_TIMED_MS)
    clocks = sampler.stop() if sampler else None

    # e2e: token from pinned host memory in, layer output back to the host, every step.  As on one GPU
    # (vib3_moe_step_run) the step of a bound layer is ONE CUDA graph — copy in from a pinned staging buffer, the whole
    # expert-parallel step with both exchanges, copy out into pinned memory — so the host pays one host-to-host copy
    # of the token, one graph launch and one wait per step instead of a dozen separate launches.
    x_host = [xs[i].cpu().pin_memory() for i in range(B.N_TOKENS)]
    x_stage = torch.zeros(sh.hidden, dtype=torch.bfloat16).pin_memory()
    out_host = torch.zeros(sh.hidden, dtype=torch.float32).pin_memory()
    out_np = out_host.numpy()
    x_dev = torch.zeros(sh.hidden, dtype=torch.bfloat16, device=dev)
    e2e_stream = torch.cuda.Stream(device=dev)
    e2e_stream.wait_stream(torch.cuda.current_stream())
    bound = []
    with torch.cuda.stream(e2e_stream):
        def body(l):
            x_dev.copy_(x_stage, non_blocking=True)
            out_host.copy_(ep.step(l, x_dev), non_blocking=True)
        for l in range(layers):
            body(l)                      # eager once: every rank runs the same steps, so the exchanges stay in step
        e2e_stream.synchronize()
        dist.barrier()
        for l in range(layers):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=e2e_stream):
                body(l)
            bound.append(g)
        checksum = 0.0

        def e2e_step(i):
            x_stage.copy_(x_host[i % B.N_TOKENS])          # the caller's token (host memory) into the staging buffer
            bound[i % layers].replay()
            e2e_stream.synchronize()
            return float(out_np[0])                      # the host reads the result
        for i in range(32):
            e2e_step(i)
        dist.barrier()
        e2e_steps = max(K, 2 * B.MIN_TIMED_STEPS)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(e2e_stream)
        for i in range(e2e_steps):
            checksum += e2e_step(i)
        e1.record(e2e_stream)
        e2e_stream.synchronize()
    torch.cuda.current_stream().wait_stream(e2e_stream)
    assert checksum == checksum
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0]) / e2e_steps
    del bound

    # where the step's time goes: the step cut short after each phase (every rank runs the same prefix, so an
    # exchange always finds its partners), each prefix in a CUDA graph of its own; a phase is the difference
    def prefix(n):
        def run(i):
            ep.route(i % layers, xs[i % B.N_TOKENS])
            if n >= 2:
                ep.gather()
            if n >= 3:
                ep.experts(i % layers)
            if n >= 4:
                ep.combine()
        return run
    cum = [timed_graph(prefix(n), 16, 64, 5.0)[0] * 1e3 for n in (1, 2, 3, 4)]
    phases = {"route": round(cum[0], 1), "exchange_tokens": round(cum[1] - cum[0], 1), "experts": round(cum[2] - cum[1], 1),
              "combine": round(cum[3] - cum[2], 1)}
    if ep.peer is not None:
        phases["note"] = ("the wait for the messages is the first warp of the pair selection, so it counts under experts; the shortened "
                          "steps lack the second exchange that normally keeps a rank from overwriting a message still being read, so "
                          "they are timings only")
    assert int(ep.dec.status.item()) == 0

    # correctness at this world size, outside every timed region
    parity = parity_check(rank, world, dev)
    extras = {}
    if not args.no_extras:
        peak = B.measured_peaks()[0]
        c4 = {"workload": f"C4 {B.STACK_LAYERS}-layer kimi-k2.5-shape MoE stack, experts sharded over {world} GPUs, hidden state replicated, "
                          "partial outputs summed by NCCL all-reduce; attention = seeded bf16 residual add",
              "layer_aliasing": f"layer l uses physical layer l mod {layers}: a rank holds {layers} x {len(local_experts(rank, sh.num_experts, world)) + 1} experts"}
        for batch in (1, 32):
            st = ExpertParallelStack(model, rank, world, B.STACK_LAYERS, batch)
            ms, n = timed_graph(lambda i: st.step(i), 1, 3, 40.0)
            assert st.status() == 0
            bound = imbalance_bound(sh.num_experts, sh.top_k, world, batch, trials=400)
            c4[f"batch{batch}"] = {"tokens_per_s": batch * 1e3 / ms, "ms_per_step": ms, "us_per_layer": ms * 1e3 / B.STACK_LAYERS,
                                   "timed_steps": n, "imbalance_bound": bound,
                                   "parity": stack_parity_check(rank, world, dev, batch)}
            del st
            torch.cuda.empty_cache()
        extras["c4"] = c4

    if rank == 0:
        b_gu, b_dn, b_r = B.algorithmic_bytes(sh)
        peak = B.measured_peaks()[0]
        per_step = (b_gu + b_dn + b_r) / (ms_step * 1e-3) / 1e9
        line = {
            "metric": B.METRIC, "value": world / (ms_step * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": B.DTYPE,
            "data": "synthetic", "config": B.workload_config(world),
            "timed": {"steps": timed_steps, "graph_steps": chunk, "physical_layers": layers, "launch_mode": "cuda-graph",
                      "collectives": "peer memory: stores and flags over NVLink (csrc/ep_peer.cu)" if ep.peer is not None else f"NCCL ({ep.collectives})",
                      "experts_per_gpu": sh.num_experts // world},
            "e2e": {"value": world / (e2e_ms * 1e-3), "unit": B.UNIT, "h2d_bytes_per_step": world * sh.hidden * 2,
                    "d2h_bytes_per_step": world * sh.hidden * 4, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "api": "one CUDA graph per bound layer and rank: copy in, ExpertParallelDecoder.step, copy out"},
            "gpu_launches": timed_steps * ep.launches_per_step * world,
            "phase_us_rank0": phases, "parity": parity,
            "imbalance_bound": imbalance_bound(sh.num_experts, sh.top_k, world, world, trials=400),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": world * per_step, "peak": world * peak, "unit": "GB/s", "frac": per_step / peak,
                         "traffic": None, "note": "whole step over all ranks, one layer-token per rank (the per-kernel roofline is reported at N=1)"},
        }
        line.update(extras)
        print(json.dumps(line))
    # leave without tearing the communicator down under live CUDA graphs that hold its kernels
    torch.cuda.synchronize()
    ep.close()
    import sys
    sys.stdout.flush()
    os._exit(0)
