"""The MoE sublayer of one decode token on the GPU: router -> experts -> accumulate.

``MoeDecoder.forward_layer`` is the fused path (3 launches, or 2 when the library is set to route inside
the gate/up kernel; no host synchronisation, graph capturable).  ``run_moe_sublayer_paged_calls`` drives the per-page entry points in the order the
reference engine does (src/runtime/engine.rs:5052-5360, :5801-6306) and exists so that path stays
exercised and comparable."""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from . import kernels
from .buffer_manager import LayerPlan, QueryPlanner
from .core_types import EXPERT_SHARED, MAX_ACTIVE_EXPERTS, SCORING_SIGMOID
from .synth import SyntheticMoe


class BoundHostStep:
    """Handle of vib3_moe_step_create with its buffers.  ``run(x_ptr)`` is vib3_moe_step_run on a host pointer: the token is
    copied in, the layer's graph launched and waited for; the fp32 [H] result is then in ``out`` (pinned host memory,
    ``out_np`` is the same memory as a numpy array), valid until the next run."""

    __slots__ = ("handle", "x_dev", "out", "out_np", "stream_ptr", "_run")

    def __init__(self, handle, x_dev: torch.Tensor, out: torch.Tensor, stream_ptr: int):
        from .lib import lib
        self.handle, self.x_dev, self.out, self.stream_ptr = handle, x_dev, out, stream_ptr
        self.out_np = out.numpy()
        self._run = lib().vib3_moe_step_run

    def run(self, x_ptr: int) -> None:
        err = self._run(self.handle, x_ptr, self.stream_ptr)
        if err:
            from .lib import check
            check("moe_step_run", err)


class MoeDecoder:
    """Device buffers and launch sequence for batch-1 decode over a SyntheticMoe (or any pool with
    the same page-table layout)."""

    def __init__(self, model: SyntheticMoe, exact_order: bool = True):
        self.model = model
        sh = model.shape
        dev = model.router_w.device
        self.exact_order = exact_order
        self.scores = torch.zeros(3 * sh.num_experts, dtype=torch.float32, device=dev)
        self.ids = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.int16, device=dev)
        self.weights = torch.zeros(MAX_ACTIVE_EXPERTS, dtype=torch.float32, device=dev)
        self.workspace = torch.zeros(4, dtype=torch.int32, device=dev)
        self.act = torch.zeros((sh.top_k + 1) * sh.intermediate, dtype=torch.float16, device=dev)
        self.out = torch.zeros(sh.hidden, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tables = [model.page_table(l) for l in range(model.n_layers)]
        self.shared_tables = [model.shared_table(l) for l in range(model.n_layers)]
        self.launches_per_layer = 3

    def _order_flags(self, hold: bool) -> int:
        return int(self.exact_order) | (kernels.EXACT_HOLD if hold else 0)

    def route(self, layer: int, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
              logit_offset: Optional[torch.Tensor] = None, hold: bool = False) -> None:
        """``hold``: x comes from a launch that lets its dependents start early (kernels.residual_rms_norm with
        early_dependents): the router then keeps the expert kernels from starting before x is complete."""
        sh = self.model.shape
        kernels.router_topk_ex(x, self.model.router_w[layer], self.scores, bias, self.ids, self.weights, sh.top_k,
                               sh.scoring, sh.scaling_factor, sh.normalize, self._order_flags(hold), self.workspace,
                               logit_offset=logit_offset)

    def experts(self, layer: int, x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                phase: int = 3) -> torch.Tensor:
        sh = self.model.shape
        out = self.out if out is None else out
        kernels.moe_layer_int4_paged(x, self.tables[layer], sh.num_experts, self.shared_tables[layer], self.ids,
                                     self.weights, sh.top_k, 1.0, self.act, out, accumulate, sh.hidden,
                                     sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page,
                                     sh.down.rows_per_page, self.status, phase=phase)
        return out

    def forward_layer(self, layer: int, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                      accumulate: bool = False, bias: Optional[torch.Tensor] = None,
                      logit_offset: Optional[torch.Tensor] = None, hold: bool = False) -> torch.Tensor:
        """x: [H] activations (bf16 / fp16 / fp32).  Returns the fp32 [H] sublayer output.  The routing is left in
        ``self.ids`` / ``self.weights``.  ``hold`` as in ``route``."""
        sh = self.model.shape
        out = self.out if out is None else out
        kernels.moe_layer_routed_int4_paged(x, self.model.router_w[layer], self.scores, bias, logit_offset, self.ids,
                                            self.weights, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize,
                                            self._order_flags(hold), self.workspace, self.tables[layer], sh.num_experts,
                                            self.shared_tables[layer], 1.0, self.act, out, accumulate, sh.hidden,
                                            sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page,
                                            sh.down.rows_per_page, self.status)
        return out

    def forward_host(self, layer: int, x_host: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """One token from and to HOST memory: x_host [H] (any of the activation dtypes, ordinary or pinned
        memory) -> pinned fp32 [H] (valid until the next call).  The copy in and the three launches are one CUDA graph per (layer, dtype), built on first use — the first call for a
        combination must therefore not happen inside somebody else's stream capture — so a step costs
        one graph launch and one stream synchronisation on the host.  The copy out is not a separate
        node: the last kernel writes its 4 H bytes into the pinned buffer directly."""
        key = (layer, x_host.dtype)
        stream = stream or torch.cuda.current_stream()
        if not hasattr(self, "_host_graphs"):
            self._host_graphs = {}
        entry = self._host_graphs.get(key)
        if entry is None:
            sh = self.model.shape
            dev = self.out.device
            x_pin = torch.zeros(sh.hidden, dtype=x_host.dtype).pin_memory()
            out_pin = torch.zeros(sh.hidden, dtype=torch.float32).pin_memory()
            x_dev = torch.zeros(sh.hidden, dtype=x_host.dtype, device=dev)

            def body():
                x_dev.copy_(x_pin, non_blocking=True)
                # the down kernel writes every output row once: it stores straight into the pinned host
                # buffer (device-addressable under unified addressing), which saves the copy-out node
                self.forward_layer(layer, x_dev, out=out_pin)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                body()  # warm-up outside capture: one-time kernel attributes and lazy loading
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    body()
            stream.wait_stream(side)
            entry = (graph, x_pin, out_pin)
            self._host_graphs[key] = entry
        graph, x_pin, out_pin = entry
        x_pin.copy_(x_host)          # host-to-host, a few microseconds for one activation vector
        with torch.cuda.stream(stream):
            graph.replay()
        stream.synchronize()
        return out_pin

    def forward_host_call(self, layer: int, x_host: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """The same step through ONE C call (vib3_moe_layer_step_host): what a binding without CUDA graphs
        uses.  Copies the token in, launches router, gate/up and down, waits for the stream; the down
        kernel stores its 4 H bytes straight into the pinned result buffer.  Measured 95 us per token
        against 91 us for the graph form (forward_host)."""
        sh = self.model.shape
        stream = stream or torch.cuda.current_stream()
        if not hasattr(self, "_host_bufs"):
            self._host_bufs = {}
        bufs = self._host_bufs.get(x_host.dtype)
        if bufs is None:
            bufs = (torch.zeros(sh.hidden, dtype=x_host.dtype, device=self.out.device),
                    torch.zeros(sh.hidden, dtype=torch.float32).pin_memory())
            self._host_bufs[x_host.dtype] = bufs
        x_dev, out_pin = bufs
        kernels.moe_layer_step_host(x_host, x_dev, self.model.router_w[layer], self.scores, None, self.ids, self.weights,
                                    sh.num_experts, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, self.exact_order,
                                    self.workspace, self.tables[layer], self.shared_tables[layer], 1.0, self.act, None, out_pin,
                                    sh.hidden, sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page,
                                    sh.down.rows_per_page, self.status, stream.cuda_stream)
        return out_pin

    def bind_host_step(self, layer: int, dtype: torch.dtype, stream: torch.cuda.Stream) -> "BoundHostStep":
        """One layer bound as a CUDA graph inside the library (vib3_moe_step_create): what a serving loop keeps per
        layer.  Built once per (layer, dtype), outside any stream capture, on a non-default stream."""
        import ctypes as C
        from .lib import check, lib
        sh = self.model.shape
        if not hasattr(self, "_bound"):
            self._bound = {}
        key = (layer, dtype)
        ent = self._bound.get(key)
        if ent is None:
            x_dev = torch.zeros(sh.hidden, dtype=dtype, device=self.out.device)
            out_pin = torch.zeros(sh.hidden, dtype=torch.float32).pin_memory()
            w = self.model.router_w[layer]
            h = C.c_void_p()
            check("moe_step_create", lib().vib3_moe_step_create(
                {torch.float32: kernels.X_F32, torch.float16: kernels.X_F16, torch.bfloat16: kernels.X_BF16}[dtype], x_dev.data_ptr(), w.data_ptr(),
                {torch.float16: 0, torch.float32: 1}[w.dtype],
                self.scores.data_ptr(), None, self.ids.data_ptr(), self.weights.data_ptr(), sh.num_experts, sh.top_k, sh.scoring,
                sh.scaling_factor, int(sh.normalize), int(self.exact_order), self.workspace.data_ptr(), self.tables[layer],
                self.shared_tables[layer] or None, 1.0, self.act.data_ptr(), out_pin.data_ptr(), sh.hidden, sh.intermediate,
                sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page, 32, self.status.data_ptr(),
                stream.cuda_stream, C.byref(h)))
            ent = BoundHostStep(h, x_dev, out_pin, stream.cuda_stream)
            self._bound[key] = ent
        return ent

    def forward_host_bound(self, layer: int, x_host: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """forward_host_call with the layer bound once as a CUDA graph inside the library (vib3_moe_step_create /
        vib3_moe_step_run): per token one C call with three arguments.  The first call for a (layer, dtype) builds the
        graph and must not happen inside a stream capture; ``stream`` must be a non-default stream.  Returns the
        pinned fp32 [H] result buffer of that (layer, dtype), valid until the next call."""
        if x_host.is_cuda:
            raise ValueError("host tensor expected")
        stream = stream or torch.cuda.current_stream()
        step = self.bind_host_step(layer, x_host.dtype, stream)
        step.run(x_host.data_ptr())
        return step.out

    def close(self) -> None:
        from .lib import lib
        for step in getattr(self, "_bound", {}).values():
            lib().vib3_moe_step_destroy(step.handle)
        self._bound = {}

    def forward_tokens(self, layer: int, xs: torch.Tensor, outs: Optional[torch.Tensor] = None,
                       logit_offset: Optional[torch.Tensor] = None, routing_out=None) -> torch.Tensor:
        """Multi-token decode, xs [T, H] -> [T, H] fp32: every token takes the batch-1 path in turn
        (the reference runs prefill the same way, src/runtime/engine.rs:1837-1838).  Experts that no
        token selects are never touched.  ``routing_out``: optional (ids int16 [T,16], weights fp32
        [T,16]) device tensors that receive each token's routing."""
        T = xs.shape[0]
        if outs is None:
            outs = torch.zeros(T, self.model.shape.hidden, dtype=torch.float32, device=xs.device)
        for t in range(T):
            self.route(layer, xs[t], None, logit_offset)
            if routing_out is not None:
                routing_out[0][t].copy_(self.ids)
                routing_out[1][t].copy_(self.weights)
            self.experts(layer, xs[t], outs[t])
        return outs

    def routing(self) -> Tuple[np.ndarray, np.ndarray]:
        k = self.model.shape.top_k
        return (self.ids[:k].cpu().numpy().view(np.uint16).copy(), self.weights[:k].cpu().numpy().copy())


def run_moe_sublayer_paged_calls(model: SyntheticMoe, layer: int, x_f32: torch.Tensor, planner: QueryPlanner,
                                 router_w_f16: torch.Tensor, bufs: Optional[dict] = None):
    """The reference engine's INT4 MoE sublayer, call by call, on this library's per-page entry
    points: router with host sync (kernels.rs:1811-1873), plan_layer, then per expert the
    (up, gate) page pairs through partial_swiglu_f32 with temps, the down pages through
    partial_matmul, weighted_accumulate_f32; shared expert last with weight 1.0.
    Returns (layer_out_f32 [H], [(expert, weight)], launches)."""
    sh = model.shape
    dev = x_f32.device
    H, I = sh.hidden, sh.intermediate
    b = bufs if bufs is not None else {}
    def buf(name, n, dt):
        if name not in b:
            b[name] = torch.zeros(n, dtype=dt, device=dev)
        return b[name]
    scores = buf("scores", sh.num_experts, torch.float32)
    ids = buf("ids", MAX_ACTIVE_EXPERTS, torch.int16)
    ws = buf("ws", MAX_ACTIVE_EXPERTS, torch.float32)
    up_tmp, gate_tmp = buf("up_tmp", I, torch.float16), buf("gate_tmp", I, torch.float16)
    expert_out = buf("expert_out", I, torch.float16)
    down_out = buf("down_out", H, torch.float16)
    layer_out = buf("layer_out", H, torch.float32)
    launches = 0
    activation = kernels.run_router_gpu_topk(x_f32, router_w_f16, scores, None, ids, ws, H, sh.num_experts, sh.top_k,
                                             sh.scoring, sh.scaling_factor)
    launches += 2
    entries = list(activation) + ([(EXPERT_SHARED, 1.0)] if sh.shared_experts else [])
    plan: LayerPlan = planner.plan_layer(layer, entries)
    layer_out.zero_()
    for ep in plan.experts:
        segs = sorted(set(p.id.segment for p in ep.pages))
        up_pages = [p for p in ep.pages if p.id.segment == segs[0]]
        gate_pages = [p for p in ep.pages if p.id.segment == segs[1]]
        down_pages = [p for p in ep.pages if p.id.segment == segs[2]]
        expert_out.zero_()
        for up, gate in zip(up_pages, gate_pages):
            kernels.partial_swiglu_f32(x_f32, up.device_ptr, gate.device_ptr, expert_out.data_ptr() + 2 * up.row_start,
                                       H, up.row_count, swiglu_temps=(up_tmp, gate_tmp))
            launches += 3
        down_out.zero_()
        for dp in down_pages:
            kernels.partial_matmul(expert_out, dp.device_ptr, down_out.data_ptr() + 2 * dp.row_start, I, dp.row_count)
            launches += 1
        kernels.weighted_accumulate_f32(layer_out, down_out, ep.weight, H)
        launches += 1
    return layer_out, activation, launches
