"""Grouped multi-token decode: T tokens through one MoE layer with every DISTINCT expert read once
(vib3_launch_moe_grouped_int4: tcgen05 tensor-core tiles over the INT4 pages).  The reference runs such a
batch token by token through its batch-1 path (src/runtime/engine.rs:1837-1838)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import kernels
from .core_types import MAX_ACTIVE_EXPERTS
from .lib import Vib3Error, check, lib
from .synth import SyntheticMoe

MAX_TOKENS = 128


def zipf_logit_offset(num_experts: int, seed: int, s: float = 1.1) -> np.ndarray:
    """The synthetic expert-load skew of the multi-token benchmark: logit offset -s * ln(rank) for a seeded
    permutation of ranks 1..E, added to the router logits before scoring."""
    rank = np.random.default_rng(seed).permutation(num_experts) + 1
    return (-s * np.log(rank)).astype(np.float32)


class GroupedDecoder:
    """Device buffers, tensor maps and launch sequence for up to ``max_tokens`` tokens per step."""

    def __init__(self, model: SyntheticMoe, max_tokens: int = MAX_TOKENS, exact_order: bool = True):
        sh = model.shape
        dev = model.router_w.device
        self.model, self.max_tokens, self.exact_order = model, max_tokens, exact_order
        nbytes = lib().vib3_moe_grouped_workspace_bytes(max_tokens, sh.top_k, sh.num_experts, sh.hidden, sh.intermediate,
                                                        sh.gate_up.rows_per_page, sh.down.rows_per_page)
        self.workspace = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=dev)
        ws_ptr = (self.workspace.data_ptr() + 1023) // 1024 * 1024
        pool = model.pool
        if pool.base_ptr % 16:
            raise Vib3Error("grouped decoder: pool base must be 16-byte aligned", -4)
        handle = C.c_void_p()
        last_gu = sh.gate_up.page_rows(sh.gate_up.num_pages - 1)[1]
        last_dn = sh.down.page_rows(sh.down.num_pages - 1)[1]
        check("moe_grouped_prewarm", lib().vib3_moe_grouped_prewarm(
            pool.base_ptr, pool.capacity_pages, sh.num_experts, sh.top_k, sh.hidden, sh.intermediate, sh.gate_up.rows_per_page,
            sh.down.rows_per_page, last_gu, last_dn, max_tokens, ws_ptr, nbytes, C.byref(handle)))
        self._h = handle
        self.scores = torch.zeros(max_tokens, 3 * sh.num_experts, dtype=torch.float32, device=dev)
        self.ids = torch.zeros(max_tokens, MAX_ACTIVE_EXPERTS, dtype=torch.int16, device=dev)
        self.weights = torch.zeros(max_tokens, MAX_ACTIVE_EXPERTS, dtype=torch.float32, device=dev)
        self.router_ws = torch.zeros(max_tokens, 4, dtype=torch.int32, device=dev)
        self.out = torch.zeros(max_tokens, sh.hidden, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tables = [model.page_table(l) for l in range(model.n_layers)]
        self.shared_tables = [model.shared_table(l) for l in range(model.n_layers)]
        # views into the workspace for inspection: GroupedWork {n_active, n_pairs}
        off = ws_ptr - self.workspace.data_ptr()
        self._work = self.workspace[off:off + 16].view(torch.int32)
        self._single = None

    def close(self) -> None:
        if self._h:
            lib().vib3_moe_grouped_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def n_distinct(self) -> torch.Tensor:
        """Distinct experts of the last step (the shared expert counts as one).  A single token with all experts
        goes through the batch-1 kernels, which keep no work list: its count is top_k (+ 1)."""
        if self._single is not None:
            return torch.tensor(self._single, dtype=torch.int32, device=self._work.device)
        return self._work[0]

    def route(self, layer: int, xs: torch.Tensor, logit_offset: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, hold: bool = False) -> None:
        """``hold``: xs comes from a launch that lets its dependents start early (see MoeDecoder.route)."""
        sh = self.model.shape
        kernels.router_topk_batch(xs, self.model.router_w[layer], self.scores, bias, logit_offset, self.ids, self.weights,
                                  sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize,
                                  int(self.exact_order) | (kernels.EXACT_HOLD if hold else 0), self.router_ws)

    def experts(self, layer: int, xs: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                expert_range=None, shared: bool = True) -> torch.Tensor:
        """expert_range (lo, hi): compute only the pairs of these experts (an expert-parallel rank's share);
        shared=False leaves the shared expert out."""
        sh = self.model.shape
        T = xs.shape[0]
        out = self.out[:T] if out is None else out
        lo, hi = expert_range if expert_range is not None else (0, sh.num_experts)
        has_shared = bool(self.shared_tables[layer]) and shared
        self._single = (sh.top_k + int(has_shared)) if (T == 1 and lo == 0 and hi == sh.num_experts) else None
        check("moe_grouped_int4", lib().vib3_launch_moe_grouped_int4(
            self._h, xs.data_ptr(), kernels.x_dtype_code(xs), xs.stride(0) * xs.element_size(), T, self.ids.data_ptr(),
            self.ids.stride(0) * 2, self.weights.data_ptr(), self.weights.stride(0) * 4, self.tables[layer],
            (self.shared_tables[layer] or None) if shared else None, 1.0, sh.pages_per_segment, lo, hi, out.data_ptr(),
            out.stride(0), int(accumulate),
            self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return out

    def forward(self, layer: int, xs: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                logit_offset: Optional[torch.Tensor] = None, hold: bool = False) -> torch.Tensor:
        """xs [T, H] (bf16 / fp16 / fp32, T <= max_tokens) -> [T, H] fp32; routing left in self.ids / self.weights."""
        if xs.shape[0] > self.max_tokens:
            raise ValueError("more tokens than the decoder was built for")
        self.route(layer, xs, logit_offset, hold=hold)
        return self.experts(layer, xs, out, accumulate)


# ── measurement helpers used by bench.py (single GPU) ───────────────────────────────────────────

def _graph_time(stream, fn, chunk, min_steps, min_ms=30.0):
    import bench as B
    return B.GraphTimer(stream, fn, chunk).time(min_steps, min_ms)


def bench_c3(model: SyntheticMoe, stream, peak_gbs: float, token_counts=(1, 8, 32, 128)) -> dict:
    """Grouped multi-token layer at 1/8/32/128 tokens with Zipf(1.1)-skewed expert load: microseconds per
    layer-step and bytes per second over the DISTINCT experts the step touches."""
    sh = model.shape
    dev = model.router_w.device
    L = model.n_layers
    gd = GroupedDecoder(model, max_tokens=max(token_counts))
    off = torch.from_numpy(zipf_logit_offset(sh.num_experts, 7)).to(dev)
    g = torch.Generator(device=dev).manual_seed(1234 + 3)
    out = {"workload": "C3 kimi-k2.5-shape MoE layer, grouped multi-token decode, router logits skewed by a Zipf(1.1) offset",
           "note": "HBM-bound by construction (90 GFLOP of tensor work against up to 7 GB of distinct expert weights at 128 tokens); "
                   "figure of merit = bytes over the distinct experts per second", "cases": []}
    from .synth import synth_activation
    for T in token_counts:
        nb = 4
        xs = synth_activation(sh, g, dev, torch.bfloat16, nb * T).view(nb, T, sh.hidden)
        distinct = []
        with torch.cuda.stream(stream):
            for b in range(nb):
                gd.forward(b % L, xs[b], logit_offset=off)
                stream.synchronize()
                distinct.append(int(gd.n_distinct.item()))
        fn = lambda i: gd.forward(i % L, xs[i % nb], logit_offset=off)  # noqa: E731
        ms, replays, steps = _graph_time(stream, fn, nb, 24 if T >= 32 else 48)
        ms_r, _, _ = _graph_time(stream, lambda i: gd.route(i % L, xs[i % nb], off), nb, 24)
        d = sum(distinct) / len(distinct)
        nbytes = d * sh.expert_bytes + sh.num_experts * sh.hidden * 4
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["cases"].append({"T": T, "distinct_experts": d, "us": ms * 1e3, "router_us": ms_r * 1e3, "tokens_per_s": T / (ms * 1e-3),
                             "bytes_over_distinct": nbytes, "hbm_gbs_over_distinct": gbs, "frac": gbs / peak_gbs, "timed_steps": steps})
    assert int(gd.status.item()) == 0
    gd.close()
    return out


def bench_c4_single(model: SyntheticMoe, stream, peak_gbs: float, n_layers: int = 61) -> dict:
    """The n_layers-deep stack on ONE GPU, batch 1 and batch 32: per layer a fused residual-add + RMS-norm launch
    (the attention block's stand-in is a seeded bf16 vector added to the hidden state), then the MoE sublayer
    adding into the hidden state.  The physical layers of the model are reused in rotation (layer l -> l mod L)."""
    from . import kernels as K
    from .moe import MoeDecoder
    from .synth import synth_activation
    sh = model.shape
    dev = model.router_w.device
    L = model.n_layers
    g = torch.Generator(device=dev).manual_seed(1234 + 4)
    T = 32
    # the attention block's stand-in: a seeded bf16 vector per layer and token, added to the hidden state
    attn = (torch.randn(n_layers, T, sh.hidden, generator=g, device=dev) * 0.3).to(torch.bfloat16)
    norm_w = (1.0 + 0.1 * torch.randn(n_layers, sh.hidden, generator=g, device=dev)).to(torch.float16)
    res = {"workload": f"C4 {n_layers}-layer kimi-k2.5-shape MoE stack on one GPU (attention = seeded bf16 residual add)",
           "layer_aliasing": f"layer l uses physical layer l mod {L} ({L} x {sh.expert_bytes * (sh.num_experts + 1) / 1e9:.1f} GB resident; "
                             f"{n_layers * sh.expert_bytes * (sh.num_experts + 1) / 1e9:.0f} GB would not fit); reuse distance {L} layers exceeds L2"}
    # batch 1
    dec = MoeDecoder(model, exact_order=True)
    h0 = synth_activation(sh, g, dev, torch.float32, 4)
    h = torch.zeros(1, sh.hidden, dtype=torch.float32, device=dev)
    x = torch.zeros(1, sh.hidden, dtype=torch.bfloat16, device=dev)

    def token1(i):
        h.copy_(h0[i % 4:i % 4 + 1])
        for l in range(n_layers):
            K.residual_rms_norm(h, attn[l, :1], norm_w[l], 1e-6, x, center=True, early_dependents=True)
            dec.forward_layer(l % L, x[0], out=h[0], accumulate=True, hold=True)
    ms, _, steps = _graph_time(stream, token1, 1, 4, 40.0)
    b_layer = 9 * sh.expert_bytes + sh.num_experts * sh.hidden * 4
    res["batch1"] = {"tokens_per_s": 1e3 / ms, "ms_per_token": ms, "us_per_layer": ms * 1e3 / n_layers,
                     "hbm_gbs": n_layers * b_layer / (ms * 1e-3) / 1e9, "frac": n_layers * b_layer / (ms * 1e-3) / 1e9 / peak_gbs,
                     "timed_tokens": steps, "launches_per_layer": 1 + dec.launches_per_layer}
    assert torch.isfinite(h).all() and int(dec.status.item()) == 0
    # batch 32
    gd = GroupedDecoder(model, max_tokens=T)
    hT0 = synth_activation(sh, g, dev, torch.float32, T)
    hT = torch.zeros(T, sh.hidden, dtype=torch.float32, device=dev)
    xT = torch.zeros(T, sh.hidden, dtype=torch.bfloat16, device=dev)
    dsum = torch.zeros(1, dtype=torch.int64, device=dev)

    def token32(i, count=False):
        hT.copy_(hT0)
        for l in range(n_layers):
            K.residual_rms_norm(hT, attn[l], norm_w[l], 1e-6, xT, center=True, early_dependents=True)
            gd.forward(l % L, xT, out=hT, accumulate=True, hold=True)
            if count:
                dsum.add_(gd.n_distinct.to(torch.int64))
    with torch.cuda.stream(stream):
        token32(0, count=True)
        stream.synchronize()
    d_avg = float(dsum.item()) / n_layers
    ms, _, steps = _graph_time(stream, token32, 1, 3, 40.0)
    nbytes = n_layers * (d_avg * sh.expert_bytes + sh.num_experts * sh.hidden * 4)
    res["batch32"] = {"tokens_per_s": T * 1e3 / ms, "ms_per_step": ms, "us_per_layer": ms * 1e3 / n_layers,
                      "distinct_experts_per_layer": d_avg, "hbm_gbs_over_distinct": nbytes / (ms * 1e-3) / 1e9,
                      "frac": nbytes / (ms * 1e-3) / 1e9 / peak_gbs, "timed_steps": steps}
    assert torch.isfinite(hT).all() and int(gd.status.item()) == 0
    gd.close()
    return res
