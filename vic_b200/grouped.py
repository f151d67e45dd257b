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
        nbytes = lib().vib3_moe_grouped_workspace_bytes(max_tokens, sh.top_k, sh.num_experts, sh.hidden, sh.intermediate)
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
        """Distinct experts of the last step (the shared expert counts as one)."""
        return self._work[0]

    def route(self, layer: int, xs: torch.Tensor, logit_offset: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None) -> None:
        sh = self.model.shape
        kernels.router_topk_batch(xs, self.model.router_w[layer], self.scores, bias, logit_offset, self.ids, self.weights,
                                  sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, self.exact_order, self.router_ws)

    def experts(self, layer: int, xs: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        sh = self.model.shape
        T = xs.shape[0]
        out = self.out[:T] if out is None else out
        check("moe_grouped_int4", lib().vib3_launch_moe_grouped_int4(
            self._h, xs.data_ptr(), kernels.x_dtype_code(xs), xs.stride(0) * xs.element_size(), T, self.ids.data_ptr(),
            self.ids.stride(0) * 2, self.weights.data_ptr(), self.weights.stride(0) * 4, self.tables[layer],
            self.shared_tables[layer] or None, 1.0, sh.pages_per_segment, out.data_ptr(), out.stride(0), int(accumulate),
            self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return out

    def forward(self, layer: int, xs: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                logit_offset: Optional[torch.Tensor] = None) -> torch.Tensor:
        """xs [T, H] (bf16 / fp16 / fp32, T <= max_tokens) -> [T, H] fp32; routing left in self.ids / self.weights."""
        if xs.shape[0] > self.max_tokens:
            raise ValueError("more tokens than the decoder was built for")
        self.route(layer, xs, logit_offset)
        return self.experts(layer, xs, out, accumulate)
