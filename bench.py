#!/usr/bin/env python
"""Benchmark of the vib3 INT4 MoE decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): one Kimi-K2.5-shape MoE layer, batch-1 decode: hidden 7168, 384 routed experts
top-8 (sigmoid, renormalised, x2.827) + 1 shared expert, intermediate 2048, INT4 group-32 weights in
2 MiB pages scattered in a VRAM pool, bf16 activations, fp32 router weights.  A step is one token
through one such layer (router -> gate/up+SiLU -> down+accumulate).  Four physical layers (38.8 GB of
pages) are used in rotation and every step has its own token, so no weight byte is re-read before
4 x 234 MB of other traffic went through the 126 MB L2.  Data is seeded synthetic.

Prints ONE JSON line (rank 0).  `value`: tokens/s with inputs resident in HBM (CUDA-graph replay,
CUDA events, at least 200 layer-steps and 50 ms whatever --steps is); `e2e`: the same through host
buffers, one call per token; `roofline`: the dominant kernel (gate/up) timed alone against the
measured HBM copy bandwidth; `cpu_baseline`: the CPU restatement of the reference's kernels (oracle/)
on this host's cores over a bounded sample; `ref_gpu`: the reference's own CUDA kernels, compiled
unmodified, driven in its engine's per-page order on this GPU; `c0`, `c3`, `c4`: the Mixtral-shape
layer, the grouped multi-token layer and the 61-layer stack, each with its own algorithmic bytes.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "Kimi-shape MoE decode tokens/s (one MoE layer per token, batch 1)"
UNIT = "tokens/s"
DTYPE = "int4 weights, 16-bit fixed-point activations, int32/fp32 accumulate"
PHYS_LAYERS = 4
N_TOKENS = 64
SEED = 1234 + 1
MIN_TIMED_STEPS = 200     # layer-steps inside a timed region, whatever --steps says
MIN_TIMED_MS = 50.0
STACK_LAYERS = 61


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def profile_figure(name: str, default=None):
    """A number committed in a summary under profiles/: the line `<name>: <value>`."""
    pdir = os.path.join(ROOT, "profiles")
    try:
        for fn in sorted(os.listdir(pdir)):
            for ln in open(os.path.join(pdir, fn)):
                if ln.startswith(name + ":"):
                    return float(ln.split(":", 1)[1].split()[0])
    except Exception:
        pass
    return default


def workload_config(n_gpus: int) -> dict:
    """The `config` of the JSON line; both arms (--impl ours / reference) print the same one."""
    from vic_b200.core_types import KIMI as sh
    cfg = {"workload": "C1 kimi-k2.5-shape single MoE layer, batch-1 decode over paged INT4 experts",
           "hidden": sh.hidden, "experts": sh.num_experts, "top_k": sh.top_k, "shared_experts": sh.shared_experts,
           "intermediate": sh.intermediate, "activations": "bf16", "router_weights": "fp32", "group_size": 32,
           "page_bytes": 2 << 20, "tokens_per_step": n_gpus,
           "l2_policy": "inputs larger than L2: the pages of consecutive steps differ (layers and tokens rotate)",
           "parallelism": "single GPU" if n_gpus == 1 else f"ep{n_gpus}: experts sharded over {n_gpus} GPUs, one token per GPU per step"}
    return cfg


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(shape, router_bytes_per_weight=4):
    """Weights + scales + router weights read once per token (activations are < 60 KB)."""
    slots = shape.top_k + shape.shared_experts
    gate_up = slots * 2 * shape.gate_up.matrix_bytes
    down = slots * shape.down.matrix_bytes
    router = shape.num_experts * shape.hidden * router_bytes_per_weight
    return gate_up, down, router


class GraphTimer:
    """Times a step function as CUDA-graph replays with CUDA events on the launching stream.

    The graph holds `chunk` consecutive steps; it is replayed R times back to back, R chosen so that
    the region holds at least MIN_TIMED_STEPS steps and lasts at least MIN_TIMED_MS — the figure does
    not depend on how few steps the caller asked for."""

    def __init__(self, stream, step_fn, chunk: int, warm: int = 3):
        import torch
        self.torch, self.stream, self.chunk = torch, stream, chunk
        with torch.cuda.stream(stream):
            for i in range(warm):
                step_fn(i)
            stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                for i in range(chunk):
                    step_fn(i)
            self.graph.replay()
            stream.synchronize()

    def _run(self, replays: int) -> float:
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(self.stream):
            self.stream.synchronize()
            e0.record(self.stream)
            for _ in range(replays):
                self.graph.replay()
            e1.record(self.stream)
            self.stream.synchronize()
        return e0.elapsed_time(e1)

    def time(self, min_steps: int = MIN_TIMED_STEPS, min_ms: float = MIN_TIMED_MS):
        """(milliseconds per step, replays, steps timed)."""
        replays = max(1, math.ceil(min_steps / self.chunk))
        ms = self._run(replays)
        if ms < min_ms:
            replays = max(replays + 1, math.ceil(replays * min_ms / max(ms, 1e-3) * 1.1))
            ms = self._run(replays)
        return ms / (replays * self.chunk), replays, replays * self.chunk


# ── CPU legs (the only code here that touches oracle/) ──────────────────────────────────────────

def host_expert_pool(O, sh, n_experts: int, seed: int):
    """`n_experts` experts' pages generated directly in host memory with the synthetic distributions
    (codes uniform, group scales |N(0, 0.02)| / 7 exact in bf16 and fp16), as the oracle's page lists."""
    import numpy as np
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for _ in range(n_experts):
        lists = []
        for geom in (sh.gate_up, sh.gate_up, sh.down):
            pages = []
            for p in range(geom.num_pages):
                r0, rc = geom.page_rows(p)
                ncode = rc * geom.packed_k
                buf = torch.empty(rc * geom.bytes_per_row, dtype=torch.uint8)
                buf[:ncode].random_(0, 256, generator=g)
                sc = torch.randn(rc * geom.num_groups, generator=g).abs_().mul_(0.02 / 7.0).clamp_(min=2.0 ** -13)
                buf[ncode:] = sc.to(torch.bfloat16).to(torch.float16).view(torch.uint8)
                pages.append(O.OraclePage(np.ascontiguousarray(buf.numpy()), r0, rc))
            lists.append(pages)
        out.append(O.OracleExpert(1.0, lists[0], lists[1], lists[2]))
    return out


class CpuLayer:
    """The CPU restatement of the reference's kernels over one Kimi-shape layer-token: router, the 8
    routed experts and the shared expert in the engine's order.  Every token walks a different set of
    nine experts out of a host pool of 27 (670 MB, larger than the CPU's caches), so weights come from
    memory as they would in a real decode.  The one procedure behind `cpu_baseline` and `--impl reference`."""

    def __init__(self):
        import torch
        from oracle import oracle as O
        from vic_b200.core_types import KIMI
        O.build()
        self.O, self.sh = O, KIMI
        self.threads = O.set_num_threads(os.cpu_count() or 1)   # torchrun exports OMP_NUM_THREADS=1 to its children
        self.flags = O.build_flags()
        self.pool = host_expert_pool(O, KIMI, 27, SEED)
        g = torch.Generator(device="cpu").manual_seed(SEED)
        self.W = [(torch.randn(KIMI.num_experts, KIMI.hidden, generator=g) * 0.02).numpy() for _ in range(2)]
        self.xs = torch.randn(8, KIMI.hidden, generator=g).to(torch.bfloat16).float().numpy()

    def step(self, i: int):
        O, sh = self.O, self.sh
        x = self.xs[i % 8]
        ids, ws, _ = O.router(x, self.W[i % 2], sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        base = (i % 3) * 9
        experts = self.pool[base:base + 9]
        for ex, w in zip(experts[:sh.top_k], ws.tolist()):
            ex.weight = w
        experts[sh.top_k].weight = 1.0
        return O.moe_layer(x, experts, sh.hidden, sh.intermediate, O.SCALE_FP16, "gpu")

    def describe(self, steps: int) -> str:
        return (f"{steps} full layer-tokens (router + 8 routed + 1 shared expert, a different set of experts every token) through the "
                f"C restatement of the reference's Rust CPU kernels, built {self.flags}; the Rust crate itself needs cargo, which this image lacks")


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path on this host's cores (kind
    "port": the C restatement under oracle/).  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuLayer()
    for i in range(max(args.warmup, 1)):
        cpu.step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        cpu.step(i)
    dt = time.perf_counter() - t0
    val = args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4 weights x f32 activations, f32 accumulate (CPU)", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cpu.threads, "kind": "port", "flags": cpu.flags,
                         "sample": cpu.describe(args.steps)},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def cpu_baseline_leg(budget_s: float = 15.0) -> dict:
    cpu = CpuLayer()
    cpu.step(0)
    done, t_total = 0, 0.0
    while t_total < budget_s and done < 200:
        t0 = time.perf_counter()
        cpu.step(1 + done)
        t_total += time.perf_counter() - t0
        done += 1
    return {"value": done / t_total, "unit": UNIT, "cores": cpu.threads, "kind": "port", "flags": cpu.flags,
            "sample": cpu.describe(done)}


# ── small cases for ncu (the commands under profiles/ run these) ───────────────────────────────

def profile_small(n, what="layer"):
    import torch
    from vic_b200.core_types import KIMI, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    dev = torch.device("cuda:0")
    if what == "router":
        # full-width router (384 experts, exact-order checks on) over a pool that holds 16 experts' pages
        model = build_synthetic_moe(KIMI, 2, dev, seed=SEED, slot_seed=99, experts=range(16))
        dec = MoeDecoder(model, exact_order=True)
        g = torch.Generator(device=dev).manual_seed(1)
        xs = synth_activation(KIMI, g, dev, torch.bfloat16, 8)
        for i in range(n):
            dec.route(i % 2, xs[i % 8])
        torch.cuda.synchronize()
        print(json.dumps({"profile_router": n}))
        return
    if what == "grouped":
        from vic_b200.grouped import GroupedDecoder, zipf_logit_offset
        sh = MoeShape("kimi48", KIMI.hidden, KIMI.intermediate, 48, KIMI.top_k, 1, KIMI.scoring, KIMI.scaling_factor, True)
        model = build_synthetic_moe(sh, 1, dev, seed=SEED, slot_seed=99)
        gd = GroupedDecoder(model, max_tokens=32)
        g = torch.Generator(device=dev).manual_seed(1)
        xs = synth_activation(sh, g, dev, torch.bfloat16, 32)
        off = torch.from_numpy(zipf_logit_offset(sh.num_experts, 7)).to(dev)
        for i in range(n):
            gd.forward(0, xs, logit_offset=off)
        torch.cuda.synchronize()
        assert int(gd.status.item()) == 0
        print(json.dumps({"profile_grouped": n, "distinct_experts": int(gd.n_distinct.item())}))
        return
    sh = MoeShape("kimi16", KIMI.hidden, KIMI.intermediate, 16, KIMI.top_k, 1, KIMI.scoring, KIMI.scaling_factor, True)
    model = build_synthetic_moe(sh, 2, dev, seed=SEED, slot_seed=99)
    dec = MoeDecoder(model, exact_order=False)
    g = torch.Generator(device=dev).manual_seed(1)
    xs = synth_activation(sh, g, dev, torch.bfloat16, 8)
    for i in range(n):
        dec.forward_layer(i % 2, xs[i % 8])
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    print(json.dumps({"profile_small": n, "status": 0}))


# ── secondary workloads of the single-GPU line ─────────────────────────────────────────────────

def bench_c0(dev, stream):
    """Mixtral-8x7B-shape layer, batch-1 decode: hidden 4096, 8 experts top-2 (softmax), intermediate
    14336, fp16 activations, fp32 router weights.  198,311,936 algorithmic bytes per token."""
    import torch
    from vic_b200.core_types import MIXTRAL as sh
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    layers = 2                                     # 2 x 0.79 GB rotate: nothing is served from L2
    model = build_synthetic_moe(sh, layers, dev, seed=1234, slot_seed=98)
    dec = MoeDecoder(model, exact_order=True)
    g = torch.Generator(device=dev).manual_seed(1234)
    xs = synth_activation(sh, g, dev, torch.float16, 16)
    outs = torch.zeros(16, sh.hidden, dtype=torch.float32, device=dev)
    timer = GraphTimer(stream, lambda i: dec.forward_layer(i % layers, xs[i % 16], out=outs[i % 16]), 32)
    ms, replays, steps = timer.time()
    assert int(dec.status.item()) == 0
    b_gu, b_dn, b_r = algorithmic_bytes(sh)
    peak, _ = measured_peaks()
    gbs = (b_gu + b_dn + b_r) / (ms * 1e-3) / 1e9
    del timer, dec, model
    torch.cuda.empty_cache()
    return {"workload": "C0 mixtral-8x7b-shape single MoE layer, batch-1 decode, fp16 activations, softmax top-2",
            "tokens_per_s": 1e3 / ms, "us_per_layer": ms * 1e3, "bytes_per_token": b_gu + b_dn + b_r, "hbm_gbs": gbs,
            "frac_of_peak": gbs / peak, "timed_steps": steps}


def bench_ref_gpu(model, xs, dev):
    """The reference's own CUDA kernels (compiled unmodified) on the same pages, in its engine's order."""
    import torch
    from oracle import ref_gpu
    w16 = model.router_w.to(torch.float16)
    r = ref_gpu.time_reference_gpu_layer(model, xs.float(), w16, iters=12)
    if r is None:
        return {"unavailable": "oracle/_ref/libvib3_ref.so is not built (needs the reference tree at build time)"}
    b_gu, b_dn, b_r = algorithmic_bytes(model.shape, 2)
    r["hbm_gbs"] = (b_gu + b_dn + b_r) / (r["us_per_layer"] * 1e-6) / 1e9
    r["note"] = ("reference cuda/src/kernels.cu, unmodified, sm_100: router GEMV, host selection after a stream synchronisation, "
                 "then one launch per page and step as src/runtime/engine.rs:6094-6107, :6215-6223, :6290-6296; CUDA events, same pages")
    return r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="only the headline workload (skip c0, c3, c4, ref_gpu)")
    ap.add_argument("--profile-small", type=int, default=0, metavar="N",
                    help="run N untimed layer-steps of a 16-expert Kimi-shape layer (same per-launch work as the full "
                         "workload: 8 routed + 1 shared expert, 223 MB of weights per step, 0.8 GB resident) and exit (for ncu)")
    ap.add_argument("--profile-router", type=int, default=0, metavar="N",
                    help="run N untimed launches of the full-width (384-expert) router and exit (for ncu)")
    ap.add_argument("--profile-grouped", type=int, default=0, metavar="N",
                    help="run N untimed grouped 32-token layer-steps of a 48-expert Kimi-shape layer (1.2 GB resident) and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_small:
        return profile_small(args.profile_small)
    if args.profile_router:
        return profile_small(args.profile_router, "router")
    if args.profile_grouped:
        return profile_small(args.profile_grouped, "grouped")
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        args.steps = min(args.steps, 200)  # ~0.05-0.1 s per CPU layer-token: keep the arm within a few minutes
        return run_reference_arm(args)

    import torch
    from vic_b200 import kernels
    from vic_b200.core_types import KIMI
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        from vic_b200 import ep
        return ep.bench_main(args)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    sh = KIMI
    model = build_synthetic_moe(sh, PHYS_LAYERS, dev, seed=SEED, slot_seed=99)
    dec = MoeDecoder(model, exact_order=True)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    xs = synth_activation(sh, gen, dev, torch.bfloat16, N_TOKENS)
    outs = torch.zeros(N_TOKENS, sh.hidden, dtype=torch.float32, device=dev)

    def step(i):
        dec.forward_layer(i % PHYS_LAYERS, xs[i % N_TOKENS], out=outs[i % N_TOKENS])

    K, W = args.steps, args.warmup
    stream = torch.cuda.Stream(device=dev)
    K = max(1, K)
    chunk = 64 if K >= 64 else K * (64 // K)   # whole groups of K steps, about 64 per graph whatever --steps is
    # ── value: device-resident inputs, graph replay, CUDA events on the launching stream ──
    timer = GraphTimer(stream, step, chunk, warm=W)
    assert int(dec.status.item()) == 0, "device status word set"
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_step, replays, timed_steps = timer.time(max(K, MIN_TIMED_STEPS))
    clocks = sampler.stop()
    value = 1e3 / ms_step

    with torch.cuda.stream(stream):
        # ── roofline: each kernel alone (graph of 32 launches over rotating layers and tokens) ──
        n_k = 32
        ids_all = torch.zeros(n_k, 16, dtype=torch.int16, device=dev)   # routing differs per launch: pre-route
        w_all = torch.zeros(n_k, 16, dtype=torch.float32, device=dev)
        for i in range(n_k):
            dec.route(i % PHYS_LAYERS, xs[i])
            ids_all[i].copy_(dec.ids)
            w_all[i].copy_(dec.weights)
        stream.synchronize()

    def phase_launch(i, phase):
        i %= n_k
        kernels.moe_layer_int4_paged(xs[i], dec.tables[i % PHYS_LAYERS], sh.num_experts, dec.shared_tables[i % PHYS_LAYERS],
                                     ids_all[i], w_all[i], sh.top_k, 1.0, dec.act, dec.out, False, sh.hidden,
                                     sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page,
                                     sh.down.rows_per_page, dec.status, phase=phase)

    def time_kernel(fn):
        us, _, _ = GraphTimer(stream, fn, n_k).time(50 * n_k, 20.0)
        return us * 1e3

    k_us = time_kernel(lambda i: phase_launch(i, 1))
    down_us = time_kernel(lambda i: phase_launch(i, 2))
    redo0 = int(dec.workspace[1].item())
    router_us = time_kernel(lambda i: dec.route(i % PHYS_LAYERS, xs[i % N_TOKENS]))
    redo_total = int(dec.workspace[1].item())

    # ── e2e: host buffers every step, one call per token through the library's host-to-host entry point
    # (MoeDecoder.bind_host_step -> vib3_moe_step_run: the token from host memory in, one graph launch — copy in,
    # router, the two expert kernels, the fp32 output stored into pinned host memory — and the wait for it) ──
    x_host = [xs[i].cpu().pin_memory() for i in range(N_TOKENS)]
    x_ptrs = [t.data_ptr() for t in x_host]
    bound = [dec.bind_host_step(l, x_host[0].dtype, stream) for l in range(PHYS_LAYERS)]   # what a serving loop keeps per layer
    checksum = 0.0
    e2e_steps = max(K, 2 * MIN_TIMED_STEPS)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for i in range(max(W, 32)):   # (the first host-driven steps after the long device-only phase run slower)
            bound[i % PHYS_LAYERS].run(x_ptrs[i % N_TOKENS])
        e0.record(stream)
        for i in range(e2e_steps):
            step = bound[i % PHYS_LAYERS]
            step.run(x_ptrs[i % N_TOKENS])      # vib3_moe_step_run(handle, host pointer, stream)
            checksum += float(step.out_np[0])   # the host reads the result
        e1.record(stream)
        stream.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    assert int(dec.status.item()) == 0 and math.isfinite(checksum)

    b_gu, b_dn, b_r = algorithmic_bytes(sh)
    peak, peak_kind = measured_peaks()
    achieved = b_gu / (k_us * 1e-6) / 1e9
    layer_gbs = (b_gu + b_dn + b_r) / (ms_step * 1e-3) / 1e9
    traffic = profile_figure("gate_up_dram_bytes_per_launch")

    cfg = workload_config(1)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": cfg,
        "timed": {"steps": timed_steps, "graph_steps": chunk, "replays": replays, "physical_layers": PHYS_LAYERS,
                  "distinct_tokens": N_TOKENS},
        "layer_hbm_gbs": layer_gbs, "layer_frac_of_peak": layer_gbs / peak, "layer_bytes": b_gu + b_dn + b_r,
        "roofline": {"bound": "hbm", "kernel": "moe_gateup_pipe_kernel (gate/up + SiLU, 9 experts)", "achieved": achieved,
                     "peak": peak, "peak_source": f"of {peak_kind} (hbm_gbs, burst: the kernel is timed alone)", "unit": "GB/s",
                     "frac": achieved / peak, "bytes_per_launch": b_gu, "us_per_launch": k_us,
                     "traffic": traffic, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu-captured launch of the same shape"},
        "e2e": {"value": 1e3 / e2e_ms, "unit": UNIT, "h2d_bytes_per_step": sh.hidden * 2, "d2h_bytes_per_step": sh.hidden * 4,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "api": "vib3_moe_step_run"},
        "kernel_us": {"router": router_us, "gate_up": k_us, "down": down_us,
                      "router_frac_of_peak": b_r / (router_us * 1e-6) / 1e9 / peak, "down_frac_of_peak": b_dn / (down_us * 1e-6) / 1e9 / peak,
                      "note": "each kernel alone, back to back in a CUDA graph over rotating layers/tokens"},
        "gpu_launches": dec.launches_per_layer * timed_steps,
        "clocks": clocks,
        "router_recomputations": redo_total,
        "router_recomputation_share_in_kernel_timing": (redo_total - redo0) / float(3 + n_k * (1 + math.ceil(50 * n_k / n_k))),
    }

    if not args.no_extras:
        t_extra = time.time()
        try:
            line["ref_gpu"] = bench_ref_gpu(model, xs, dev)
        except Exception as exc:  # noqa: BLE001
            line["ref_gpu"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        try:
            from vic_b200 import grouped
            line["c3"] = grouped.bench_c3(model, stream, measured_peaks()[0])
            line["c4"] = grouped.bench_c4_single(model, stream, measured_peaks()[0], STACK_LAYERS)
        except ImportError:
            pass
        del timer
        line["c0"] = None
        free_model = time.time() - t_extra < 120
        if free_model:
            del dec, model
            torch.cuda.empty_cache()
            try:
                line["c0"] = bench_c0(dev, stream)
            except Exception as exc:  # noqa: BLE001
                line["c0"] = {"unavailable": f"{type(exc).__name__}: {exc}"}

    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg()
    print(json.dumps(line))


if __name__ == "__main__":
    main()
