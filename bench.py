#!/usr/bin/env python
"""Benchmark of the vib3 INT4 MoE decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE.json configs[1] — one Kimi-K2.5-shape MoE layer, batch-1 decode:
hidden 7168, 384 routed experts top-8 (sigmoid, renormalised, x2.827) + 1 shared expert,
intermediate 2048, INT4 group-32 weights in 2 MiB pages scattered in a VRAM pool, bf16
activations, fp32 router weights.  A step is one token through one such layer (router ->
gate/up+SiLU -> down+accumulate).  Four physical layers (38.8 GB of pages) are used in rotation
and every step has its own token, so no weight byte is re-read before 4 x 234 MB of other
traffic went through the 126 MB L2.  Data is seeded synthetic (no checkpoint, no dataset).

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM (CUDA-graph
replay, CUDA events); `e2e` = the same through host buffers (MoeDecoder.forward_host: pinned H2D of
the token and the three launches as one CUDA graph, the fp32 layer output written by the last kernel
straight into pinned host memory, one stream synchronisation, every step); `roofline` = the dominant kernel (gate/up) timed alone with CUDA
events against the measured HBM copy bandwidth; `cpu_baseline` = the CPU restatement of the
reference's kernels (oracle/) on this host's cores over a bounded sample.
"""
from __future__ import annotations

import argparse
import json
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
PHYS_LAYERS = 4
N_TOKENS = 64
SEED = 1234 + 1  # configs[1]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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


def cpu_reference_layer_tokens(model, xs_host, routes, n_tokens, budget_s=25.0):
    """Time the CPU restatement of the reference's kernels (router + engine-order expert chain) on
    host copies of the pages a token touches.  Returns (tokens_per_s, threads, tokens_timed)."""
    from oracle import oracle as O
    from tests.parity import oracle_experts
    sh = model.shape
    Wn = [model.router_w[l].float().cpu().numpy() for l in range(model.n_layers)]
    done, t_total = 0, 0.0
    for t in range(n_tokens):
        ids, ws, layer = routes[t]
        experts = oracle_experts(O, model, layer, list(zip(ids, ws)))  # host copies, untimed
        x32 = xs_host[t]
        t0 = time.perf_counter()
        O.router(x32, Wn[layer], sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        O.moe_layer(x32, experts, sh.hidden, sh.intermediate, O.SCALE_FP16, "gpu")
        t_total += time.perf_counter() - t0
        done += 1
        if t_total > budget_s:
            break
    threads = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return done / t_total, threads, done


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path.  The Rust crate cannot be
    built here (no cargo), so this times the C restatement of its CPU kernels (oracle/, kind
    "port") with all host threads, on the same config and metric.  Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch
    from vic_b200.core_types import KIMI, MoeShape
    from vic_b200.synth import build_synthetic_moe
    from oracle import oracle as O
    O.build()
    sh = KIMI
    # Host-only: the pages a token touches are generated directly in host memory (same
    # distributions), 9 experts' worth; routing comes from the oracle router.
    g = torch.Generator(device="cpu").manual_seed(SEED)
    sub = MoeShape(sh.name, sh.hidden, sh.intermediate, sh.top_k, sh.top_k, 1, sh.scoring, sh.scaling_factor, sh.normalize)
    model = build_synthetic_moe(sub, 1, "cpu", seed=SEED, slot_seed=99)
    W = (torch.randn(sh.num_experts, sh.hidden, generator=g) * 0.02).numpy()
    from tests.parity import oracle_experts
    experts = oracle_experts(O, model, 0, [(e, 1.0 / sh.top_k) for e in range(sh.top_k)])
    xs = torch.randn(8, sh.hidden, generator=g).to(torch.bfloat16).float().numpy()

    def step(i):
        x = xs[i % 8]
        ids, ws, _ = O.router(x, W, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        for ex, w in zip(experts[:sh.top_k], ws.tolist()):
            ex.weight = w
        return O.moe_layer(x, experts, sh.hidden, sh.intermediate, O.SCALE_FP16, "gpu")

    for i in range(max(args.warmup, 1)):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(i)
    dt = time.perf_counter() - t0
    threads = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    val = args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4 weights x f32 activations, f32 accumulate (CPU)", "data": "synthetic",
        "config": {"workload": "C1 kimi-k2.5-shape single MoE layer, batch-1 decode, CPU kernels", "hidden": sh.hidden,
                   "experts": sh.num_experts, "top_k": sh.top_k, "shared_experts": 1, "intermediate": sh.intermediate},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} full layer-tokens (router + 8 routed + 1 shared expert), CPU restatement of the reference's Rust kernels; the Rust crate itself needs cargo, which this image lacks"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def profile_small(n, router_only=False):
    import torch
    from vic_b200.core_types import KIMI, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    dev = torch.device("cuda:0")
    if router_only:
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
    sh = MoeShape("kimi16", KIMI.hidden, KIMI.intermediate, 16, KIMI.top_k, 1, KIMI.scoring, KIMI.scaling_factor, True)
    model = build_synthetic_moe(sh, 2, dev, seed=SEED, slot_seed=99)
    dec = MoeDecoder(model, exact_order=False)
    if os.environ.get("VIB3_BENCH_DIRECT") == "1":   # A/B: direct-load kernels instead of the staged ones
        from vic_b200.lib import lib
        lib().vib3_config_set(0, 0)
    g = torch.Generator(device=dev).manual_seed(1)
    xs = synth_activation(sh, g, dev, torch.bfloat16, 8)
    for i in range(n):
        dec.forward_layer(i % 2, xs[i % 8])
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    print(json.dumps({"profile_small": n, "status": 0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-small", type=int, default=0, metavar="N",
                    help="run N untimed layer-steps of a 16-expert Kimi-shape layer (same per-launch work as the full "
                         "workload: 8 routed + 1 shared expert, 223 MB of weights per step, 0.8 GB resident) and exit; "
                         "this is the command the ncu captures under profiles/ run")
    ap.add_argument("--profile-router", type=int, default=0, metavar="N",
                    help="run N untimed launches of the full-width (384-expert) router and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_small:
        profile_small(args.profile_small)
        return
    if args.profile_router:
        profile_small(args.profile_router, router_only=True)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200  # ~0.1-0.3 s per CPU layer-token: keep the arm within a few minutes
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    from vic_b200 import kernels
    from vic_b200.core_types import KIMI
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        from vic_b200 import ep
        ep.bench_main(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    sh = KIMI
    model = build_synthetic_moe(sh, PHYS_LAYERS, dev, seed=SEED, slot_seed=99)
    dec = MoeDecoder(model, exact_order=True)
    if os.environ.get("VIB3_BENCH_ROUTER_SMEM_KB"):   # A/B: shared memory the gate/up kernel leaves to a co-resident router CTA
        from vic_b200.lib import lib as _l
        _l().vib3_config_set(3, int(os.environ["VIB3_BENCH_ROUTER_SMEM_KB"]))
    gen = torch.Generator(device=dev).manual_seed(SEED)
    xs = synth_activation(sh, gen, dev, torch.bfloat16, N_TOKENS)
    outs = torch.zeros(N_TOKENS, sh.hidden, dtype=torch.float32, device=dev)

    def step(i):
        dec.forward_layer(i % PHYS_LAYERS, xs[i % N_TOKENS], out=outs[i % N_TOKENS])

    K, W = args.steps, args.warmup
    stream = torch.cuda.Stream(device=dev)
    chunk = min(K, 64)
    with torch.cuda.stream(stream):
        for i in range(W):
            step(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(chunk):
                step(i)
        graph.replay()
        stream.synchronize()
        assert int(dec.status.item()) == 0, "device status word set"

        # ── value: device-resident inputs, graph replay, CUDA events on the launching stream ──
        sampler = ClockSampler(local_rank)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(K // chunk):
            graph.replay()
        for i in range(K % chunk):
            step(i)
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        value = K / (ms * 1e-3)

        # ── roofline: the dominant kernel (gate/up + SiLU) alone ──
        for i in range(4):
            dec.route(i % PHYS_LAYERS, xs[i])
        n_k = 32
        # routing differs per launch: pre-route into separate id/weight buffers
        ids_all = torch.zeros(n_k, 16, dtype=torch.int16, device=dev)
        w_all = torch.zeros(n_k, 16, dtype=torch.float32, device=dev)
        for i in range(n_k):
            dec.route(i % PHYS_LAYERS, xs[i])
            ids_all[i].copy_(dec.ids)
            w_all[i].copy_(dec.weights)
        stream.synchronize()

        def phase_launch(i, phase):
            kernels.moe_layer_int4_paged(xs[i], dec.tables[i % PHYS_LAYERS], sh.num_experts, dec.shared_tables[i % PHYS_LAYERS],
                                         ids_all[i], w_all[i], sh.top_k, 1.0, dec.act, dec.out, False, sh.hidden,
                                         sh.intermediate, sh.pages_per_segment, sh.gate_up.rows_per_page,
                                         sh.down.rows_per_page, dec.status, phase=phase)

        def time_kernel(fn):
            """Average duration of one launch: CUDA graph of n_k launches (rotating layers and tokens),
            CUDA events on the launching stream around `reps` replays."""
            for i in range(3):
                fn(i)
            stream.synchronize()
            gk = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gk, stream=stream):
                for i in range(n_k):
                    fn(i)
            gk.replay()
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                gk.replay()
            e1.record(stream)
            stream.synchronize()
            return e0.elapsed_time(e1) * 1e3 / (reps * n_k)

        reps = 8
        k_us = time_kernel(lambda i: phase_launch(i, 1))
        down_us = time_kernel(lambda i: phase_launch(i, 2))
        redo0 = int(dec.workspace[1].item())
        router_us = time_kernel(lambda i: dec.route(i % PHYS_LAYERS, xs[i]))
        # share of the timed router launches that recomputed near-tied logits in sequential order
        router_redo_share = (int(dec.workspace[1].item()) - redo0) / float(3 + n_k * (reps + 1))

        variants = {}
        if os.environ.get("VIB3_BENCH_VARIANTS") == "1":   # A/B of library options in one process
            from vic_b200.lib import lib as _lib
            for v in (3, 0):
                _lib().vib3_config_set(2, v)
                variants[f"router_variant_{v}"] = time_kernel(lambda i: dec.route(i % PHYS_LAYERS, xs[i]))
            w16 = [model.router_w[l].to(torch.float16) for l in range(PHYS_LAYERS)]
            x32 = xs.float()
            sc = torch.zeros(sh.num_experts, dtype=torch.float32, device=dev)
            variants["router_gemv_only_f16w"] = time_kernel(lambda i: kernels.router_gemv_f32(x32[i], w16[i % PHYS_LAYERS], sc, sh.hidden, sh.num_experts))
            dec.exact_order = False
            variants["router_no_exact"] = time_kernel(lambda i: dec.route(i % PHYS_LAYERS, xs[i]))
            dec.exact_order = True
            _lib().vib3_config_set(1, 0)
            variants["gate_up_no_pdl"] = time_kernel(lambda i: phase_launch(i, 1))
            variants["down_no_pdl"] = time_kernel(lambda i: phase_launch(i, 2))
            _lib().vib3_config_set(1, 1)
            _lib().vib3_config_set(0, 0)
            variants["gate_up_direct"] = time_kernel(lambda i: phase_launch(i, 1))
            variants["down_direct"] = time_kernel(lambda i: phase_launch(i, 2))
            _lib().vib3_config_set(0, 1)

        # ── e2e: host buffers every step, through the public host-to-host call (one CUDA graph per
        # layer: copy in from pinned memory, router, gate/up, down storing into pinned host memory; one
        # synchronisation).  The single C call vib3_moe_layer_step_host does the same without a graph
        # and measures about 4 us slower per token. ──
        x_host = [xs[i].cpu().pin_memory() for i in range(N_TOKENS)]
        checksum = 0.0

        def e2e_step(i):
            return dec.forward_host(i % PHYS_LAYERS, x_host[i % N_TOKENS], stream)
        for i in range(max(W, PHYS_LAYERS)):
            e2e_step(i)
        e0.record(stream)
        for i in range(K):
            checksum += float(e2e_step(i)[0])   # the host reads the step's result
        e1.record(stream)
        stream.synchronize()
        e2e_ms = e0.elapsed_time(e1)
        e2e_value = K / (e2e_ms * 1e-3)
        assert int(dec.status.item()) == 0

    b_gu, b_dn, b_r = algorithmic_bytes(sh)
    peak, peak_kind = measured_peaks()
    achieved = b_gu / (k_us * 1e-6) / 1e9
    layer_gbs = (b_gu + b_dn + b_r) / (ms * 1e-3 / K) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights, 16-bit fixed-point activations, int32/fp32 accumulate", "data": "synthetic",
        "config": {"workload": "C1 kimi-k2.5-shape single MoE layer, batch-1 decode over paged INT4 experts",
                   "hidden": sh.hidden, "experts": sh.num_experts, "top_k": sh.top_k, "shared_experts": sh.shared_experts,
                   "intermediate": sh.intermediate, "activations": "bf16", "router_weights": "fp32", "page_bytes": 2 << 20,
                   "physical_layers": PHYS_LAYERS, "l2_policy": "inputs larger than L2: 4 layers x 234 MB rotate, 64 distinct tokens",
                   "parallelism": "single GPU"},
        "layer_hbm_gbs": layer_gbs, "layer_frac_of_peak": layer_gbs / peak,
        "roofline": {"bound": "hbm", "kernel": "moe_gateup_pipe_kernel (gate/up + SiLU, 9 experts)", "achieved": achieved,
                     "peak": peak, "peak_source": f"of {peak_kind} (MEASURED_PEAKS.json hbm_gbs, burst)", "unit": "GB/s",
                     "frac": achieved / peak, "bytes_per_launch": b_gu, "us_per_launch": k_us,
                     "traffic": 153.06e6, "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of the same shape (profiles/moe_gateup_down_kimi_batch1.md)"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": sh.hidden * 2, "d2h_bytes_per_step": sh.hidden * 4,
                "ms_per_step": e2e_ms / K},
        "kernel_us": {"router": router_us, "gate_up": k_us, "down": down_us,
                      "note": "each kernel alone, back to back in a CUDA graph over rotating layers/tokens"},
        "variants_us": variants,
        "gpu_launches": dec.launches_per_layer * K,
        "clocks": clocks,
        "router_recomputations": int(dec.workspace[1].item()),
        "router_recomputation_share_in_kernel_timing": router_redo_share,
    }

    if not args.no_cpu_baseline:
        routes = []
        n_cpu = 12
        for t in range(n_cpu):
            dec.route(t % PHYS_LAYERS, xs[t])
            torch.cuda.synchronize()
            ids, ws = dec.routing()
            routes.append((ids.tolist(), ws.tolist(), t % PHYS_LAYERS))
        xs_host32 = [xs[t].float().cpu().numpy() for t in range(n_cpu)]
        tps, threads, done = cpu_reference_layer_tokens(model, xs_host32, routes, n_cpu)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{done} layer-tokens of the same workload (router + 8 routed + 1 shared expert) through the CPU restatement of the reference's kernels"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
