"""The fused MoE sublayer (router -> gate/up+SiLU -> down+accumulate over a device page table)
against the CPU oracle's restatement of the reference engine's call chain, against the per-page
call sequence, and against the reference's own CUDA kernels driven in that sequence."""
import numpy as np
import pytest
import torch

from tests.parity import assert_close, load_ref_lib, oracle_experts, ref_moe_sublayer

pytestmark = pytest.mark.gpu


def _shapes():
    from vic_b200.core_types import KIMI, MIXTRAL, SCORING_SIGMOID, SCORING_SOFTMAX, MoeShape
    tiny = MoeShape("tiny", 64, 96, 4, 2, 1, SCORING_SOFTMAX, 1.0, True)
    # several ragged pages per segment at small size: gate/up 3640+360 rows, down 932+92 rows
    mid = MoeShape("mid", 1024, 4000, 6, 3, 1, SCORING_SIGMOID, 2.5, True)
    noshared = MoeShape("noshared", 256, 512, 8, 2, 0, SCORING_SOFTMAX, 1.0, True)
    return {"tiny": tiny, "mid": mid, "noshared": noshared, "kimi": KIMI, "mixtral": MIXTRAL}


_cache = {}


def _model(name, dev, seed=1234, slot_seed=99):
    from vic_b200.synth import build_synthetic_moe
    key = (name, seed, slot_seed)
    if key not in _cache:
        _cache.clear()  # one big model resident at a time
        torch.cuda.empty_cache()
        _cache[key] = build_synthetic_moe(_shapes()[name], 1, dev, seed=seed, slot_seed=slot_seed)
    return _cache[key]


@pytest.mark.parametrize("name,xdt,ntok", [
    ("tiny", torch.float16, 4), ("tiny", torch.float32, 2), ("noshared", torch.bfloat16, 3),
    ("mid", torch.bfloat16, 3), ("mid", torch.float32, 2),
    ("mixtral", torch.float16, 2), ("kimi", torch.bfloat16, 3), ("kimi", torch.float32, 1),
])
def test_fused_layer_vs_oracle(cuda_dev, oracle, name, xdt, ntok):
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model(name, cuda_dev)
    sh = model.shape
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(1234 + ntok)
    xs = synth_activation(sh, g, cuda_dev, xdt, ntok)
    Wn = model.router_w[0].cpu().numpy()
    for t in range(ntok):
        out = dec.forward_layer(0, xs[t]).cpu().numpy()
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        ids, w = dec.routing()
        x32 = xs[t].float().cpu().numpy()
        oi, ow, _ = oracle.router(x32, Wn, sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize, None, oracle.ORDER_SEQUENTIAL)
        assert np.array_equal(ids, oi)
        assert np.allclose(w, ow, rtol=1e-4)
        want = oracle.moe_layer(x32, oracle_experts(oracle, model, 0, list(zip(oi.tolist(), ow.tolist()))), sh.hidden,
                                sh.intermediate, oracle.SCALE_FP16, order="gpu")
        assert_close(out, want, f"{name} {xdt} token {t}")
        assert np.all(np.isfinite(out))


@pytest.mark.parametrize("name,xdt", [("kimi", torch.bfloat16), ("kimi", torch.float32), ("mixtral", torch.float16)])
def test_staged_kernels_equal_direct_kernels_bit_for_bit(cuda_dev, name, xdt):
    """The bulk-copy staged kernels and the direct-load kernels share their arithmetic: same bits (experts wider
    than 2048: same bits for gate/up, agreement to rounding for down, whose staged form splits K across warps)."""
    from vic_b200.lib import lib
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model(name, cuda_dev)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(77)
    xs = synth_activation(model.shape, g, cuda_dev, xdt, 3)
    try:
        for t in range(3):
            lib().vib3_config_set(0, 1)
            a = dec.forward_layer(0, xs[t]).clone()
            act_a = dec.act.clone()
            lib().vib3_config_set(0, 0)
            b = dec.forward_layer(0, xs[t]).clone()
            torch.cuda.synchronize()
            assert int(dec.status.item()) == 0
            assert torch.equal(act_a, dec.act)
            if model.shape.intermediate <= 2048:
                assert torch.equal(a, b)
            else:
                # wide experts: the staged down kernel splits K across warps (another fp32 association)
                assert float((a - b).abs().max()) <= 2e-3 * max(1.0, float(b.abs().max()))
    finally:
        lib().vib3_config_set(0, 1)


def test_host_to_host_step_equals_device_step(cuda_dev):
    """forward_host (one CUDA graph: copy in, three launches, copy out) returns the same bits as the
    device-resident call, for pinned and ordinary host tensors, several tokens in a row."""
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model("mid", cuda_dev)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(6)
    xs = synth_activation(model.shape, g, cuda_dev, torch.bfloat16, 4)
    side = torch.cuda.Stream()
    for t in range(4):
        want = dec.forward_layer(0, xs[t]).clone().cpu()
        xh = xs[t].cpu()
        if t % 2:
            xh = xh.pin_memory()
        got = dec.forward_host(0, xh)
        assert got.is_pinned() and torch.equal(got, want)
        got2 = dec.forward_host_call(0, xh)      # the single C call with host pointers
        assert got2.is_pinned() and torch.equal(got2, want)
        got3 = dec.forward_host_bound(0, xh, side)   # the layer bound once as a graph inside the library
        assert got3.is_pinned() and torch.equal(got3, want)
    assert int(dec.status.item()) == 0


def test_accumulate_into_residual(cuda_dev):
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model("mid", cuda_dev)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(5)
    x = synth_activation(model.shape, g, cuda_dev, torch.bfloat16, 1)[0]
    base = dec.forward_layer(0, x).clone()
    resid = torch.randn(model.shape.hidden, device=cuda_dev, dtype=torch.float32)
    want = resid + base
    dec.forward_layer(0, x, out=resid, accumulate=True)
    assert torch.equal(resid, want)


def test_norm_with_early_dependents_and_holding_router_equal_the_plain_chain(cuda_dev):
    """A stack of norm -> router -> experts launches in a CUDA graph: with the norm letting the router start early and
    the router holding the expert kernels back until the token is complete, the hidden state after twelve layers
    equals, bit for bit, that of the chain without either flag (both on the batch-1 and on the grouped path)."""
    from vic_b200 import kernels as K
    from vic_b200.grouped import GroupedDecoder
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model("kimi", cuda_dev)
    sh = model.shape
    L, depth, T = model.n_layers, 12, 4
    g = torch.Generator(device=cuda_dev).manual_seed(21)
    attn = (torch.randn(depth, T, sh.hidden, generator=g, device=cuda_dev) * 0.3).to(torch.bfloat16)
    norm_w = (1.0 + 0.1 * torch.randn(depth, sh.hidden, generator=g, device=cuda_dev)).to(torch.float16)
    h0 = synth_activation(sh, g, cuda_dev, torch.float32, T)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        dec, gd = MoeDecoder(model), GroupedDecoder(model, max_tokens=T)
        for batch in (1, T):
            h = torch.zeros(batch, sh.hidden, dtype=torch.float32, device=cuda_dev)
            x = torch.zeros(batch, sh.hidden, dtype=torch.bfloat16, device=cuda_dev)

            def stack(early):   # (nothing between the layers: the norm follows the previous layer's last kernel)
                h.copy_(h0[:batch])
                for l in range(depth):
                    K.residual_rms_norm(h, attn[l, :batch], norm_w[l], 1e-6, x, center=True, early_dependents=early)
                    if batch == 1:
                        dec.forward_layer(l % L, x[0], out=h[0], accumulate=True, hold=early)
                    else:
                        gd.forward(l % L, x, out=h, accumulate=True, hold=early)
            got = {}
            for early in (False, True):
                stack(early)
                stream.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=stream):
                    stack(early)
                for _ in range(3):
                    gr.replay()
                stream.synchronize()
                got[early] = h.clone()
            assert torch.isfinite(got[False]).all()
            assert torch.equal(got[False], got[True])
        assert int(dec.status.item()) == 0 and int(gd.status.item()) == 0
        gd.close()


def test_paged_equals_contiguous_bit_for_bit(cuda_dev):
    """Same page contents, different slots: scattered pool vs back-to-back pool give identical bits."""
    from vic_b200.buffer_manager import PageBufferManager
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import SyntheticMoe, synth_activation
    for name in ("mid", "kimi"):
        model = _model(name, cuda_dev)
        sh = model.shape
        dec = MoeDecoder(model)
        g = torch.Generator(device=cuda_dev).manual_seed(8)
        xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, 2)
        outs, routes = [], []
        for t in range(2):
            outs.append(dec.forward_layer(0, xs[t]).clone())
            routes.append(dec.routing()[0].tolist())
        needed = sorted(set(sum(routes, []))) + [0xFFFF]
        pages = [p for p in model.pages if p.pid.expert in needed]
        for slot_seed in (0, 4242):
            pool2 = PageBufferManager(len(pages), device=cuda_dev, slot_seed=slot_seed)
            for p in pages:
                s2 = pool2.load_page(p.pid, p.row_start, p.row_count, None, p.nbytes)
                pool2.slot_view(s2, p.nbytes).copy_(model.pool.slot_view(p.slot, p.nbytes))
            pool2.freeze()
            m2 = SyntheticMoe(sh, 1, pool2, model.router_w, pages)
            dec2 = MoeDecoder(m2)
            for t in range(2):
                o2 = dec2.forward_layer(0, xs[t])
                assert int(dec2.status.item()) == 0
                assert torch.equal(o2, outs[t]), f"{name} slot_seed={slot_seed} token {t}"


def test_missing_page_sets_status_and_does_not_fault(cuda_dev):
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    sh = _shapes()["noshared"]
    model = build_synthetic_moe(sh, 1, cuda_dev, seed=3, slot_seed=5, experts=[0, 1, 2])  # experts 3..7 absent
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(2)
    hit_missing = False
    for t in range(12):
        x = synth_activation(sh, g, cuda_dev, torch.bfloat16, 1)[0]
        dec.status.zero_()
        out = dec.forward_layer(0, x)
        torch.cuda.synchronize()
        ids = dec.routing()[0]
        assert torch.isfinite(out).all()
        if any(int(e) > 2 for e in ids):
            hit_missing = True
            assert int(dec.status.item()) & 1
        else:
            assert int(dec.status.item()) == 0
    assert hit_missing
    # the host planner reports the same condition as an error before any launch
    from vic_b200.buffer_manager import QueryPlanner
    from vic_b200.lib import Vib3Error
    with pytest.raises(Vib3Error):
        QueryPlanner(model.pool, sh.pages_per_segment).plan_layer(0, [(5, 1.0)])


def test_fused_vs_per_page_sequence_and_reference_kernels(cuda_dev, oracle):
    from vic_b200.buffer_manager import QueryPlanner
    from vic_b200.moe import MoeDecoder, run_moe_sublayer_paged_calls
    from vic_b200.synth import synth_activation
    ref = load_ref_lib()
    for name in ("mid", "kimi"):
        model = _model(name, cuda_dev)
        sh = model.shape
        dec = MoeDecoder(model, exact_order=False)
        planner = QueryPlanner(model.pool, sh.pages_per_segment)
        g = torch.Generator(device=cuda_dev).manual_seed(31)
        x = synth_activation(sh, g, cuda_dev, torch.bfloat16, 1)[0]
        x32 = x.float()
        w16 = model.router_w[0].to(torch.float16)
        seq_out, activation, launches = run_moe_sublayer_paged_calls(model, 0, x32, planner, w16)
        # drive the fused experts with the same routing
        k = sh.top_k
        dec.ids[:k] = torch.tensor([e for e, _ in activation], dtype=torch.int32).to(torch.int16).to(cuda_dev)
        dec.weights[:k] = torch.tensor([w for _, w in activation], dtype=torch.float32, device=cuda_dev)
        fused = dec.experts(0, x).clone()
        torch.cuda.synchronize()
        assert_close(fused.cpu().numpy(), seq_out.cpu().numpy(), f"{name}: fused vs per-page sequence")
        per_expert = 3 * sh.gate_up.num_pages + sh.down.num_pages + 1
        assert launches == 2 + (k + sh.shared_experts) * per_expert
        if ref is not None:
            ref_out, ref_launches = ref_moe_sublayer(ref, model, 0, x32, activation, planner)
            torch.cuda.synchronize()
            assert_close(fused.cpu().numpy(), ref_out.cpu().numpy(), f"{name}: fused vs reference kernels")
            assert_close(seq_out.cpu().numpy(), ref_out.cpu().numpy(), f"{name}: per-page vs reference kernels")


def test_device_side_slot_count_and_local_selection(cuda_dev, oracle):
    """vib3_launch_select_local_experts keeps a rank's experts in order; the `_var` launcher over the
    kept slots equals the plain launcher given the same experts explicitly (bit for bit)."""
    from vic_b200 import kernels
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model("kimi", cuda_dev)
    sh = model.shape
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(41)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, 3)
    ids_loc = torch.zeros(16, dtype=torch.int16, device=cuda_dev)
    w_loc = torch.zeros(16, dtype=torch.float32, device=cuda_dev)
    n_loc = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    out_var = torch.zeros(sh.hidden, dtype=torch.float32, device=cuda_dev)
    out_ref = torch.zeros(sh.hidden, dtype=torch.float32, device=cuda_dev)
    for t, (lo, hi, shared) in enumerate([(0, 192, True), (192, 384, False), (380, 384, False)] * 2):
        if t >= 3:   # second round: ranges that leave exactly one or two slots
            dec.route(0, xs[t % 3])
            one = int(dec.routing()[0][t % 3 + 1])
            lo, hi, shared = one, one + 1, (t == 5)
        dec.route(0, xs[t % 3])
        ids, ws = dec.routing()
        kernels.select_local_experts(dec.ids, dec.weights, sh.top_k, lo, hi, ids_loc, w_loc, n_loc)
        torch.cuda.synchronize()
        keep = [(int(e), float(w)) for e, w in zip(ids, ws) if lo <= int(e) < hi]
        n = int(n_loc.item())
        assert n == len(keep)
        assert ids_loc[:n].cpu().numpy().view(np.uint16).tolist() == [e for e, _ in keep]
        assert w_loc[:n].cpu().tolist() == [w for _, w in keep]
        sp = dec.shared_tables[0] if shared else 0
        kernels.moe_layer_int4_paged_var(xs[t % 3], dec.tables[0], sh.num_experts, sp, ids_loc, w_loc, sh.top_k, 1.0, dec.act,
                                         out_var, False, sh.hidden, sh.intermediate, sh.pages_per_segment,
                                         sh.gate_up.rows_per_page, sh.down.rows_per_page, n_loc, dec.status)
        if n + (1 if shared else 0) > 0:
            kernels.moe_layer_int4_paged(xs[t % 3], dec.tables[0], sh.num_experts, sp, ids_loc, w_loc, n, 1.0, dec.act, out_ref,
                                         False, sh.hidden, sh.intermediate, sh.pages_per_segment,
                                         sh.gate_up.rows_per_page, sh.down.rows_per_page, dec.status) if n > 0 or shared else None
        else:
            out_ref.zero_()
        torch.cuda.synchronize()
        assert int(dec.status.item()) == 0
        assert torch.equal(out_var, out_ref), (t, n)
        if t >= 3:   # one or two slots: check against the oracle as well
            ex = oracle_experts(oracle, model, 0, keep)
            if not shared:
                ex = ex[:len(keep)]
            want = oracle.moe_layer(xs[t % 3].float().cpu().numpy(), ex, sh.hidden, sh.intermediate, oracle.SCALE_FP16, "gpu")
            assert_close(out_var.cpu().numpy(), want, f"{n} routed slot(s), shared={shared}")


@pytest.mark.parametrize("name,T,lo_hi", [("grp", 3, (4, 12)), ("grp", 6, (0, 16)), ("kimi", 4, (96, 288)), ("kimi", 8, (0, 48))])
def test_grouped_pairs_equal_per_token_launches_bit_for_bit(cuda_dev, name, T, lo_hi):
    """The grouped launch (pairs of several tokens, as an expert-parallel rank sees them) writes, for
    every token, the same bits as that token's own launch over its local experts; also with more than 9
    slots (one warp per slot in the down kernel) and more than 16 pairs (a second, accumulating launch)."""
    from vic_b200 import kernels
    from vic_b200.core_types import KIMI, SCORING_SIGMOID, X_BF16, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    if name == "grp":
        sh = MoeShape("grp", 1024, 1024, 16, 4, 1, SCORING_SIGMOID, 2.5, True)
        _cache.clear()
        model = build_synthetic_moe(sh, 1, cuda_dev, seed=21, slot_seed=5)
    else:
        model = _model("kimi", cuda_dev)
        sh = model.shape
    dec = MoeDecoder(model)
    lo, hi = lo_hi
    g = torch.Generator(device=cuda_dev).manual_seed(90 + T)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, T)          # [T, H] contiguous: stride 2H bytes
    ids_all = torch.zeros(T, 16, dtype=torch.int16, device=cuda_dev)
    w_all = torch.zeros(T, 16, dtype=torch.float32, device=cuda_dev)
    for t in range(T):
        dec.route(0, xs[t])
        ids_all[t].copy_(dec.ids)
        w_all[t].copy_(dec.weights)
    shared_token = T // 2
    # per-token launches over the local experts
    want = torch.zeros(T, sh.hidden, dtype=torch.float32, device=cuda_dev)
    ids_loc = torch.zeros(16, dtype=torch.int16, device=cuda_dev)
    w_loc = torch.zeros(16, dtype=torch.float32, device=cuda_dev)
    n_loc = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    total = 0
    for t in range(T):
        kernels.select_local_experts(ids_all[t], w_all[t], sh.top_k, lo, hi, ids_loc, w_loc, n_loc)
        kernels.moe_layer_int4_paged_var(xs[t], dec.tables[0], sh.num_experts, dec.shared_tables[0] if t == shared_token else 0,
                                         ids_loc, w_loc, sh.top_k, 1.0, dec.act, want[t], False, sh.hidden, sh.intermediate,
                                         sh.pages_per_segment, sh.gate_up.rows_per_page, sh.down.rows_per_page, n_loc, dec.status)
        torch.cuda.synchronize()
        total += int(n_loc.item())
    # grouped
    cap = T * sh.top_k
    pe = torch.zeros(cap, dtype=torch.int16, device=cuda_dev)
    pw = torch.zeros(cap, dtype=torch.float32, device=cuda_dev)
    pt = torch.zeros(cap, dtype=torch.int16, device=cuda_dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    kernels.select_local_pairs(ids_all, 32, w_all, 64, T, sh.top_k, lo, hi, pe, pw, pt, cap, cnt)
    torch.cuda.synchronize()
    assert int(cnt.item()) == total
    toks = pt[:total].cpu().tolist()
    assert toks == sorted(toks)
    act = torch.zeros(17 * sh.intermediate, dtype=torch.float16, device=cuda_dev)
    got = torch.full((T, sh.hidden), 7.0, dtype=torch.float32, device=cuda_dev)
    for j in range((cap + 15) // 16):
        kernels.moe_layer_int4_paged_grouped(xs, X_BF16, sh.hidden * 2, T, dec.tables[0], sh.num_experts,
                                             dec.shared_tables[0] if j == 0 else 0, shared_token, pe, pw, pt, 16, 16 * j, cnt, 1.0,
                                             act, got, sh.hidden, j > 0, sh.hidden, sh.intermediate, sh.pages_per_segment,
                                             sh.gate_up.rows_per_page, sh.down.rows_per_page, dec.status)
    torch.cuda.synchronize()
    assert int(dec.status.item()) == 0
    assert torch.equal(got, want), (name, T, total)


def test_sum_rows_and_pair_list_overflow(cuda_dev):
    """Helpers of the expert-parallel step: the row sum adds in row order (bit-exact against the same
    additions in torch); the pair selection reports the full count even when the lists are too short."""
    from vic_b200 import kernels
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    rows = torch.randn(5, 1000, generator=g, device=cuda_dev)[:, :996]      # stride 1000, 996 columns
    out = torch.zeros(996, device=cuda_dev)
    kernels.sum_rows_f32(rows, out)
    want = rows[0].clone()
    for r in range(1, 5):
        want = want + rows[r]
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    ids = torch.arange(32, dtype=torch.int16, device=cuda_dev).view(4, 8).contiguous()
    ws = torch.arange(32, dtype=torch.float32, device=cuda_dev).view(4, 8).contiguous()
    pe = torch.full((6,), -1, dtype=torch.int16, device=cuda_dev)
    pw = torch.zeros(6, dtype=torch.float32, device=cuda_dev)
    pt = torch.zeros(6, dtype=torch.int16, device=cuda_dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    kernels.select_local_pairs(ids, 16, ws, 32, 4, 8, 4, 28, pe, pw, pt, 6, cnt)   # experts 4..27 are local: 24 pairs
    torch.cuda.synchronize()
    assert int(cnt.item()) == 24
    assert pe.cpu().tolist() == [4, 5, 6, 7, 8, 9] and pt.cpu().tolist() == [0, 0, 0, 0, 1, 1]
    assert pw.cpu().tolist() == [4.0, 5.0, 6.0, 7.0, 8.0, 9.0]


def test_fused_launcher_refusals(cuda_dev):
    from vic_b200.lib import lib
    L = lib()
    t = torch.zeros(4096, dtype=torch.float32, device=cuda_dev)
    p = t.data_ptr()
    ok = dict(x=p, xd=2, tab=p, E=8, sh=None, ids=p, w=p, k=2, sw=1.0, act=p, out=p, acc=0, H=256, I=512, P=1, rg=512, rd=256, g=32, st=None, s=None)
    def call(**kw):
        a = {**ok, **kw}
        return L.vib3_launch_moe_layer_int4_paged(a["x"], a["xd"], a["tab"], a["E"], a["sh"], a["ids"], a["w"], a["k"], a["sw"], a["act"],
                                                  a["out"], a["acc"], a["H"], a["I"], a["P"], a["rg"], a["rd"], a["g"], a["st"], a["s"])
    assert call(x=None) == -3 and call(tab=None) == -3 and call(out=None) == -3 and call(act=None) == -3
    assert call(g=128) == -1 and call(xd=7) == -1
    assert call(H=250) == -5 and call(I=0) == -5
    assert call(k=17) == -2 and call(k=0) == -2 and call(P=17) == -2 and call(E=0) == -2
    assert call(rg=100) == -5            # pages cannot cover the matrix: row range out of [0, M)
    assert call(tab=p + 8) == -4 and call(x=p + 4) == -4
    torch.cuda.synchronize()


@pytest.mark.parametrize("name,xdt", [("kimi", torch.bfloat16), ("mid", torch.float32)])
def test_routing_inside_the_gate_up_kernel_equals_separate_router(cuda_dev, name, xdt):
    """Library option 2: the gate/up kernel streams the router's rows and selects in its prologue.  Same
    arithmetic as the router kernel: identical routing and identical layer output."""
    from vic_b200.lib import lib
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    from vic_b200.synth import build_synthetic_moe
    if name == "kimi":
        model = _model("kimi", cuda_dev)
    else:
        model = build_synthetic_moe(MoeShape("routed-mid", 1024, 2048, 40, 4, 1, SCORING_SIGMOID, 2.5, True), 1, cuda_dev, seed=5, slot_seed=2)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(78)
    xs = synth_activation(model.shape, g, cuda_dev, xdt, 6)
    try:
        for t in range(6):
            lib().vib3_config_set(2, 0)
            a = dec.forward_layer(0, xs[t]).clone()
            ids_a, w_a = dec.routing()
            lib().vib3_config_set(2, 1)
            b = dec.forward_layer(0, xs[t]).clone()
            b2 = dec.forward_layer(0, xs[t]).clone()     # back to back: the grid-wide counter was reset
            torch.cuda.synchronize()
            ids_b, w_b = dec.routing()
            assert int(dec.status.item()) == 0
            assert int(dec.workspace[0].item()) == 0 and int(dec.workspace[2].item()) == 0
            assert np.array_equal(ids_a, ids_b) and np.array_equal(w_a, w_b)
            assert torch.equal(a, b) and torch.equal(a, b2)
    finally:
        lib().vib3_config_set(2, 0)


def test_back_to_back_layers_on_one_scratch_without_a_router(cuda_dev, oracle):
    """Two launch pairs in a row that share the activation scratch, small hidden size (fewer CTAs than SMs, so
    the second gate/up kernel finds free SMs while the first down kernel still runs) and a shared expert, whose
    rows the gate/up kernel writes before its dependency wait: the down kernel lets its successor go only after
    every consumer warp has read the scratch."""
    from vic_b200 import kernels
    from vic_b200.core_types import SCORING_SIGMOID, MoeShape
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import build_synthetic_moe, synth_activation
    sh = MoeShape("b2b", 512, 1024, 6, 2, 1, SCORING_SIGMOID, 2.0, True)
    model = build_synthetic_moe(sh, 1, cuda_dev, seed=31, slot_seed=4)
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(9)
    xs = synth_activation(sh, g, cuda_dev, torch.bfloat16, 8)
    routes = []
    for t in range(8):
        dec.route(0, xs[t])
        torch.cuda.synchronize()
        routes.append((dec.ids.clone(), dec.weights.clone()))
    outs = torch.zeros(8, sh.hidden, dtype=torch.float32, device=cuda_dev)
    for rep in range(20):
        for t in range(8):      # no router in between: gate/up follows down directly
            kernels.moe_layer_int4_paged(xs[t], dec.tables[0], sh.num_experts, dec.shared_tables[0], routes[t][0], routes[t][1],
                                         sh.top_k, 1.0, dec.act, outs[t], False, sh.hidden, sh.intermediate, sh.pages_per_segment,
                                         sh.gate_up.rows_per_page, sh.down.rows_per_page, dec.status)
        torch.cuda.synchronize()
        if rep == 0:
            first = outs.clone()
        assert torch.equal(outs, first)
    assert int(dec.status.item()) == 0
    x32 = xs.float().cpu().numpy()
    for t in (0, 7):
        ids = routes[t][0][:sh.top_k].cpu().numpy().view(np.uint16)
        ws = routes[t][1][:sh.top_k].cpu().numpy()
        want = oracle.moe_layer(x32[t], oracle_experts(oracle, model, 0, list(zip(ids.tolist(), ws.tolist()))), sh.hidden,
                                sh.intermediate, oracle.SCALE_FP16, "gpu")
        assert_close(first[t].cpu().numpy(), want, f"back-to-back token {t}")


def test_activation_outliers_stay_inside_the_tolerance(cuda_dev, oracle):
    """The staged kernels hold each 32-column chunk of the activation vector as 16-bit fixed point against the
    chunk's largest magnitude.  Worst case for that: every chunk carries one value 100x larger than the rest, so
    the small values keep only 9-10 significant bits.  The layer output must still meet the layer tolerance."""
    from vic_b200.moe import MoeDecoder
    from vic_b200.synth import synth_activation
    model = _model("kimi", cuda_dev)
    sh = model.shape
    dec = MoeDecoder(model)
    g = torch.Generator(device=cuda_dev).manual_seed(41)
    for t in range(2):
        x = synth_activation(sh, g, cuda_dev, torch.float32, 1)[0]
        x.view(-1, 32)[:, (3 + 7 * t) % 32] *= 100.0
        x = x.to(torch.bfloat16)
        out = dec.forward_layer(0, x).cpu().numpy()
        torch.cuda.synchronize()
        ids, w = dec.routing()
        x32 = x.float().cpu().numpy()
        oi, ow, _ = oracle.router(x32, model.router_w[0].cpu().numpy(), sh.top_k, sh.scoring, sh.scaling_factor, sh.normalize)
        assert np.array_equal(ids, oi)
        want = oracle.moe_layer(x32, oracle_experts(oracle, model, 0, list(zip(oi.tolist(), ow.tolist()))), sh.hidden, sh.intermediate,
                                oracle.SCALE_FP16, "gpu")
        # max-abs scales with the output magnitude here (outputs are ~100x larger than for N(0,1) tokens)
        scale = max(1.0, float(np.abs(want).max()) / 2.5)
        assert_close(out, want, f"outlier token {t}", max_abs_tol=2e-2 * scale)
