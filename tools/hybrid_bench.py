#!/usr/bin/env python
"""Prefill and decode throughput of the hybrid decoder family beside the Qwen2 engine at equal width / depth / ff /
heads (random weights), and the new kernels alone against their rooflines.  One JSON line.

    python tools/hybrid_bench.py [--sizes w2048,w4096] [--prompt 4096] [--context 2048] [--batch 32] [--steps 20]

End to end: `prefill` = one prompt through EngineCore.run_prefill (chunks of 1024 rows), `decode` = token steps of
`batch` sequences that hold `context` tokens each (CUDA graph + sampler + state advance), both timed with CUDA events.
Kernels: each launched alone on the engine's buffers at the same shapes, L2 flushed between timed launches; the
memory-bound ones against the measured copy bandwidth, the sequential scans against the fp32 FMA rate of the SMs.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

SIZES = {
    # width, layers, ff, heads, kv_heads, vocab
    "w1024": dict(width=1024, layers=8, ff=4096, heads=8, kv=2, vocab=32768),
    "w2048": dict(width=2048, layers=8, ff=8192, heads=16, kv=4, vocab=32768),
    "w4096": dict(width=4096, layers=8, ff=14336, heads=32, kv=8, vocab=32768),
}


def hybrid_config(s):
    """Alternating GLA / (attention + state-space) layers, every one with a feed-forward: the same width, depth, ff,
    attention heads (size 128) and vocabulary as the Qwen2 model it is compared with."""
    W = s["width"]
    gla = dict(type="gla", mixer=dict(heads=W // 256, dim=128, vdim=256, tau=16.0, rank=64),
               mlp=dict(kind="dense", ff=s["ff"], limit=7.0))
    par = dict(type="parallel",
               mixer=dict(left=dict(heads=s["heads"], kv_heads=s["kv"], dim=128, vdim=128, rot=dict(dims=64, base=1e6), scale=128 ** -0.5),
                          right=dict(heads=W // 64, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                          left_scale=1.0, right_scale=1.0),
               mlp=dict(kind="dense", ff=s["ff"], limit=7.0))
    return dict(architecture="Povurax", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), embedding=dict(scale=1.0),
                layers=[gla if i % 2 == 0 else par for i in range(s["layers"])])


def belelorn_config(s):
    """Six layers of which the first two run twice (eight layer runs, the depth of the models beside it): attention
    (windowed, values = keys, head size 128) beside lightning attention alternating with matrix-memory LSTM layers,
    squared-ReLU feed-forwards of the same ff alternating with routed ones of the same active width (two of sixteen
    experts of ff / 4 each plus a shared expert of ff / 2)."""
    W, ff = s["width"], s["ff"]
    par = dict(type="parallel",
               mixer=dict(left=dict(heads=s["heads"], kv_heads=s["kv"], dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                                    mask=dict(size=1024, keep_first=4)),
                          right=dict(heads=W // 128, dim=128, vdim=128,
                                     decay=[1.0 - 2.0 ** -(3 + 6 * h / max(1, W // 128 - 1)) for h in range(W // 128)])))
    cell = dict(type="mlstm", mixer=dict(heads=W // 256, dim=128, vdim=256, gate_cap=15.0))
    dense = dict(kind="dense", ff=ff)
    routed = dict(kind="moe", router=dict(experts=16, top=2), expert=dict(ff=ff // 4, limit=7.0), shared=dict(ff=ff // 2, limit=7.0))
    layers = []
    for i in range(s["layers"] - 2):
        layers.append(dict(par if i % 2 == 0 else cell, mlp=dense if i % 2 == 0 else routed))
    return dict(architecture="Belelorn", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), logit_scale=1.0, layers=layers,
                loop=dict(start=0, stop=2, times=2))


def pametar_config(s):
    """Six layers of which the first two run twice (eight layer runs, the depth of the models beside it): latent attention
    (head size 128 + 64 rotated channels, latent of 256, query latent of 3/8 width) alternating with a delta-rule memory
    (heads of 64), every layer with routed experts of the same active width as the dense ff (four of sixteen experts of
    ff / 4), four residual streams, a token-pair table."""
    W, ff = s["width"], s["ff"]
    att = dict(type="latent_attention",
               mixer=dict(heads=s["heads"], dim=128, rot_dim=64, vdim=128, kv_rank=256, q_rank=3 * W // 8,
                          rot=dict(dims=64, base=1e4), scale=192 ** -0.5))
    mem = dict(type="general_delta", mixer=dict(heads=W // 64, dim=64, rank=64))
    routed = dict(kind="moe", router=dict(experts=16, top=4, scale=1.0), expert=dict(ff=ff // 4))
    layers = [dict(att if i % 2 == 0 else mem, mlp=routed) for i in range(s["layers"] - 2)]
    return dict(architecture="Pametar", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), streams=4,
                embedding=dict(scale=1.0, bigram=dict(buckets=65521, mul_prev=131, mul_cur=17)), layers=layers,
                loop=dict(start=0, stop=2, times=2))


def kolotar_config(s):
    """Eight layers, (windowed attention, windowed attention, latent attention, attention without a softmax beside the
    gated delta rule) twice: attention heads of 128 with 64 rotated channels and a window of 1024, a latent of 256 with 64
    rotated channels, delta-rule heads of 128 x 128 on half as many q / k heads, every layer with routed experts of the
    same active width as the dense ff (four of sixteen experts of ff / 4)."""
    W, ff, H, G = s["width"], s["ff"], s["heads"], s["kv"]
    routed = dict(kind="moe", router=dict(experts=16, top=4), expert=dict(ff=ff // 4))
    att = dict(type="attention", mlp=routed,
               mixer=dict(heads=H, kv_heads=G, dim=128, vdim=128, mask=dict(size=1024), scale=128 ** -0.5, v_mix=True,
                          rot=dict(base=1e6, dims=64, scaling=dict(factor=4.0, original=2048, fast=32.0, slow=1.0))))
    lat = dict(type="latent_attention", mlp=routed,
               mixer=dict(heads=H, dim=128, rot_dim=64, vdim=128, kv_rank=256, mask=dict(size=1024), rot=dict(dims=64, base=1e4),
                          scale=192 ** -0.5))
    par = dict(type="parallel", mlp=routed,
               mixer=dict(left=dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                                    q_temp=dict(coef=0.1, every=256)),
                          right=dict(heads=W // 128, kv_heads=max(1, W // 256), dim=128, vdim=128, conv=4),
                          left_scale=0.5, right_scale=0.5))
    return dict(architecture="Kolotar", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), postln_alpha=2.0,
                layers=[[att, att, lat, par][i % 4] for i in range(s["layers"])])


def peaks():
    try:
        p = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def events(self, fn, iters=10, warm=3, flush=True):
        for _ in range(warm):
            fn()
        total = 0.0
        for _ in range(iters):
            if flush:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters


def end_to_end(eng, vocab, prompt, context, batch, steps, warm):
    from pipelinerl_b200.engine import SamplingParams
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(8, vocab - 8, (n,), generator=g).tolist()  # noqa: E731
    sp = SamplingParams(max_tokens=2, greedy=True, ignore_eos=True)

    def drain():
        while eng.slot_req:
            eng.step()
            eng.harvest()
    eng.add_request(rnd(1100), sp)                      # warm-up: buffers, kernel attributes
    eng.run_prefill()
    drain()
    ms = []
    for _ in range(2):
        eng.add_request(rnd(prompt), sp)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.run_prefill()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
        drain()
    prefill_ms = min(ms)
    spd = SamplingParams(max_tokens=warm + steps + 4, greedy=False, temperature=1.0, ignore_eos=True)
    for _ in range(batch):
        eng.add_request(rnd(context), spd)
    eng.run_prefill()
    for _ in range(warm):
        eng.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        eng.step()
    b.record()
    torch.cuda.synchronize()
    step_ms = a.elapsed_time(b) / steps
    drain()
    return {"prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round((prompt - 1) / prefill_ms * 1e3),
            "decode_ms_per_step": round(step_ms, 3), "decode_tokens_per_s": round(batch / step_ms * 1e3)}


def kernel_table(eng, s, batch, chunk, timer):
    """The new kernels alone, at the decode shape (`batch` one-token segments) and the prefill shape (one segment of
    `chunk` rows), with the Qwen2 engine's closest row kernels on the same row counts."""
    import ctypes as C  # noqa: F401
    from pipelinerl_b200 import _lib
    from pipelinerl_b200.hybrid import _Rows
    lib, cfg = eng.lib, eng.cfg
    hbm, _, how = peaks()
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12          # fp32 FMA rate of the SMs at the maximum clock (nominal)
    W = cfg.width
    g = next(L.gla for L in cfg.layers if L.kind == "gla")
    par = next(L for L in cfg.layers if L.kind == "parallel")
    a, ss = par.attn, par.ssd
    gi = next(i for i, L in enumerate(cfg.layers) if L.kind == "gla")
    pi = next(i for i, L in enumerate(cfg.layers) if L.kind == "parallel")
    st = _lib.stream_ptr()
    out = {}
    i32 = dict(dtype=torch.int32, device=eng.dev)
    for shape, n, ns in (("decode", batch, batch), ("prefill", chunk, 1)):
        R = _Rows(eng, n, pieces=shape == "prefill")
        R.P.normal_(0, 0.5)
        R.aux.uniform_(0.9, 1.0)                           # decays (GLA) / convolved inputs (state-space)
        if shape == "decode":
            R.seg.copy_(torch.stack([torch.arange(n, **i32), torch.ones(n, **i32), torch.full((n,), 64, **i32), torch.arange(n, **i32)]))
            R.row_slot.copy_(torch.arange(n, **i32)); R.row_pos.fill_(64); R.row_back.zero_()
        else:
            R.seg[:, :1].copy_(torch.tensor([[0], [n], [0], [0]], **i32))
            R.row_slot.zero_(); R.row_pos.copy_(torch.arange(n, **i32)); R.row_back.copy_(torch.arange(n, **i32))
            step = eng.piece_tokens                            # the one segment as side-by-side pieces
            n_sub = (n + step - 1) // step
            R.sub[0, :n_sub].copy_(torch.arange(0, n, step, **i32))
            R.sub[1, :n_sub].copy_(torch.tensor([min(step, n - c) for c in range(0, n, step)], **i32))
            R.seg_sub[:, :1].copy_(torch.tensor([[0], [n_sub]], **i32))
            pieces = (R.seg_sub[0].data_ptr(), R.seg_sub[1].data_ptr(), R.sub[0].data_ptr(), R.sub[1].data_ptr(), n_sub,
                      R.scratch.data_ptr(), R.cdec.data_ptr())
        seg = [R.seg[k].data_ptr() for k in range(4)]
        vec = eng.vec
        nq, nv = g.heads * g.dim, g.heads * g.vdim
        ldg = 2 * nq + 2 * nv + g.rank
        w = f"l{cfg.layers[gi].weights_of}."

        def gla():
            _lib.check(lib.prl_gla_scan(R.P.data_ptr(), ldg, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                        g.vdim, seg[0], seg[1], seg[3], ns, eng.gla_state[gi].data_ptr(), R.o.data_ptr(), nv, st))
        ms = timer.events(gla)
        state_b = 2 * ns * g.heads * g.dim * g.vdim * 4
        io_b = n * (3 * nq + 2 * nv) * 4
        flops = 5.0 * n * g.heads * g.dim * g.vdim
        out[f"gla_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                        fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))
        if shape == "prefill":
            def gla_split():
                _lib.check(lib.prl_gla_scan_split(R.P.data_ptr(), ldg, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads,
                                                  g.dim, g.vdim, seg[3], ns, *pieces, eng.gla_state[gi].data_ptr(),
                                                  R.o.data_ptr(), nv, st))
            ms = timer.events(gla_split)
            out["gla_scan_split/prefill"] = dict(ms=round(ms, 4), hbm_frac=round((state_b * (1 + 2 * n_sub) + io_b) / ms / 1e6 / hbm, 3),
                                                 fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))
        wp = f"l{par.weights_of}."
        left = a.heads * a.dim + a.kv_heads * (a.dim + a.vdim) + a.heads * a.vdim
        ldp, inner, ch = left + ss.in_rows, ss.inner, ss.conv_channels

        def ssd():
            _lib.check(lib.prl_ssd_scan(R.P.data_ptr(), ldp, left + inner + ch, R.aux.data_ptr(), ch,
                                        vec[wp + "mix.right.dt_bias"].data_ptr(), vec[wp + "mix.right.A_log"].data_ptr(),
                                        vec[wp + "mix.right.D"].data_ptr(), ss.heads, ss.groups, ss.state, ss.vdim, seg[0], seg[1],
                                        seg[3], ns, eng.ssd_state[pi].data_ptr(), R.o2.data_ptr(), inner, st))
        ms = timer.events(ssd)
        state_b = 2 * ns * ss.heads * ss.state * ss.vdim * 4
        io_b = n * (2 * inner + 2 * ss.groups * ss.state) * 4
        flops = 5.0 * n * ss.heads * ss.state * ss.vdim
        out[f"ssd_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                        fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))

        if shape == "prefill":
            def ssd_split():
                _lib.check(lib.prl_ssd_scan_split(R.P.data_ptr(), ldp, left + inner + ch, R.aux.data_ptr(), ch,
                                                  vec[wp + "mix.right.dt_bias"].data_ptr(), vec[wp + "mix.right.A_log"].data_ptr(),
                                                  vec[wp + "mix.right.D"].data_ptr(), ss.heads, ss.groups, ss.state, ss.vdim,
                                                  seg[3], ns, *pieces, eng.ssd_state[pi].data_ptr(), R.o2.data_ptr(), inner, st))
            ms = timer.events(ssd_split)
            out["ssd_scan_split/prefill"] = dict(ms=round(ms, 4), hbm_frac=round((state_b * (1 + 2 * n_sub) + io_b) / ms / 1e6 / hbm, 3),
                                                 fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))

        def conv():
            _lib.check(lib.prl_conv_silu(R.P.data_ptr(), ldp, left + inner, n, ch, ss.conv, vec[wp + "mix.right.conv"].data_ptr(),
                                         vec[wp + "mix.right.conv.b"].data_ptr(), R.row_slot.data_ptr(), R.row_back.data_ptr(),
                                         eng.conv_state[pi].data_ptr(), R.aux.data_ptr(), st))
        ms = timer.events(conv)
        out[f"conv_silu/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * ch * 8 / ms / 1e6 / hbm, 3))

        def post():
            _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, 1, R.y1.data_ptr(), W, 1.0, 1, vec[wp + "norm1"].data_ptr(),
                                                 cfg.eps, n, W, R.x.data_ptr(), R.xa.data_ptr(), 0, st))
        ms = timer.events(post)
        out[f"postnorm_residual/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (4 * 4 + 2) / ms / 1e6 / hbm, 3))

        def gate():
            _lib.check(lib.prl_gate_norm(R.o2.data_ptr(), 1, inner, R.P.data_ptr() + 4 * left, ldp, vec[wp + "mix.right.norm"].data_ptr(),
                                         inner, inner // ss.norm_groups, n, inner, 0, 1, 1, cfg.eps, R.yb.data_ptr(), 0, st))
        ms = timer.events(gate)
        out[f"gate_norm/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * inner * (4 + 4 + 2) / ms / 1e6 / hbm, 3))
        F = par.mlp.ff

        def glu():
            _lib.check(lib.prl_glu_clamped(R.P.data_ptr(), 2 * F, n, F, par.mlp.limit, par.mlp.beta, R.act.data_ptr(), 0, st))
        if 2 * F <= R.P.numel() // n:
            ms = timer.events(glu)
            out[f"glu_clamped/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (8 + 2) / ms / 1e6 / hbm, 3))
        # the Qwen2 engine's row kernels on the same rows (their bytes: fp32 partial in, fp32 residual in/out, bf16 out)
        h = torch.zeros(n, W, dtype=torch.float32, device=eng.dev)
        xb = torch.zeros(n, W, dtype=torch.bfloat16, device=eng.dev)
        gam = torch.ones(W, dtype=torch.bfloat16, device=eng.dev)
        part = torch.randn(n, 2 * F, dtype=torch.float32, device=eng.dev)
        actb = torch.zeros(n, F, dtype=torch.bfloat16, device=eng.dev)

        def qres():
            _lib.check(lib.prl_residual_rmsnorm(part.data_ptr(), 1, n, W, gam.data_ptr(), 1e-6, h.data_ptr(), xb.data_ptr(), None, 0, st))
        ms = timer.events(qres)
        out[f"qwen2.residual_rmsnorm/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (3 * 4 + 2) / ms / 1e6 / hbm, 3))

        def qsilu():
            _lib.check(lib.prl_silu_mul(part.data_ptr(), 1, n, F, actb.data_ptr(), None, 0, st))
        ms = timer.events(qsilu)
        out[f"qwen2.silu_mul/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (8 + 2) / ms / 1e6 / hbm, 3))
        del R
    out["_denominators"] = {"hbm_gbs": hbm, "hbm": how, "fp32_fma_tflops_nominal": round(fma_tflops, 1)}
    return out


def kernel_table_belelorn(eng, s, batch, chunk, timer):
    """The kernels the Belelorn layers add, alone, at the decode shape (`batch` one-token segments at position 2047) and
    the prefill shape (one segment of `chunk` rows at the start of a sequence): memory-bound ones against the measured
    copy bandwidth, the recurrences and the CUDA-core products also against the SMs' fp32 FMA rate."""
    from pipelinerl_b200 import _lib
    from pipelinerl_b200.cache import PAGE_SIZE
    from pipelinerl_b200.hybrid import _Rows
    lib, cfg = eng.lib, eng.cfg
    hbm, _, how = peaks()
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12
    W = cfg.width
    pi = next(i for i, L in enumerate(cfg.layers) if L.kind == "parallel_lin")
    mi = next(i for i, L in enumerate(cfg.layers) if L.kind == "mlstm")
    par, cell = cfg.layers[pi], cfg.layers[mi]
    a, r, c = par.attn, par.lin, cell.mlstm
    e = cell.mlp.moe
    st = _lib.stream_ptr()
    out = {}
    i32 = dict(dtype=torch.int32, device=eng.dev)
    ctx = 2047
    pages_per = (ctx + PAGE_SIZE) // PAGE_SIZE
    for b in range(batch):
        eng.block_table[b, :pages_per].copy_(torch.arange(1 + b * pages_per, 1 + (b + 1) * pages_per, **i32))
    for shape, n, ns in (("decode", batch, batch), ("prefill", chunk, 1)):
        R = _Rows(eng, n, pieces=shape == "prefill")
        R.P.normal_(0, 0.5)
        if shape == "decode":
            R.seg.copy_(torch.stack([torch.arange(n, **i32), torch.ones(n, **i32), torch.full((n,), ctx, **i32), torch.arange(n, **i32)]))
            R.row_slot.copy_(torch.arange(n, **i32)); R.row_pos.fill_(ctx)
        else:
            R.seg[:, :1].copy_(torch.tensor([[0], [n], [0], [0]], **i32))
            R.row_slot.zero_(); R.row_pos.copy_(torch.arange(n, **i32))
            step = eng.piece_tokens
            n_sub = (n + step - 1) // step
            R.sub[0, :n_sub].copy_(torch.arange(0, n, step, **i32))
            R.sub[1, :n_sub].copy_(torch.tensor([min(step, n - k) for k in range(0, n, step)], **i32))
            R.seg_sub[:, :1].copy_(torch.tensor([[0], [n_sub]], **i32))
            pieces = (R.seg_sub[0].data_ptr(), R.seg_sub[1].data_ptr(), R.sub[0].data_ptr(), R.sub[1].data_ptr(), n_sub,
                      R.scratch.data_ptr(), R.cdec.data_ptr())
        seg = [R.seg[k].data_ptr() for k in range(4)]
        vec = eng.vec
        max_q = 1 if shape == "decode" else n
        # -- attention: front end and the windowed kernel
        nq, nk = a.heads * a.dim, a.kv_heads * a.dim
        rq, rv = r.heads * r.dim, r.heads * r.vdim
        ld = nq + nk + 2 * rq + 2 * rv
        wp = f"l{par.weights_of}."
        qb = vec[wp + "mix.left.b"].data_ptr()

        def front():
            _lib.check(lib.prl_qk_headnorm_cache(R.P.data_ptr(), ld, 0, nq, -1, n, a.heads, a.kv_heads, a.dim, a.vdim, qb, qb + 4 * nq,
                                                 None, None, cfg.eps, R.row_pos.data_ptr(), R.row_slot.data_ptr(),
                                                 eng.block_table.data_ptr(), eng.max_blocks, PAGE_SIZE, R.q.data_ptr(),
                                                 eng.k_pool[pi].data_ptr(), eng.v_pool[pi].data_ptr(), 0, st))
        ms = timer.events(front)
        out[f"qk_headnorm_cache/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * ((nq + nk) * 4 + (nq + 2 * nk) * 2) / ms / 1e6 / hbm, 3))

        def attn():
            _lib.check(lib.prl_attn_any_masked(R.q.data_ptr(), eng.k_pool[pi].data_ptr(), eng.v_pool[pi].data_ptr(), 0,
                                               eng.block_table.data_ptr(), eng.max_blocks, PAGE_SIZE, seg[0], seg[1], seg[2], seg[3],
                                               ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first,
                                               a.softcap, 1, R.ya.data_ptr(), st))
        ms = timer.events(attn)
        keys = (min(ctx + 1, a.window + a.keep_first) * n) if shape == "decode" else sum(min(t + 1, a.window + a.keep_first) for t in range(n))
        flops = 4.0 * keys * a.heads * a.dim
        kv_b = (ns * min(ctx + 1, a.window + a.keep_first) if shape == "decode" else n) * a.kv_heads * a.dim * 2 * 2
        out[f"attn_window/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((kv_b + n * nq * 4) / ms / 1e6 / hbm, 3),
                                           fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3), tflops=round(flops / ms / 1e9, 2))
        # -- lightning attention
        off = nq + nk
        head = (R.P.data_ptr(), ld, off, off + rq, 1.0, R.P.data_ptr(), ld, off + 2 * rq, None, 0, 0, eng.lin_decay[pi].data_ptr(),
                r.heads, r.dim, r.vdim)

        def silu():
            _lib.check(lib.prl_act_cols(R.P.data_ptr(), ld, off, n, 2 * rq + rv, 0, st))
        ms = timer.events(silu)
        out[f"act_cols/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * (2 * rq + rv) * 8 / ms / 1e6 / hbm, 3))

        def lin():
            _lib.check(lib.prl_decay_scan(*head, seg[0], seg[1], seg[3], ns, eng.lin_state[pi].data_ptr(), R.o2.data_ptr(), rv, st))
        ms = timer.events(lin)
        state_b, io_b = 2 * ns * r.heads * r.dim * r.vdim * 4, n * (2 * rq + 2 * rv) * 4
        flops = 5.0 * n * r.heads * r.dim * r.vdim
        out[f"lightning_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                              fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))
        if shape == "prefill":
            def lin_split():
                _lib.check(lib.prl_decay_scan_split(*head, seg[3], ns, *pieces, eng.lin_state[pi].data_ptr(), R.o2.data_ptr(), rv, st))
            ms = timer.events(lin_split)
            out["lightning_scan_split/prefill"] = dict(ms=round(ms, 4), fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))
        # -- matrix-memory LSTM
        H, mq, mv = c.heads, c.heads * c.dim, c.heads * c.vdim
        ldm = 2 * mq + 2 * mv + 2 * H
        wm = f"l{cell.weights_of}."
        gb = vec[wm + "mix.gate.b"].data_ptr()

        def gates():
            _lib.check(lib.prl_mlstm_gates(R.P.data_ptr(), ldm, 2 * mq + 2 * mv, 2 * mq + 2 * mv + H, gb, gb + 4 * H, c.gate_cap, H,
                                           seg[0], seg[1], seg[3], ns, eng.mlstm_m[mi].data_ptr(), R.gates.data_ptr(),
                                           R.minv.data_ptr(), st))
        out[f"mlstm_gates/{shape}"] = dict(ms=round(timer.events(gates), 4))

        def one():
            _lib.check(lib.prl_append_one(R.P.data_ptr(), ldm, 2 * mq, n, H, c.vdim, R.aux.data_ptr(), st))
        ms = timer.events(one)
        out[f"append_one/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * mv * 8 / ms / 1e6 / hbm, 3))
        dv = c.vdim + 1
        mhead = (R.P.data_ptr(), ldm, 0, mq, c.dim ** -0.5, R.aux.data_ptr(), H * dv, 0, R.gates.data_ptr(), 2 * H, 0, None, H, c.dim, dv)

        def cellscan():
            _lib.check(lib.prl_decay_scan(*mhead, seg[0], seg[1], seg[3], ns, eng.mlstm_state[mi].data_ptr(), R.o.data_ptr(), H * dv, st))
        ms = timer.events(cellscan)
        state_b, io_b = 2 * ns * H * c.dim * dv * 4, n * (2 * mq + 2 * H * dv) * 4
        flops = 5.0 * n * H * c.dim * dv
        out[f"mlstm_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                          fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))
        if shape == "prefill":
            def cell_split():
                _lib.check(lib.prl_decay_scan_split(*mhead, seg[3], ns, *pieces, eng.mlstm_state[mi].data_ptr(), R.o.data_ptr(), H * dv, st))
            ms = timer.events(cell_split)
            out["mlstm_scan_split/prefill"] = dict(ms=round(ms, 4), fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))

        def cellout():
            _lib.check(lib.prl_mlstm_out(R.o.data_ptr(), n, H, c.vdim, R.minv.data_ptr(), c.den_eps, R.P.data_ptr() + 4 * (2 * mq + mv),
                                         ldm, vec[wm + "mix.norm"].data_ptr(), cfg.eps, R.ya.data_ptr(), 0, st))
        ms = timer.events(cellout)
        out[f"mlstm_out/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * mv * (4 + 4 + 2) / ms / 1e6 / hbm, 3))
        # -- the closing kernel with both branches (the Qwen2 engine's residual + norm kernel is its counterpart)
        def close():
            eng._st = st
            eng._close(R, n, R.y0, 1, gain0=vec[wp + "mix.left.out"], s0=0.5, y1=R.y1, k1=1, gain1=vec[wp + "mix.right.out"], s1=0.5,
                       post_gain=vec[wp + "norm1b"], next_gain=vec[wp + "norm2"])
        ms = timer.events(close)
        out[f"sublayer_close/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (4 * 4 + 2) / ms / 1e6 / hbm, 3))
        # -- routed feed-forward
        eng._st = st
        R.xa.normal_(0, 1.0)

        def routed():
            eng._routed_ff(R, n, wm, e, cell.mlp.beta)
        ms = timer.events(routed)
        flops = 2.0 * n * e.top * 3 * e.ff * W
        wbytes = min(e.experts, n * e.top) * 3 * e.ff * W * 2
        out[f"routed_ff/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(wbytes / ms / 1e6 / hbm, 3), tflops=round(flops / ms / 1e9, 2),
                                         fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))
        F = par.mlp.ff

        def relu2():
            _lib.check(lib.prl_act_store(R.P.data_ptr(), F, n, F, 0, R.act.data_ptr(), 0, st))
        ms = timer.events(relu2)
        out[f"relu2/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (4 + 2) / ms / 1e6 / hbm, 3))
        h = torch.zeros(n, W, dtype=torch.float32, device=eng.dev)
        xb = torch.zeros(n, W, dtype=torch.bfloat16, device=eng.dev)
        gam = torch.ones(W, dtype=torch.bfloat16, device=eng.dev)
        part = torch.randn(n, 2 * F, dtype=torch.float32, device=eng.dev)
        actb = torch.zeros(n, F, dtype=torch.bfloat16, device=eng.dev)

        def qres():
            _lib.check(lib.prl_residual_rmsnorm(part.data_ptr(), 1, n, W, gam.data_ptr(), 1e-6, h.data_ptr(), xb.data_ptr(), None, 0, st))
        ms = timer.events(qres)
        out[f"qwen2.residual_rmsnorm/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (3 * 4 + 2) / ms / 1e6 / hbm, 3))

        def qsilu():
            _lib.check(lib.prl_silu_mul(part.data_ptr(), 1, n, F, actb.data_ptr(), None, 0, st))
        ms = timer.events(qsilu)
        out[f"qwen2.silu_mul/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (8 + 2) / ms / 1e6 / hbm, 3))
        del R
    eng.block_table.zero_()
    out["_denominators"] = {"hbm_gbs": hbm, "hbm": how, "fp32_fma_tflops_nominal": round(fma_tflops, 1)}
    return out


def run_belelorn(sizes, prompt, context, batch, steps, warm, kernels=True, e2e=True, others=True):
    """Belelorn beside the Povurax hybrid and the Qwen2 engine at equal width / depth / ff / attention heads."""
    from pipelinerl_b200.engine import DecodeEngine
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ModelConfig, ParamArena
    dev = torch.device("cuda:0")
    timer = Timer()
    res = {}
    for name in sizes:
        s = SIZES[name]
        kw = dict(max_batch=batch, max_seq_len=max(prompt, context) + 256, max_new_tokens=warm + steps + 8, device=dev,
                  prefill_chunk=1024)
        entry = {}
        if e2e and others:
            qcfg = ModelConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_layers=s["layers"],
                               num_q_heads=s["heads"], num_kv_heads=s["kv"])
            eng = DecodeEngine(qcfg, ParamArena(qcfg, dev).init_random(seed=1), **kw)
            entry["qwen2"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["qwen2"]["params_M"] = round(qcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
            hcfg = HybridConfig.from_povurax(hybrid_config(s))
            eng = HybridEngine(hcfg, ParamArena(hcfg, dev).init_random(seed=1), **kw)
            entry["povurax"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["povurax"]["params_M"] = round(hcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
        bcfg = HybridConfig.from_belelorn(belelorn_config(s))
        eng = HybridEngine(bcfg, ParamArena(bcfg, dev).init_random(seed=1), **kw)
        if e2e:
            entry["belelorn"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["belelorn"]["params_M"] = round(bcfg.num_params() / 1e6)
            for other in ("qwen2", "povurax"):
                if other in entry:
                    entry[f"belelorn_over_{other}"] = {k: round(entry["belelorn"][f"{k}_tokens_per_s"] / entry[other][f"{k}_tokens_per_s"], 3)
                                                       for k in ("prefill", "decode")}
        if kernels:
            entry["kernels"] = kernel_table_belelorn(eng, s, batch, 1024, timer)
        res[name] = entry
        del eng
        torch.cuda.empty_cache()
    return res


def run_pametar(sizes, prompt, context, batch, steps, warm, kernels=True, e2e=True, others=True):
    """Pametar beside Belelorn (the closest design: attention + recurrent mixers, routed experts, a repeated block) and
    the Qwen2 engine at equal width / depth / active ff / attention heads."""
    from pipelinerl_b200.engine import DecodeEngine
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ModelConfig, ParamArena
    dev = torch.device("cuda:0")
    timer = Timer()
    res = {}
    for name in sizes:
        s = SIZES[name]
        kw = dict(max_batch=batch, max_seq_len=max(prompt, context) + 256, max_new_tokens=warm + steps + 8, device=dev,
                  prefill_chunk=1024)
        entry = {}
        if e2e and others:
            qcfg = ModelConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_layers=s["layers"],
                               num_q_heads=s["heads"], num_kv_heads=s["kv"])
            eng = DecodeEngine(qcfg, ParamArena(qcfg, dev).init_random(seed=1), **kw)
            entry["qwen2"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["qwen2"]["params_M"] = round(qcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
            bcfg = HybridConfig.from_belelorn(belelorn_config(s))
            eng = HybridEngine(bcfg, ParamArena(bcfg, dev).init_random(seed=1), **kw)
            entry["belelorn"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["belelorn"]["params_M"] = round(bcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
        pcfg = HybridConfig.from_pametar(pametar_config(s))
        eng = HybridEngine(pcfg, ParamArena(pcfg, dev).init_random(seed=1), **kw)
        if e2e:
            entry["pametar"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["pametar"]["params_M"] = round(pcfg.num_params() / 1e6)
            for other in ("qwen2", "belelorn"):
                if other in entry:
                    entry[f"pametar_over_{other}"] = {k: round(entry["pametar"][f"{k}_tokens_per_s"] / entry[other][f"{k}_tokens_per_s"], 3)
                                                      for k in ("prefill", "decode")}
        if kernels:
            entry["kernels"] = kernel_table_pametar(eng, s, batch, 1024, timer)
        res[name] = entry
        del eng
        torch.cuda.empty_cache()
    return res


def run_kolotar(sizes, prompt, context, batch, steps, warm, kernels=True, e2e=True, others=True):
    """Kolotar beside Pametar (the closest design: latent attention, a delta-rule memory, routed experts in every layer)
    and the Qwen2 engine at equal width / depth / active ff / attention heads."""
    from pipelinerl_b200.engine import DecodeEngine
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ModelConfig, ParamArena
    dev = torch.device("cuda:0")
    timer = Timer()
    res = {}
    for name in sizes:
        s = SIZES[name]
        kw = dict(max_batch=batch, max_seq_len=max(prompt, context) + 256, max_new_tokens=warm + steps + 8, device=dev,
                  prefill_chunk=1024)
        entry = {}
        if e2e and others:
            qcfg = ModelConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_layers=s["layers"],
                               num_q_heads=s["heads"], num_kv_heads=s["kv"])
            eng = DecodeEngine(qcfg, ParamArena(qcfg, dev).init_random(seed=1), **kw)
            entry["qwen2"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["qwen2"]["params_M"] = round(qcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
            pcfg = HybridConfig.from_pametar(pametar_config(s))
            eng = HybridEngine(pcfg, ParamArena(pcfg, dev).init_random(seed=1), **kw)
            entry["pametar"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["pametar"]["params_M"] = round(pcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
        kcfg = HybridConfig.from_kolotar(kolotar_config(s))
        eng = HybridEngine(kcfg, ParamArena(kcfg, dev).init_random(seed=1), **kw)
        if e2e:
            entry["kolotar"] = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            entry["kolotar"]["params_M"] = round(kcfg.num_params() / 1e6)
            for other in ("qwen2", "pametar"):
                if other in entry:
                    entry[f"kolotar_over_{other}"] = {k: round(entry["kolotar"][f"{k}_tokens_per_s"] / entry[other][f"{k}_tokens_per_s"], 3)
                                                      for k in ("prefill", "decode")}
        if kernels:
            entry["kernels"] = kernel_table_kolotar(eng, s, batch, 1024, timer)
        res[name] = entry
        del eng
        torch.cuda.empty_cache()
    return res


def kernel_table_kolotar(eng, s, batch, chunk, timer):
    """The parts of the three Kolotar layer kinds alone, at the decode shape (`batch` one-token segments at position 2047)
    and the prefill shape (one segment of `chunk` rows whose sequence already holds `chunk` tokens): the engine's own
    mixer and feed-forward methods on its buffers, then single kernels; memory-bound ones against the measured copy
    bandwidth, attention products against the measured bf16 GEMM rate, the recurrence against the SMs' fp32 FMA rate."""
    from pipelinerl_b200 import _lib
    from pipelinerl_b200.cache import PAGE_SIZE
    from pipelinerl_b200.hybrid import _Rows
    lib, cfg = eng.lib, eng.cfg
    hbm, tflops, how = peaks()
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12
    W = cfg.width
    idx = {k: next(i for i, L in enumerate(cfg.layers) if L.kind == k) for k in ("attention", "latent_attention", "sigmoid_delta")}
    ai, ti, pi = idx["attention"], idx["latent_attention"], idx["sigmoid_delta"]
    LA, LT, LP = cfg.layers[ai], cfg.layers[ti], cfg.layers[pi]
    a, t_, left, g, e = LA.attn, LT.latent, LP.attn, LP.gdelta, LA.mlp.moe
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "fp32_fma_tflops": round(fma_tflops, 1), "source": how}}
    i32 = dict(dtype=torch.int32, device=eng.dev)
    ctx = 2047
    pages_per = (ctx + PAGE_SIZE) // PAGE_SIZE
    for b in range(batch):
        eng.block_table[b, :pages_per].copy_(torch.arange(1 + b * pages_per, 1 + (b + 1) * pages_per, **i32))
    for pools in (eng.lat_pool, eng.k_pool, eng.v_pool):
        for pool in pools.values():
            pool.normal_(0, 0.5)
    for shape, n, ns in (("decode", batch, batch), ("prefill", chunk, 1)):
        R = _Rows(eng, n)
        R.P.normal_(0, 0.5); R.xa.normal_(0, 0.5); R.x.normal_(0, 0.5); R.q.normal_(0, 0.5)
        pos0 = ctx if shape == "decode" else chunk
        if shape == "decode":
            R.seg.copy_(torch.stack([torch.arange(n, **i32), torch.ones(n, **i32), torch.full((n,), ctx, **i32), torch.arange(n, **i32)]))
            R.row_slot.copy_(torch.arange(n, **i32)); R.row_pos.fill_(ctx)
        else:
            R.seg[:, :1].copy_(torch.tensor([[0], [n], [pos0], [0]], **i32))
            R.row_slot.zero_(); R.row_pos.copy_(torch.arange(pos0, pos0 + n, **i32)); R.row_back.copy_(torch.arange(n, **i32))
        eng._st = _lib.stream_ptr()
        segs = (R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr(), ns)
        max_q = 1 if shape == "decode" else n
        wa, wt_, wp = f"l{LA.weights_of}.", f"l{LT.weights_of}.", f"l{LP.weights_of}."
        t = {}
        t["attention_mixer"] = timer.events(lambda: eng._window_attn_mixer(R, n, ai, LA, wa, segs, max_q, R.row_pos, R.seg[2]))
        t["latent_mixer"] = timer.events(lambda: eng._latent_direct_mixer(R, n, ti, LT, wt_, segs, max_q, R.row_pos, R.seg[2]))
        t["sigmoid_delta_mixer"] = timer.events(lambda: eng._sigmoid_delta_mixer(R, n, pi, LP, wp, segs, max_q, R.row_pos, R.seg[2]))
        t["routed_ff"] = timer.events(lambda: eng._routed_ff(R, n, wa, e, 1.0))
        t["postln_close"] = timer.events(lambda: eng._postln_close(R, n, wa, "1", R.y0, 1))
        bt, mb = eng.block_table.data_ptr(), eng.max_blocks

        def win_attn():
            _lib.check(lib.prl_attn_any_sink(R.q.data_ptr(), eng.k_pool[ai].data_ptr(), eng.v_pool[ai].data_ptr(), a.vdim, 0, bt, mb,
                                             PAGE_SIZE, *segs[:2], R.seg[2].data_ptr(), segs[2], ns, max_q, a.heads, a.kv_heads, a.dim,
                                             a.vdim, a.scale, a.window, 0, 0.0, eng.vec[wa + "mix.sink"].data_ptr(), 0, R.o.data_ptr(),
                                             eng._st))
        kd = t_.kv_rank + t_.rot_dim
        pool = eng.lat_pool[ti].data_ptr()

        def lat_attn():
            eng._latent_attention(R, ti, t_, segs, max_q, R.seg[2])

        def sig_attn():
            _lib.check(lib.prl_attn_sigmoid(R.q.data_ptr(), eng.k_pool[pi].data_ptr(), eng.v_pool[pi].data_ptr(), 0, bt, mb, PAGE_SIZE,
                                            *segs[:2], R.seg[2].data_ptr(), segs[2], ns, max_q, left.heads, left.kv_heads, left.dim,
                                            left.vdim, left.scale, left.softcap, left.q_temp[0], left.q_temp[1],
                                            eng.vec[wp + "mix.left.pb"].data_ptr(), eng.vec[wp + "mix.left.talk"].data_ptr(), 1,
                                            R.ya.data_ptr(), n, 1, eng.attn_ws.data_ptr(), eng.attn_ws.numel(), eng._st))
        gq, gv, ch = g.kv_heads * g.dim, g.heads * g.vdim, g.conv_channels
        nleft = left.heads * left.dim + left.kv_heads * (left.dim + left.vdim)
        ldp = nleft + g.in_rows

        def scan():
            _lib.check(lib.prl_gated_delta_scan(R.aux.data_ptr(), ch, 0, gq, 2 * gq, R.P.data_ptr(), ldp, nleft + ch, nleft + ch + g.heads,
                                                eng.vec[wp + "mix.right.A_log"].data_ptr(), eng.vec[wp + "mix.right.dt_bias"].data_ptr(),
                                                g.unit_eps, g.heads, g.kv_heads, g.dim, g.vdim, n, R.dprep.data_ptr(), *segs[:3], ns, max_q,
                                                eng.delta_state[pi].data_ptr(), R.o.data_ptr(), gv, eng._st))
        t["window_attention"] = timer.events(win_attn)
        t["latent_attention"] = timer.events(lat_attn)
        t["sigmoid_attention"] = timer.events(sig_attn, iters=3, warm=1)
        t["gated_delta_scan"] = timer.events(scan)
        row = {k: {"us": round(v * 1e3, 1)} for k, v in t.items()}
        # (query, key) pairs a row really sees
        seen_w = [min(a.window, p + 1) for p in (range(pos0, pos0 + n) if shape == "prefill" else [ctx] * n)]
        seen_t = [min(t_.window, p + 1) for p in (range(pos0, pos0 + n) if shape == "prefill" else [ctx] * n)]
        seen_all = [p + 1 for p in (range(pos0, pos0 + n) if shape == "prefill" else [ctx] * n)]
        fl = {"window_attention": 2.0 * sum(seen_w) * a.heads * (a.dim + a.vdim),
              "latent_attention": 2.0 * sum(seen_t) * t_.heads * (kd + t_.kv_rank),
              "sigmoid_attention": 2.0 * sum(seen_all) * left.heads * (left.dim + left.vdim + left.heads)}
        for k, f in fl.items():
            row[k]["tflops"] = round(f / t[k] / 1e9, 1)
            row[k]["of_bf16_peak"] = round(f / t[k] / 1e9 / tflops, 4)
        if shape == "decode":
            row["window_attention"]["of_hbm"] = round(sum(seen_w) * a.kv_heads * (a.dim + a.vdim) * 2 / t["window_attention"] / 1e6 / hbm, 3)
            row["latent_attention"]["of_hbm"] = round(sum(seen_t) * kd * 2 / t["latent_attention"] / 1e6 / hbm, 3)
            row["sigmoid_attention"]["of_hbm"] = round(sum(seen_all) * left.kv_heads * (left.dim + left.vdim) * 2 / t["sigmoid_attention"] / 1e6 / hbm, 3)
            row["gated_delta_scan"]["of_hbm"] = round(2 * n * g.heads * g.dim * g.vdim * 4 / t["gated_delta_scan"] / 1e6 / hbm, 3)
        else:
            row["gated_delta_scan"]["of_fp32_fma"] = round(n * g.heads * g.dim * g.vdim * 5 * 2 / t["gated_delta_scan"] / 1e9 / fma_tflops, 3)
        row["postln_close"]["of_hbm"] = round((n * W * 4 * 3 + n * W * 2) / t["postln_close"] / 1e6 / hbm, 3)
        out[shape] = row
        del R
    eng.block_table.zero_()
    eng.states.reset(0)
    return out


def kernel_table_pametar(eng, s, batch, chunk, timer):
    """The parts of a Pametar layer alone, at the decode shape (`batch` one-token segments at position 2047) and the
    prefill shape (one segment of `chunk` rows whose sequence already holds `chunk` tokens): the engine's own mixer and
    feed-forward methods on its buffers, then single kernels; memory-bound ones against the measured copy bandwidth, the
    attention product against the measured bf16 GEMM rate, the recurrence against the SMs' fp32 FMA rate."""
    from pipelinerl_b200 import _lib
    from pipelinerl_b200.cache import PAGE_SIZE
    from pipelinerl_b200.hybrid import _Rows
    lib, cfg = eng.lib, eng.cfg
    hbm, tflops, how = peaks()
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12
    W, S = cfg.width, cfg.streams
    ai = next(i for i, L in enumerate(cfg.layers) if L.kind == "latent")
    di = next(i for i, L in enumerate(cfg.layers) if L.kind == "delta")
    A, D = cfg.layers[ai], cfg.layers[di]
    a, c, e = A.latent, D.delta, A.mlp.moe
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "fp32_fma_tflops": round(fma_tflops, 1), "source": how}}
    i32 = dict(dtype=torch.int32, device=eng.dev)
    ctx = 2047
    pages_per = (ctx + PAGE_SIZE) // PAGE_SIZE
    for b in range(batch):
        eng.block_table[b, :pages_per].copy_(torch.arange(1 + b * pages_per, 1 + (b + 1) * pages_per, **i32))
    for pool in eng.lat_pool.values():
        pool.normal_(0, 0.5)
    for shape, n, ns in (("decode", batch, batch), ("prefill", chunk, 1)):
        R = _Rows(eng, n)
        R.P.normal_(0, 0.5); R.xa.normal_(0, 0.5); R.xs.normal_(0, 0.5)
        pos0 = ctx if shape == "decode" else chunk
        if shape == "decode":
            R.seg.copy_(torch.stack([torch.arange(n, **i32), torch.ones(n, **i32), torch.full((n,), ctx, **i32), torch.arange(n, **i32)]))
            R.row_slot.copy_(torch.arange(n, **i32)); R.row_pos.fill_(ctx)
        else:
            R.seg[:, :1].copy_(torch.tensor([[0], [n], [pos0], [0]], **i32))
            R.row_slot.zero_(); R.row_pos.copy_(torch.arange(pos0, pos0 + n, **i32)); R.row_back.copy_(torch.arange(n, **i32))
        R.tokens.copy_(torch.randint(0, cfg.vocab_size, (n,), device=eng.dev).int())
        eng._st = _lib.stream_ptr()
        segs = (R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr(), ns)
        max_q = 1 if shape == "decode" else n
        wa, wd = f"l{A.weights_of}.", f"l{D.weights_of}."
        keys = (ctx + 1) * n if shape == "decode" else n * pos0 + n * (n + 1) // 2      # (query, key) pairs
        kd = a.kv_rank + a.rot_dim
        t = {}
        t["latent_mixer"] = timer.events(lambda: eng._latent_mixer(R, n, ai, A, wa, segs, max_q, R.row_pos, R.seg[2]))
        t["delta_mixer"] = timer.events(lambda: eng._delta_mixer(R, n, di, D, wd, segs, max_q))
        t["routed_ff"] = timer.events(lambda: eng._routed_ff(R, n, wa, e, 1.0))
        t["stream_close"] = timer.events(lambda: eng._stream_close(R, n, ai, "1", R.y0, 1, R.P.data_ptr(), W))
        t["embed_pair"] = timer.events(lambda: eng._embed(R, n, R.tokens, R.row_pos, ns))
        pool = eng.lat_pool[ai].data_ptr()

        def attn():
            _lib.check(lib.prl_attn_latent(R.q.data_ptr(), pool, eng.block_table.data_ptr(), eng.max_blocks, PAGE_SIZE, *segs[:2],
                                           R.seg[2].data_ptr(), segs[2], ns, max_q, a.heads, kd, a.kv_rank, a.scale, 0,
                                           eng.vec[wa + "mix.sink"].data_ptr(), R.ya.data_ptr(), eng.attn_ws.data_ptr(),
                                           eng.attn_ws.numel(), eng._st))

        def attn_plain():
            _lib.check(lib.prl_attn_any_sink(R.q.data_ptr(), pool, pool, kd, 0, eng.block_table.data_ptr(), eng.max_blocks, PAGE_SIZE,
                                             *segs[:2], R.seg[2].data_ptr(), segs[2], ns, max_q, a.heads, 1, kd, a.kv_rank, a.scale, 0, 0,
                                             0.0, eng.vec[wa + "mix.sink"].data_ptr(), 1, R.ya.data_ptr(), eng._st))
        t["latent_attention"] = timer.events(attn)
        t["latent_attention_cuda_cores"] = timer.events(attn_plain, iters=3, warm=1)
        nq = c.heads * c.dim

        def scan():
            _lib.check(lib.prl_delta_scan(R.P.data_ptr(), 5 * nq + c.rank + W, 0, nq, 2 * nq, 4 * nq, R.aux.data_ptr(), nq,
                                          eng.vec[wd + "mix.w0"].data_ptr(), eng.vec[wd + "mix.a.b"].data_ptr(), c.decay_scale,
                                          c.unit_eps, c.heads, c.dim, c.dim, n, R.o2.data_ptr(), *segs[:3], ns, max_q, eng.delta_state[di].data_ptr(),
                                          R.o.data_ptr(), nq, eng._st))
        t["delta_scan"] = timer.events(scan)
        row = {k: {"us": round(v * 1e3, 1)} for k, v in t.items()}
        attn_flops = 2.0 * keys * a.heads * (kd + a.kv_rank)
        row["latent_attention"]["tflops"] = round(attn_flops / t["latent_attention"] / 1e9, 1)
        row["latent_attention"]["of_bf16_peak"] = round(attn_flops / t["latent_attention"] / 1e9 / tflops, 3)
        if shape == "decode":
            cache = n * (ctx + 1) * kd * 2
            row["latent_attention"]["of_hbm"] = round(cache / t["latent_attention"] / 1e6 / hbm, 3)
            state = 2 * n * c.heads * c.dim * c.dim * 4
            row["delta_scan"]["of_hbm"] = round(state / t["delta_scan"] / 1e6 / hbm, 3)
        else:
            row["delta_scan"]["of_fp32_fma"] = round(n * c.heads * c.dim * c.dim * 5 * 2 / t["delta_scan"] / 1e9 / fma_tflops, 3)
        stream_bytes = n * W * 4 * (2 * S + 2) + n * W * 2
        row["stream_close"]["of_hbm"] = round(stream_bytes / t["stream_close"] / 1e6 / hbm, 3)
        out[shape] = row
        del R
    eng.block_table.zero_()
    eng.states.reset(0)
    return out


def run(sizes, prompt, context, batch, steps, warm, kernels=True, e2e=True):
    from pipelinerl_b200.engine import DecodeEngine
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ModelConfig, ParamArena
    dev = torch.device("cuda:0")
    timer = Timer()
    res = {}
    for name in sizes:
        s = SIZES[name]
        kw = dict(max_batch=batch, max_seq_len=max(prompt, context) + 256, max_new_tokens=warm + steps + 8, device=dev,
                  prefill_chunk=1024)
        qcfg = ModelConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_layers=s["layers"],
                           num_q_heads=s["heads"], num_kv_heads=s["kv"])
        hcfg = HybridConfig.from_povurax(hybrid_config(s))
        entry = {}
        if e2e:
            eng = DecodeEngine(qcfg, ParamArena(qcfg, dev).init_random(seed=1), **kw)
            q = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            q["params_M"] = round(qcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
        eng = HybridEngine(hcfg, ParamArena(hcfg, dev).init_random(seed=1), **kw)
        if e2e:
            h = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            h["params_M"] = round(hcfg.num_params() / 1e6)
            entry = {"qwen2": q, "hybrid": h,
                     "hybrid_over_qwen2": {"prefill": round(h["prefill_tokens_per_s"] / q["prefill_tokens_per_s"], 3),
                                           "decode": round(h["decode_tokens_per_s"] / q["decode_tokens_per_s"], 3)}}
        if kernels:
            entry["kernels"] = kernel_table(eng, s, batch, 1024, timer)
        res[name] = entry
        del eng
        torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="w2048,w4096")
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--only-kernels", action="store_true", help="skip the end-to-end runs (a small case for a profiler)")
    ap.add_argument("--design", default="povurax", choices=["povurax", "belelorn", "pametar", "kolotar"], help="which hybrid design is measured")
    ap.add_argument("--alone", action="store_true", help="--design belelorn: skip the Qwen2 and Povurax runs beside it")
    a = ap.parse_args()
    from pipelinerl_b200 import _lib
    before = _lib.launch_count()
    if a.design == "kolotar":
        res = run_kolotar(a.sizes.split(","), a.prompt, a.context, a.batch, a.steps, a.warmup, kernels=not a.no_kernels,
                          e2e=not a.only_kernels, others=not a.alone)
    elif a.design == "pametar":
        res = run_pametar(a.sizes.split(","), a.prompt, a.context, a.batch, a.steps, a.warmup, kernels=not a.no_kernels,
                          e2e=not a.only_kernels, others=not a.alone)
    elif a.design == "belelorn":
        res = run_belelorn(a.sizes.split(","), a.prompt, a.context, a.batch, a.steps, a.warmup, kernels=not a.no_kernels,
                           e2e=not a.only_kernels, others=not a.alone)
    else:
        res = run(a.sizes.split(","), a.prompt, a.context, a.batch, a.steps, a.warmup, kernels=not a.no_kernels, e2e=not a.only_kernels)
    print(json.dumps({"bench": f"{a.design}_vs_qwen2", "dtype": "bf16", "data": "synthetic", "prompt": a.prompt,
                      "context": a.context, "batch": a.batch, "steps": a.steps, "warmup": a.warmup,
                      "gpu_launches": _lib.launch_count() - before, "sizes": res}), flush=True)


if __name__ == "__main__":
    main()
