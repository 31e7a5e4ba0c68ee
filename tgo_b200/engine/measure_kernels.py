"""Kernel by kernel: the kernels of the layers that norm their sublayers' outputs, mix the
heads' attention weights and carry a retention state, each timed alone beside the like kernel
of the plain pre-norm attention layer at equal sizes, with what each reaches of its roofline.

Timing: CUDA events around the replay of a CUDA graph that holds one call (one to three
launches), an L2 flush before each, the mean of `repeats` after three warm-up calls. Denominators: the
measured copy bandwidth and library bfloat16 product of this pool for memory- and tensor-bound
kernels; for the float32 recurrence, which no tensor-core mode computes in true 32 bits, the
float32 FMA rate of the device (multiprocessors x 128 lanes x 2 x the SM clock seen).
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..kernels import ops
from ..parts.attention import splits_for, step_tiles
from ..parts.attention_mixed import decode_ranges
from ..parts.base import StepContext
from ..parts.retention import step_chunks
from .measure import L2Flusher, load_peaks


def _timed(fn, flush, repeats: int = 5) -> float:
    """Mean milliseconds of fn() on the device, cold L2: fn is captured into a CUDA graph after
    three plain calls and the replays are timed, so that the host's share of a call that makes
    scratch tensors and launches two or three kernels does not count."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    graph.replay()
    times = []
    for _ in range(repeats):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sum(times) / len(times)


def _paged(requests: int, length: int, heads: int, width: int, page: int, dev):
    """A cache plane with `requests` requests of `length` keys, and its block tables."""
    per = -(-length // page)
    plane = torch.randn((requests * per + 1, heads, page, width), device=dev).to(torch.bfloat16)
    table = (torch.arange(requests * per, dtype=torch.int32, device=dev) + 1).view(requests, per)
    return plane, table.contiguous()


def _fma_tflops(dev) -> float:
    props = torch.cuda.get_device_properties(dev)
    mhz = getattr(props, "clock_rate", 1_965_000) / 1e3
    return props.multi_processor_count * 128 * 2 * mhz * 1e6 / 1e12


def measure_kernels(width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                    ret_heads: int, ret_key: int, ret_value: int, inter: int,
                    prompt: int = 2048, batch: int = 64, context: int = 1024,
                    page: int = 16, device="cuda:0") -> List[Dict[str, object]]:
    dev = torch.device(device)
    peaks = load_peaks()
    hbm, tc, fma = peaks["hbm_gbs"], peaks["bf16_tflops"], _fma_tflops(dev)
    flush = L2Flusher(dev)
    out: List[Dict[str, object]] = []
    bf = torch.bfloat16

    def row(name, ms, like, like_ms, bound, work, like_work=None):
        """work: bytes (bound 'hbm') or floating-point operations (bound 'tensor', 'fma')."""
        peak = {"hbm": hbm * 1e9, "tensor": tc * 1e12, "fma": fma * 1e12}[bound]
        rec = {"kernel": name, "us": round(ms * 1e3, 1), "bound": bound,
               "frac": round(work / (ms * 1e-3) / peak, 3)}
        if like:
            rec.update(like=like, like_us=round(like_ms * 1e3, 1),
                       like_frac=round((like_work or work) / (like_ms * 1e-3) / peak, 3))
        out.append(rec)

    def context_of(n_req, extent, first):
        T = n_req * extent
        pos = (torch.arange(extent, dtype=torch.int32, device=dev) + first).repeat(n_req)
        seq = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(extent)
        qs = torch.arange(n_req + 1, dtype=torch.int32, device=dev) * extent
        z = torch.zeros(n_req, dtype=torch.int32, device=dev)
        return StepContext(T, n_req, pos, pos, seq, qs, z, torch.arange(n_req, dtype=torch.int32, device=dev),
                           z, bf, extents=[extent] * n_req, first_positions=[first] * n_req,
                           max_extent=extent, max_context=first + extent, decode_only=extent == 1)

    # ---- attention over a prompt: the mixed-head tile kernel beside the plain one
    H, G, dk, dv = heads, kv_heads, key_dim, value_dim
    mix = torch.eye(H, device=dev) * 0.7 + 0.3 * torch.randn(H, H, device=dev)
    scale = 1.0 / math.sqrt(dk)
    kc, table = _paged(1, prompt, G, dk, page, dev)
    vc, _ = _paged(1, prompt, G, dv, page, dev)
    ctx = context_of(1, prompt, 0)
    q = torch.randn((prompt, H * dk), device=dev).to(bf)
    o = torch.empty((prompt, H * dv), dtype=bf, device=dev)
    keys = prompt * (prompt + 1) / 2
    flops = 2.0 * H * (dk + dv) * keys
    tok0, ntok = step_tiles(ctx, 16)
    ms = _timed(lambda: ops.attention_mixed_tile(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                 ctx.positions, mix, scale, tok0, ntok), flush)
    like, like_ms, like_flops = None, 0.0, 4.0 * H * dk * keys
    vk, _ = _paged(1, prompt, G, dk, page, dev)
    o2 = torch.empty((prompt, H * dk), dtype=bf, device=dev)
    group = H // G
    if dk == 128 and ops.attention_tc_supports(dk, group, page):
        t0, n0 = step_tiles(ctx, 128 // group)
        like = "attention_tc_prefill"
        like_ms = _timed(lambda: ops.attention_tc_prefill(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                          ctx.seq_ids, t0, n0, scale, 0), flush)
    elif ops.flash_supports(dk, group):
        t0, n0 = step_tiles(ctx, ops.flash_tile_rows() // group)
        like = "attention_flash (tiles)"
        like_ms = _timed(lambda: ops.attention_flash(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                     ctx.seq_ids, t0, n0, scale, 0), flush)
    row(f"attention_mixed_tile, {prompt} tokens", ms, like, like_ms, "tensor", flops, like_flops)

    # ---- attention of a decode step
    kc, table = _paged(batch, context, G, dk, page, dev)
    vc, _ = _paged(batch, context, G, dv, page, dev)
    vk, _ = _paged(batch, context, G, dk, page, dev)
    ctx = context_of(batch, 1, context - 1)
    q = torch.randn((batch, H * dk), device=dev).to(bf)
    o = torch.empty((batch, H * dv), dtype=bf, device=dev)
    o2 = torch.empty((batch, H * dk), dtype=bf, device=dev)
    ranges = decode_ranges(batch, context, ops.num_sms(dev))
    ms = _timed(lambda: ops.attention_mixed_decode(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                   ctx.positions, mix, scale, ranges, context), flush)
    like, like_ms = None, 0.0
    if ops.flash_supports(dk, group):
        like = "attention_flash (decode)"
        n_splits = splits_for(batch * G, context, 0, ops.num_sms(dev))
        like_ms = _timed(lambda: ops.attention_flash(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                     ctx.seq_ids, None, None, scale, 0, n_splits=n_splits), flush)
    row(f"attention_mixed_decode, batch {batch} x {context} keys", ms, like, like_ms, "hbm",
        2.0 * batch * context * G * (dk + dv), 2.0 * batch * context * G * 2 * dk)

    # ---- retention: a prompt, and a decode step
    Hr, a, b = ret_heads, ret_key, ret_value
    decay = torch.linspace(0.9, 0.999, Hr, device=dev)
    for n_req, extent, first, what in ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch}")):
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        z = torch.randn((T, Hr * (2 * a + 2 * b)), device=dev).to(bf)
        qk = Hr * a
        state = torch.zeros((n_req + 1, Hr, a, b), dtype=torch.float32, device=dev)
        oo = torch.empty((T, Hr * b), dtype=torch.float32, device=dev)
        rope = torch.randn((T, a), device=dev)
        args = (z[:, :qk], z[:, qk:2 * qk], z[:, 2 * qk:2 * qk + Hr * b], oo, n_req, Hr, a, b, decay,
                a ** -0.5, rope, a, ctx.q_start, ctx.state_slots, state)
        lists = () if extent == 1 else step_chunks(ctx, ops.retention_chunk_tokens())
        ms = _timed(lambda: ops.retention_chunked(*args, *lists), flush)
        in_order = _timed(lambda: ops.retention(*args), flush, repeats=2)
        if extent > 1:
            # by the chunked form's own count: per token and head 2 dk dv for the summaries, as
            # much for the state's part of the outputs, and chunk x (dk + dv) inside the chunk
            C = ops.retention_chunk_tokens()
            row(f"retention (summaries, scan, outputs), {what}", ms, "retention in order", in_order, "fma",
                2.0 * T * Hr * (2 * a * b + C * (a + b) / 2.0))
        else:
            row(f"retention (single tokens), {what}", ms, "retention in order", in_order, "hbm",
                8.0 * n_req * Hr * a * b)
        y = torch.empty((T, Hr * b), dtype=bf, device=dev)
        ms = _timed(lambda: ops.head_norm_gate(oo, z[:, 2 * qk + Hr * b:], y, Hr, b, 1e-6), flush)
        row(f"head_norm_gate, {what}", ms, None, 0.0, "hbm", T * Hr * b * (4 + 2 + 2.0))

    # ---- the add into the stream with its norm, beside the pre-norm layer's
    for T in (prompt, batch):
        h = torch.randn((T, width), device=dev)
        y32 = torch.randn((T, width), device=dev)
        ybf = y32.to(bf)
        gain = torch.ones(width, device=dev)
        act = torch.empty((T, width), dtype=bf, device=dev)
        ms = _timed(lambda: ops.group_norm_scale_add(h, y32, gain, gain, 1e-6, 2, act), flush)
        like_ms = _timed(lambda: ops.add_rmsnorm(h, ybf, gain, 1e-6, act), flush)
        row(f"group_norm_scale_add, {T} rows", ms, "add_rmsnorm", like_ms, "hbm",
            T * width * (4 + 4 + 4 + 2.0), T * width * (4 + 2 + 4 + 2.0))
    T = prompt
    gu = torch.randn((T, 2 * inter), device=dev).to(bf)
    go = torch.empty((T, inter), dtype=bf, device=dev)
    ms = _timed(lambda: ops.gated_act(gu, go, True, "relu"), flush)
    like_ms = _timed(lambda: ops.swiglu(gu, go, True), flush)
    row(f"gated_act relu, {T} rows", ms, "swiglu", like_ms, "hbm", T * inter * 6.0)
    # ---- values normed, blended, stored, beside the q/k-norm kernel that stores k and v
    v = torch.randn((T, G * dv), device=dev).to(bf)
    shared = torch.empty((T, G * dv), dtype=torch.float32, device=dev)
    vcache, _ = _paged(1, T, G, dv, page, dev)
    slots = torch.arange(T, dtype=torch.int32, device=dev) + page
    lam = torch.tensor([0.3], device=dev)
    ops.value_norm_share_cache(v, G, dv, True, 1e-6, None, shared, 1, slots, vcache, page)
    ms = _timed(lambda: ops.value_norm_share_cache(v, G, dv, True, 1e-6, lam, shared, 2, slots, vcache, page),
                flush)
    row(f"value_norm_share_cache, {T} rows", ms, None, 0.0, "hbm", T * G * dv * (2 + 4 + 2.0))
    return out


def measure_totatar_kernels(width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                            window: int, ssm_heads: int, ssm_channels: int, ssm_state: int,
                            ssm_groups: int, taps: int, experts: int, top: int, expert_ff: int,
                            dense_ff: int, prompt: int = 2048, batch: int = 64, context: int = 1024,
                            page: int = 16, device="cuda:0") -> List[Dict[str, object]]:
    """The kernels of the layers that run a windowed attention with a sink beside linear
    attention, a selective state-space scan and routed experts, each timed alone beside the
    like kernel of the framework's closest layers at equal sizes, with what each reaches of its
    roofline (same timing and denominators as `measure_kernels`)."""
    dev = torch.device(device)
    peaks = load_peaks()
    hbm, tc, fma = peaks["hbm_gbs"], peaks["bf16_tflops"], _fma_tflops(dev)
    flush = L2Flusher(dev)
    out: List[Dict[str, object]] = []
    bf = torch.bfloat16

    def row(name, ms, like, like_ms, bound, work, like_work=None):
        peak = {"hbm": hbm * 1e9, "tensor": tc * 1e12, "fma": fma * 1e12}[bound]
        rec = {"kernel": name, "us": round(ms * 1e3, 1), "bound": bound,
               "frac": round(work / (ms * 1e-3) / peak, 4)}
        if like:
            rec.update(like=like, like_us=round(like_ms * 1e3, 1),
                       like_frac=round((like_work or work) / (like_ms * 1e-3) / peak, 4))
        out.append(rec)

    def context_of(n_req, extent, first):
        T = n_req * extent
        pos = (torch.arange(extent, dtype=torch.int32, device=dev) + first).repeat(n_req)
        seq = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(extent)
        qs = torch.arange(n_req + 1, dtype=torch.int32, device=dev) * extent
        z = torch.zeros(n_req, dtype=torch.int32, device=dev)
        return StepContext(T, n_req, pos, pos, seq, qs, z, torch.arange(n_req, dtype=torch.int32, device=dev),
                           z, bf, extents=[extent] * n_req, first_positions=[first] * n_req,
                           max_extent=extent, max_context=first + extent, decode_only=extent == 1)

    H, G, dk, dv = heads, kv_heads, key_dim, value_dim
    group = H // G
    scale = 1.0 / math.sqrt(dk)
    sinks = torch.randn(H, device=dev)
    # ---- attention over a prompt: window + sink beside the plain windowed tile kernel
    kc, table = _paged(1, prompt, G, dk, page, dev)
    vc, _ = _paged(1, prompt, G, dv, page, dev)
    ctx = context_of(1, prompt, 0)
    q = torch.randn((prompt, H * dk), device=dev).to(bf)
    o = torch.empty((prompt, H * dv), dtype=bf, device=dev)
    keys = sum(min(t + 1, window) for t in range(prompt))
    tok0, ntok = step_tiles(ctx, ops.attention_sink_tile_tokens(group))
    ms = _timed(lambda: ops.attention_sink_tile(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                ctx.positions, scale, window, sinks, tok0, ntok), flush)
    like, like_ms = None, 0.0
    if dk == dv and ops.flash_supports(dk, group):
        t0, n0 = step_tiles(ctx, ops.flash_tile_rows() // group)
        like = "attention_flash (tiles, same window)"
        like_ms = _timed(lambda: ops.attention_flash(q, o, H, G, dk, kc, vc, page, table, ctx.positions,
                                                     ctx.seq_ids, t0, n0, scale, window), flush)
    row(f"attention_sink, {prompt} tokens, window {window}", ms, like, like_ms, "tensor",
        2.0 * H * (dk + dv) * keys)
    # ---- attention of a decode step
    kc, table = _paged(batch, context, G, dk, page, dev)
    vc, _ = _paged(batch, context, G, dv, page, dev)
    ctx = context_of(batch, 1, context - 1)
    q = torch.randn((batch, H * dk), device=dev).to(bf)
    o = torch.empty((batch, H * dv), dtype=bf, device=dev)
    reach = min(window, context)
    n_splits = splits_for(batch * G, reach, window, ops.num_sms(dev))
    ms = _timed(lambda: ops.attention_sink_tile(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                ctx.positions, scale, window, sinks, n_splits=n_splits), flush)
    like, like_ms = None, 0.0
    if dk == dv and ops.flash_supports(dk, group):
        like = "attention_flash (decode, same window)"
        like_ms = _timed(lambda: ops.attention_flash(q, o, H, G, dk, kc, vc, page, table, ctx.positions,
                                                     ctx.seq_ids, None, None, scale, window,
                                                     n_splits=n_splits), flush)
    row(f"attention_sink (a tile a token, keys in {n_splits} shares), batch {batch} x {reach} keys", ms, like, like_ms, "hbm",
        2.0 * batch * reach * G * (dk + dv))
    # ---- projection rows: bias, rotation, cache write, beside the q/k-norm kernel
    T = prompt
    ctx = context_of(1, T, 0)
    qkv = torch.randn((T, (H + G) * dk + G * dv), device=dev).to(bf)
    qq, kk, vv = qkv[:, :H * dk], qkv[:, H * dk:(H + G) * dk], qkv[:, (H + G) * dk:]
    kc, _ = _paged(1, T, G, dk, page, dev)
    vc, _ = _paged(1, T, G, dv, page, dev)
    slots = torch.arange(T, dtype=torch.int32, device=dev) + page
    rope = torch.randn((T, dk // 2), device=dev)
    bq, bk, bv = (torch.randn(n, device=dev) for n in (H * dk, G * dk, G * dv))
    ms = _timed(lambda: ops.qkv_bias_rope_cache(qq, kk, vv, H, G, dk, dv, bq, bk, bv, rope, dk // 2, True,
                                                slots, kc, vc, page), flush)
    like, like_ms = None, 0.0
    if dk == dv:
        gain = torch.ones(dk, device=dev)
        rope2 = torch.randn((T, dk), device=dev)
        like = "qk_norm_rope_cache"
        like_ms = _timed(lambda: ops.qk_norm_rope_cache(qq, kk, vv, H, G, dk, gain, gain, 1e-6, rope2, dk,
                                                        slots, kc, vc, page), flush)
    row(f"qkv_bias_rope_cache, {T} rows", ms, like, like_ms, "hbm", 2.0 * T * (2 * H * dk + 2 * G * (dk + dv)))

    # ---- the state-space mixer: convolution, scan, gated norm; a prompt and a decode step
    Hs, P, N, Gs = ssm_heads, ssm_channels, ssm_state, ssm_groups
    inner, C = Hs * P, Hs * P + 2 * Gs * N
    floats = Hs * N * P + (taps - 1) * C
    w = torch.randn((C, taps), device=dev) * 0.3
    cb = torch.zeros(C, device=dev)
    dtb, alog, dsk = torch.zeros(Hs, device=dev), torch.zeros(Hs, device=dev), torch.ones(Hs, device=dev)
    gain = torch.ones(inner, device=dev)
    # the like kernels: retention with heads of 128 x 256 and a state of the same size
    Hr = max(1, (Hs * N * P) // (128 * 256))
    decay = torch.linspace(0.9, 0.999, Hr, device=dev)
    for n_req, extent, first, what in ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch}")):
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        zall = (torch.randn((T, 2 * inner + 2 * Gs * N + Hs), device=dev) * 0.5).to(bf)
        state = torch.zeros((n_req + 1, floats), dtype=torch.float32, device=dev)
        xbc = torch.empty((T, C), dtype=torch.float32, device=dev)
        ms = _timed(lambda: ops.causal_conv_act(zall[:, inner:inner + C], w, cb, xbc, n_req, ctx.seq_ids,
                                                ctx.q_start, ctx.state_slots, state, Hs * N * P), flush)
        row(f"causal_conv_act (+ kept inputs), {what}", ms, None, 0.0, "hbm", T * C * (2 + 4.0))
        y = torch.empty((T, inner), dtype=torch.float32, device=dev)
        ms = _timed(lambda: ops.selective_scan(xbc, zall[:, inner + C:], dtb, alog, dsk, y, n_req, Hs, Gs, N, P,
                                               ctx.q_start, ctx.state_slots, state, 0), flush)
        zr = torch.randn((T, Hr * (2 * 128 + 2 * 256)), device=dev).to(bf)
        rstate = torch.zeros((n_req + 1, Hr, 128, 256), dtype=torch.float32, device=dev)
        oo = torch.empty((T, Hr * 256), dtype=torch.float32, device=dev)
        rargs = (zr[:, :Hr * 128], zr[:, Hr * 128:Hr * 256], zr[:, Hr * 256:Hr * 512], oo, n_req, Hr, 128, 256,
                 decay, 1.0, None, 0, ctx.q_start, ctx.state_slots, rstate)
        lists = () if extent == 1 else step_chunks(ctx, ops.retention_chunk_tokens())
        like_ms = _timed(lambda: ops.retention_chunked(*rargs, *lists), flush)
        if extent > 1:
            Cc = ops.retention_chunk_tokens()
            row(f"selective_scan, {what}", ms, "retention by chunks (state of equal size)", like_ms, "fma",
                6.0 * T * Hs * N * P, 2.0 * T * Hr * (2 * 128 * 256 + Cc * (128 + 256) / 2.0))
        else:
            row(f"selective_scan, {what}", ms, "retention single tokens (state of equal size)", like_ms,
                "hbm", 8.0 * n_req * Hs * N * P, 8.0 * n_req * Hr * 128 * 256)
        g = torch.empty((T, inner), dtype=bf, device=dev)
        ms = _timed(lambda: ops.gated_group_norm(y, zall[:, :inner], gain, g, Gs, 1e-6, "silu", True), flush)
        yb = torch.empty((T, Hr * 256), dtype=bf, device=dev)
        like_ms = _timed(lambda: ops.head_norm_gate(oo, zr[:, Hr * 512:], yb, Hr, 256, 1e-6), flush)
        row(f"gated_group_norm, {what}", ms, "head_norm_gate", like_ms, "hbm", T * inner * (4 + 2 + 2.0),
            T * Hr * 256 * (4 + 2 + 2.0))

    # ---- routed experts beside a dense gated feed-forward of as many active rows of weights
    E, ff = experts, expert_ff
    wr = torch.randn((E, width), device=dev) * 0.05
    wg, wu = (torch.randn((E, ff, width), device=dev) * 0.02).to(bf), (torch.randn((E, ff, width), device=dev) * 0.02).to(bf)
    wd = (torch.randn((E, width, ff), device=dev) * 0.02).to(bf)
    act_ff = top * ff                                    # width of the dense feed-forward of equal work
    wgu = (torch.randn((2 * act_ff, width), device=dev) * 0.02).to(bf)
    wdn = (torch.randn((width, act_ff), device=dev) * 0.02).to(bf)
    for T, what in ((prompt, f"{prompt} tokens"), (batch, f"batch {batch}"), (8, "batch 8")):
        x = torch.randn((T, width), device=dev).to(bf)
        ms = _timed(lambda: ops.moe_feed_forward(x, wr, None, wg, wu, wd, top, "silu"), flush)
        like_ms = _timed(lambda: ops.linear(ops.gated_linear(x, wgu, True), wdn, out_dtype=torch.float32), flush)
        if T >= 1024:
            row(f"routed experts ({E} experts, top {top}, ff {ff}), {what}", ms,
                "dense gated feed-forward of equal work", like_ms, "tensor", 2.0 * T * top * 3 * width * ff)
        else:
            touched = min(E, T * top)
            row(f"routed experts ({E} experts, top {top}, ff {ff}), {what}", ms,
                "dense gated feed-forward of equal work", like_ms, "hbm", 2.0 * touched * 3 * width * ff,
                2.0 * 3 * width * act_ff)
    return out


def measure_derosun_kernels(width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                            softcap: float, latent_rank: int, rope_dim: int, query_rank: int,
                            mem_heads: int, mem_key: int, mem_value: int, ff: int, prompt: int = 2048,
                            batch: int = 64, context: int = 1024, page: int = 16,
                            device="cuda:0") -> List[Dict[str, object]]:
    """The kernels of the layers that norm the scaled sum, cap their attention scores, attend
    over one cached latent row per token and carry a gated matrix memory, each timed alone
    beside the like kernel of the framework's closest layers at equal sizes, with what each
    reaches of its roofline (same timing and denominators as `measure_kernels`)."""
    from types import SimpleNamespace

    from ..parts.attention_sink import sink_attention
    dev = torch.device(device)
    peaks = load_peaks()
    hbm, tc, fma = peaks["hbm_gbs"], peaks["bf16_tflops"], _fma_tflops(dev)
    flush = L2Flusher(dev)
    out: List[Dict[str, object]] = []
    bf = torch.bfloat16

    def row(name, ms, like, like_ms, bound, work, like_work=None):
        peak = {"hbm": hbm * 1e9, "tensor": tc * 1e12, "fma": fma * 1e12}[bound]
        rec = {"kernel": name, "us": round(ms * 1e3, 1), "bound": bound,
               "frac": round(work / (ms * 1e-3) / peak, 4)}
        if like:
            rec.update(like=like, like_us=round(like_ms * 1e3, 1),
                       like_frac=round((like_work or work) / (like_ms * 1e-3) / peak, 4))
        out.append(rec)

    def context_of(n_req, extent, first):
        T = n_req * extent
        pos = (torch.arange(extent, dtype=torch.int32, device=dev) + first).repeat(n_req)
        seq = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(extent)
        qs = torch.arange(n_req + 1, dtype=torch.int32, device=dev) * extent
        z = torch.zeros(n_req, dtype=torch.int32, device=dev)
        return StepContext(T, n_req, pos, pos, seq, qs, z, torch.arange(n_req, dtype=torch.int32, device=dev),
                           z, bf, extents=[extent] * n_req, first_positions=[first] * n_req,
                           max_extent=extent, max_context=first + extent, decode_only=extent == 1)

    H, G, dk, dv = heads, kv_heads, key_dim, value_dim
    group = H // G
    scale = 1.0 / math.sqrt(dk)
    cases = ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch} x {context} keys"))
    # ---- attention with capped scores beside the plain tile kernel
    for n_req, extent, first, what in cases:
        kc, table = _paged(n_req, first + extent, G, dk, page, dev)
        vc, _ = _paged(n_req, first + extent, G, dv, page, dev)
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        q = torch.randn((T, H * dk), device=dev).to(bf)
        o = torch.empty((T, H * dv), dtype=bf, device=dev)
        cache = SimpleNamespace(k=kc, v=vc, page_size=page, block_tables=table)
        ms = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, 0, None, softcap=softcap), flush)
        like, like_ms = None, 0.0
        if dk == dv and ops.flash_supports(dk, group):
            like = "attention_flash (no cap)"
            if extent > 1:
                t0, n0 = step_tiles(ctx, ops.flash_tile_rows() // group)
                like_ms = _timed(lambda: ops.attention_flash(q, o, H, G, dk, kc, vc, page, table, ctx.positions,
                                                             ctx.seq_ids, t0, n0, scale, 0), flush)
            else:
                n_splits = splits_for(n_req * G, context, 0, ops.num_sms(dev))
                like_ms = _timed(lambda: ops.attention_flash(q, o, H, G, dk, kc, vc, page, table, ctx.positions,
                                                             ctx.seq_ids, None, None, scale, 0,
                                                             n_splits=n_splits), flush)
        ms0 = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, 0, None), flush)
        if extent > 1:
            row(f"attention with capped scores, {what}", ms, like, like_ms, "tensor",
                2.0 * H * (dk + dv) * (prompt * (prompt + 1) / 2))
            row(f"the same kernel without the cap, {what}", ms0, None, 0.0, "tensor",
                2.0 * H * (dk + dv) * (prompt * (prompt + 1) / 2))
        else:
            row(f"attention with capped scores, {what}", ms, like, like_ms, "hbm",
                2.0 * n_req * context * G * (dk + dv))
            row(f"the same kernel without the cap, {what}", ms0, None, 0.0, "hbm",
                2.0 * n_req * context * G * (dk + dv))
    # ---- projection rows: norm over the whole row, banded rotation, cache write
    T = prompt
    qkv = torch.randn((T, (H + G) * dk + G * dv), device=dev).to(bf)
    qq, kk, vv = qkv[:, :H * dk], qkv[:, H * dk:(H + G) * dk], qkv[:, (H + G) * dk:]
    kc, _ = _paged(1, T, G, dk, page, dev)
    vc, _ = _paged(1, T, G, dv, page, dev)
    slots = torch.arange(T, dtype=torch.int32, device=dev) + page
    rope = torch.randn((T, dk // 2), device=dev)
    gq, gk = torch.ones(H * dk, device=dev), torch.ones(G * dk, device=dev)
    ms = _timed(lambda: ops.qk_rownorm_rope_cache(qq, kk, vv, H, G, dk, dv, gq, gk, 1e-6, rope, dk // 2, False,
                                                  slots, kc, vc, page), flush)
    like, like_ms = None, 0.0
    if dk == dv:
        gain = torch.ones(dk, device=dev)
        rope2 = torch.randn((T, dk), device=dev)
        like = "qk_norm_rope_cache (norm per head)"
        like_ms = _timed(lambda: ops.qk_norm_rope_cache(qq, kk, vv, H, G, dk, gain, gain, 1e-6, rope2, dk,
                                                        slots, kc, vc, page), flush)
    row(f"qk_rownorm_rope_cache, {T} rows", ms, like, like_ms, "hbm", 2.0 * T * (2 * H * dk + 2 * G * (dk + dv)))

    # ---- latent attention: the cache row, the query as the cache sees it, the attention, the values
    rank, dr, rowl = latent_rank, rope_dim, latent_rank + rope_dim
    lscale = 1.0 / math.sqrt(dk + dr)
    w_uk_t = (torch.randn((H, rank, dk), device=dev) * 0.05).to(bf)
    w_uv = (torch.randn((H, dv, rank), device=dev) * 0.05).to(bf)
    gl = torch.ones(rank, device=dev)
    for n_req, extent, first, what in cases:
        T = n_req * extent
        ctx = context_of(n_req, extent, first)
        plane, table = _paged(n_req, first + extent, 1, rowl, page, dev)
        cache = SimpleNamespace(k=plane, v=None, page_size=page, block_tables=table)
        kv = torch.randn((T, rowl), device=dev).to(bf)
        q = torch.randn((T, H * (dk + dr)), device=dev).to(bf)
        tab = torch.randn((T, dr), device=dev)
        slots = (torch.arange(T, dtype=torch.int32, device=dev) % (first + extent)) + page
        qa = torch.empty((T, H * rowl), dtype=bf, device=dev)
        lat = torch.empty((T, H * rank), dtype=bf, device=dev)
        a = torch.empty((T, H * dv), dtype=bf, device=dev)

        def before():
            ops.latent_row_cache(kv, rank, dr, gl, 1e-6, tab, dr, True, slots, plane, page)
            ops.head_linear(q, dk + dr, w_uk_t, qa, rowl)
            ops.rope_slice(q, dk + dr, dk, qa, rowl, rank, H, dr, tab, dr, True)
        ms = _timed(before, flush)
        weights = 2.0 * H * rank * dk
        if extent > 1:
            row(f"latent row to the cache, query through the key expansion, rotated slice, {what}", ms, None,
                0.0, "tensor", 2.0 * T * H * dk * rank)
        else:
            row(f"latent row to the cache, query through the key expansion, rotated slice, {what}", ms, None,
                0.0, "hbm", weights + 2.0 * T * (rowl * 2 + H * (dk + dr) + H * rowl))
        ms = _timed(lambda: sink_attention(qa, lat, H, 1, rowl, rank, cache, ctx, lscale, 0, None, value_row=rowl),
                    flush)
        like, like_ms, like_work = None, 0.0, None
        if dk == dv and ops.flash_supports(dk, group):
            kc, table2 = _paged(n_req, first + extent, G, dk, page, dev)
            vc, _ = _paged(n_req, first + extent, G, dv, page, dev)
            q2 = torch.randn((T, H * dk), device=dev).to(bf)
            o2 = torch.empty((T, H * dv), dtype=bf, device=dev)
            like = f"attention_flash ({H}/{G} heads of {dk})"
            if extent > 1:
                t0, n0 = step_tiles(ctx, ops.flash_tile_rows() // group)
                like_ms = _timed(lambda: ops.attention_flash(q2, o2, H, G, dk, kc, vc, page, table2, ctx.positions,
                                                             ctx.seq_ids, t0, n0, scale, 0), flush)
                like_work = 2.0 * H * (dk + dv) * (prompt * (prompt + 1) / 2)
            else:
                n_splits = splits_for(n_req * G, context, 0, ops.num_sms(dev))
                like_ms = _timed(lambda: ops.attention_flash(q2, o2, H, G, dk, kc, vc, page, table2, ctx.positions,
                                                             ctx.seq_ids, None, None, scale, 0,
                                                             n_splits=n_splits), flush)
                like_work = 2.0 * n_req * context * G * (dk + dv)
        if extent > 1:
            row(f"attention over latent rows ({rowl} wide, values the first {rank}), {what}", ms, like, like_ms,
                "tensor", 2.0 * H * (rowl + rank) * (prompt * (prompt + 1) / 2), like_work)
        else:
            row(f"attention over latent rows ({rowl} wide, values the first {rank}), {what}", ms, like, like_ms,
                "hbm", 2.0 * n_req * context * rowl, like_work)
        ms = _timed(lambda: ops.head_linear(lat, rank, w_uv, a, dv), flush)
        if extent > 1:
            row(f"value expansion per head, {what}", ms, None, 0.0, "tensor", 2.0 * T * H * dv * rank)
        else:
            row(f"value expansion per head, {what}", ms, None, 0.0, "hbm",
                2.0 * H * dv * rank + 2.0 * T * H * (rank + dv))

    # ---- the gated matrix memory beside retention with a state of equal size
    Hm, mk, mv = mem_heads, mem_key, mem_value
    floats = ops.mlstm_state_floats(Hm, mk, mv)
    bi, bfg = torch.zeros(Hm, device=dev), torch.full((Hm,), 3.0, device=dev)
    gain = torch.ones(Hm * mv, device=dev)
    decay = torch.linspace(0.9, 0.999, Hm, device=dev)
    for n_req, extent, first, what in ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch}")):
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        z = (torch.randn((T, Hm * (2 * mk + 2 * mv)), device=dev) * 0.5).to(bf)
        qm, km, vm = z[:, :Hm * mk], z[:, Hm * mk:2 * Hm * mk], z[:, 2 * Hm * mk:2 * Hm * mk + Hm * mv]
        gate = z[:, 2 * Hm * mk + Hm * mv:]
        g = torch.randn((T, 2 * Hm), device=dev)
        state = torch.zeros((n_req + 1, floats), dtype=torch.float32, device=dev)
        oo = torch.empty((T, Hm * mv), dtype=torch.float32, device=dev)
        margs = (qm, km, vm, g[:, :Hm], g[:, Hm:], bi, bfg, 15.0, mk ** -0.5, oo, n_req, Hm, mk, mv,
                 ctx.q_start, ctx.state_slots, state)
        rstate = torch.zeros((n_req + 1, Hm, mk, mv), dtype=torch.float32, device=dev)
        rargs = (qm, km, vm, oo, n_req, Hm, mk, mv, decay, 1.0, None, 0, ctx.q_start, ctx.state_slots, rstate)
        if extent > 1:
            lists = step_chunks(ctx, ops.mlstm_chunk_tokens())
            ms = _timed(lambda: ops.mlstm_chunked(*margs, *lists), flush)
            rl = step_chunks(ctx, ops.retention_chunk_tokens())
            like_ms = _timed(lambda: ops.retention_chunked(*rargs, *rl), flush)
            Cc = ops.mlstm_chunk_tokens()
            row(f"matrix memory by chunks, {what}", ms, "retention by chunks (state of equal size)", like_ms,
                "fma", 2.0 * T * Hm * (2 * mk * mv + Cc * (mk + mv) / 2.0))
            ms = _timed(lambda: ops.mlstm(*margs), flush)
            row(f"matrix memory in order (the form for sizes the chunked kernels refuse), {what}", ms, None,
                0.0, "fma", 2.0 * T * Hm * (2 * mk * mv + 32 * (mk + mv) / 2.0))
        else:
            ms = _timed(lambda: ops.mlstm_chunked(*margs), flush)
            like_ms = _timed(lambda: ops.retention_chunked(*rargs), flush)
            row(f"matrix memory, single tokens, {what}", ms, "retention single tokens (state of equal size)",
                like_ms, "hbm", 8.0 * n_req * Hm * mk * mv)
        yb = torch.empty((T, Hm * mv), dtype=bf, device=dev)
        ms = _timed(lambda: ops.gated_group_norm(oo, gate, gain, yb, Hm, 1e-6, "sigmoid", False), flush)
        like_ms = _timed(lambda: ops.head_norm_gate(oo, gate, yb, Hm, mv, 1e-6), flush)
        row(f"gated_group_norm (sigmoid gate, gain), {what}", ms, "head_norm_gate", like_ms, "hbm",
            T * Hm * mv * (4 + 2 + 2.0))

    # ---- the block's norm of the scaled sum, and the feed-forward's activation with biases
    for T, what in ((prompt, f"{prompt} rows"), (batch, f"{batch} rows")):
        h = torch.randn((T, width), device=dev)
        y = torch.randn((T, width), device=dev).to(bf)
        bias = torch.randn(width, device=dev)
        gain = torch.ones(width, device=dev)
        act = torch.empty((T, width), dtype=bf, device=dev)
        ms = _timed(lambda: ops.scaled_add_norm(h, y, bias, 2.0, gain, 1e-6, act), flush)
        like_ms = _timed(lambda: ops.add_rmsnorm(h, y, gain, 1e-6, act), flush)
        row(f"scaled_add_norm (+ bias), {what}", ms, "add_rmsnorm", like_ms, "hbm", T * width * (4 + 2 + 4 + 2.0))
        gu = torch.randn((T, 2 * ff), device=dev).to(bf)
        b2 = torch.randn(2 * ff, device=dev)
        go = torch.empty((T, ff), dtype=bf, device=dev)
        ms = _timed(lambda: ops.gated_act(gu, go, True, "silu", b2), flush)
        like_ms = _timed(lambda: ops.swiglu(gu, go, True), flush)
        row(f"gated_act with biases, {what}", ms, "swiglu", like_ms, "hbm", T * ff * 6.0)
    return out


def measure_vimelorn_kernels(width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                             window: int, keep_first: int, taps: int, streams: int, experts: int,
                             identity: int, top: int, expert_ff: int, prompt: int = 2048, batch: int = 64,
                             context: int = 2048, page: int = 16, device="cuda:0") -> List[Dict[str, object]]:
    """The kernels of the layers that keep several residual streams, convolve their projection
    rows, keep the first keys beside a window, add a bias by distance and route to small experts
    among which some are the identity, each timed alone beside the like kernel of the framework's
    closest layers at equal sizes (same timing and denominators as `measure_kernels`)."""
    from types import SimpleNamespace

    from ..parts.attention_sink import bias_by_distance, sink_attention
    dev = torch.device(device)
    peaks = load_peaks()
    hbm, tc, fma = peaks["hbm_gbs"], peaks["bf16_tflops"], _fma_tflops(dev)
    flush = L2Flusher(dev)
    out: List[Dict[str, object]] = []
    bf = torch.bfloat16

    def row(name, ms, like, like_ms, bound, work, like_work=None):
        peak = {"hbm": hbm * 1e9, "tensor": tc * 1e12, "fma": fma * 1e12}[bound]
        rec = {"kernel": name, "us": round(ms * 1e3, 1), "bound": bound,
               "frac": round(work / (ms * 1e-3) / peak, 4)}
        if like:
            rec.update(like=like, like_us=round(like_ms * 1e3, 1),
                       like_frac=round((like_work or work) / (like_ms * 1e-3) / peak, 4))
        out.append(rec)

    def context_of(n_req, extent, first):
        T = n_req * extent
        pos = (torch.arange(extent, dtype=torch.int32, device=dev) + first).repeat(n_req)
        seq = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(extent)
        qs = torch.arange(n_req + 1, dtype=torch.int32, device=dev) * extent
        z = torch.zeros(n_req, dtype=torch.int32, device=dev)
        return StepContext(T, n_req, pos, pos, seq, qs, z, torch.arange(n_req, dtype=torch.int32, device=dev),
                           z, bf, extents=[extent] * n_req, first_positions=[first] * n_req,
                           max_extent=extent, max_context=first + extent, decode_only=extent == 1)

    H, G, dk, dv = heads, kv_heads, key_dim, value_dim
    scale = 1.0 / math.sqrt(dk)
    table_rel = bias_by_distance(torch.randn((32, H), device=dev), 4 * window)
    cases = ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch} x {context} keys"))
    # ---- attention: the window with kept first keys beside the window alone; the bias by
    # distance beside plain causal attention (the same tile kernels without the extra)
    for n_req, extent, first, what in cases:
        kc, table = _paged(n_req, first + extent, G, dk, page, dev)
        vc, _ = _paged(n_req, first + extent, G, dv, page, dev)
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        q = torch.randn((T, H * dk), device=dev).to(bf)
        o = torch.empty((T, H * dv), dtype=bf, device=dev)
        cache = SimpleNamespace(k=kc, v=vc, page_size=page, block_tables=table)
        ms = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, window, None,
                                           keep_first=keep_first), flush)
        like_ms = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, window, None), flush)
        ms_b = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, 0, None,
                                             dist_bias=table_rel), flush)
        like_b = _timed(lambda: sink_attention(q, o, H, G, dk, dv, cache, ctx, scale, 0, None), flush)
        if extent > 1:
            keys = sum(min(t + 1, window) + min(keep_first, max(0, t + 1 - window)) for t in range(prompt))
            row(f"attention, window {window} + first {keep_first}, {what}", ms, "the window alone", like_ms,
                "tensor", 2.0 * H * (dk + dv) * keys, 2.0 * H * (dk + dv) * sum(min(t + 1, window) for t in range(prompt)))
            row(f"attention with a bias by distance, {what}", ms_b, "plain causal", like_b, "tensor",
                2.0 * H * (dk + dv) * (prompt * (prompt + 1) / 2))
        else:
            reach = min(window, context)
            row(f"attention, window {window} + first {keep_first}, {what}", ms, "the window alone", like_ms,
                "hbm", 2.0 * n_req * (reach + keep_first) * G * (dk + dv), 2.0 * n_req * reach * G * (dk + dv))
            row(f"attention with a bias by distance, {what}", ms_b, "plain causal", like_b, "hbm",
                2.0 * n_req * context * G * (dk + dv))
    # ---- projection rows: convolution, rotation, unit norm, cache write, beside the biased rows
    C = H * dk + G * (dk + dv)
    conv = torch.randn((C, taps), device=dev)
    for n_req, extent, first, what in ((1, prompt, 0, f"{prompt} rows"), (batch, 1, context - 1, f"batch {batch}")):
        T = n_req * extent
        ctx = context_of(n_req, extent, first)
        qkv = torch.randn((T, C), device=dev).to(bf)
        qq, kk, vv = qkv[:, :H * dk], qkv[:, H * dk:(H + G) * dk], qkv[:, (H + G) * dk:]
        q_out = torch.empty((T, H * dk), dtype=bf, device=dev)
        kc, _ = _paged(1, T, G, dk, page, dev)
        vc, _ = _paged(1, T, G, dv, page, dev)
        slots = torch.arange(T, dtype=torch.int32, device=dev) + page
        rope = torch.randn((T, dk), device=dev)
        state = torch.zeros((n_req + 1, (taps - 1) * C), device=dev)
        ms = _timed(lambda: ops.qkv_conv_rope_norm_cache(qkv, q_out, H, G, dk, dv, conv, n_req, ctx.seq_ids,
                                                         ctx.q_start, ctx.state_slots, state, 0, rope, dk, False,
                                                         True, 1e-6, slots, kc, vc, page), flush)
        bq, bk, bv = (torch.randn(n, device=dev) for n in (H * dk, G * dk, G * dv))
        like_ms = _timed(lambda: ops.qkv_bias_rope_cache(qq, kk, vv, H, G, dk, dv, bq, bk, bv, rope, dk, False,
                                                         slots, kc, vc, page), flush)
        row(f"qkv_conv_rope_norm_cache + kept rows, {what}", ms, "qkv_bias_rope_cache", like_ms, "hbm",
            2.0 * T * (2 * H * dk + 2 * G * (dk + dv)) + 8.0 * n_req * (taps - 1) * C,
            2.0 * T * (2 * H * dk + 2 * G * (dk + dv)))
    # ---- the streams: read with the norm, write with the next read, beside add + norm
    S = streams
    for T, what in ((prompt, f"{prompt} rows"), (batch, f"batch {batch}")):
        x = torch.randn((S, T, width), device=dev)
        y = torch.randn((T, width), device=dev)
        h = torch.randn((T, width), device=dev)
        cin, cout, mix = torch.randn(S, device=dev), torch.randn(S, device=dev), torch.randn((S, S), device=dev)
        gain = torch.ones(width, device=dev)
        n = torch.empty((T, width), dtype=bf, device=dev)
        ms = _timed(lambda: ops.stream_read_norm(x, cin, gain, 1e-6, n), flush)
        like_ms = _timed(lambda: ops.add_rmsnorm(h, None, gain, 1e-6, n), flush)
        row(f"stream_read_norm ({S} streams), {what}", ms, "add_rmsnorm", like_ms, "hbm",
            T * width * (4.0 * S + 2), T * width * (4.0 + 2))
        ms = _timed(lambda: ops.stream_write(x, y, mix, cout, 1e-6, cin, gain, n), flush)
        like_ms = _timed(lambda: ops.add_rmsnorm(h, y, gain, 1e-6, n), flush)
        row(f"stream_write with the next read ({S} streams), {what}", ms, "add_rmsnorm with the add", like_ms,
            "hbm", T * width * (8.0 * S + 4 + 2), T * width * (4.0 + 4 + 4 + 2))
    # ---- routed experts: small ones without a gate, identity experts, scores over all, beside
    # the gated routed experts of equal active width
    E, ff = experts, expert_ff
    wr = torch.randn((E + identity + 1, width), device=dev) * 0.05
    corr = torch.randn(E + identity, device=dev) * 0.01
    wu = (torch.randn((E, ff, width), device=dev) * 0.02).to(bf)
    wd = (torch.randn((E, width, ff), device=dev) * 0.02).to(bf)
    ffg = 2 * ff // 3 // 8 * 8                           # a gated expert of about equal work
    wr2 = torch.randn((E, width), device=dev) * 0.05
    wg2, wu2 = ((torch.randn((E, ffg, width), device=dev) * 0.02).to(bf) for _ in range(2))
    wd2 = (torch.randn((E, width, ffg), device=dev) * 0.02).to(bf)
    for T, what in ((prompt, f"{prompt} tokens"), (batch, f"batch {batch}"), (8, "batch 8")):
        x = torch.randn((T, width), device=dev).to(bf)
        extra = torch.randn((T, width), device=dev)
        ms = _timed(lambda: ops.moe_feed_forward(x, wr, None, None, wu, wd, top, "relu_squared", extra, "all",
                                                 corr, identity, True), flush)
        like_ms = _timed(lambda: ops.moe_feed_forward(x, wr2, None, wg2, wu2, wd2, top, "silu", extra), flush)
        like = f"gated routed experts (ff {ffg}, scores over the chosen)"
        share = E / (E + identity)                       # of the chosen, about this many have matrices
        if T >= 1024:
            row(f"routed experts ({E} + {identity} identity, top {top}, ff {ff}, no gate), {what}", ms, like,
                like_ms, "tensor", 2.0 * T * top * share * 2 * width * ff, 2.0 * T * top * 3 * width * ffg)
        else:
            touched = min(E, T * top)
            row(f"routed experts ({E} + {identity} identity, top {top}, ff {ff}, no gate), {what}", ms, like,
                like_ms, "hbm", 2.0 * touched * 2 * width * ff, 2.0 * touched * 3 * width * ffg)
    return out


if __name__ == "__main__":
    # python -m tgo_b200.engine.measure_kernels vimelorn|derosun|totatar|gafonex [width]: the kernels of one design
    # at one size, a JSON line each (small enough to run under a profiler)
    import json
    import sys
    design = sys.argv[1] if len(sys.argv) > 1 else "totatar"
    w = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
    ff = 3 * w
    if design == "vimelorn":
        recs = measure_vimelorn_kernels(w, 16, 4, 128, 128, 1024, 4, 4, 4, 32, 2, 4, ff // 8)
    elif design == "derosun":
        recs = measure_derosun_kernels(w, 16, 4, 128, 128, 30.0, 512, 64, 3 * w // 4, w // 256, 128, 256, ff)
    elif design == "totatar":
        recs = measure_totatar_kernels(w, 16, 4, 128, 128, 1024, 2 * w // 64, 64, 128, 8, 4, 32, 4, ff // 8, ff)
    else:
        recs = measure_kernels(w, 16, 4, 128, 128, w // 256, 128, 256, ff)
    for rec in recs:
        print(json.dumps(rec), flush=True)
