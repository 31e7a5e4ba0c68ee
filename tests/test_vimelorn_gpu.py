"""Vimelorn on the GPU: every new kernel alone against the plain statement of its mechanism
(with inputs made so that a dropped far key, a window or a kept range that is one token off, a
lost convolution state or a forgotten bias shows), then the engine against the plain model:
whole prompts, decoding, portions down to two tokens, mixed batches with pages and state slots
that come back, first tokens, long decoding, a long prompt, and greedy generation through the
library's entry point, the scheduler and the command line."""
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vimelorn as plain
import tiny
import vimelorn_tiny as vt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(device=DEV, dtype=dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def close(got, want, tol, what=""):
    err = np.abs(host(got) - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err}"


# ------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,T,d", [(3, 7, 48), (1, 1, 36), (8, 70, 200), (2, 5, 13), (4, 3, 4100), (3, 2, 13000),
                                   (2, 3, 12289), (5, 9, 1026)])
def test_streams_read_and_written(S, T, d, ydtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(S * 100 + d)
    h = rng.normal(size=(T, d)).astype(np.float32).astype(np.float64)
    x = torch.empty((S, T, d), dtype=torch.float32, device=DEV)
    ops.stream_spread(dev(h), x)
    assert np.array_equal(host(x), np.broadcast_to(h, (S, T, d)))
    xs = rng.normal(size=(S, T, d)).astype(np.float32).astype(np.float64)
    cin = rng.normal(size=S).astype(np.float32).astype(np.float64)
    cout = rng.normal(size=S).astype(np.float32).astype(np.float64)
    mix = (np.eye(S) + 0.3 * rng.normal(size=(S, S))).astype(np.float32).astype(np.float64)
    gain = (1 + 0.2 * rng.normal(size=d)).astype(np.float32).astype(np.float64)
    y = vt.bf16_values(rng.normal(size=(T, d)) * 3)
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.empty((T, d), dtype=out_dtype, device=DEV)
        ops.stream_read_norm(dev(xs), dev(cin), dev(gain), 1e-5, out)
        close(out, plain.rmsnorm(np.tensordot(cin, xs, 1), gain, 1e-5), TOL[out_dtype], "read")
    new = np.stack([np.tensordot(mix[:, t], xs, 1) + cout[t] * y for t in range(S)])
    # the write alone, with the sum, and with the next sublayer's input
    x = dev(xs)
    total = torch.empty((T, d), dtype=torch.float32, device=DEV)
    ops.stream_write(x, dev(y, ydtype), dev(mix), dev(cout), sum_out=total)
    close(x, new, 3e-6, "write")
    close(total, new.sum(axis=0), 3e-6, "sum")
    for out_dtype in (torch.float32, torch.bfloat16):
        x = dev(xs)
        nxt = torch.empty((T, d), dtype=out_dtype, device=DEV)
        ops.stream_write(x, dev(y, ydtype), dev(mix), dev(cout), 1e-5, dev(cin), dev(gain), nxt)
        close(x, new, 3e-6, "write")
        close(nxt, plain.rmsnorm(np.tensordot(cin, new, 1), gain, 1e-5), TOL[out_dtype], "next")


def _paged(rows, page_size, table, pages_total, dtype):
    n, heads, width = rows.shape
    plane = torch.full((pages_total, heads, page_size, width), float("nan"), dtype=dtype, device=DEV)
    for j in range(n):
        plane[table[j // page_size], :, j % page_size, :] = dev(rows[j], dtype)
    return plane


def _table(rot, base, positions):
    from tgo_b200.config.spec import PositionSpec
    from tgo_b200.registry import POSITIONS
    part = POSITIONS.get("rope_half_split")(PositionSpec("rope_half_split", rotary_dim=rot, theta=base),
                                            rot, DEV)
    return part.table(SimpleNamespace(positions=ints(positions), aux={}))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,taps,rot,ps", [(4, 2, 12, 20, 3, 8, 8), (1, 1, 24, 24, 1, 24, 16),
                                               (6, 3, 10, 6, 5, 6, 4), (4, 1, 80, 80, 4, 80, 16),
                                               (2, 2, 16, 8, 2, 0, 8), (3, 1, 8, 8, 0, 4, 8)])
def test_projection_rows_convolved_rotated_normed_and_stored(H, G, a, b, taps, rot, ps, dtype):
    """Three requests (150, 9 and 1 tokens) cut into portions down to one token, in state slots
    that hold NaN elsewhere; the first token of the long one is loud, so a convolution that
    loses its kept rows at a portion's start shows at once. The first step holds all three, so
    that tokens whose taps all meet rows of the step lie beside tokens at the start of another
    request's portion, whose taps meet kept rows or nothing."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * 10 + taps)
    C = H * a + G * (a + b)
    eps = 1e-5
    lengths = [150, 9, 1]
    cuts = {0: [37, 1, 2, 1, 1, 60, 3, 45], 1: [2, 7], 2: [1]}
    raw = [vt.bf16_values(rng.normal(size=(n, C))) for n in lengths]
    raw[0][0] *= 6.0
    w = rng.normal(0, 0.7, (C, max(taps, 1))).astype(np.float32).astype(np.float64) if taps else None
    want = []
    for u in raw:
        n = u.shape[0]
        c = plain.short_conv(u, w) if taps else u
        q = c[:, :H * a].reshape(n, H, a)
        k = c[:, H * a:H * a + G * a].reshape(n, G, a)
        v = c[:, H * a + G * a:].reshape(n, G, b)
        if rot:
            q, k = plain.rotate_half_split(q, range(n), rot, 70.0), plain.rotate_half_split(k, range(n), rot, 70.0)
        want.append((plain.rms_unit(q, eps), plain.rms_unit(k, eps), v))
    keep = max(taps - 1, 0) * C
    slots_of = [3, 0, 2]
    state = torch.full((5, keep + 2), float("nan"), dtype=torch.float32, device=DEV)
    if keep:
        state[slots_of, :] = 0.0
    pages = [(n + ps - 1) // ps for n in lengths]
    perm = list(np.random.default_rng(3).permutation(np.arange(1, sum(pages) + 3)))
    tables = [perm[sum(pages[:i]):sum(pages[:i + 1])] for i in range(3)]
    total_pages = sum(pages) + 3
    kc = torch.full((total_pages, G, ps, a), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((total_pages, G, ps, b), float("nan"), dtype=dtype, device=DEV)
    got_q = [np.zeros((n, H, a)) for n in lengths]
    done = [0, 0, 0]
    for r in range(max(len(c) for c in cuts.values())):
        live = [i for i in range(3) if r < len(cuts[i])]
        spans = [(i, done[i], done[i] + cuts[i][r]) for i in live]
        T = sum(e - s for _, s, e in spans)
        rows = np.concatenate([raw[i][s:e] for i, s, e in spans])
        wide = dev(np.concatenate([np.zeros((T, 3)), rows, np.zeros((T, 5))], axis=1), dtype)
        qkv = wide[:, 3:3 + C]                                              # a view with a row stride
        positions = [p for _, s, e in spans for p in range(s, e)]
        seq = [j for j, (_, s, e) in enumerate(spans) for _ in range(s, e)]
        starts = np.cumsum([0] + [e - s for _, s, e in spans])
        slots = [tables[i][p // ps] * ps + p % ps for i, s, e in spans for p in range(s, e)]
        q_out = torch.empty((T, H * a), dtype=dtype, device=DEV)
        ops.qkv_conv_rope_norm_cache(qkv, q_out, H, G, a, b, dev(w) if taps else None, len(spans), ints(seq),
                                     ints(starts), ints([slots_of[i] for i, _, _ in spans]),
                                     state if keep else None, 0, _table(rot, 70.0, positions) if rot else None,
                                     rot, False, True, eps, ints(slots), kc, vc, ps)
        qh = host(q_out).reshape(T, H, a)
        for (i, s, e), at in zip(spans, starts):
            got_q[i][s:e] = qh[at:at + e - s]
            done[i] = e
    tol = TOL[dtype]
    for i, n in enumerate(lengths):
        close(torch.from_numpy(got_q[i]), want[i][0], tol, f"q of request {i}")
        for j in range(n):
            page, off = tables[i][j // ps], j % ps
            close(kc[page, :, off], want[i][1][j], tol, f"k {i} {j}")
            close(vc[page, :, off], want[i][2][j], tol, f"v {i} {j}")
    if keep:
        assert torch.isnan(state[[1, 4]]).all() and not torch.isnan(state[slots_of, :keep]).any()
        # the kept rows of the long request are its last taps - 1 projected rows
        close(state[3, :keep].reshape(taps - 1, C), raw[0][-(taps - 1):], 1e-6, "kept rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,coef,every", [(3, 1, 8, 16, 0.4, 5), (1, 1, 24, 24, 0.2, 1),
                                              (4, 2, 48, 48, 0.25, 32), (5, 5, 6, 7, 1.5, 3)])
def test_whole_row_norm_with_a_query_temperature(H, G, a, b, coef, every, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + a)
    positions = [0, 1, every - 1, every, 2 * every - 1, 2 * every, 63, 64, 700, 1000]
    T = len(positions)
    q = vt.bf16_values(rng.normal(size=(T, H * a)) * 2)
    k = vt.bf16_values(rng.normal(size=(T, G * a)))
    v = vt.bf16_values(rng.normal(size=(T, G * b)))
    gq = (1.5 + 0.4 * rng.normal(size=H * a)).astype(np.float32).astype(np.float64)
    gk = (1.5 + 0.4 * rng.normal(size=G * a)).astype(np.float32).astype(np.float64)
    wide = dev(np.concatenate([q, k, v], axis=1), dtype)
    qv, kv, vv = wide[:, :H * a], wide[:, H * a:H * a + G * a], wide[:, H * a + G * a:]
    ps = 4
    kc = torch.full((T + 1, G, ps, a), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((T + 1, G, ps, b), float("nan"), dtype=dtype, device=DEV)
    slots = [(t + 1) * ps + t % ps for t in range(T)]
    ops.qk_rownorm_rope_cache(qv, kv, vv, H, G, a, b, dev(gq), dev(gk), 1e-5, None, 0, False, ints(slots),
                              kc, vc, ps, ints(positions), coef, every)
    want_q = plain.rmsnorm(q, gq, 1e-5) * plain.query_temperature(positions, coef, every)[:, None]
    assert plain.query_temperature(positions, coef, every)[-1] > 1.0 + coef
    close(qv, want_q, TOL[dtype], "q")
    want_k = plain.rmsnorm(k, gk, 1e-5).reshape(T, G, a)
    for t in range(T):
        close(kc[t + 1, :, t % ps], want_k[t], TOL[dtype], "k")
        close(vc[t + 1, :, t % ps], v[t].reshape(G, b), TOL[dtype], "v")


def _attention_case(H, G, a, b, n, loud, rng, strength=4.0):
    """One request of n tokens whose keys in `loud` stand out for every query (a multiple of a
    direction all queries share), each with a value of its own: a key that is wrongly dropped
    or wrongly seen changes the result visibly."""
    q = rng.normal(size=(n, H, a))
    k = rng.normal(size=(n, G, a))
    v = rng.normal(size=(n, G, b))
    direction = rng.normal(size=a)
    direction /= np.linalg.norm(direction)
    q += 3.0 * direction
    for i, j in enumerate(loud):
        k[j] = (strength + 1.5 * math.sqrt(a)) * direction
        v[j] = 10.0 + 3.0 * i
    return vt.bf16_values(q), vt.bf16_values(k), vt.bf16_values(v)


def _plain_attention(q, k, v, scale, window, keep, rel, bias_max):
    n, H = q.shape[0], q.shape[1]
    vis = plain.visible_window_keep(n, window if window else n + 1, keep)
    bias = None
    if rel is not None:
        bias = np.zeros((H, n, n))
        for dist in range(n):
            idx = np.arange(dist, n)
            bias[:, idx, idx - dist] = rel[plain.distance_bucket(dist, rel.shape[0], bias_max)][:, None]
    return plain.softmax_attention(q, k, v, scale, vis, bias)


def _run_attention(fn, q, k, v, H, b, ps, dtype, positions):
    n = k.shape[0]
    pages = (n + ps - 1) // ps
    table = list(np.random.default_rng(7).permutation(np.arange(1, pages + 3))[:pages])
    kc = _paged(k, ps, table, pages + 3, dtype)
    vc = _paged(v, ps, table, pages + 3, dtype)
    bt = torch.zeros((2, pages + 2), dtype=torch.int32, device=DEV)
    bt[1, :pages] = ints(table)
    qq = dev(q[positions].reshape(len(positions), -1), dtype)
    out = torch.empty((len(positions), H * b), dtype=dtype, device=DEV)
    fn(qq, out, kc, vc, bt, ints([1] * len(positions)), ints(positions))
    return out


# (heads, kv heads, key size, value size, page, window, kept first)
WINDOWS = [(4, 2, 12, 20, 8, 7, 2), (4, 1, 80, 80, 16, 44, 5), (6, 3, 10, 6, 4, 3, 9), (2, 2, 16, 16, 8, 64, 64),
           (8, 2, 64, 64, 16, 70, 3), (3, 1, 32, 48, 16, 129, 70), (1, 1, 24, 24, 16, 300, 1)]


def _window_cases(window, keep, n):
    """Loud keys: the last kept one, the first that is not kept, the oldest key inside the
    window of the last query and the newest outside it."""
    last = n - 1
    return [[keep - 1] if keep else [], [keep], [last - window + 1], [last - window],
            [j for j in (keep - 1, last - window) if j >= 0], []]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,ps,window,keep", WINDOWS)
def test_window_with_kept_first_tokens_generic(H, G, a, b, ps, window, keep, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + a + window)
    n = 330
    picks = sorted(p for p in {0, 1, keep - 1 if keep else 0, keep, keep + 1, window - 1, window, window + 1,
                               window + keep - 1, window + keep, window + keep + 1, 63, 64, 65, 127, 128, 200,
                               n - 2, n - 1} if p < n)
    for loud in _window_cases(window, keep, n):
        q, k, v = _attention_case(H, G, a, b, n, loud, rng)
        want = _plain_attention(q, k, v, 0.3, window, keep, None, 0)

        def fn(qq, out, kc, vc, bt, seq, pos):
            ops.attention_generic(qq, out, H, G, a, kc, vc, ps, bt, seq, pos, 0.3, window, value_dim=b,
                                  keep_first=keep)
        close(_run_attention(fn, q, k, v, H, b, ps, dtype, picks), want[picks], TOL[dtype], f"loud {loud}")
    # the test sees what it is for: the kept key and the window's edge each move the last row
    q, k, v = _attention_case(H, G, a, b, n, [keep - 1] if keep else [n - window], rng)
    with_it = _plain_attention(q, k, v, 0.3, window, keep, None, 0)[n - 1]
    without = _plain_attention(q, k, v, 0.3, window, max(keep - 1, 0), None, 0)[n - 1] if keep else \
        _plain_attention(q, k, v, 0.3, window - 1, 0, None, 0)[n - 1]
    assert np.abs(with_it - without).max() > 1.0


TILE_WINDOWS = [(4, 2, 16, 24, 8, 7, 2), (4, 1, 80, 80, 16, 44, 5), (8, 2, 64, 64, 16, 70, 3), (3, 1, 32, 48, 16, 129, 70),
                (2, 2, 128, 128, 16, 64, 64), (20, 1, 16, 16, 16, 33, 5), (5, 5, 40, 40, 8, 200, 130)]


@pytest.mark.parametrize("H,G,a,b,ps,window,keep", TILE_WINDOWS)
def test_window_with_kept_first_tokens_on_the_tensor_cores(H, G, a, b, ps, window, keep):
    """The tile kernel over a prompt (tiles of consecutive tokens) and over single tokens whose
    keys are cut into 1, 2 and 5 shares."""
    from tgo_b200.kernels import ops
    assert ops.attention_sink_supports(H, G, a, b)
    rng = np.random.default_rng(H + a + window)
    n = 330
    per = ops.attention_sink_tile_tokens(H // G)
    for loud in _window_cases(window, keep, n):
        q, k, v = _attention_case(H, G, a, b, n, loud, rng)
        want = _plain_attention(q, k, v, 0.3, window, keep, None, 0)

        def tiles(qq, out, kc, vc, bt, seq, pos):
            T = qq.shape[0]
            tok0 = list(range(0, T, per))
            ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, window, None,
                                    ints(tok0), ints([min(per, T - t) for t in tok0]), keep_first=keep)
        close(_run_attention(tiles, q, k, v, H, b, ps, torch.bfloat16, list(range(n))), want, 2e-2,
              f"prompt, loud {loud}")
        picks = sorted(p for p in {0, keep, keep + 1, window - 1, window, window + keep, 63, 64, 127, 128, 129,
                                   n - 2, n - 1} if p < n)
        for splits in (1, 2, 5):
            def single(qq, out, kc, vc, bt, seq, pos):
                ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, window, None,
                                        n_splits=splits, keep_first=keep)
            close(_run_attention(single, q, k, v, H, b, ps, torch.bfloat16, picks), want[picks], 2e-2,
                  f"single tokens in {splits} shares, loud {loud}")


BIASES = [(3, 1, 8, 16, 8, 10, 30), (1, 1, 24, 24, 16, 2, 3), (4, 2, 64, 32, 16, 30, 110), (5, 5, 6, 7, 4, 7, 17),
          (20, 1, 16, 16, 16, 32, 200)]


@pytest.mark.parametrize("H,G,a,b,ps,rows,bias_max", BIASES)
def test_bias_by_distance(H, G, a, b, ps, rows, bias_max):
    """The table's buckets against the plain bucket function, then both attention kernels with
    a table in which one far bucket is loud for one head: the bias moves that head alone."""
    from tgo_b200.kernels import ops
    from tgo_b200.parts.attention_sink import bias_by_distance
    rng = np.random.default_rng(rows + bias_max)
    rel = vt.bf16_values(rng.normal(0, 1.5, (rows, H)))
    rel[rows - 1, 0] = 6.0
    table = bias_by_distance(dev(rel), bias_max)
    full = host(table)
    for dist in range(2 * bias_max + 5):
        assert np.array_equal(full[min(dist, full.shape[0] - 1)],
                              rel[plain.distance_bucket(dist, rows, bias_max)]), dist
    n = 2 * bias_max + 140
    q, k, v = _attention_case(H, G, a, b, n, [], rng)
    want = _plain_attention(q, k, v, 0.3, 0, 0, rel, bias_max)
    assert np.abs(want - _plain_attention(q, k, v, 0.3, 0, 0, None, 0)).max() > 0.1
    picks = sorted({0, 1, rows // 2 - 1, rows // 2, rows // 2 + 1, bias_max - 1, bias_max, bias_max + 1, 63, 64, n - 1})
    for dtype in (torch.float32, torch.bfloat16):
        def fn(qq, out, kc, vc, bt, seq, pos):
            ops.attention_generic(qq, out, H, G, a, kc, vc, ps, bt, seq, pos, 0.3, 0, value_dim=b,
                                  dist_bias=table)
        close(_run_attention(fn, q, k, v, H, b, ps, dtype, picks), want[picks], TOL[dtype], "generic")
    if not ops.attention_sink_supports(H, G, a, b):
        return
    per = ops.attention_sink_tile_tokens(H // G)

    def tiles(qq, out, kc, vc, bt, seq, pos):
        T = qq.shape[0]
        tok0 = list(range(0, T, per))
        ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, 0, None, ints(tok0),
                                ints([min(per, T - t) for t in tok0]), dist_bias=table)
    close(_run_attention(tiles, q, k, v, H, b, ps, torch.bfloat16, list(range(n))), want, 2e-2, "prompt")
    for splits in (1, 3):
        def single(qq, out, kc, vc, bt, seq, pos):
            ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, 0, None,
                                    n_splits=splits, dist_bias=table)
        close(_run_attention(single, q, k, v, H, b, ps, torch.bfloat16, picks), want[picks], 2e-2,
              f"single tokens in {splits} shares")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,E,ident,top,ff,shared", [(9, 48, 5, 1, 2, 24, 28), (1, 40, 3, 0, 1, 40, 0),
                                                      (150, 64, 12, 2, 3, 32, 40), (33, 36, 2, 2, 3, 20, 12),
                                                      (70, 64, 4, 0, 2, 64, 0), (5, 32, 1, 3, 4, 8, 8)])
def test_experts_chosen_by_corrected_scores_with_identity_and_a_gated_shared_one(T, d, E, ident, top, ff,
                                                                                shared, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(T + E)
    W = {}
    for e in range(E):
        W[f"e{e}.up"] = vt.bf16_values(rng.normal(0, 1.5 / math.sqrt(d), (ff, d)))
        W[f"e{e}.down"] = vt.bf16_values(rng.normal(0, 1 / math.sqrt(ff), (d, ff)))
    W["router"] = vt.bf16_values(rng.normal(0, 3 / math.sqrt(d), (E + ident, d)))
    # a correction large enough to change who is chosen, which must not change the weights
    W["correction"] = vt.bf16_values(rng.normal(0, 0.3, E + ident))
    mlp = {"router": {"experts": E, "identity": ident, "top": top}}
    if shared:
        W["shared.up"] = vt.bf16_values(rng.normal(0, 1.5 / math.sqrt(d), (shared, d)))
        W["shared.down"] = vt.bf16_values(rng.normal(0, 1 / math.sqrt(shared), (d, shared)))
        W["shared.sg"] = vt.bf16_values(rng.normal(0, 2 / math.sqrt(d), (1, d)))
        mlp["shared"] = {"ff": shared}
    x = vt.bf16_values(rng.normal(size=(T, d)))
    want = plain.routed_feed_forward(x, W, "", mlp)
    chosen, _ = plain.route(x, W, "", mlp["router"])
    plainly, _ = plain.route(x, {k: v for k, v in W.items() if k != "correction"}, "", mlp["router"])
    if T > 8 and E + ident > top:
        assert (np.sort(chosen, 1) != np.sort(plainly, 1)).any()          # the correction decides somewhere
        assert ident == 0 or (chosen >= E).any()                          # identity experts are used
    stack = lambda r: torch.stack([dev(W[f"e{e}.{r}"], dtype) for e in range(E)]).contiguous()   # noqa: E731
    router = W["router"] if not shared else np.concatenate([W["router"], W["shared.sg"]])
    extra = None
    if shared:
        extra = dev(plain.small_expert(x, W, "shared."))
    got = ops.moe_feed_forward(dev(x, dtype), dev(router), None, None, stack("up"), stack("down"), top,
                               "relu_squared", extra, "all", dev(W["correction"]), ident, bool(shared))
    close(got, want, 3e-5 if dtype == torch.float32 else 2e-2, "routed")


# ------------------------------------------------------------------- the engine, end to end
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page) in vt.CONFIGS.items():
        W = vt.make_weights(cfg, 13, vt.REL_ROWS[name])
        d = vt.write_model_dir(str(tmp_path_factory.mktemp("vimelorn" + name)), cfg, W)
        out[name] = (d, cfg, W, page)
    return out


def spread(d):
    d = d - d.mean()
    return math.sqrt((d * d).mean())


def bounds(cfg, W, requests, dtype):
    """Plain logits per request and the allowed spread of a difference. float32: rounding.
    bfloat16: three times what rounding the activations to bfloat16 does to the plain model's
    own logits on the same requests (the largest over their positions)."""
    want = {rid: plain.forward(cfg, W, toks) for rid, toks in requests.items()}
    if dtype == "float32":
        return want, None
    allowed = 3.0 * max(spread(row - want[rid][p]) for rid, toks in requests.items()
                        for p, row in enumerate(plain.forward_rounded(cfg, W, toks)))
    return want, allowed


def rows_close(got, cfg, W, requests, dtype):
    want, allowed = bounds(cfg, W, requests, dtype)
    assert got
    for (rid, p), row in got.items():
        err = spread(row.astype(np.float64) - want[rid][p])
        bound = 1e-4 * want[rid][p].std() if allowed is None else allowed
        assert err <= bound, (rid, p, err, bound)


FAMILIES = {"whole": tiny.trace_whole, "tail": lambda r: tiny.trace_tail(r, 12),
            "portions": tiny.trace_portions,
            "mixed": lambda r: tiny.trace_mixed(r, seed=4, max_live=4, tail=9)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("name", sorted(vt.CONFIGS))
def test_replay_against_plain(models, tmp_path, name, family, dtype):
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [90, 9, 1, 45, 33, 21], seed=6)
    trace = FAMILIES[family](requests)
    got = tiny.run_trace_program(d, dtype, trace, tmp_path / "out", cfg["vocab"],
                                 extra=["--page-size", str(page), "--max-live", "4"])
    assert len(got) == sum(len(t) for t in requests.values())
    rows_close(got, cfg, W, requests, dtype)


@pytest.mark.parametrize("name", ["V1", "V3", "V4"])
def test_float32_cuts_agree_and_pages_and_slots_come_back(models, name):
    """Every cutting gives the same float32 logits to rounding, with NaN in every page nobody
    holds (the pages a window has passed among them, the kept first ones not) and three state
    slots for six requests."""
    import tgo_b200
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [100, 17, 2, 40, 33, 65], seed=7)
    model = tgo_b200.open(d, dtype="float32")
    base = None
    for family in ("whole", "portions", "mixed"):
        trace = tiny.trace_mixed(requests, seed=1, max_live=3, tail=7) if family == "mixed" \
            else FAMILIES[family](requests)
        eng = model.new_engine(page_size=page, max_tokens=tiny.max_tokens_of(trace, page), num_slots=3)
        owners = [dict() for _ in eng.cache.groups]
        got = tiny.run_trace_engine(eng, trace, poison=True, owners=owners)
        rows_close(got, cfg, W, requests, "float32")
        if base is None:
            base = got
        for key, row in got.items():
            assert np.abs(row - base[key]).max() <= 2e-4 * max(1.0, np.abs(base[key]).max()), key
        if family == "mixed":
            assert any(len(ids) > 1 for g in owners for ids in g.values())


def test_a_window_gives_pages_back_and_keeps_the_first(models):
    """While a long request decodes, its window group holds the kept first pages and the
    window's, and nothing in between."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["V3"]
    model = tgo_b200.open(d, dtype="float32")
    toks = tiny.random_requests(cfg["vocab"], [200], seed=2)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=256, num_slots=1)
    eng.admit("a")
    eng.step([StepEntry("a", toks[:150], [])])
    for t in toks[150:]:
        eng.step([StepEntry("a", [t], [0])])
    held = tiny.held_pages(eng)
    windows = [g for g, grp in enumerate(eng.cache.groups) if grp.kind == "window"]
    assert windows
    for g in windows:
        grp = eng.cache.groups[g]
        most = (grp.keep_first + page - 1) // page + (grp.window + page - 1) // page + 1
        assert 0 < len(held[g]) <= most < 200 // page, (len(held[g]), most)


def test_a_batch_gives_each_request_what_it_gets_alone(models):
    """Unequal requests in one step (a long portion, a short one, single tokens) against the
    same requests each in an engine of its own: float32, to rounding."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["V1"]
    model = tgo_b200.open(d, dtype="float32")
    reqs = tiny.random_requests(cfg["vocab"], [41, 6, 19, 2], seed=21)
    alone = {}
    for rid, toks in reqs.items():
        eng = model.new_engine(page_size=page, max_tokens=64, num_slots=1)
        eng.admit(rid)
        head = max(1, len(toks) - 3)
        lg = eng.step([StepEntry(rid, toks[:head], [head - 1])]).float().cpu().numpy()
        alone[(rid, head - 1)] = lg[0]
        for p in range(head, len(toks)):
            alone[(rid, p)] = eng.step([StepEntry(rid, [toks[p]], [0])])[0].float().cpu().numpy()
    eng = model.new_engine(page_size=page, max_tokens=256, num_slots=4)
    for rid in reqs:
        eng.admit(rid)
    got = {}
    heads = {rid: max(1, len(t) - 3) for rid, t in reqs.items()}
    lg = eng.step([StepEntry(rid, reqs[rid][:heads[rid]], [heads[rid] - 1]) for rid in reqs])
    for i, rid in enumerate(reqs):
        got[(rid, heads[rid] - 1)] = lg[i].float().cpu().numpy()
    for r in range(3):
        live = [rid for rid in reqs if heads[rid] + r < len(reqs[rid])]
        if not live:
            break
        lg = eng.step([StepEntry(rid, [reqs[rid][heads[rid] + r]], [0]) for rid in live])
        for i, rid in enumerate(live):
            got[(rid, heads[rid] + r)] = lg[i].float().cpu().numpy()
    assert set(got) == set(alone)
    for key, row in got.items():
        assert np.abs(row - alone[key]).max() <= 2e-4 * max(1.0, np.abs(alone[key]).max()), key
    rows_close(got, cfg, W, reqs, "float32")


@pytest.mark.parametrize("name", ["V1", "V3"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_first_tokens_and_a_long_prompt(models, dtype, name):
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models[name]
    model = tgo_b200.open(d, dtype=dtype)
    toks = tiny.random_requests(cfg["vocab"], [150], seed=3)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=192, num_slots=2)
    eng.admit("a")
    got = {}
    for p, t in enumerate(toks):                       # from an empty cache, one by one (graphs)
        got[("a", p)] = eng.step([StepEntry("a", [t], [0])])[0].float().cpu().numpy()
    rows_close(got, cfg, W, {"a": toks}, dtype)
    # 1100 tokens in one step: the many-row products; then a few decoded
    long = tiny.random_requests(cfg["vocab"], [1106], seed=4)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=1152, num_slots=2)
    eng.admit("b")
    picks = [0, 7, 511, 1023, 1024, 1099]
    lg = eng.step([StepEntry("b", long[:1100], picks)]).float().cpu().numpy()
    rows = {("b", p): lg[i] for i, p in enumerate(picks)}
    for p in range(1100, 1106):
        rows[("b", p)] = eng.step([StepEntry("b", [long[p]], [0])])[0].float().cpu().numpy()
    want, allowed = bounds(cfg, W, {"b": long}, dtype)
    for (rid, p), g in rows.items():
        err = spread(g.astype(np.float64) - want["b"][p])
        assert err <= (2e-4 * want["b"][p].std() if allowed is None else allowed), (p, err)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_equal_portions_replayed_from_a_graph(models, dtype):
    """Portions of 256 tokens of one prompt: from the second on they run as a captured graph
    (the convolution's kept rows and the cache advance with every replay)."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["V1"]
    model = tgo_b200.open(d, dtype=dtype)
    toks = tiny.random_requests(cfg["vocab"], [256 * 3 + 5], seed=12)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=832, num_slots=2)
    eng.admit("p")
    got = {}
    for o in range(0, 768, 256):
        lg = eng.step([StepEntry("p", toks[o:o + 256], [0, 255])]).float().cpu().numpy()
        got[("p", o)], got[("p", o + 255)] = lg[0], lg[1]
    assert len(eng._portion_graphs) >= 1
    for p in range(768, len(toks)):
        got[("p", p)] = eng.step([StepEntry("p", [toks[p]], [0])])[0].float().cpu().numpy()
    want, allowed = bounds(cfg, W, {"p": toks}, dtype)
    for (_, p), g in got.items():
        err = spread(g.astype(np.float64) - want["p"][p])
        assert err <= (2e-4 * want["p"][p].std() if allowed is None else allowed), (p, err)


def test_greedy_generation_through_entry_point_scheduler_and_command_line(models):
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    d, cfg, W, page = models["V1"]
    prompts = list(tiny.random_requests(cfg["vocab"], [5, 17, 33, 1, 12], seed=8).values())
    want = [plain.greedy(cfg, W, p, 8) for p in prompts]
    assert len({t for o in want for t in o}) > 4
    model = tgo_b200.open(d, dtype="float32")
    assert model.generate(prompts, Policy(max_tokens=8), slots=3, chunk=16, page_size=page) == want
    # so few pages and slots that requests wait for others' to come back
    assert model.generate(prompts, Policy(max_tokens=8), slots=2, chunk=7, pool_tokens=96,
                          page_size=page) == want
    got = tgo_b200.open(d, dtype="bfloat16").generate(prompts, Policy(max_tokens=8), slots=4,
                                                      page_size=page)
    for p, o in zip(prompts, got):                       # bfloat16: each pick is near the best
        seq = list(p)
        for tok in o:
            z = plain.forward(cfg, W, seq)[-1]
            assert z.max() - z[tok] <= 0.25 * z.std()
            seq.append(tok)
    tgo = os.path.join(tiny.ROOT, "bin", "tgo")
    r = subprocess.run([sys.executable, tgo, "run", "--prompt", " ".join(map(str, prompts[1])),
                        "--max-tokens", "8", "--precision", "f32", "--context", "64", d],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == want[1]
    r = subprocess.run([sys.executable, tgo, "info", d], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "Vimelorn" in r.stdout
