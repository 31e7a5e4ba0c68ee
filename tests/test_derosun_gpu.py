"""Derosun on the GPU: every new kernel alone against the plain statement of its mechanism
(with inputs made so that a far key, an ignored cap, a lost or foreign state shows), then the
engine against the plain model: whole prompts, decoding, portions down to two tokens, mixed
batches with pages and state slots that come back, first tokens, long decoding, a long prompt,
and greedy generation through the library's entry point, the scheduler and the command line."""
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import derosun_tiny as dt
import plain_derosun as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(device=DEV, dtype=dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def close(got, want, tol, what=""):
    err = np.abs(host(got) - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err}"


TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}
BANDS = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
RAMP = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def table_of(kind, rot, base, scaling, positions):
    """The package's table of cosines and sines for these positions, from its position part."""
    from tgo_b200.config.spec import PositionSpec
    from tgo_b200.registry import POSITIONS
    keys = {"rope_banded": ("factor", "low", "high", "original"),
            "rope_stretched_interleaved": ("factor", "original", "fast", "slow")}[kind]
    sc = tuple(float(scaling[k]) for k in keys) if scaling else None
    part = POSITIONS.get(kind)(PositionSpec(kind, rotary_dim=rot, theta=base, scaling=sc), rot, DEV)
    return part.table(SimpleNamespace(positions=ints(positions), aux={}))


def rotated(x, positions, rot, base, scaling, interleaved):
    """x [T, heads, width] with the first `rot` channels of every head turned, plainly."""
    if interleaved:
        f, mag = plain.stretched_frequencies(rot, base, scaling)
    else:
        f, mag = plain.banded_frequencies(rot, base, scaling), 1.0
    out = np.array(x, dtype=np.float64)
    for t, p in enumerate(positions):
        for j in range(x.shape[1]):
            out[t, j] = plain.rotate(x[t, j], p, f, rot, interleaved, mag)
    return out


# ------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,alpha,bias", [(7, 48, 2.0, True), (1, 36, 1.0, False), (70, 200, 0.5, True),
                                            (3, 1030, 3.0, False)])
def test_norm_of_the_scaled_sum(T, d, alpha, bias, ydtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(T + d)
    h = rng.normal(size=(T, d)) * 3.0
    y = dt.bf16_values(rng.normal(size=(T, d)))
    g = rng.normal(size=d) + 1.0
    b = rng.normal(size=d) if bias else None
    want = plain.rms_norm(alpha * h.astype(np.float32).astype(np.float64) + y + (b if bias else 0.0),
                          g.astype(np.float32), 1e-5)
    for with_copy in (False, True):
        hh = dev(h)
        act = torch.empty((T, d), dtype=torch.bfloat16, device=DEV) if with_copy else None
        ops.scaled_add_norm(hh, dev(y, ydtype), dev(b) if bias else None, alpha, dev(g), 1e-5, act)
        close(hh, want, 3e-5, "stream")
        if with_copy:
            close(act, want, 1e-2, "the copy in the activation type")


def test_embedding_rows_times_a_factor():
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(0)
    table = dt.bf16_values(rng.normal(size=(37, 44)))
    ids = [5, 0, 36, 5]
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.empty((4, 44), dtype=torch.float32, device=DEV)
        ops.embed(dev(table, dtype), ints(ids), out, 0.3)
        close(out, table[ids] * np.float64(np.float32(0.3)), 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,f", [(5, 40), (1, 7), (66, 136)])
def test_gated_activation_with_biases(T, f, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(f)
    gu = dt.bf16_values(rng.normal(size=(T, 2 * f)) * 2.0)
    b = rng.normal(size=2 * f)
    b32 = b.astype(np.float32).astype(np.float64)
    out = torch.empty((T, f), dtype=dtype, device=DEV)
    ops.gated_act(dev(gu, dtype), out, False, "silu", dev(b))
    want = plain.silu(gu[:, :f] + b32[:f]) * (gu[:, f:] + b32[f:])
    close(out, want, TOL[dtype])


def _paged(rows, page_size, table, pages_total, dtype):
    """rows [n, heads, width] of one request laid into a plane [pages, heads, page, width]
    through its block table; unheld pages are NaN."""
    n, heads, width = rows.shape
    plane = torch.full((pages_total, heads, page_size, width), float("nan"), dtype=dtype, device=DEV)
    for j in range(n):
        plane[table[j // page_size], :, j % page_size, :] = dev(rows[j], dtype)
    return plane


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,rot,ps", [(4, 2, 12, 20, 8, 8), (1, 1, 24, 24, 24, 16), (6, 3, 10, 6, 6, 4),
                                            (8, 2, 64, 48, 32, 16), (5, 5, 8, 8, 0, 4)])
def test_rows_normed_whole_rotated_in_bands_and_stored(H, G, a, b, rot, ps, dtype):
    """q and k normed over ALL their heads at once (a norm per head gives other numbers), the
    first `rot` channels of every head turned in half-split pairs with banded frequencies, k
    and v stored at shuffled slots."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * a)
    positions = [0, 1, 63, 64, 500, 4000, 7]
    T = len(positions)
    q = dt.bf16_values(rng.normal(size=(T, H, a)) * np.linspace(0.2, 3.0, H)[None, :, None])
    k = dt.bf16_values(rng.normal(size=(T, G, a)) * np.linspace(3.0, 0.2, G)[None, :, None])
    v = dt.bf16_values(rng.normal(size=(T, G, b)))
    gq, gk = rng.normal(size=H * a) + 1.5, rng.normal(size=G * a) + 1.5
    eps = 1e-5
    qn = plain.rms_norm(q.reshape(T, -1), gq.astype(np.float32), eps).reshape(T, H, a)
    kn = plain.rms_norm(k.reshape(T, -1), gk.astype(np.float32), eps).reshape(T, G, a)
    if H > 1:
        per_head = plain.rms_norm(q, None, eps) * gq.astype(np.float32).reshape(H, a)
        assert np.abs(per_head - qn).max() > 0.1
    table = None
    if rot:
        qn = rotated(qn, positions, rot, 500.0, BANDS, False)
        kn = rotated(kn, positions, rot, 500.0, BANDS, False)
        table = table_of("rope_banded", rot, 500.0, BANDS, positions)
    qkv = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1), dtype)
    qw, kw = H * a, G * a
    pages = 6
    kc = torch.zeros((pages, G, ps, a), dtype=dtype, device=DEV)
    vc = torch.zeros((pages, G, ps, b), dtype=dtype, device=DEV)
    slots = list(rng.permutation(pages * ps)[:T])
    ops.qk_rownorm_rope_cache(qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:], H, G, a, b, dev(gq),
                              dev(gk), eps, table, rot, False, ints(slots), kc, vc, ps)
    close(qkv[:, :qw], qn.reshape(T, -1), TOL[dtype], "q")
    for t, s in enumerate(slots):
        close(kc[s // ps, :, s % ps, :], kn[t], TOL[dtype], "k")
        close(vc[s // ps, :, s % ps, :], v[t], TOL[dtype], "v")
    assert int((kc != 0).any(-1).any(1).sum()) <= T        # nothing else was written


def _attention_case(H, G, a, b, n, loud, rng, strength=4.0):
    """One request of n tokens whose key `loud` stands out for every query (a multiple of a
    direction that all queries share), with a value of its own: a far key that is dropped, or
    a cap that is left out, changes the result visibly."""
    q = rng.normal(size=(n, H, a))
    k = rng.normal(size=(n, G, a))
    v = rng.normal(size=(n, G, b))
    direction = rng.normal(size=a)
    direction /= np.linalg.norm(direction)
    q += 3.0 * direction
    if loud is not None:
        k[loud] = (strength + 1.5 * math.sqrt(a)) * direction
        v[loud] = 10.0
    return dt.bf16_values(q), dt.bf16_values(k), dt.bf16_values(v)


def _run_attention(fn, q, k, v, H, b, ps, dtype, positions, one_plane=False):
    """Queries at `positions` of one request whose n keys lie in shuffled pages."""
    n = k.shape[0]
    pages = (n + ps - 1) // ps
    table = list(np.random.default_rng(7).permutation(np.arange(1, pages + 3))[:pages])
    kc = _paged(k, ps, table, pages + 3, dtype)
    vc = kc if one_plane else _paged(v, ps, table, pages + 3, dtype)
    bt = torch.zeros((2, pages + 2), dtype=torch.int32, device=DEV)
    bt[1, :pages] = ints(table)
    qq = dev(q[positions].reshape(len(positions), -1), dtype)
    out = torch.empty((len(positions), H * b), dtype=dtype, device=DEV)
    fn(qq, out, kc, vc, bt, ints([1] * len(positions)), ints(positions))
    return out


CAP_SIZES = [(4, 2, 12, 20, 8), (8, 2, 64, 48, 16), (3, 3, 16, 8, 4), (6, 2, 88, 72, 16), (1, 1, 24, 24, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,ps", CAP_SIZES)
def test_capped_scores_generic(H, G, a, b, ps, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + a)
    n = 300
    for loud, cap in ((3, 2.5), (3, None), (250, 2.5), (None, 30.0), (0, 1.0)):
        q, k, v = _attention_case(H, G, a, b, n, loud, rng)
        want = plain.capped_softmax_attention(q, k, v, 0.3, cap).reshape(n, -1)

        def fn(qq, out, kc, vc, bt, seq, pos):
            ops.attention_generic(qq, out, H, G, a, kc, vc, ps, bt, seq, pos, 0.3, 0, value_dim=b,
                                  softcap=cap or 0.0)
        picks = [0, 1, 2, 3, 4, 63, 64, 65, 249, 250, 251, 299]
        close(_run_attention(fn, q, k, v, H, b, ps, dtype, picks), want[picks], TOL[dtype],
              f"loud {loud} cap {cap}")
    # the cap decides: with it the far loud key is one voice among many, without it the only one
    q, k, v = _attention_case(H, G, a, b, n, 3, rng)
    capped = plain.capped_softmax_attention(q, k, v, 0.3, 2.5)[299]
    free = plain.capped_softmax_attention(q, k, v, 0.3, None)[299]
    assert np.abs(capped - free).max() > 1.0
    q2, k2, v2 = q.copy(), k.copy(), v.copy()
    k2[3], v2[3] = k[4], v[4]
    assert np.abs(plain.capped_softmax_attention(q2, k2, v2, 0.3, 2.5)[299] - capped).max() > 0.02


TILE_CAP_SIZES = [(4, 2, 16, 24, 8), (12, 1, 64, 48, 16), (6, 2, 88, 72, 16), (2, 2, 128, 128, 16),
                  (40, 1, 8, 16, 16), (5, 5, 40, 40, 8)]


@pytest.mark.parametrize("H,G,a,b,ps", TILE_CAP_SIZES)
def test_capped_scores_on_the_tensor_cores(H, G, a, b, ps):
    """The tile kernel over a whole request, over a portion that starts in the middle of a page
    and of a key tile, and over single tokens with their keys in 1, 2 and 5 shares."""
    from tgo_b200.kernels import ops
    assert ops.attention_sink_supports(H, G, a, b)
    rng = np.random.default_rng(H + a)
    n, bf = 333, torch.bfloat16
    per = ops.attention_sink_tile_tokens(H // G)

    def tiles_of(count):
        t0 = list(range(0, count, per))
        return ints(t0), ints([min(per, count - t) for t in t0])

    for loud, cap in ((3, 2.5), (200, 2.5), (3, None), (None, 20.0), (64, 0.7)):
        q, k, v = _attention_case(H, G, a, b, n, loud, rng)
        want = plain.capped_softmax_attention(q, k, v, 0.3, cap).reshape(n, -1)
        for first, count in ((0, n), (123, 150), (200, 1)):
            def fn(qq, out, kc, vc, bt, seq, pos):
                t0, nt = tiles_of(count)
                ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, 0, None,
                                        t0, nt, softcap=cap or 0.0)
            picks = list(range(first, first + count))
            close(_run_attention(fn, q, k, v, H, b, ps, bf, picks), want[picks], 2e-2,
                  f"loud {loud} cap {cap} from {first}")
        for splits in (1, 2, 5):
            def single(qq, out, kc, vc, bt, seq, pos):
                ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, 0, None,
                                        n_splits=splits, softcap=cap or 0.0)
            picks = [0, 1, 2, 3, 4, 63, 64, 65, 199, 200, 201, 332]
            close(_run_attention(single, q, k, v, H, b, ps, bf, picks), want[picks], 2e-2,
                  f"single tokens in {splits} shares, loud {loud} cap {cap}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,rank,width,ps,tile", [(3, 20, 8, 8, False), (20, 48, 16, 16, True),
                                                  (4, 32, 32, 16, True), (5, 11, 6, 4, False),
                                                  (1, 40, 2, 16, False), (16, 96, 32, 16, True),
                                                  (2, 700, 20, 16, False)])
def test_attention_whose_values_are_the_head_of_its_key_rows(H, rank, width, ps, tile, dtype):
    """One cache plane, rows rank + width wide: the key is the whole row, the value its first
    `rank` channels. A far loud row must be found; the channels after `rank` must not leak."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + rank)
    n, row = 210, rank + width
    for loud in (2, 150, None):
        q, k, _ = _attention_case(H, 1, row, rank, n, loud, rng)
        k[:, :, rank:] *= 5.0                     # loud tails: a value that read them would show
        k = dt.bf16_values(k)
        v = k[:, :, :rank]
        want = plain.capped_softmax_attention(q, k, v, 0.1, None).reshape(n, -1)
        picks = [0, 1, 2, 3, 63, 64, 65, 149, 150, 151, 209]

        def generic(qq, out, kc, vc, bt, seq, pos):
            ops.attention_generic(qq, out, H, 1, row, kc, vc, ps, bt, seq, pos, 0.1, 0, value_dim=rank,
                                  value_row=row)
        close(_run_attention(generic, q, k, v, H, rank, ps, dtype, picks, one_plane=True), want[picks],
              TOL[dtype], f"generic, loud {loud}")
        if not tile or dtype != torch.bfloat16:
            continue
        assert ops.attention_sink_supports(H, 1, row, rank)
        per = ops.attention_sink_tile_tokens(H)

        def tiles(qq, out, kc, vc, bt, seq, pos):
            t0 = list(range(0, n, per))
            ops.attention_sink_tile(qq, out, H, 1, row, rank, kc, vc, ps, bt, seq, pos, 0.1, 0, None,
                                    ints(t0), ints([min(per, n - t) for t in t0]), value_row=row)
        close(_run_attention(tiles, q, k, v, H, rank, ps, dtype, list(range(n)), one_plane=True), want,
              2e-2, f"tiles, loud {loud}")
        for splits in (1, 3):
            def single(qq, out, kc, vc, bt, seq, pos):
                ops.attention_sink_tile(qq, out, H, 1, row, rank, kc, vc, ps, bt, seq, pos, 0.1, 0, None,
                                        n_splits=splits, value_row=row)
            close(_run_attention(single, q, k, v, H, rank, ps, dtype, picks, one_plane=True), want[picks],
                  2e-2, f"single tokens in {splits} shares, loud {loud}")


@pytest.mark.parametrize("H,rank,width,ps,cap", [(16, 512, 64, 16, None), (3, 200, 24, 8, None),
                                                 (70, 136, 16, 16, 3.0), (5, 104, 40, 4, None),
                                                 (2, 512, 8, 16, 2.0)])
def test_wide_rows_on_the_tensor_cores(H, rank, width, ps, cap):
    """Rows wider than 128 (up to 512 + 64), more heads than a tile has rows, a tile's key
    halves and value halves in different warps: tiles over a prompt, and single tokens with
    their keys in 1, 2 and 5 shares. A far loud row must be found in both."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + rank)
    n, row = 150, rank + width
    assert ops.attention_sink_wide_supports(H, 1, row, rank) and not ops.attention_sink_supports(H, 1, row, rank)
    per = ops.attention_sink_wide_tile_tokens(H)
    for loud in (1, 97, None):
        q, k, _ = _attention_case(H, 1, row, rank, n, loud, rng)
        k[:, :, rank:] *= 3.0
        k = dt.bf16_values(k)
        v = k[:, :, :rank]
        want = plain.capped_softmax_attention(q, k, v, 0.05, cap).reshape(n, -1)

        def tiles(qq, out, kc, vc, bt, seq, pos):
            t0 = list(range(0, n, per))
            ops.attention_sink_wide(qq, out, H, 1, row, rank, kc, ps, bt, seq, pos, 0.05, 0, None,
                                    ints(t0), ints([min(per, n - t) for t in t0]), softcap=cap or 0.0)
        close(_run_attention(tiles, q, k, v, H, rank, ps, torch.bfloat16, list(range(n)), one_plane=True),
              want, 2e-2, f"tiles, loud {loud}")
        picks = [0, 1, 2, 31, 32, 33, 63, 64, 96, 97, 98, 149]
        for splits in (1, 2, 5):
            def single(qq, out, kc, vc, bt, seq, pos):
                ops.attention_sink_wide(qq, out, H, 1, row, rank, kc, ps, bt, seq, pos, 0.05, 0, None,
                                        n_splits=splits, softcap=cap or 0.0)
            close(_run_attention(single, q, k, v, H, rank, ps, torch.bfloat16, picks, one_plane=True),
                  want[picks], 2e-2, f"single tokens in {splits} shares, loud {loud}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,width,rot,ps", [(20, 8, 8, 8), (11, 6, 4, 4), (40, 2, 2, 16), (48, 16, 16, 16),
                                               (64, 32, 0, 16)])
def test_latent_rows_normed_rotated_and_stored(rank, width, rot, ps, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(rank)
    positions = [0, 1, 31, 32, 33, 900, 5]
    T = len(positions)
    kv = dt.bf16_values(rng.normal(size=(T, rank + width)) * 2.0)
    gain = rng.normal(size=rank) + 1.5
    want = np.concatenate([plain.rms_norm(kv[:, :rank], gain.astype(np.float32), 1e-5), kv[:, rank:]], axis=1)
    table = None
    if rot:
        want[:, rank:] = rotated(kv[:, None, rank:], positions, rot, 100.0, RAMP, True)[:, 0]
        table = table_of("rope_stretched_interleaved", rot, 100.0, RAMP, positions)
    pages = 5
    cache = torch.zeros((pages, 1, ps, rank + width), dtype=dtype, device=DEV)
    slots = list(rng.permutation(pages * ps)[:T])
    wide = dev(np.concatenate([np.zeros((T, 8)), kv], axis=1), dtype)        # a view with a stride
    ops.latent_row_cache(wide[:, 8:], rank, width, dev(gain), 1e-5, table, rot, True, ints(slots),
                         cache, ps)
    for t, s in enumerate(slots):
        close(cache[s // ps, 0, s % ps], want[t], TOL[dtype], f"row {t}")
    assert int((cache != 0).any(-1).sum()) <= T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 9, 70])
@pytest.mark.parametrize("H,K,N", [(3, 12, 20), (5, 7, 11), (8, 24, 72), (1, 16, 40)])
def test_a_product_per_head_and_the_rotated_slice(H, K, N, T, dtype):
    """y_h = W_h x_h into rows wider than the result (the rest is another kernel's), and a slice
    of every head copied and turned beside it: together the query as the latent cache sees it."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * K + T)
    extra = 6
    x = dt.bf16_values(rng.normal(size=(T, H, K + extra)))
    w = dt.bf16_values(rng.normal(size=(H, N, K)) / math.sqrt(K))
    y = torch.zeros((T, H * (N + extra)), dtype=dtype, device=DEV)
    xx = dev(x.reshape(T, -1), dtype)
    ops.head_linear(xx, K + extra, dev(w, dtype), y, N + extra)
    positions = list(range(40, 40 + T))
    table = table_of("rope_stretched_interleaved", 4, 100.0, RAMP, positions)
    ops.rope_slice(xx, K + extra, K, y, N + extra, N, H, extra, table, 4, True)
    want = np.zeros((T, H, N + extra))
    want[:, :, :N] = np.einsum("thk,hnk->thn", x[:, :, :K], w)
    want[:, :, N:] = rotated(x[:, :, K:], positions, 4, 100.0, RAMP, True)
    close(y, want.reshape(T, -1), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("form", ["in order", "by chunks"])
@pytest.mark.parametrize("H,dk,dv", [(3, 8, 12), (1, 24, 24), (2, 5, 7), (2, 32, 48), (4, 16, 40), (2, 128, 72)])
def test_matrix_memory_over_portions_and_slots(H, dk, dv, form, dtype):
    """Three requests of unequal length in one call, then each continued in portions that end
    before, on and after the kernels' chunks of tokens, in state slots given out of order, by
    the kernels that walk a request in order and by those that take its chunks side by side
    (and, when every request brings one token, stream the state through once); one
    early token of the long request is written loudly (a wide-open input gate, forget gates
    nearly 1 after it), so that a state that is lost, reset or taken from another slot shows
    in every later output. A slot that is used again starts from zeros the caller wrote."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * dk + dv)
    cap, q_scale = 9.0, dk ** -0.5
    lengths = [297, 33, 1]
    cuts = {0: [31, 1, 32, 2, 64, 1, 1, 165], 1: [32, 1], 2: [1]}
    reqs = []
    for n in lengths:
        q = dt.bf16_values(rng.normal(size=(n, H, dk)))
        k = dt.bf16_values(rng.normal(size=(n, H, dk)))
        v = dt.bf16_values(rng.normal(size=(n, H, dv)))
        a = rng.normal(size=(n, H)) * 3.0
        c = rng.normal(size=(n, H)) * 3.0 + 2.0
        if n > 50:
            a[3], c[4:] = 30.0, 25.0
            v[3] *= 4.0
        reqs.append((q, k, v, a.astype(np.float32).astype(np.float64),
                     c.astype(np.float32).astype(np.float64)))
    bi = rng.normal(size=H).astype(np.float32).astype(np.float64)
    bf = rng.normal(size=H).astype(np.float32).astype(np.float64)
    want = []
    for q, k, v, a, c in reqs:
        gi, gf = plain.log_gates(a + bi, c + bf, cap)
        want.append(plain.gated_memory(q * q_scale, k, v, gi, gf)[0])
    floats = ops.mlstm_state_floats(H, dk, dv)
    slots = [4, 0, 2]
    state = torch.full((5, floats + 3), float("nan"), dtype=torch.float32, device=DEV)
    state[slots] = 0.0
    got = [np.zeros_like(w) for w in want]
    done = [0, 0, 0]
    rounds = max(len(c) for c in cuts.values())
    for r in range(rounds):
        live = [i for i in range(3) if r < len(cuts[i])]
        spans = [(i, done[i], done[i] + cuts[i][r]) for i in live]
        cat = lambda j: np.concatenate([reqs[i][j][s:e] for i, s, e in spans])
        T = sum(e - s for _, s, e in spans)
        pad = 5                                                        # views with a row stride
        wide = dev(np.concatenate([cat(0).reshape(T, -1), np.zeros((T, pad)), cat(1).reshape(T, -1),
                                   cat(2).reshape(T, -1)], axis=1), dtype)
        qv, kv_ = wide[:, :H * dk], wide[:, H * dk + pad:2 * H * dk + pad]
        vv = wide[:, 2 * H * dk + pad:]
        g = dev(np.concatenate([cat(3), cat(4)], axis=1))
        out = torch.empty((T, H * dv), dtype=torch.float32, device=DEV)
        starts = np.cumsum([0] + [e - s for _, s, e in spans])
        args = (qv, kv_, vv, g[:, :H], g[:, H:], dev(bi), dev(bf), cap, q_scale, out, len(spans),
                H, dk, dv, ints(starts), ints([slots[i] for i, _, _ in spans]), state)
        if form == "in order":
            ops.mlstm(*args)
        elif all(e - s == 1 for _, s, e in spans):
            ops.mlstm_chunked(*args)
        else:
            most = ops.mlstm_chunk_tokens()
            tok0, ntok, first = [], [], []
            for (_, s, e), at in zip(spans, starts):
                first.append(len(tok0))
                for o in range(0, e - s, most):
                    tok0.append(int(at) + o)
                    ntok.append(min(most, e - s - o))
            ops.mlstm_chunked(*args, ints(tok0), ints(ntok), ints(first))
        o = host(out).reshape(T, H, dv)
        for (i, s, e), at in zip(spans, starts):
            got[i][s:e] = o[at:at + e - s]
            done[i] = e
    for i in range(3):
        assert done[i] == lengths[i]
        # per token: where n . q passes near zero the read-out is large and as ill-conditioned
        # as that sum of terms of both signs, in any float32 order
        size = np.maximum(np.abs(want[i]).max(axis=(1, 2)), np.median(np.abs(want[i]).max(axis=(1, 2))))
        err = np.abs(got[i] - want[i]).max(axis=(1, 2))
        assert (err <= 1e-3 * size).all() and np.median(err / size) <= 2e-5, (i, (err / size).max())
    assert torch.isnan(state[[1, 3]]).all() and not torch.isnan(state[slots, :floats]).any()
    # the loud token is still there at the end of the long request
    quiet = plain.gated_memory(reqs[0][0][4:] * q_scale, reqs[0][1][4:], reqs[0][2][4:],
                               *plain.log_gates(reqs[0][3][4:] + bi, reqs[0][4][4:] + bf, cap))[0]
    assert np.abs(quiet[-1] - want[0][-1]).max() > 0.05 * np.abs(want[0][-1]).max()


# ------------------------------------------------------------------- the engine, end to end
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page) in dt.CONFIGS.items():
        W = dt.make_weights(cfg, 13)
        d = dt.write_model_dir(str(tmp_path_factory.mktemp("derosun" + name)), cfg, W)
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
                        for p, row in enumerate(plain.forward(cfg, W, toks, rnd=dt.bf16_values)))
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
@pytest.mark.parametrize("name", sorted(dt.CONFIGS))
def test_replay_against_plain(models, tmp_path, name, family, dtype):
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [70, 9, 1, 45, 33, 21], seed=6)
    trace = FAMILIES[family](requests)
    got = tiny.run_trace_program(d, dtype, trace, tmp_path / "out", cfg["vocab"],
                                 extra=["--page-size", str(page), "--max-live", "4"])
    assert len(got) == sum(len(t) for t in requests.values())
    rows_close(got, cfg, W, requests, dtype)


@pytest.mark.parametrize("name", ["D1", "D4", "D5"])
def test_float32_cuts_agree_and_pages_and_slots_come_back(models, name):
    """Every cutting gives the same float32 logits to rounding, with NaN in every page nobody
    holds and three state slots for six requests."""
    import tgo_b200
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [64, 17, 2, 40, 33, 65], seed=7)
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


def test_a_batch_gives_each_request_what_it_gets_alone(models):
    """Unequal requests in one step (a long portion, a short one, single tokens) against the
    same requests each in an engine of its own: float32, to rounding."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["D1"]
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


@pytest.mark.parametrize("name", ["D1", "D5"])
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
    (the memory's state and the cache advance with every replay)."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["D1"]
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
    d, cfg, W, page = models["D1"]
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
    assert r.returncode == 0 and "Derosun" in r.stdout
