"""The Vimelorn design stated plainly: numpy float64, one function per mechanism, a whole
sequence at a time, no cache, no batching. It shares no code with the package and is what the
tests hold the engine to.

A model is (config dict as config.json gives it, dict name -> float64/int array).

    x_0 = embed[token] * embedding.scale, copied into `streams` streams
    per layer and sublayer q (mixer, feed-forward):
        u   = sum_s in_q[s] x_s
        y   = sublayer(rmsnorm(u) * w)
        x_t = sum_s mix_q[s, t] x_s + out_q[t] y            (all t from the old streams)
    logits = head (rmsnorm(sum_s x_s) * final.norm)

Without `streams` in the config a layer is the ordinary pre-norm residual pair.
"""
import math

import numpy as np


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rmsnorm(x, w, eps):
    return rms_unit(x, eps) * w


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * w[:, j][None, :]
    return y


def rotate_half_split(x, positions, dims, base):
    """x [T, heads, dim]: the first `dims` channels of every head rotated, channel i paired with
    i + dims/2, angle position * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]       # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def visible_window_keep(T, size, keep_first):
    """[T, T] booleans: i sees j if j <= i and (i - j < size or j < keep_first)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def distance_bucket(n, rows, bias_max):
    """Row of the distance table for a distance n >= 0: the distance itself below rows/2, then
    logarithmic steps up to bias_max, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half)
                                               * (rows - half))))


def softmax_attention(q, k, v, scale, visible, bias=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; visible [T, T]; bias [H, T, T] or None.
    Query head h reads kv head h // (H / G). -> [T, H * dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if bias is not None:
            s = s + bias[h]
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w /= w.sum(axis=1, keepdims=True)
        out[:, h] = w @ v[:, g]
    return out.reshape(T, -1)


def mixer_attention(h, W, p, m, eps):
    """The windowed mixer: projections, a short convolution on each, rotation, unit norm per
    head of q and k, a window that keeps the first tokens."""
    T = h.shape[0]
    H, G, dk = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", dk)
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, W[p + "q.conv"]), short_conv(k, W[p + "k.conv"]), \
            short_conv(v, W[p + "v.conv"])
    q, k, v = q.reshape(T, H, dk), k.reshape(T, G, dk), v.reshape(T, G, dv)
    pos = np.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half_split(q, pos, rot["dims"], rot["base"])
        k = rotate_half_split(k, pos, rot["dims"], rot["base"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    mask = m.get("mask")
    vis = visible_window_keep(T, mask["size"], mask.get("keep_first", 0)) if mask else \
        visible_window_keep(T, T + 1, 0)
    a = softmax_attention(q, k, v, m["scale"], vis)
    return a @ W[p + "o"].T


def query_temperature(positions, coef, every):
    return 1.0 + coef * np.log(np.floor((np.asarray(positions) + 1) / every) + 1.0)


def mixer_attention_2(h, W, p, m, eps):
    """The causal mixer: q and k normed over their whole rows, no rotation, a query temperature
    that grows with the position, a learned bias by distance."""
    T = h.shape[0]
    H, G, dk = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", dk)
    q = rmsnorm(h @ W[p + "q"].T, W[p + "q.norm"], eps)
    k = rmsnorm(h @ W[p + "k"].T, W[p + "k.norm"], eps)
    v = h @ W[p + "v"].T
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(np.arange(T), qt["coef"], qt["every"])[:, None]
    q, k, v = q.reshape(T, H, dk), k.reshape(T, G, dk), v.reshape(T, G, dv)
    rel = W[p + "rel"]                                    # [rows, H]
    rows = rel.shape[0]
    bias = np.zeros((H, T, T))
    for n in range(T):
        b = rel[distance_bucket(n, rows, m["bias_max"])]
        idx = np.arange(n, T)
        bias[:, idx, idx - n] = b[:, None]
    vis = visible_window_keep(T, T + 1, 0)
    a = softmax_attention(q, k, v, m["scale"], vis, bias)
    return a @ W[p + "o"].T


def silu(z):
    return z / (1.0 + np.exp(-z))


def relu_squared(z):
    return np.maximum(z, 0.0) ** 2


def dense_feed_forward(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def small_expert(h, W, p):
    return relu_squared(h @ W[p + "up"].T) @ W[p + "down"].T


def route(h, W, p, r):
    """-> (chosen [T, top] expert indices, weights [T, top]). Softmax over all experts (identity
    ones included); the choice adds the correction, the weights do not."""
    z = h @ W[p + "router"].T
    z = z - z.max(axis=1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=1, keepdims=True)
    choice = s + W[p + "correction"][None, :] if (p + "correction") in W else s
    top = r["top"]
    chosen = np.argsort(-choice, axis=1, kind="stable")[:, :top]
    w = np.take_along_axis(s, chosen, axis=1)
    return chosen, w / (w.sum(axis=1, keepdims=True) + 1e-20)


def routed_feed_forward(h, W, p, mlp):
    r = mlp["router"]
    E, n_id = r["experts"], r.get("identity", 0)
    chosen, w = route(h, W, p, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t], w[t]):
            if e >= E:
                assert e < E + n_id
                out[t] += we * h[t]
            else:
                out[t] += we * small_expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        gate = 1.0 / (1.0 + np.exp(-(h @ W[p + "shared.sg"].T)))            # [T, 1]
        out += gate * small_expert(h, W, p + "shared.")
    return out


def feed_forward(h, W, p, mlp):
    if mlp.get("kind", "dense") == "dense":
        return dense_feed_forward(h, W, p)
    return routed_feed_forward(h, W, p, mlp)


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2}


def forward(cfg, W, tokens, layer_outputs=None):
    """Logits [T, vocab] of one sequence. `layer_outputs`, a list, gets the stream (the sum of
    the streams) after every layer."""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    S = cfg.get("streams")
    xs = [x0.copy() for _ in range(S)] if S else None
    x = x0
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [(1, lambda u, L=layer, p=p: MIXERS[L["type"]](u, W, p + "mix.", L["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda u, L=layer, p=p: feed_forward(u, W, p + "mlp.", L["mlp"])))
        for qn, fn in subs:
            gain = W[f"{p}norm{qn}"]
            if S:
                cin, cout, mix = W[f"{p}hc{qn}.in"], W[f"{p}hc{qn}.out"], W[f"{p}hc{qn}.mix"]
                u = sum(cin[s] * xs[s] for s in range(S))
                y = fn(rmsnorm(u, gain, eps))
                xs = [sum(mix[s, t] * xs[s] for s in range(S)) + cout[t] * y for t in range(S)]
            else:
                x = x + fn(rmsnorm(x, gain, eps))
        if S:
            x = sum(xs)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return rmsnorm(x, W["final.norm"], eps) @ W["head"].T


def forward_rounded(cfg, W, tokens):
    """The same with every sublayer's input rounded to bfloat16: what rounding the activations
    does to the logits, the yardstick of the bfloat16 engine's bound."""
    def bf16(a):
        b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return r.view(np.float32).astype(np.float64)

    saved = globals()["rmsnorm"]

    def rounded(x, w, eps):
        return bf16(saved(x, w, eps))

    globals()["rmsnorm"] = rounded
    try:
        return forward(cfg, W, tokens)
    finally:
        globals()["rmsnorm"] = saved


def greedy(cfg, W, prompt, n):
    """n tokens after `prompt`, each the most likely next one (ties: the lower id)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(np.argmax(forward(cfg, W, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
