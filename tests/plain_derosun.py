"""Plain statement of the Derosun design in numpy float64: one function per mechanism, whole
sequences from position 0, no cache, no batching. The tests hold the engine to it; it shares
no code with the package.

A model is (config dict in the form of the design's config.json, dict of numpy arrays by
tensor name). Matrices are [out, in] and applied as W x.
"""
from __future__ import annotations

import math

import numpy as np


# ------------------------------------------------------------------ small pieces

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    x = np.asarray(x, dtype=np.float64)
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * np.asarray(w, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def softmax(s):
    s = s - np.max(s)
    e = np.exp(s)
    return e / np.sum(e)


# ------------------------------------------------------------------ rotations

def base_frequencies(dims, base):
    i = np.arange(dims // 2, dtype=np.float64)
    return base ** (-2.0 * i / dims)


def banded_frequencies(dims, base, scaling):
    """Frequencies slowed by wavelength bands: short waves keep f, long waves get f / factor,
    those between are blended linearly in original / wavelength."""
    f = base_frequencies(dims, base)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out[i] = fi
        elif wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def stretched_frequencies(dims, base, scaling):
    """(frequencies, magnitude) of the rotation stretched by a ramp over the pairs."""
    f = base_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))

    def turns(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns(fast)), 0)
    hi = min(math.ceil(turns(slow)), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, position, freqs, dims, interleaved, magnitude=1.0):
    """The first `dims` entries of the vector x turned by position * freqs: pair i is
    (i, i + dims/2), or (2i, 2i + 1) if `interleaved`."""
    x = np.array(x, dtype=np.float64)
    out = x.copy()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + dims // 2)
        ang = position * freqs[i]
        c, s = math.cos(ang) * magnitude, math.sin(ang) * magnitude
        out[a] = x[a] * c - x[b] * s
        out[b] = x[b] * c + x[a] * s
    return out


# ------------------------------------------------------------------ mixers

def _same(x):
    return x


def capped_softmax_attention(q, k, v, scale, cap=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], already normed and rotated: causal softmax of
    the scaled scores, each bounded by cap tanh(s / cap) if cap is given -> [T, H, dv]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for j in range(H):
            g = j // (H // G)
            s = (k[:t + 1, g] @ q[t, j]) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            out[t, j] = softmax(s) @ v[:t + 1, g]
    return out


def attention(h, w, m, eps, prefix, rnd=_same):
    """Grouped-query softmax attention: q and k normed over their whole projection rows,
    half-split rotation with banded frequencies, scores through a soft cap. h [T, d]."""
    T = h.shape[0]
    H, G, dk = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", dk)
    q = rms_norm(rnd(h @ w[prefix + "q"].T), w[prefix + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(rnd(h @ w[prefix + "k"].T), w[prefix + "k.norm"], eps).reshape(T, G, dk)
    v = rnd(h @ w[prefix + "v"].T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        f = banded_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        for t in range(T):
            for j in range(H):
                q[t, j] = rotate(q[t, j], t, f, rot["dims"], False)
            for j in range(G):
                k[t, j] = rotate(k[t, j], t, f, rot["dims"], False)
    out = capped_softmax_attention(rnd(q), rnd(k), v, m["scale"], m.get("softcap"))
    return rnd(out).reshape(T, H * dv) @ w[prefix + "o"].T


def latent_attention(h, w, m, eps, prefix, rnd=_same):
    """Attention whose keys and values are expanded from one small latent per token, with one
    rotated key part shared by all heads; queries through a latent of their own."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rnd(rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps))
    q = rnd(cq @ w[prefix + "uq"].T).reshape(T, H, dn + dr)
    kv = rnd(h @ w[prefix + "dkv"].T)
    c = rnd(rms_norm(kv[:, :rank], w[prefix + "dkv.norm"], eps))
    kr = kv[:, rank:].copy()
    kn = (c @ w[prefix + "uk"].T).reshape(T, H, dn)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, dv)
    rot = m.get("rot")
    if rot:
        f, mag = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        for t in range(T):
            kr[t] = rotate(kr[t], t, f, rot["dims"], True, mag)
            for j in range(H):
                q[t, j, dn:] = rotate(q[t, j, dn:], t, f, rot["dims"], True, mag)
    kr, q = rnd(kr), rnd(q)
    out = np.zeros((T, H, dv))
    for t in range(T):
        for j in range(H):
            s = (kn[:t + 1, j] @ q[t, j, :dn] + kr[:t + 1] @ q[t, j, dn:]) * m["scale"]
            out[t, j] = softmax(s) @ v[:t + 1, j]
    return rnd(out).reshape(T, H * dv) @ w[prefix + "o"].T


def gated_memory(q, k, v, gi, gf, state=None):
    """The recurrence alone. q, k [T, H, dk] (q already scaled), v [T, H, dv], log gates gi, gf
    [T, H]; per head m_t = max(gf + m, gi), S_t = e^(gf + m - m_t) S + e^(gi - m_t) k v^T, n_t
    likewise with k, o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6); S, n and m start at 0.
    Returns (o [T, H, dv], (S, n, m))."""
    T, H, dk = q.shape
    dv = v.shape[2]
    if state is None:
        S, n, mx = np.zeros((H, dk, dv)), np.zeros((H, dk)), np.zeros(H)
    else:
        S, n, mx = (np.array(a, dtype=np.float64) for a in state)
    o = np.zeros((T, H, dv))
    for t in range(T):
        for j in range(H):
            m_new = max(gf[t, j] + mx[j], gi[t, j])
            keep, take = math.exp(gf[t, j] + mx[j] - m_new), math.exp(gi[t, j] - m_new)
            S[j] = keep * S[j] + take * np.outer(k[t, j], v[t, j])
            n[j] = keep * n[j] + take * k[t, j]
            mx[j] = m_new
            o[t, j] = (S[j].T @ q[t, j]) / (max(abs(n[j] @ q[t, j]), math.exp(-m_new)) + 1e-6)
    return o, (S, n, mx)


def log_gates(a, c, cap):
    """Raw gate rows a (input), c (forget) with their biases added -> (log input gate, log
    forget gate): cap tanh(a / cap) and logsigmoid(cap tanh(c / cap))."""
    return cap * np.tanh(a / cap), log_sigmoid(cap * np.tanh(c / cap))


def mlstm(h, w, m, eps, prefix, state=None, rnd=_same):
    """Matrix memory with exponential gates kept stable by a running maximum that starts at
    0. Returns (output [T, d], final state (S, n, m) per head)."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m.get("vdim", m["dim"]), m["gate_cap"]
    q = rnd(h @ w[prefix + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = rnd(h @ w[prefix + "k"].T).reshape(T, H, dk)
    v = rnd(h @ w[prefix + "v"].T).reshape(T, H, dv)
    gi, gf = log_gates(h @ w[prefix + "i"].T + w[prefix + "i.b"],
                       h @ w[prefix + "f"].T + w[prefix + "f.b"], cap)
    o, state = gated_memory(q, k, v, gi, gf, state)
    o = rms_norm(o, None, eps).reshape(T, H * dv) * w[prefix + "norm"]
    o = o * sigmoid(rnd(h @ w[prefix + "g"].T))
    return rnd(o) @ w[prefix + "o"].T, state


MIXERS = {"attention": attention, "latent_attention": latent_attention,
          "mlstm": lambda h, w, m, eps, p, rnd=_same: mlstm(h, w, m, eps, p, rnd=rnd)[0]}


# ------------------------------------------------------------------ the rest

def feed_forward(h, w, prefix, rnd=_same):
    g = rnd(h @ w[prefix + "gate"].T) + w[prefix + "gate.b"]
    u = rnd(h @ w[prefix + "up"].T) + w[prefix + "up.b"]
    return rnd(silu(g) * u) @ w[prefix + "down"].T + w[prefix + "down.b"]


def forward(cfg, w, tokens, layers_out=None, rnd=None):
    """Logits [T, vocab] of a whole sequence; `layers_out`, a list, receives the stream after
    every layer. `rnd`, a rounding of arrays (to bfloat16, say), is applied where an engine
    that keeps activations in that type would round: what the sublayers read, what the
    projections give, what the last products read."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    rnd = rnd or _same
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    x = w["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](rnd(x), w, layer["mixer"], eps, p + "mix.", rnd)
        x = rms_norm(alpha * x + y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = rms_norm(alpha * x + feed_forward(rnd(x), w, p + "mlp.", rnd), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def greedy(cfg, w, prompt, n):
    """The n tokens that picking the largest logit (the lowest id among equals) appends."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(np.argmax(forward(cfg, w, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def round_bf16(a):
    """Values rounded to bfloat16 (nearest even), as float64."""
    a = np.asarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64)
