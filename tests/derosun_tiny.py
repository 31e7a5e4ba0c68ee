"""Small Derosun configurations with weights of the tests' own making.

  D1: every size different from every other: a matrix-memory layer with three heads and a
      feed-forward, grouped attention (4/2 heads, values wider than keys, a partial rotation
      whose pairs fall into all three wavelength bands, a soft cap) without a feed-forward,
      latent attention (latents of 20 and 28, 12 unrotated and 8 rotated channels, a ramp
      that leaves one pair alone, blends one and slows two), a second matrix-memory layer
      without a feed-forward; the stream doubled before each norm, the embedding halved.
  D2: the values a model may happen to make equal or 1: kv heads = heads, key size = value
      size, a rotation of the whole head without scaling, no soft cap, one attention head, one
      memory head, a rotated part of one pair, stream factor 1, no embedding factor, a latent
      as wide as the model.
  D3: matrix-memory layers only: no layer owns a paged cache.
  D4: sizes that no kernel's fast form takes (a width, head sizes, latents, a feed-forward and
      a vocabulary that are not multiples of 8).
  D5: sizes the tensor-core attention takes (head sizes and the latent row multiples of 16),
      more attention heads per kv head than a decode tile of 16 rows in one layer and fewer in
      the other.
  D6: latent rows wider than 128 (the tensor-core kernel whose key tiles serve as values), more
      heads than one of its tiles has rows in one layer and three in the other.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def _attn(H, G, dim, vdim, rot, scale, cap):
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if cap is not None:
        m["softcap"] = cap
    return m


def _latent(H, dim, rot_dim, vdim, kv_rank, q_rank, rot, scale):
    return {"heads": H, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "q_rank": q_rank, "rot": rot, "scale": scale}


def _mem(H, dim, vdim, cap):
    return {"heads": H, "dim": dim, "vdim": vdim, "gate_cap": cap}


D1 = {
    "architecture": "Derosun", "vocab": 89, "width": 48, "norm": {"eps": 1e-5},
    "postln_alpha": 2.0, "embedding": {"scale": 0.5},
    "layers": [
        {"type": "mlstm", "mixer": _mem(3, 8, 12, 10.0), "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention",
         "mixer": _attn(4, 2, 12, 20, {"dims": 8, "base": 500.0,
                                       "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                        0.3, 5.0),
         "mlp": None},
        {"type": "latent_attention",
         "mixer": _latent(3, 12, 8, 10, 20, 28,
                          {"dims": 8, "base": 100.0,
                           "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}, 0.25),
         "mlp": {"kind": "dense", "ff": 56}},
        {"type": "mlstm", "mixer": _mem(2, 16, 4, 6.0), "mlp": None},
    ],
}

D2 = {
    "architecture": "Derosun", "vocab": 70, "width": 40, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "layers": [
        {"type": "attention", "mixer": _attn(1, 1, 24, 24, {"dims": 24, "base": 30.0}, 0.2, None),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "mlstm", "mixer": _mem(1, 24, 24, 15.0), "mlp": None},
        {"type": "latent_attention",
         "mixer": _latent(1, 16, 2, 16, 40, 40, {"dims": 2, "base": 7.0}, 0.3),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": _attn(5, 5, 8, 8, None, 0.35, 30.0), "mlp": None},
    ],
}

D3 = {
    "architecture": "Derosun", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
    "embedding": {"scale": 2.0},
    "layers": [
        {"type": "mlstm", "mixer": _mem(2, 16, 20, 8.0), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "mlstm", "mixer": _mem(8, 4, 6, 20.0), "mlp": None},
    ],
}

D4 = {
    "architecture": "Derosun", "vocab": 53, "width": 36, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
    "embedding": {"scale": 0.7},
    "layers": [
        {"type": "latent_attention",
         "mixer": _latent(5, 6, 6, 7, 11, 13,
                          {"dims": 4, "base": 40.0,
                           "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}}, 0.4),
         "mlp": None},
        {"type": "mlstm", "mixer": _mem(3, 5, 7, 12.0), "mlp": {"kind": "dense", "ff": 44}},
        {"type": "attention",
         "mixer": _attn(6, 3, 10, 6, {"dims": 6, "base": 30.0,
                                      "scaling": {"factor": 3.0, "low": 2.0, "high": 5.0, "original": 40}},
                        0.35, 2.5),
         "mlp": {"kind": "dense", "ff": 20}},
    ],
}

D5 = {
    "architecture": "Derosun", "vocab": 96, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
    "embedding": {"scale": 0.5},
    "layers": [
        {"type": "attention",
         "mixer": _attn(4, 1, 32, 48, {"dims": 16, "base": 10000.0,
                                       "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 128}},
                        0.2, 8.0),
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "latent_attention",
         "mixer": _latent(20, 16, 16, 24, 48, 40,
                          {"dims": 16, "base": 1000.0,
                           "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}, 0.18),
         "mlp": {"kind": "dense", "ff": 80}},
        {"type": "mlstm", "mixer": _mem(2, 16, 32, 15.0), "mlp": None},
        {"type": "latent_attention",
         "mixer": _latent(4, 16, 32, 16, 32, 24,
                          {"dims": 32, "base": 5000.0,
                           "scaling": {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 2.0}}, 0.15),
         "mlp": None},
    ],
}

D6 = {
    "architecture": "Derosun", "vocab": 80, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 1.5,
    "embedding": {"scale": 0.8},
    "layers": [
        {"type": "latent_attention",
         "mixer": _latent(3, 16, 16, 24, 144, 40,
                          {"dims": 16, "base": 1000.0,
                           "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}, 0.18),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "mlstm", "mixer": _mem(2, 16, 24, 15.0), "mlp": None},
        {"type": "latent_attention",
         "mixer": _latent(72, 8, 8, 8, 264, 48, {"dims": 8, "base": 300.0}, 0.2),
         "mlp": None},
    ],
}

CONFIGS = {"D1": (D1, 8), "D2": (D2, 16), "D3": (D3, 16), "D4": (D4, 4), "D5": (D5, 16),
           "D6": (D6, 16)}   # config, page size


def bf16_values(x: np.ndarray) -> np.ndarray:
    """float64 values that bfloat16 holds exactly (what a checkpoint would store)."""
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def make_weights(cfg, seed):
    """name -> float64 array of bfloat16-exact values; lively enough that tokens differ, that
    the gates of the memory open and shut and that biases and caps matter."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = rng.normal(0, gain / np.sqrt(inp), (out, inp))

    def vec(name, n, mean=0.0, sd=0.2):
        W[name] = mean + sd * rng.normal(0, 1, n)

    W["embed"] = rng.normal(0, 1.0, (V, d))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", d, 1.0)
        if L["type"] == "attention":
            H, dim = m["heads"], m["dim"]
            G, vdim = m.get("kv_heads", H), m.get("vdim", dim)
            mat(p + "mix.q", H * dim, d, 2.0)
            mat(p + "mix.k", G * dim, d, 2.0)
            mat(p + "mix.v", G * vdim, d)
            vec(p + "mix.q.norm", H * dim, 1.5, 0.4)
            vec(p + "mix.k.norm", G * dim, 1.5, 0.4)
            mat(p + "mix.o", d, H * vdim)
        elif L["type"] == "latent_attention":
            H, dim, rd, vdim = m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"])
            mat(p + "mix.dq", m["q_rank"], d)
            vec(p + "mix.dq.norm", m["q_rank"], 1.5, 0.3)
            mat(p + "mix.uq", H * (dim + rd), m["q_rank"], 1.5)
            mat(p + "mix.dkv", m["kv_rank"] + rd, d, 2.0)
            vec(p + "mix.dkv.norm", m["kv_rank"], 1.5, 0.3)
            mat(p + "mix.uk", H * dim, m["kv_rank"], 1.5)
            mat(p + "mix.uv", H * vdim, m["kv_rank"])
            mat(p + "mix.o", d, H * vdim)
        else:
            H, dim, vdim = m["heads"], m["dim"], m.get("vdim", m["dim"])
            mat(p + "mix.q", H * dim, d, 1.5)
            mat(p + "mix.k", H * dim, d, 1.5)
            mat(p + "mix.v", H * vdim, d)
            mat(p + "mix.g", H * vdim, d, 1.5)
            mat(p + "mix.o", d, H * vdim)
            vec(p + "mix.norm", H * vdim, 1.0)
            mat(p + "mix.i", H, d, 3.0)
            vec(p + "mix.i.b", H, 0.0, 1.0)
            mat(p + "mix.f", H, d, 3.0)
            vec(p + "mix.f.b", H, 2.0, 1.0)
        mlp = L.get("mlp")
        if mlp:
            vec(p + "norm2", d, 1.0)
            f = mlp["ff"]
            mat(p + "mlp.gate", f, d, 1.5)
            vec(p + "mlp.gate.b", f, 0.0, 0.5)
            mat(p + "mlp.up", f, d)
            vec(p + "mlp.up.b", f, 0.0, 0.5)
            mat(p + "mlp.down", d, f)
            vec(p + "mlp.down.b", d, 0.0, 0.5)
    vec("final.norm", d, 1.0)
    mat("head", V, d, 2.0)
    return {k: bf16_values(v) for k, v in W.items()}


def write_model_dir(path, cfg, W):
    """config.json + model.safetensors (bfloat16) of these weights."""
    from tgo_b200.weights.safetensors import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16)
                       for k, v in W.items()})
    return str(path)


def bind_model(cfg, W, dtype, device):
    """A tgo_b200 Model with these weights, without a folder."""
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    model = Model(model_spec_from_config(cfg), dtype, device)
    weights = {}
    for ws in model.weight_specs():
        if ws.optional and ws.name not in W:
            continue
        store = torch.float32 if ws.role in ("gain", "constant") else dtype
        weights[ws.name] = torch.from_numpy(np.asarray(W[ws.name], dtype=np.float32)).to(
            device=device, dtype=store)
    model.bind(weights)
    return model
