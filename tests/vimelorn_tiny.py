"""Small Vimelorn configurations with weights of the tests' own making.

  V1: every size different from every other: three streams; a windowed layer (4/2 heads,
      values wider than keys, three taps, a partial rotation, a window of 7 that keeps the
      first 2) with a dense feed-forward; a causal layer (3/1 heads, a temperature every 5
      positions, a distance table of 10 rows up to 30) with routed experts (5 and 1 identity,
      top 2, a shared expert); a windowed layer without a feed-forward and without kept tokens.
  V2: the values a model may happen to make equal or 1: one stream, kv heads = heads, key size
      = value size, the whole head rotated, one tap, a window wider than any prompt here, top
      1 of experts without identity or shared expert, a temperature every position, a table
      of two rows, one head.
  V3: sizes the tensor-core kernels take (head sizes multiples of 16, expert widths multiples
      of 8), a window of 44 with 5 kept on pages of 16, more query heads per kv head than a
      decode tile of 16 rows in the causal layer, many experts.
  V4: sizes that no kernel's fast form takes (a width, head sizes, expert widths and a
      vocabulary that are not multiples of 8), more kept tokens than a page holds, a window
      narrower than a page, five taps, two identity experts among three outputs chosen.
  V5: no `streams` key: the ordinary pre-norm residual pair around the same parts.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def _win(H, G, dim, vdim, conv, rot, size, keep, scale):
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
         "mask": {"size": size, "keep_first": keep}}
    if rot is not None:
        m["rot"] = rot
    return m


def _causal(H, G, dim, vdim, coef, every, bias_max, scale):
    return {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
            "q_temp": {"coef": coef, "every": every}}


def _moe(E, ident, top, ff, shared_ff):
    m = {"kind": "moe", "router": {"experts": E, "identity": ident, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


V1 = {
    "architecture": "Vimelorn", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "streams": 3,
    "embedding": {"scale": 3.0},
    "layers": [
        {"type": "attention", "mixer": _win(4, 2, 12, 20, 3, {"dims": 8, "base": 500.0}, 7, 2, 0.3),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention_2", "mixer": _causal(3, 1, 8, 16, 0.4, 5, 30, 0.35),
         "mlp": _moe(5, 1, 2, 24, 28)},
        {"type": "attention", "mixer": _win(2, 1, 16, 10, 2, {"dims": 16, "base": 50.0}, 5, 0, 0.25),
         "mlp": None},
    ],
}
V2 = {
    "architecture": "Vimelorn", "vocab": 70, "width": 40, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        {"type": "attention_2", "mixer": _causal(1, 1, 24, 24, 0.2, 1, 3, 0.2),
         "mlp": _moe(3, 0, 1, 40, 0)},
        {"type": "attention", "mixer": _win(5, 5, 8, 8, 1, {"dims": 8, "base": 30.0}, 500, 0, 0.35),
         "mlp": {"kind": "dense", "ff": 72}},
    ],
}
V3 = {
    "architecture": "Vimelorn", "vocab": 96, "width": 64, "norm": {"eps": 1e-6}, "streams": 2,
    "embedding": {"scale": 8.0},
    "layers": [
        {"type": "attention", "mixer": _win(4, 1, 32, 48, 4, {"dims": 16, "base": 10000.0}, 44, 5, 0.18),
         "mlp": _moe(12, 3, 4, 32, 40)},
        {"type": "attention_2", "mixer": _causal(20, 1, 16, 16, 0.25, 32, 150, 0.25),
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": _win(8, 2, 64, 64, 3, {"dims": 64, "base": 100000.0}, 70, 3, 0.125),
         "mlp": None},
        {"type": "attention_2", "mixer": _causal(4, 2, 64, 32, 0.3, 16, 200, 0.125),
         "mlp": _moe(4, 0, 2, 64, 0)},
    ],
}
V4 = {
    "architecture": "Vimelorn", "vocab": 53, "width": 36, "norm": {"eps": 1e-5}, "streams": 4,
    "embedding": {"scale": 0.7},
    "layers": [
        {"type": "attention", "mixer": _win(6, 3, 10, 6, 5, {"dims": 6, "base": 40.0}, 3, 9, 0.4),
         "mlp": _moe(2, 2, 3, 20, 12)},
        {"type": "attention_2", "mixer": _causal(5, 5, 6, 7, 1.5, 3, 17, 0.4),
         "mlp": {"kind": "dense", "ff": 44}},
    ],
}
V5 = {
    "architecture": "Vimelorn", "vocab": 61, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _win(2, 2, 16, 16, 2, None, 9, 1, 0.25),
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention_2", "mixer": _causal(2, 1, 16, 8, 0.5, 4, 12, 0.3),
         "mlp": _moe(3, 1, 2, 16, 16)},
    ],
}

CONFIGS = {"V1": (V1, 8), "V2": (V2, 16), "V3": (V3, 16), "V4": (V4, 4), "V5": (V5, 8)}   # config, page
REL_ROWS = {"V1": 10, "V2": 2, "V3": 24, "V4": 7, "V5": 6}     # rows of the distance tables


def bf16_values(x: np.ndarray) -> np.ndarray:
    """float64 values that bfloat16 holds exactly (what a checkpoint would store)."""
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def make_weights(cfg, seed, rel_rows=8):
    """name -> float64 array of bfloat16-exact values, lively enough that tokens differ, that
    the routing spreads over the experts (identity ones too) and that the kept tokens, the
    distance bias and the temperature matter."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams")
    W = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = rng.normal(0, gain / np.sqrt(inp), (out, inp))

    def vec(name, n, mean=0.0, sd=0.2):
        W[name] = mean + sd * rng.normal(0, 1, n)

    W["embed"] = rng.normal(0, 1.0, (V, d))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, dim = m["heads"], m["dim"]
        G, vdim = m.get("kv_heads", H), m.get("vdim", dim)
        vec(p + "norm1", d, 1.0)
        mat(p + "mix.q", H * dim, d, 2.0)
        mat(p + "mix.k", G * dim, d, 2.0)
        mat(p + "mix.v", G * vdim, d)
        mat(p + "mix.o", d, H * vdim)
        if L["type"] == "attention":
            for t, n in (("q", H * dim), ("k", G * dim), ("v", G * vdim)):
                W[f"{p}mix.{t}.conv"] = rng.normal(0, 0.6, (n, m["conv"])) + \
                    np.eye(1, m["conv"], m["conv"] - 1)
        else:
            vec(p + "mix.q.norm", H * dim, 1.5, 0.4)
            vec(p + "mix.k.norm", G * dim, 1.5, 0.4)
            W[p + "mix.rel"] = rng.normal(0, 1.5, (rel_rows, H))
        mlp = L.get("mlp")
        if mlp:
            vec(p + "norm2", d, 1.0)
            if mlp["kind"] == "dense":
                mat(p + "mlp.gate", mlp["ff"], d, 1.5)
                mat(p + "mlp.up", mlp["ff"], d)
                mat(p + "mlp.down", d, mlp["ff"])
            else:
                r, f = mlp["router"], mlp["expert"]["ff"]
                outputs = r["experts"] + r.get("identity", 0)
                for e in range(r["experts"]):
                    mat(f"{p}mlp.e{e}.up", f, d, 1.5)
                    mat(f"{p}mlp.e{e}.down", d, f)
                mat(p + "mlp.router", outputs, d, 3.0)
                vec(p + "mlp.correction", outputs, 0.0, 0.15)
                if mlp.get("shared"):
                    mat(p + "mlp.shared.up", mlp["shared"]["ff"], d, 1.5)
                    mat(p + "mlp.shared.down", d, mlp["shared"]["ff"])
                    mat(p + "mlp.shared.sg", 1, d, 2.0)
        if S:
            for q in ("hc1", "hc2") if mlp else ("hc1",):
                vec(f"{p}{q}.in", S, 1.0 / S, 0.3)
                vec(f"{p}{q}.out", S, 1.0, 0.4)
                W[f"{p}{q}.mix"] = np.eye(S) + rng.normal(0, 0.25, (S, S))
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
