"""Typed reading of a Derosun config.json, and its translation to a ModelSpec.

Derosun is a decoder whose layers are listed one by one in the file. A layer norms the SUM of
the scaled stream and each sublayer's output, so that the stream itself is what the norm
leaves (post-LN):

    x <- norm1(a x + mixer(x));  x <- norm2(a x + feed_forward(x)),   a = postln_alpha

The embedding rows are multiplied by `embedding.scale`. Its mixers: "attention", grouped-query
softmax attention with q and k normed over their whole projection rows, a half-split rotation
slowed by wavelength bands and scores through a soft cap; "latent_attention", attention over
one small cached latent per token with a rotated key part that all heads share, an
interleaved rotation stretched by a ramp; "mlstm", a matrix memory with exponential gates and
a 32-bit state per request. Its feed-forward is dense, SiLU-gated, with a bias on every
projection, or absent. The head has a matrix of its own.

Every size and constant comes from the file; a value the engine cannot honour is refused
with its key in the message.
"""
from __future__ import annotations

from typing import Optional

from .gafonex import _int, _number, _positive
from .qwen3 import ConfigError
from .spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

ARCHITECTURE = "Derosun"

ATTENTION_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"),
                     ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"))
LATENT_TENSORS = (("q_down", "mix.dq"), ("q_down_norm", "mix.dq.norm"), ("q_up", "mix.uq"),
                  ("kv_down", "mix.dkv"), ("kv_norm", "mix.dkv.norm"), ("k_up", "mix.uk"),
                  ("v_up", "mix.uv"), ("o", "mix.o"))
MLSTM_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("gate", "mix.g"), ("o", "mix.o"),
                 ("out_norm", "mix.norm"), ("input_gate", "mix.i"), ("input_gate_bias", "mix.i.b"),
                 ("forget_gate", "mix.f"), ("forget_gate_bias", "mix.f.b"))
FEED_FORWARD_TENSORS = (("gate", "mlp.gate"), ("up", "mlp.up"), ("down", "mlp.down"),
                        ("gate_bias", "mlp.gate.b"), ("up_bias", "mlp.up.b"),
                        ("down_bias", "mlp.down.b"))
BLOCK_TENSORS = (("mixer_norm", "norm1"), ("ffn_norm", "norm2"))


def _rotation(rot, width: int, where: str, kind: str, keys: tuple) -> Optional[PositionSpec]:
    """`rot` {dims, base, scaling?} -> a PositionSpec of `kind`, whose `scaling` tuple holds the
    file's rot.scaling values in the order of `keys`; without `rot` positions do not enter."""
    if rot is None:
        return None
    if not isinstance(rot, dict):
        raise ConfigError(f"config: {where}rot must be an object")
    dims = _int(rot, "dims", where + "rot.")
    if dims % 2 or dims > width:
        raise ConfigError(f"config: {where}rot.dims is {dims}; it must be even and at most the "
                          f"rotated width {width}")
    base = _positive(rot, "base", where + "rot.")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config: {where}rot.scaling must be an object or null")
        scaling = tuple(_positive(sc, key, where + "rot.scaling.") for key in keys)
        if base == 1.0:
            raise ConfigError(f"config: {where}rot.base is 1; a scaled rotation needs a base "
                              "whose logarithm is not zero")
    return PositionSpec(kind, rotary_dim=dims, theta=base, scaling=scaling)


def _scale(m: dict, where: str) -> Optional[float]:
    return _positive(m, "scale", where) if m.get("scale") is not None else None


def _attention(m: dict, where: str, eps: float) -> MixerSpec:
    H = _int(m, "heads", where)
    G = _int(m, "kv_heads", where, default=H)
    if H % G:
        raise ConfigError(f"config: {where}heads ({H}) is not a multiple of kv_heads ({G})")
    dim = _int(m, "dim", where)
    cap = _positive(m, "softcap", where) if m.get("softcap") is not None else None
    return MixerSpec("sink_attention", num_heads=H, num_kv_heads=G, head_dim=dim, qk_norm=True,
                     qk_norm_scope="row", norm_eps=eps, scale=_scale(m, where), softcap=cap,
                     position=_rotation(m.get("rot"), dim, where, "rope_banded",
                                        ("factor", "low", "high", "original")),
                     tensors=ATTENTION_TENSORS, value_dim=_int(m, "vdim", where, default=dim))


def _latent_attention(m: dict, where: str, eps: float) -> MixerSpec:
    dim = _int(m, "dim", where)
    rot_dim = _int(m, "rot_dim", where)
    return MixerSpec("latent_attention", num_heads=_int(m, "heads", where), num_kv_heads=1,
                     head_dim=dim, value_dim=_int(m, "vdim", where, default=dim),
                     latent_rank=_int(m, "kv_rank", where), query_rank=_int(m, "q_rank", where),
                     rope_dim=rot_dim, norm_eps=eps, scale=_scale(m, where),
                     position=_rotation(m.get("rot"), rot_dim, where, "rope_stretched_interleaved",
                                        ("factor", "original", "fast", "slow")),
                     tensors=LATENT_TENSORS)


def _mlstm(m: dict, where: str, eps: float) -> MixerSpec:
    H = _int(m, "heads", where)
    dim = _int(m, "dim", where)
    return MixerSpec("mlstm", num_heads=H, num_kv_heads=H, head_dim=dim,
                     value_dim=_int(m, "vdim", where, default=dim), norm_eps=eps,
                     gate_cap=_positive(m, "gate_cap", where), tensors=MLSTM_TENSORS)


MIXER_READERS = {"attention": _attention, "latent_attention": _latent_attention, "mlstm": _mlstm}


def _feed_forward(mlp, where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config: {where}mlp must be an object or null")
    kind = mlp.get("kind", "dense")
    if kind != "dense":
        raise ConfigError(f"config: {where}mlp.kind is {kind!r}; known kinds: dense")
    return FeedForwardSpec("gated_dense", intermediate_size=_int(mlp, "ff", where + "mlp."),
                           tensors=FEED_FORWARD_TENSORS, activation="silu", bias=True)


def derosun_model_spec(raw: dict) -> ModelSpec:
    """config.json (as a dict) -> ModelSpec. Tensor names: `embed`, `l<i>.norm1|norm2`,
    `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`."""
    if not isinstance(raw, dict):
        raise ConfigError("config: the top level must be an object")
    d = _int(raw, "width", "")
    V = _int(raw, "vocab", "")
    norm = raw.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config: norm is required (eps)")
    eps = _positive(norm, "eps", "norm.")
    nspec = NormSpec("rmsnorm", eps)
    alpha = _number(raw, "postln_alpha", "") if raw.get("postln_alpha") is not None else 1.0
    emb = raw.get("embedding")
    if emb is not None and not isinstance(emb, dict):
        raise ConfigError("config: embedding must be an object")
    emb_scale = _number(emb, "scale", "embedding.") if emb and emb.get("scale") is not None else 1.0
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config: layers must list at least one layer")
    layers = []
    for i, e in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(e, dict) or not isinstance(e.get("mixer"), dict):
            raise ConfigError(f"config: {where}mixer is required")
        kind = e.get("type")
        if kind not in MIXER_READERS:
            raise ConfigError(f"config: {where}type is {kind!r}; known mixers are "
                              + ", ".join(sorted(MIXER_READERS)))
        mixer = MIXER_READERS[kind](e["mixer"], where + "mixer.", eps)
        layers.append(LayerSpec("postnorm_residual", f"l{i}.", mixer,
                                _feed_forward(e.get("mlp"), where), nspec, BLOCK_TENSORS,
                                residual_scale=alpha))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=d, vocab_size=V, layers=layers,
        run_order=[LayerCall(i) for i in range(len(layers))], final_norm=nspec,
        embedding_name="embed", final_norm_name="final.norm", head_name="head",
        embedding_scale=emb_scale, source=dict(raw))
    spec.validate()
    return spec
