"""Typed reading of a Vimelorn config.json, and its translation to a ModelSpec.

Vimelorn is a decoder whose layers are listed one by one in the file. It keeps `streams`
copies of the residual stream; every sublayer reads a learned combination of them through
an RMS norm and writes back through a learned mixing matrix (the `hyper_connections` block).
Without `streams` a layer is the ordinary pre-norm residual pair. The embedding rows are
multiplied by `embedding.scale`.

Mixers: "attention", grouped-query softmax attention whose q, k and v pass a short causal
convolution over time after their projections, with a half-split rotation of the first
`rot.dims` channels, q and k heads divided by their root mean square after the rotation, and
a sliding window (`mask.size`) beside which the first `mask.keep_first` tokens stay visible;
"attention_2", causal grouped-query attention without a rotation, q and k normed over their
whole projection rows, a query temperature that grows with the logarithm of the position
(`q_temp.coef`, `q_temp.every`) and a learned bias by distance in logarithmic buckets up to
`bias_max`. Feed-forwards: dense and SiLU-gated, or routed small experts (down of the squared
relu of up) chosen among `router.experts` real and `router.identity` identity experts by
softmax scores plus a correction, with a shared expert behind a logistic gate; or none.
The head has a matrix of its own.

Every size and constant comes from the file; a value the engine cannot honour is refused
with its key in the message.
"""
from __future__ import annotations

from typing import Optional

from .gafonex import _int, _number, _positive
from .qwen3 import ConfigError
from .spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)
from .totatar import _object

ARCHITECTURE = "Vimelorn"

WINDOW_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"),
                  ("q_conv", "mix.q.conv"), ("k_conv", "mix.k.conv"), ("v_conv", "mix.v.conv"))
CAUSAL_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"),
                  ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"), ("distance_bias", "mix.rel"))
DENSE_TENSORS = (("gate", "mlp.gate"), ("up", "mlp.up"), ("down", "mlp.down"))
ROUTED_TENSORS = (("expert_up", "mlp.e{e}.up"), ("expert_down", "mlp.e{e}.down"),
                  ("router", "mlp.router"), ("router_correction", "mlp.correction"),
                  ("shared_gate", "mlp.shared.sg"))
SHARED_TENSORS = (("up", "mlp.shared.up"), ("down", "mlp.shared.down"))
BLOCK_TENSORS = (("mixer_norm", "norm1"), ("ffn_norm", "norm2"),
                 ("mixer_in", "hc1.in"), ("mixer_out", "hc1.out"), ("mixer_mix", "hc1.mix"),
                 ("ffn_in", "hc2.in"), ("ffn_out", "hc2.out"), ("ffn_mix", "hc2.mix"))

EXPERT_ACTIVATION = "relu_squared"      # the design fixes it


def _count(raw: dict, key: str, where: str, default: int = 0) -> int:
    """A whole number that may be zero."""
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config: {where}{key} is {v!r}; it must be a whole number, zero or more")
    return v


def _heads(m: dict, where: str):
    H = _int(m, "heads", where)
    G = _int(m, "kv_heads", where, default=H)
    if H % G:
        raise ConfigError(f"config: {where}heads ({H}) is not a multiple of kv_heads ({G})")
    dim = _int(m, "dim", where)
    return H, G, dim, _int(m, "vdim", where, default=dim)


def _windowed_attention(m: dict, where: str, eps: float) -> MixerSpec:
    H, G, dim, vdim = _heads(m, where)
    position = None
    rot = _object(m, "rot", where, required=False)
    if rot is not None:
        dims = _int(rot, "dims", where + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config: {where}rot.dims is {dims}; it must be even and at most "
                              f"dim ({dim})")
        position = PositionSpec("rope_half_split", rotary_dim=dims,
                                theta=_positive(rot, "base", where + "rot."))
    window, keep = None, 0
    mask = _object(m, "mask", where, required=False)
    if mask is not None:
        window = _int(mask, "size", where + "mask.")
        keep = _count(mask, "keep_first", where + "mask.")
    taps = _count(m, "conv", where)
    if taps > 64:
        raise ConfigError(f"config: {where}conv is {taps}; at most 64 taps")
    return MixerSpec("sink_attention", num_heads=H, num_kv_heads=G, head_dim=dim, value_dim=vdim,
                     window=window, keep_first=keep, scale=_positive(m, "scale", where),
                     position=position, norm_eps=eps, qk_unit_norm=True, conv_taps=taps,
                     tensors=WINDOW_TENSORS)


def _causal_attention(m: dict, where: str, eps: float) -> MixerSpec:
    H, G, dim, vdim = _heads(m, where)
    temperature = None
    qt = _object(m, "q_temp", where, required=False)
    if qt is not None:
        temperature = (_number(qt, "coef", where + "q_temp."), _int(qt, "every", where + "q_temp."))
    bias_max = _int(m, "bias_max", where)
    return MixerSpec("sink_attention", num_heads=H, num_kv_heads=G, head_dim=dim, value_dim=vdim,
                     scale=_positive(m, "scale", where), norm_eps=eps, qk_norm=True,
                     qk_norm_scope="row", query_temperature=temperature,
                     distance_bias_max=bias_max, tensors=CAUSAL_TENSORS)


MIXER_READERS = {"attention": _windowed_attention, "attention_2": _causal_attention}


def _feed_forward(mlp, where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config: {where}mlp must be an object or null")
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return FeedForwardSpec("gated_dense", intermediate_size=_int(mlp, "ff", where + "mlp."),
                               tensors=DENSE_TENSORS, activation="silu")
    if kind == "moe":
        router = _object(mlp, "router", where + "mlp.")
        E = _int(router, "experts", where + "mlp.router.")
        n_id = _count(router, "identity", where + "mlp.router.")
        top = _int(router, "top", where + "mlp.router.")
        if top > E + n_id or top > 32:
            raise ConfigError(f"config: {where}mlp.router.top is {top}; at most the number of "
                              f"router outputs ({E + n_id}) and at most 32")
        expert = _object(mlp, "expert", where + "mlp.")
        shared = _object(mlp, "shared", where + "mlp.", required=False)
        shared_spec = None
        if shared is not None:
            shared_spec = FeedForwardSpec("plain_dense",
                                          intermediate_size=_int(shared, "ff", where + "mlp.shared."),
                                          tensors=SHARED_TENSORS, activation=EXPERT_ACTIVATION)
        return FeedForwardSpec("routed_experts",
                               intermediate_size=_int(expert, "ff", where + "mlp.expert."),
                               tensors=ROUTED_TENSORS, activation=EXPERT_ACTIVATION, experts=E,
                               top=top, gated=False, router_scores="all", router_correction=True,
                               identity_experts=n_id, shared=shared_spec,
                               shared_gate=shared_spec is not None)
    raise ConfigError(f"config: {where}mlp.kind is {kind!r}; known kinds: dense, moe")


def vimelorn_model_spec(raw: dict) -> ModelSpec:
    """config.json (as a dict) -> ModelSpec. Tensor names: `embed`, `l<i>.norm1|norm2`,
    `l<i>.hc1.*|hc2.*`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`."""
    if not isinstance(raw, dict):
        raise ConfigError("config: the top level must be an object")
    d = _int(raw, "width", "")
    V = _int(raw, "vocab", "")
    norm = raw.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config: norm is required (eps)")
    eps = _positive(norm, "eps", "norm.")
    nspec = NormSpec("rmsnorm", eps)
    emb = raw.get("embedding")
    if emb is not None and not isinstance(emb, dict):
        raise ConfigError("config: embedding must be an object")
    emb_scale = _number(emb, "scale", "embedding.") if emb and emb.get("scale") is not None else 1.0
    streams = raw.get("streams")
    if streams is not None:
        streams = _int(raw, "streams", "")
        if streams > 8:
            raise ConfigError(f"config: streams is {streams}; at most 8")
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
        ff = _feed_forward(e.get("mlp"), where)
        if streams is None:
            if ff is None:
                raise ConfigError(f"config: {where}mlp is null; without streams a layer is the "
                                  "pre-norm pair and needs a feed-forward")
            layers.append(LayerSpec("prenorm_residual", f"l{i}.", mixer, ff, nspec, BLOCK_TENSORS[:2]))
        else:
            layers.append(LayerSpec("hyper_connections", f"l{i}.", mixer, ff, nspec, BLOCK_TENSORS,
                                    streams=streams))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=d, vocab_size=V, layers=layers,
        run_order=[LayerCall(i) for i in range(len(layers))], final_norm=nspec,
        embedding_name="embed", final_norm_name="final.norm", head_name="head",
        embedding_scale=emb_scale, source=dict(raw))
    spec.validate()
    return spec
