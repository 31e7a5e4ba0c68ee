"""Architecture-neutral description of a model: what the engine builds from.

An architecture's config reader (for instance `config/qwen3.py`) turns its own
config.json keys into these records. Everything below the reader (parts, cache,
step function, kernels) sees only these records, never a model's name, so another
architecture is another reader plus, where needed, new part kinds.

The reference keeps the same split between a typed `Config` and the blocks that
take their constants as parameters (model/config.go:20-87, nn/attention.go:60-94,
model/layerkind.go:21-59).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional


def tensor_names(tensors, prefix: str, roles: Iterable[str], what: str) -> Dict[str, str]:
    """The checkpoint names a part asks for: `tensors` is the (role, name) table its spec
    carries (names relative to the layer's prefix), `roles` the roles the part needs. A role
    the table does not name is an error of the architecture's config reader, which owns the
    table (model/qwen3.go:57-67 keeps it per architecture in the same way)."""
    table = dict(tensors)
    out = {}
    for role in roles:
        if role not in table:
            raise ValueError(f"{what}: the spec names no tensor for the role {role!r}; "
                             f"it names {sorted(table) or 'none'}")
        out[role] = prefix + table[role]
    return out


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis. kind names a registered norm part."""
    kind: str
    eps: float
    groups: int = 1                      # grouped kinds: equal consecutive parts, each normed alone
    unit_offset: bool = False            # a zero-centred weight: the gain is 1 + w


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer. kind names a registered position encoding.
    `rotary_dim` channels of each head are rotated; the rest are left alone."""
    kind: str
    rotary_dim: int = 0
    theta: float = 0.0
    # frequency interpolation of a rotation trained on `original` positions and stretched by
    # `factor` (kinds that know it): (factor, original, fast, slow), or None
    scaling: Optional[tuple] = None


@dataclass(frozen=True)
class MixerSpec:
    """The token-mixing part of a layer. kind names a registered mixer.

    For attention kinds: `window` is None when a query reads every earlier key,
    else the number of most recent keys (its own included) that it reads.
    `tensors` is the (role, checkpoint name relative to the layer's prefix) table of the
    mixer's weights; the roles are the mixer kind's own (attention: q, k, v or qkv joined, o,
    q_norm, k_norm). `extra` carries what a mixer kind outside this package needs.
    """
    kind: str
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None        # None: 1/sqrt(head_dim)
    position: Optional[PositionSpec] = None
    norm_eps: float = 0.0                # eps of the per-head q/k norm
    tensors: tuple = ()
    extra: tuple = ()
    value_dim: Optional[int] = None      # per-head width of the values; None: head_dim
    value_norm: bool = False             # each head's value divided by its root mean square
    head_mix: bool = False               # attention weights mixed across heads by a matrix
    # values blended with those an earlier layer made for the same token: "source" (this layer
    # makes them), "blend" (this layer reads them), None
    value_share: Optional[str] = None
    decay: tuple = ()                    # linear-attention kinds: one decay per head
    output_gate: bool = False            # the mixer's output multiplied by a gate projection
    gate_activation: str = "silu"        # what the gate projection goes through: silu | sigmoid
    input_activation: Optional[str] = None   # linear-attention kinds: q, k, v through this (silu)
    # linear-attention kinds: how the heads' outputs are normed: "head_unit" (each head by its
    # own root mean square, no gain) or "joint_gain" (all heads as one row, times a gain)
    output_norm: str = "head_unit"
    bias: bool = False                   # attention kinds: q, k and v projections carry biases
    sink: bool = False                   # attention kinds: a learned term per head in the
                                         # softmax's denominator that stands for no token
    # state-space kinds: num_heads heads of value_dim channels, num_kv_heads groups of B and C,
    # head_dim the state size; taps of the causal convolution; parts of the output norm
    conv_taps: int = 0
    norm_groups: int = 1
    # composite kinds: the mixers that share one input, and the factor on
    # each one's result
    branches: tuple = ()
    branch_scales: tuple = ()
    # attention kinds: c > 0 bounds every scaled score by c tanh(score / c); None: no bound
    softcap: Optional[float] = None
    # where qk_norm takes its mean: "head" (every head's channels alone, a gain of head_dim) or
    # "row" (all heads of a token at once, a gain as wide as the whole projection)
    qk_norm_scope: str = "head"
    # latent attention kinds: width of the latent that keys and values are expanded from and
    # of the latent the queries go through; width of the rotated key part all heads share
    # (head_dim then counts the unrotated channels of a head's query and key)
    latent_rank: int = 0
    query_rank: int = 0
    rope_dim: int = 0
    # gated recurrences: the bound c of a gate's pre-activation, c tanh(x / c)
    gate_cap: float = 0.0
    # attention kinds with a window: the first `keep_first` tokens of a request stay visible to
    # every later query, at their true positions
    keep_first: int = 0
    # attention kinds: every q and k head divided by its root mean square AFTER the rotation,
    # no gain (eps is norm_eps); and, with conv_taps > 0, q, k and v each through a causal
    # convolution of that many taps over time, straight after their projections
    qk_unit_norm: bool = False
    # attention kinds: (coef, every): the query at position p is multiplied by
    # 1 + coef * ln(floor((p + 1) / every) + 1); None: no such factor
    query_temperature: Optional[tuple] = None
    # attention kinds: a learned bias by distance, a table [rows, heads] (role distance_bias)
    # whose row for distance n is n below rows/2 and then grows by logarithmic steps up to
    # this distance, beyond which the last row stands; None: no bias
    distance_bias_max: Optional[int] = None


@dataclass(frozen=True)
class FeedForwardSpec:
    """The per-token part of a layer. kind names a registered feed-forward. `tensors` as in
    MixerSpec (gated feed-forward: gate, up or gate_up joined, down)."""
    kind: str
    intermediate_size: int = 0
    tensors: tuple = ()
    extra: tuple = ()
    activation: str = "silu"             # what the gate goes through
    # routed kinds: `experts` gated feed-forwards of intermediate_size, of which a token uses
    # `top`; the router may carry a bias; `shared` is a feed-forward every token also takes
    experts: int = 0
    top: int = 0
    router_bias: bool = False
    shared: Optional["FeedForwardSpec"] = None
    bias: bool = False                   # dense kinds: every projection carries a bias
    # routed kinds: experts without a gate matrix (down act(up x)) when False
    gated: bool = True
    # routed kinds: "chosen": softmax over the chosen logits; "all": softmax over every logit,
    # the chosen scores divided by their sum
    router_scores: str = "chosen"
    router_correction: bool = False      # a per-expert term added to the scores for the choice only
    identity_experts: int = 0            # router outputs past `experts` whose expert is the input itself
    shared_gate: bool = False            # the shared feed-forward times a logistic gate per token


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts inside it.
    `prefix` is the tensor-name prefix of the layer's weights ("model.layers.3."); every
    part of the layer gets it and adds the names of its own spec's `tensors` table.
    `tensors` names the block's own weights (pre-norm block: mixer_norm, ffn_norm)."""
    block: str
    prefix: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]      # None: the layer has no feed-forward
    norm: NormSpec
    tensors: tuple = ()
    # blocks that norm the sum: the factor on the stream in stream <- norm(factor * stream +
    # sublayer(stream))
    residual_scale: float = 1.0
    # blocks that keep several copies of the residual stream and learn how the sublayers read
    # and write them: how many
    streams: int = 1


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes ModelSpec.layers (a layer may be named by several calls, which
    then share weights). `cache_from` is None when the call owns a cache of its
    own, else the index of an earlier call whose cache it reads without writing.
    """
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    """A whole decoder: embedding, layers, their run order, final norm and head."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list                     # list[LayerSpec]
    run_order: list                  # list[LayerCall]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]         # None: the head is the embedding table (tied)
    tied_head_alias: Optional[str] = None   # name a tied checkpoint may ship anyway
    max_positions: int = 0           # advisory, as in the reference
    logit_softcap: Optional[float] = None   # c: logits <- c tanh(logits / c)
    embedding_scale: float = 1.0     # the embedding rows are multiplied by this
    source: dict = field(default_factory=dict)   # the config.json it came from

    @property
    def tied_head(self) -> bool:
        return self.head_name is None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("model spec: no layers")
        for i, call in enumerate(self.run_order):
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"model spec: run_order[{i}] names layer {call.layer}, "
                                 f"there are {len(self.layers)}")
            if call.cache_from is not None:
                if not (0 <= call.cache_from < i):
                    raise ValueError(f"model spec: run_order[{i}] reads the cache of call "
                                     f"{call.cache_from}, which does not run before it")
                if self.run_order[call.cache_from].cache_from is not None:
                    raise ValueError(f"model spec: run_order[{i}] reads the cache of call "
                                     f"{call.cache_from}, which owns none")
