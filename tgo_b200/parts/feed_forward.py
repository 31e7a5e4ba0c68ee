"""Dense gated feed-forward: (act(x Wg^T) * (x Wu^T)) Wd^T, act = SiLU unless the
spec names another activation (nn/blocks.go:57-66); without biases unless the spec's `bias` is
set, then (act(x Wg^T + bg) * (x Wu^T + bu)) Wd^T + bd (roles gate_bias, up_bias, down_bias). The gate and up matrices are joined at bind time so that one
matrix product makes both, and one kernel applies the gate. The checkpoint names of the
three matrices come from the spec's `tensors` table (roles gate, up or gate_up for a
matrix that is shipped joined, gate rows first; down)."""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import FeedForwardSpec, tensor_names
from ..kernels import ops
from ..registry import FEED_FORWARDS
from ..weights.binder import WeightSpec
from .base import Part


class SwiGLU(Part):
    def __init__(self, spec: FeedForwardSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.inter = spec.intermediate_size
        self.activation = getattr(spec, "activation", "silu") or "silu"
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward: activation {self.activation!r}; known: "
                             f"{sorted(ops.ACTIVATIONS)}")
        self.joined = "gate_up" in dict(spec.tensors)
        self.bias = bool(getattr(spec, "bias", False))
        if self.bias and self.joined:
            raise ValueError("feed-forward: biases come with separate gate and up matrices")
        roles = (["gate_up"] if self.joined else ["gate", "up"]) + ["down"] + \
            (["gate_bias", "up_bias", "down_bias"] if self.bias else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "feed-forward")
        self.w_gate_up = None
        self.w_down = None
        self.interleaved = False
        self.b_gate_up = None            # float32 [2 ff], in the order of w_gate_up's rows
        self.output_bias = None          # float32 [hidden]: the down product's bias

    def weight_specs(self):
        n = self.names
        if self.joined:
            first = [WeightSpec(n["gate_up"], (2 * self.inter, self.hidden))]
        else:
            first = [WeightSpec(n["gate"], (self.inter, self.hidden)),
                     WeightSpec(n["up"], (self.inter, self.hidden))]
        out = first + [WeightSpec(n["down"], (self.hidden, self.inter))]
        if self.bias:
            out += [WeightSpec(n["gate_bias"], (self.inter,), "gain"),
                    WeightSpec(n["up_bias"], (self.inter,), "gain"),
                    WeightSpec(n["down_bias"], (self.hidden,), "gain")]
        return out

    def bind(self, weights):
        n = self.names
        f, d = self.inter, self.hidden
        if self.joined:
            both = weights.pop(n["gate_up"])
            gate, up = both[:f], both[f:]
        else:
            gate, up = weights.pop(n["gate"]), weights.pop(n["up"])
        # eight gate rows, then the eight matching up rows, and so on: one 16-row tile of the
        # weight-streaming product then holds a gate column and its up column together
        self.interleaved = f % 8 == 0
        if self.interleaved:
            self.w_gate_up = torch.stack([gate.reshape(f // 8, 8, d), up.reshape(f // 8, 8, d)],
                                         dim=1).reshape(2 * f, d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights.pop(n["down"]).contiguous()
        if self.bias:
            bg = weights.pop(n["gate_bias"]).to(torch.float32)
            bu = weights.pop(n["up_bias"]).to(torch.float32)
            if self.interleaved:
                self.b_gate_up = torch.stack([bg.reshape(f // 8, 8), bu.reshape(f // 8, 8)],
                                             dim=1).reshape(2 * f).contiguous()
            else:
                self.b_gate_up = torch.cat([bg, bu]).contiguous()
            self.output_bias = weights.pop(n["down_bias"]).to(torch.float32).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        extra = ["layer_ops"] if self.activation != "silu" or self.bias else []
        return (["sgemm"] if dtype == torch.float32 else ["gemm_skinny"]) + extra

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        return 2.0 * sum(extents) * self.hidden * 3 * self.inter

    lazy_rows = True        # x may come as ops.NormedRows; the gate/up product folds the norm in

    def forward(self, x, ctx, residual=None):
        """With `residual` (the float32 stream) the result may be added to it, and None is
        then returned; otherwise the result is returned for the caller to add."""
        if self.bias:
            act = ops.gated_linear(x, self.w_gate_up, self.interleaved, self.activation,
                                   bias=self.b_gate_up)
            y = ops.linear(act, self.w_down, out_dtype=self.out_dtype)
            if not self.defer_output_bias:
                ops.add_bias(y, self.output_bias)
            if residual is not None:
                ops.residual_add(residual, y)
                return None
            return y
        if self.activation == "silu":
            act = ops.gated_linear(x, self.w_gate_up, self.interleaved)
        else:
            act = ops.gated_linear(x, self.w_gate_up, self.interleaved, self.activation)
        return ops.linear(act, self.w_down, residual=residual, out_dtype=self.out_dtype)

    out_dtype = None        # a block that norms the result in float32 asks for float32 rows
    defer_output_bias = False   # a block that adds `output_bias` itself sets this


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("gated_dense", SwiGLU)      # the gate's activation is the spec's


class PlainDense(Part):
    """A feed-forward without a gate: W_down act(W_up x), act one of `ops.PLAIN_ACTIVATIONS`
    (the spec's `activation`), no biases. Tensor roles: up, down."""
    out_dtype = None

    def __init__(self, spec: FeedForwardSpec, hidden: int, prefix: str, device=None):
        self.hidden, self.inter = hidden, spec.intermediate_size
        self.activation = spec.activation or "silu"
        if self.activation not in ops.PLAIN_ACTIVATIONS:
            raise ValueError(f"feed-forward: activation {self.activation!r}; known: "
                             f"{sorted(ops.PLAIN_ACTIVATIONS)}")
        self.names = tensor_names(spec.tensors, prefix, ["up", "down"], "feed-forward")
        self.w_up = self.w_down = None

    def weight_specs(self):
        return [WeightSpec(self.names["up"], (self.inter, self.hidden)),
                WeightSpec(self.names["down"], (self.hidden, self.inter))]

    def bind(self, weights):
        self.w_up = weights.pop(self.names["up"]).contiguous()
        self.w_down = weights.pop(self.names["down"]).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm" if dtype == torch.float32 else "gemm_skinny", "layer_ops"]

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        return 2.0 * sum(extents) * self.hidden * 2 * self.inter

    def forward(self, x, ctx, residual=None):
        hidden = ops.linear(ops.rows_of(x), self.w_up)
        ops.act_rows(hidden, self.activation)
        return ops.linear(hidden, self.w_down, residual=residual, out_dtype=self.out_dtype)


FEED_FORWARDS.register("plain_dense", PlainDense)


class RoutedExperts(Part):
    """A routed feed-forward (mixture of experts): `experts` gated feed-forwards without
    biases, of which every token uses the `top` with the largest router logits,

        z = W_router x + b_router                      float32 sums
        out = sum over the top experts e of softmax(z over the chosen)_e * expert_e(x)
              + shared(x)                              a feed-forward every token also takes

    expert_e(x) = W_down_e (act(W_gate_e x) * (W_up_e x)). The experts' matrices are stacked at
    bind time ([E, ff, d] and [E, d, ff]); routing, the products over each expert's tokens and
    the weighted sum run on the device without a word to the host. The spec's `tensors` table
    names expert tensors with a `{e}` in them: roles expert_gate, expert_up, expert_down, router
    and, with `router_bias`, router_bias. `shared` is a FeedForwardSpec of its own kind.

    What the spec may change: `gated` False, experts W_down act(W_up x) without a gate matrix
    (no role expert_gate); `router_scores` "all", the scores are the softmax over every router
    output, the weights the chosen scores divided by their sum (+ 1e-20), and with
    `router_correction` (role router_correction) the choice is by score + correction while the
    weights are not; `identity_experts` n, the router has n more outputs after the experts,
    whose expert gives back its input; `shared_gate` (role shared_gate, [1, hidden]), the shared
    feed-forward's output is multiplied by a logistic gate per token (the gate's row rides as
    the router matrix's last row, so its logit is a float32 sum too)."""
    out_dtype = None        # the result is float32 rows when a block asks, else the activations'

    def __init__(self, spec: FeedForwardSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.inter = spec.intermediate_size
        self.E, self.top = int(spec.experts), int(spec.top)
        self.gated = bool(getattr(spec, "gated", True))
        self.identity = int(getattr(spec, "identity_experts", 0) or 0)
        self.scores = "all" if getattr(spec, "router_scores", "chosen") == "all" else "chosen"
        self.correction = bool(getattr(spec, "router_correction", False))
        self.shared_gate = bool(getattr(spec, "shared_gate", False))
        if not 0 < self.top <= self.E + self.identity:
            raise ValueError(f"routed feed-forward: top {self.top} of {self.E + self.identity} experts")
        if self.shared_gate and spec.shared is None:
            raise ValueError("routed feed-forward: a gate on the shared feed-forward needs one")
        if self.correction and self.scores != "all":
            raise ValueError("routed feed-forward: the correction belongs to scores over all experts")
        self.activation = spec.activation or "silu"
        known = ops.ACTIVATIONS if self.gated else ops.PLAIN_ACTIVATIONS
        if self.activation not in known:
            raise ValueError(f"feed-forward: activation {self.activation!r}; known: {sorted(known)}")
        self.router_bias = bool(spec.router_bias)
        roles = (["expert_gate"] if self.gated else []) + ["expert_up", "expert_down", "router"] + \
            (["router_bias"] if self.router_bias else []) + \
            (["router_correction"] if self.correction else []) + \
            (["shared_gate"] if self.shared_gate else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "routed feed-forward")
        self.shared = None
        if spec.shared is not None:
            self.shared = FEED_FORWARDS.get(spec.shared.kind)(spec.shared, hidden, prefix, device)
            if hasattr(self.shared, "out_dtype"):
                self.shared.out_dtype = torch.float32       # it joins a float32 sum
        self.w_gate = self.w_up = self.w_down = self.w_router = self.b_router = None
        self.router_correction = None

    def _expert(self, role: str, e: int) -> str:
        return self.names[role].replace("{e}", str(e))

    def parts(self):
        return [self.shared] if self.shared is not None else []

    def weight_specs(self):
        f, d = self.inter, self.hidden
        out = []
        outputs = self.E + self.identity
        for e in range(self.E):
            if self.gated:
                out.append(WeightSpec(self._expert("expert_gate", e), (f, d)))
            out += [WeightSpec(self._expert("expert_up", e), (f, d)),
                    WeightSpec(self._expert("expert_down", e), (d, f))]
        out.append(WeightSpec(self.names["router"], (outputs, d), "constant"))
        if self.router_bias:
            out.append(WeightSpec(self.names["router_bias"], (outputs,), "gain"))
        if self.correction:
            out.append(WeightSpec(self.names["router_correction"], (outputs,), "gain"))
        if self.shared_gate:
            out.append(WeightSpec(self.names["shared_gate"], (1, d), "constant"))
        if self.shared is not None:
            out += self.shared.weight_specs()
        return out

    def bind(self, weights):
        stack = lambda role: torch.stack(                                       # noqa: E731
            [weights.pop(self._expert(role, e)) for e in range(self.E)], dim=0).contiguous()
        self.w_gate = stack("expert_gate") if self.gated else None
        self.w_up, self.w_down = stack("expert_up"), stack("expert_down")
        self.w_router = weights.pop(self.names["router"]).to(torch.float32).contiguous()
        if self.shared_gate:
            gate_row = weights.pop(self.names["shared_gate"]).to(torch.float32).reshape(1, -1)
            self.w_router = torch.cat([self.w_router, gate_row], dim=0).contiguous()
        if self.router_bias:
            self.b_router = weights.pop(self.names["router_bias"]).to(torch.float32).contiguous()
        if self.correction:
            self.router_correction = weights.pop(self.names["router_correction"]).to(
                torch.float32).contiguous()
        if self.shared is not None:
            self.shared.bind(weights)

    def libraries(self, dtype, page_size) -> List[str]:
        out = ["moe", "layer_ops"]
        if self.shared is not None:
            out += self.shared.libraries(dtype, page_size)
        return out

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        total = 2.0 * n * self.hidden * (self.E + self.identity) + \
            2.0 * n * self.top * self.hidden * (3 if self.gated else 2) * self.inter
        if self.shared is not None:
            total += self.shared.flops(extents, first_positions, writes_cache)
        return total

    def forward(self, x, ctx):
        x = ops.rows_of(x)
        extra = self.shared.forward(x, ctx) if self.shared is not None else None
        y = ops.moe_feed_forward(x, self.w_router, self.b_router, self.w_gate, self.w_up,
                                 self.w_down, self.top, self.activation, extra, self.scores,
                                 self.router_correction, self.identity, self.shared_gate)
        want = self.out_dtype or ctx.act_dtype
        if want == torch.float32:
            return y
        out = torch.empty(y.shape, dtype=want, device=y.device)
        ops.cast_rows(y, out)
        return out


FEED_FORWARDS.register("routed_experts", RoutedExperts)
