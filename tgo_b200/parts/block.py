"""Arrangements of a layer's parts. The first: pre-norm with two residual adds,

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))

(model/qwen3_graph.go:76-100). The residual stream h is float32. Each add is left
pending and handed to the next norm, which does it in its own kernel. The two norms'
checkpoint names come from the layer spec's `tensors` table (roles mixer_norm, ffn_norm).
The second, `PostNormScaledResidual` below, norms and scales each sublayer's output instead;
the third norms a sublayer's input and its output; the fourth, `PostNormResidual`, norms the
sum, so that the stream itself is what the norm leaves.
"""
from __future__ import annotations

import inspect

import torch

from ..config.spec import LayerSpec, tensor_names
from ..kernels import ops
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from ..weights.binder import WeightSpec
from .base import Part, offered


class PreNormResidual(Part):
    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        names = tensor_names(spec.tensors, p, ["mixer_norm", "ffn_norm"], "pre-norm block")
        self.norm1 = NORMS.get(spec.norm.kind)(spec.norm, hidden, names["mixer_norm"])
        self.norm2 = NORMS.get(spec.norm.kind)(spec.norm, hidden, names["ffn_norm"])
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        if spec.feed_forward is None:
            raise ValueError("pre-norm block: a layer needs a feed-forward")
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
            spec.feed_forward, hidden, p, device)
        # a part whose forward takes `residual` may add its result to the stream itself
        self._mixer_adds = "residual" in inspect.signature(self.mixer.forward).parameters
        self._ffn_adds = "residual" in inspect.signature(self.feed_forward.forward).parameters
        # a part with `lazy_rows` set takes its input as ops.NormedRows (a norm it may fold
        # into its first product), if the norm knows how to hand that on
        self._lazy1 = getattr(self.mixer, "lazy_rows", False) and \
            "lazy" in inspect.signature(self.norm1.forward).parameters
        self._lazy2 = getattr(self.feed_forward, "lazy_rows", False) and \
            "lazy" in inspect.signature(self.norm2.forward).parameters

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def libraries(self, dtype, page_size):
        out = []
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    def forward(self, h, pending, ctx, cache):
        n = self.norm1.forward(h, pending, ctx.act_dtype, lazy=True) if self._lazy1 else \
            self.norm1.forward(h, pending, ctx.act_dtype)
        if self._mixer_adds:
            a = self.mixer.forward(n, ctx, cache, residual=h)
        else:
            a = self.mixer.forward(n, ctx, cache)
        n = self.norm2.forward(h, a, ctx.act_dtype, lazy=True) if self._lazy2 else \
            self.norm2.forward(h, a, ctx.act_dtype)
        if self._ffn_adds:
            return h, self.feed_forward.forward(n, ctx, residual=h)
        return h, self.feed_forward.forward(n, ctx)


BLOCKS.register("prenorm_residual", PreNormResidual)


class PostNormScaledResidual(Part):
    """Arrangement with the norm on each sublayer's OUTPUT and a per-channel scale on it:

        h = h + s1 * norm1(mixer(h));  h = h + s2 * norm2(feed_forward(h))

    The sublayers read the stream itself (narrowed to the activation type in a bfloat16
    engine: the kernel that adds to the stream writes that copy too). The stream, the norms
    and the adds are float32. A layer may have no feed-forward. Tensor roles of the layer
    spec: mixer_norm, ffn_norm (gains) and, optional, mixer_scale, ffn_scale."""

    STREAM_KEY = "stream_rows"       # ctx.aux: (the stream tensor, its activation-type copy)

    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        has_ffn = spec.feed_forward is not None
        table = dict(spec.tensors)
        roles = ["mixer_norm"] + (["ffn_norm"] if has_ffn else [])
        self.scaled = "mixer_scale" in table
        if self.scaled:
            roles += ["mixer_scale"] + (["ffn_scale"] if has_ffn else [])
        self.names = tensor_names(spec.tensors, p, roles, "post-norm block")
        self.hidden = hidden
        self.norm1 = NORMS.get(spec.norm.kind)(spec.norm, hidden, self.names["mixer_norm"])
        if not hasattr(self.norm1, "add_scaled"):
            raise ValueError(f"post-norm block: the norm {spec.norm.kind!r} cannot norm a "
                             "sublayer's output into the stream (no add_scaled)")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        self.norm2 = self.feed_forward = None
        if has_ffn:
            self.norm2 = NORMS.get(spec.norm.kind)(spec.norm, hidden, self.names["ffn_norm"])
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
                spec.feed_forward, hidden, p, device)
        # the sublayers' last products keep float32 rows: the norm that follows is float32
        for part in (self.mixer, self.feed_forward):
            if part is not None and hasattr(part, "out_dtype"):
                part.out_dtype = torch.float32
        self.scale1 = self.scale2 = None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        if self.scaled:
            out.append(WeightSpec(self.names["mixer_scale"], (self.hidden,), "gain"))
            if self.feed_forward is not None:
                out.append(WeightSpec(self.names["ffn_scale"], (self.hidden,), "gain"))
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)
        if self.scaled:
            self.scale1 = weights[self.names["mixer_scale"]].contiguous()
            if self.feed_forward is not None:
                self.scale2 = weights[self.names["ffn_scale"]].contiguous()

    def libraries(self, dtype, page_size):
        out = ["layer_ops"]
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    def _rows(self, h, ctx):
        """The stream as the sublayers read it: itself in a float32 engine, else the copy the
        last add left, or a fresh one."""
        if ctx.act_dtype == torch.float32:
            return h
        got = ctx.aux.get(self.STREAM_KEY)
        if got is not None and got[0] is h:
            return got[1]
        x = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        ops.cast_rows(h, x)
        return x

    def _add(self, norm, h, y, scale, ctx):
        act = None
        if ctx.act_dtype != torch.float32:
            act = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        norm.add_scaled(h, y, scale, act)
        ctx.aux[self.STREAM_KEY] = (h, act)

    def forward(self, h, pending, ctx, cache):
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.aux.pop(self.STREAM_KEY, None)
        self._add(self.norm1, h, self.mixer.forward(self._rows(h, ctx), ctx, cache), self.scale1,
                  ctx)
        if self.feed_forward is not None:
            self._add(self.norm2, h, self.feed_forward.forward(self._rows(h, ctx), ctx),
                      self.scale2, ctx)
        return h, None


BLOCKS.register("postnorm_scaled_residual", PostNormScaledResidual)


class SandwichNormResidual(Part):
    """Arrangement with a norm before AND after each sublayer:

        h = h + norm1b(mixer(norm1(h)));  h = h + norm2b(feed_forward(norm2(h)))

    The stream, the four norms and the adds are float32; the sublayers read the normed rows
    in the activation type and hand back float32 rows. A layer may have no feed-forward (it
    then has no second pair of norms). Tensor roles of the layer spec: mixer_norm,
    mixer_out_norm, ffn_norm, ffn_out_norm."""

    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        has_ffn = spec.feed_forward is not None
        roles = ["mixer_norm", "mixer_out_norm"] + (["ffn_norm", "ffn_out_norm"] if has_ffn else [])
        self.names = tensor_names(spec.tensors, p, roles, "sandwich-norm block")
        make = NORMS.get(spec.norm.kind)
        self.norm1 = make(spec.norm, hidden, self.names["mixer_norm"])
        self.norm1b = make(spec.norm, hidden, self.names["mixer_out_norm"])
        if not hasattr(self.norm1b, "add_scaled"):
            raise ValueError(f"sandwich-norm block: the norm {spec.norm.kind!r} cannot norm a "
                             "sublayer's output into the stream (no add_scaled)")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        self.norm2 = self.norm2b = self.feed_forward = None
        if has_ffn:
            self.norm2 = make(spec.norm, hidden, self.names["ffn_norm"])
            self.norm2b = make(spec.norm, hidden, self.names["ffn_out_norm"])
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
                spec.feed_forward, hidden, p, device)
        # the norm that follows a sublayer is float32: its last product keeps float32 rows
        for part in (self.mixer, self.feed_forward):
            if part is not None and hasattr(part, "out_dtype"):
                part.out_dtype = torch.float32
        # a layer without a feed-forward has no use for the second pair of norms; a checkpoint
        # that ships them anyway is not refused for that
        table = dict(spec.tensors)
        self.unused = [] if has_ffn else [(p + table[r], hidden) for r in ("ffn_norm", "ffn_out_norm")
                                          if r in table]

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm1b, self.norm2, self.feed_forward,
                            self.norm2b) if p is not None]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        out += [WeightSpec(name, (width,), "gain", optional=True) for name, width in self.unused]
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def libraries(self, dtype, page_size):
        out = ["layer_ops"]
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    def forward(self, h, pending, ctx, cache):
        y = self.mixer.forward(self.norm1.forward(h, pending, ctx.act_dtype), ctx, cache)
        self.norm1b.add_scaled(h, y, None)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(self.norm2.forward(h, None, ctx.act_dtype), ctx)
            self.norm2b.add_scaled(h, y, None)
        return h, None


BLOCKS.register("sandwich_norm_residual", SandwichNormResidual)


class PostNormResidual(Part):
    """Arrangement with the norm AFTER the sum (post-LN), the stream scaled before it:

        h = norm1(a * h + mixer(h));  h = norm2(a * h + feed_forward(h))

    with a = the layer spec's `residual_scale`. The sublayers read the stream itself (in a
    bfloat16 engine the copy that the norm's kernel writes beside the float32 stream); the
    sum, the norm and the stream are float32. A layer may have no feed-forward (it then has
    no second norm). A sublayer that offers `output_bias` (its last product's bias, left
    unadded when the block sets `defer_output_bias`) has it added in the norm's kernel.
    Tensor roles of the layer spec: mixer_norm, ffn_norm."""

    STREAM_KEY = PostNormScaledResidual.STREAM_KEY

    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        has_ffn = spec.feed_forward is not None
        roles = ["mixer_norm"] + (["ffn_norm"] if has_ffn else [])
        self.names = tensor_names(spec.tensors, p, roles, "post-norm block")
        self.alpha = float(spec.residual_scale)
        make = NORMS.get(spec.norm.kind)
        self.norm1 = make(spec.norm, hidden, self.names["mixer_norm"])
        if not hasattr(self.norm1, "scaled_add_norm"):
            raise ValueError(f"post-norm block: the norm {spec.norm.kind!r} cannot norm the "
                             "stream in place (no scaled_add_norm)")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        self.norm2 = self.feed_forward = None
        if has_ffn:
            self.norm2 = make(spec.norm, hidden, self.names["ffn_norm"])
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
                spec.feed_forward, hidden, p, device)
        for part in (self.mixer, self.feed_forward):
            if part is None:
                continue
            if hasattr(part, "out_dtype"):
                part.out_dtype = torch.float32      # the sum that follows is float32
            if hasattr(part, "defer_output_bias"):
                part.defer_output_bias = True       # added in the norm's kernel

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def libraries(self, dtype, page_size):
        out = ["layer_ops"]
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    _rows = PostNormScaledResidual._rows

    def _norm(self, norm, h, y, part, ctx):
        act = None
        if ctx.act_dtype != torch.float32:
            act = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        norm.scaled_add_norm(h, y, getattr(part, "output_bias", None), self.alpha, act)
        ctx.aux[self.STREAM_KEY] = (h, act)

    def forward(self, h, pending, ctx, cache):
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.aux.pop(self.STREAM_KEY, None)
        self._norm(self.norm1, h, self.mixer.forward(self._rows(h, ctx), ctx, cache), self.mixer, ctx)
        if self.feed_forward is not None:
            self._norm(self.norm2, h, self.feed_forward.forward(self._rows(h, ctx), ctx),
                       self.feed_forward, ctx)
        return h, None


BLOCKS.register("postnorm_residual", PostNormResidual)


class HyperConnections(Part):
    """Arrangement with `streams` copies x_1 .. x_S of the residual stream and learned
    coefficients for how each sublayer reads them and writes back. For sublayer q (the mixer,
    then the feed-forward) with coefficients in_q [S], out_q [S] and mix_q [S, S] ([from, to]):

        u   = sum_s in_q[s] x_s
        y   = sublayer_q(norm_q(u))
        x_t = sum_s mix_q[s, t] x_s + out_q[t] y          all t at once, from the old streams

    All streams equal the block's input when it is the first of its kind to run; what the
    block hands on as the stream is the sum of its streams, and the streams themselves stay
    in the step's context for the next block of this kind. Streams, coefficients, norms and
    sums are float32. The write of the mixer's result also makes the feed-forward's input.
    A layer may have no feed-forward. Tensor roles of the layer spec: mixer_norm, mixer_in,
    mixer_out, mixer_mix and ffn_norm, ffn_in, ffn_out, ffn_mix."""

    STREAMS_KEY = "residual_streams"     # ctx.aux: (the summed stream it belongs to, x [S, T, d])

    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        self.S = int(spec.streams)
        if not 1 <= self.S <= ops.MAX_STREAMS:
            raise ValueError(f"hyper-connections block: {self.S} streams; 1 to {ops.MAX_STREAMS}")
        has_ffn = spec.feed_forward is not None
        roles = ["mixer_norm", "mixer_in", "mixer_out", "mixer_mix"] + \
            (["ffn_norm", "ffn_in", "ffn_out", "ffn_mix"] if has_ffn else [])
        self.names = tensor_names(spec.tensors, p, roles, "hyper-connections block")
        self.hidden = hidden
        make = NORMS.get(spec.norm.kind)
        self.norm1 = make(spec.norm, hidden, self.names["mixer_norm"])
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        self.norm2 = self.feed_forward = None
        if has_ffn:
            self.norm2 = make(spec.norm, hidden, self.names["ffn_norm"])
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
                spec.feed_forward, hidden, p, device)
        for norm in (self.norm1, self.norm2):
            if norm is not None and (not hasattr(norm, "gain") or getattr(norm, "groups", 1) != 1):
                raise ValueError(f"hyper-connections block: the norm {spec.norm.kind!r} is not a "
                                 "plain RMS norm with a gain")
        # the write into the streams is float32: the sublayers' last products keep float32 rows
        for part in (self.mixer, self.feed_forward):
            if part is not None and hasattr(part, "out_dtype"):
                part.out_dtype = torch.float32
        self.coef = {}

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        S = self.S
        for q in ("mixer", "ffn") if self.feed_forward is not None else ("mixer",):
            out += [WeightSpec(self.names[q + "_in"], (S,), "gain"),
                    WeightSpec(self.names[q + "_out"], (S,), "gain"),
                    WeightSpec(self.names[q + "_mix"], (S, S), "constant")]
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)
        for role, name in self.names.items():
            if role.endswith(("_in", "_out", "_mix")):
                self.coef[role] = weights[name].to(torch.float32).contiguous()

    def libraries(self, dtype, page_size):
        out = ["layer_ops"]
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    def forward(self, h, pending, ctx, cache):
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.aux.pop(self.STREAMS_KEY, None)
        got = ctx.aux.get(self.STREAMS_KEY)
        if got is not None and got[0] is h and got[1].shape[0] == self.S:
            x = got[1]
        else:
            x = torch.empty((self.S,) + tuple(h.shape), dtype=torch.float32, device=h.device)
            ops.stream_spread(h, x)
        c, eps = self.coef, self.norm1.eps
        n = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        ops.stream_read_norm(x, c["mixer_in"], self.norm1.gain, eps, n)
        y = self.mixer.forward(n, ctx, cache)
        if self.feed_forward is None:
            ops.stream_write(x, y, c["mixer_mix"], c["mixer_out"], sum_out=h)
        else:
            n = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
            ops.stream_write(x, y, c["mixer_mix"], c["mixer_out"], self.norm2.eps, c["ffn_in"],
                             self.norm2.gain, n)
            y = self.feed_forward.forward(n, ctx)
            ops.stream_write(x, y, c["ffn_mix"], c["ffn_out"], sum_out=h)
        ctx.aux[self.STREAMS_KEY] = (h, x)
        return h, None


BLOCKS.register("hyper_connections", HyperConnections)
