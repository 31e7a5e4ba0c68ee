"""Rotary position encoding with half-split pairing: channel i of a head is paired with
channel i + rot/2 and the pair is rotated by position * theta^(-2i/rot)
(internal/oracle/rope.go:83-146; nn/attention.go:203-211). The reference reaches the same
pairing by permuting channels at load and running an interleaved kernel
(weights/convert.go:88-125); here the weights stay as the checkpoint has them and the
kernel pairs across the half."""
from __future__ import annotations

import torch

from ..config.spec import PositionSpec
from ..kernels import ops
from ..registry import POSITIONS
from .base import Part


class RopeHalfSplit(Part):
    fusable = True      # rotary() describes it fully; the mixer's kernel does the rotation
    pairing = "half_split"

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        rot = spec.rotary_dim or head_dim
        if rot % 2 or rot <= 0 or rot > head_dim:
            raise ValueError(f"rotary_dim {rot} must be even and within head_dim {head_dim}")
        self.rotary_dim = rot
        self.theta = float(spec.theta)
        self.magnitude = 1.0
        self.inv_freq = self.frequencies(spec, rot).to(device)
        self._key = ("rope_table", rot, self.theta, getattr(spec, "scaling", None))

    def frequencies(self, spec: PositionSpec, rot: int) -> torch.Tensor:
        i = torch.arange(rot // 2, dtype=torch.float64)
        return self.theta ** (-2.0 * i / rot)

    def table(self, ctx):
        """Cosines and sines of this step's positions, made once per step and shared by
        every layer with the same rotary_dim, theta and stretch."""
        got = ctx.aux.get(self._key)
        if got is None:
            got = ops.rope_table(ctx.positions, self.inv_freq, self.magnitude)
            ctx.aux[self._key] = got
        return got

    def rotary(self, ctx):
        """(table, rotary_dim): lets a mixer do the rotation inside its own kernel."""
        return self.table(ctx), self.rotary_dim

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        """Rotate q [T, H*dh] and k [T, Hkv*dh] in place."""
        ops.qk_norm_rope_cache(q, k, None, num_heads, num_kv_heads, head_dim, None, None, 0.0,
                               self.table(ctx), self.rotary_dim, None, None, None, 0)


class RopeStretched(RopeHalfSplit):
    """The half-split rotation with its frequencies stretched for contexts longer than the
    `original` one it was made for (the scheme known as YaRN): with f_i = theta^(-2i/rot),
    pairs that turn more than `fast` times over the original context keep f_i, pairs that
    turn fewer than `slow` times get f_i / factor, and between them a linear ramp blends the
    two. With turns(t) = rot ln(original / (2 pi t)) / (2 ln theta): lo = max(floor(turns(fast)),
    0), hi = min(ceil(turns(slow)), rot - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    frequency_i = (f_i / factor) r_i + f_i (1 - r_i). Cosines and sines are both multiplied by
    0.1 ln(factor) + 1."""

    def frequencies(self, spec: PositionSpec, rot: int) -> torch.Tensor:
        import math
        base = super().frequencies(spec, rot)
        if not spec.scaling:
            return base
        factor, original, fast, slow = (float(x) for x in spec.scaling)

        def turns(t: float) -> float:
            return rot * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(turns(fast)), 0)
        hi = min(math.ceil(turns(slow)), rot - 1)
        i = torch.arange(rot // 2, dtype=torch.float64)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        self.magnitude = 0.1 * math.log(factor) + 1.0
        return base / factor * ramp + base * (1.0 - ramp)


class RopeInterleaved(RopeHalfSplit):
    """The rotation with neighbouring channels paired: channel 2i of a head turns with channel
    2i + 1 by position * theta^(-2i/rot), for the first `rot` channels; the rest pass. With
    `scaling` = (factor,) every frequency is divided by the factor (linear position
    interpolation). The table of cosines and sines is the half-split one's (pair i has column
    i); `pairing` tells a mixer's kernel which channels belong to pair i. A mixer that only
    knows the half-split pairing calls `apply`."""
    fusable = False
    pairing = "interleaved"

    def frequencies(self, spec: PositionSpec, rot: int) -> torch.Tensor:
        base = super().frequencies(spec, rot)
        if spec.scaling:
            base = base / float(spec.scaling[0])
        return base

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        table = self.table(ctx)
        for x, heads in ((q, num_heads), (k, num_kv_heads)):
            if x is not None:
                ops.qkv_bias_rope_cache(x, None, None, heads, 0, head_dim, head_dim, None, None,
                                        None, table, self.rotary_dim, True, None, None, None, 0)


class RopeStretchedInterleaved(RopeStretched):
    """The stretched rotation (ramp over the pairs, enlarged cosines and sines) with
    neighbouring channels paired: pair i is channels 2i and 2i + 1."""
    fusable = False
    pairing = "interleaved"

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        RopeInterleaved.apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim)


class RopeBanded(RopeHalfSplit):
    """The half-split rotation slowed by wavelength bands (the scheme Llama 3.1 uses):
    `scaling` = (factor, low, high, original). With f_i = theta^(-2i/rot) and the wavelength
    l_i = 2 pi / f_i: short waves, l_i < original / high, keep f_i; long waves, l_i > original
    / low, get f_i / factor; between them, with s = (original / l_i - low) / (high - low), the
    frequency is (1 - s) f_i / factor + s f_i."""

    def frequencies(self, spec: PositionSpec, rot: int) -> torch.Tensor:
        import math
        base = super().frequencies(spec, rot)
        if not spec.scaling:
            return base
        factor, low, high, original = (float(x) for x in spec.scaling)
        wave = 2.0 * math.pi / base
        s = (original / wave - low) / (high - low) if high != low else torch.ones_like(wave)
        out = (1.0 - s) * base / factor + s * base
        out = torch.where(wave < original / high, base, out)
        out = torch.where(wave > original / low, base / factor, out)
        return out


class NoPosition(Part):
    """Positions do not enter the mixer."""
    fusable = True

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        pass

    def rotary(self, ctx):
        return None, 0

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        pass


POSITIONS.register("rope_half_split", RopeHalfSplit)
POSITIONS.register("rope_stretched", RopeStretched)
POSITIONS.register("rope_interleaved", RopeInterleaved)
POSITIONS.register("rope_stretched_interleaved", RopeStretchedInterleaved)
POSITIONS.register("rope_banded", RopeBanded)
POSITIONS.register("none", NoPosition)
