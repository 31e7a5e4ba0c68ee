"""RMSNorm over the last axis, with the residual add (and the row selection before the
head) fused into the same kernel, or, for the few rows of a decode step, left to the product
that consumes them: y = (x * rsqrt(mean x^2 + eps)) * gain, eps inside
the root, sums in float32 (nn/blocks.go:53-55; internal/oracle/oracle.go:31-67)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import NormSpec
from ..kernels import ops
from ..registry import NORMS
from ..weights.binder import WeightSpec
from .base import Part


def stored_gain(w: torch.Tensor, unit_offset: bool) -> torch.Tensor:
    """The gain a norm multiplies by, in float32: the stored weight itself, or, for a weight
    that is zero-centred (`unit_offset`), 1 + w (added in float32)."""
    w = w.to(torch.float32)
    return (w + 1.0).contiguous() if unit_offset else w.contiguous()


class RMSNorm(Part):
    def __init__(self, spec: NormSpec, width: int, name: str):
        self.eps = float(spec.eps)
        self.width = width
        self.name = name
        self.unit_offset = bool(getattr(spec, "unit_offset", False))
        self.gain: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.width,), "gain")]

    def bind(self, weights):
        self.gain = stored_gain(weights[self.name], self.unit_offset)

    def libraries(self, dtype, page_size):
        return ["elementwise"]

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, lazy: bool = False):
        """With `lazy` (the consumer takes `ops.NormedRows`), a few bfloat16 rows with nothing
        to add are handed on uncomputed: the product that reads them norms them itself."""
        if lazy and delta is None and rows is None and out_dtype == torch.bfloat16 and \
                h.is_cuda and h.shape[0] <= ops.SKINNY_MAX_ROWS:
            return ops.NormedRows(h, self.gain, self.eps, out_dtype)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=h.device)
        ops.add_rmsnorm(h, delta, self.gain, self.eps, out, rows)
        return out

    def scaled_add_norm(self, h: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor],
                        alpha: float, act: Optional[torch.Tensor] = None) -> None:
        """h <- gain * norm(alpha * h + y + bias): the stream itself is normed, in place, for
        blocks that norm AFTER the sum; `act` also gets the new stream in the activation type."""
        ops.scaled_add_norm(h, y, bias, alpha, self.gain, self.eps, act)


class GroupRMSNorm(Part):
    """RMSNorm in groups: the row is cut into `groups` equal consecutive parts, each divided by
    sqrt(mean of its squares + eps), and the whole multiplied by the gain (groups = 1 is the
    plain norm). Besides the norm of the stream's rows it offers `add_scaled`, for blocks that
    norm a sublayer's output instead of its input."""

    def __init__(self, spec: NormSpec, width: int, name: str):
        self.eps = float(spec.eps)
        self.groups = int(getattr(spec, "groups", 1) or 1)
        if width % self.groups:
            raise ValueError(f"group norm: {self.groups} groups do not divide {width} channels")
        self.width = width
        self.name = name
        self.unit_offset = bool(getattr(spec, "unit_offset", False))
        self.gain: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.width,), "gain")]

    def bind(self, weights):
        self.gain = stored_gain(weights[self.name], self.unit_offset)

    def libraries(self, dtype, page_size):
        return ["elementwise", "layer_ops"]

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None):
        if delta is not None:
            ops.residual_add(h, delta)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=h.device)
        ops.group_norm_rows(h, rows, self.gain, self.eps, self.groups, out)
        return out

    def add_scaled(self, h: torch.Tensor, y: torch.Tensor, scale: Optional[torch.Tensor],
                   act: Optional[torch.Tensor] = None) -> None:
        """h += scale * gain * norm(y), the stream h in float32; `act` also gets the new
        stream in the activation type."""
        ops.group_norm_scale_add(h, y, self.gain, scale, self.eps, self.groups, act)

    def scaled_add_norm(self, h: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor],
                        alpha: float, act: Optional[torch.Tensor] = None) -> None:
        """h <- gain * norm(alpha * h + y + bias), in place (one group only)."""
        if self.groups != 1:
            raise ValueError("group norm: the norm of the stream itself is not grouped")
        ops.scaled_add_norm(h, y, bias, alpha, self.gain, self.eps, act)


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("group_rmsnorm", GroupRMSNorm)
