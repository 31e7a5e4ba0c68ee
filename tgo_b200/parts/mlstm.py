"""The matrix memory of xLSTM (mLSTM) as a mixer: linear attention whose state is gated by
an exponential input gate and a forget gate per head and token, kept stable by a running
maximum, with a fixed-size float32 state per request instead of a cache that grows.

    q = Wq x * dk^-1/2, k = Wk x (heads x dk), v = Wv x (heads x dv)
    i_t = c tanh((Wi x + bi) / c)                      log input gate, c = gate_cap
    f_t = logsigmoid(c tanh((Wf x + bf) / c))          log forget gate
    m_t = max(f_t + m_(t-1), i_t)                      m starts at 0
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T      (n_t likewise with k_t)
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    y   = Wo ( o_t / rms(o_t per head) * g * sigmoid(Wg x) )

The q, k, v and gate projections may run in the activation type; the two gates' projections
keep float32 rows, and the gates, the recurrence, its state and the per-head norm are float32.
Tensor roles: q, k, v, gate, o, out_norm, input_gate, input_gate_bias, forget_gate,
forget_gate_bias.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS
from ..weights.binder import WeightSpec
from .base import LayerCache, Part, StateNeed
from .retention import step_chunks

USE_CHUNKED = True                   # False: every step through the kernels that walk a request in order


class MLSTM(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.dk = spec.num_heads, spec.head_dim
        self.dv = spec.value_dim or spec.head_dim
        self.cap = float(spec.gate_cap)
        if self.H <= 0 or self.dk <= 0 or self.dv <= 0:
            raise ValueError("mlstm: heads, head_dim and value_dim must be positive")
        if not self.cap > 0:
            raise ValueError(f"mlstm: gate_cap is {self.cap}; the gates' bound must be positive")
        self.eps = float(spec.norm_eps)
        self.q_scale = float(self.dk) ** -0.5 if spec.scale is None else float(spec.scale)
        self.names = tensor_names(spec.tensors, prefix,
                                  ["q", "k", "v", "gate", "o", "out_norm", "input_gate",
                                   "input_gate_bias", "forget_gate", "forget_gate_bias"], "mlstm")
        self.w_in = self.w_gates = self.w_o = self.out_gain = self.b_i = self.b_f = None

    def weight_specs(self):
        n, d, H = self.names, self.hidden, self.H
        return [WeightSpec(n["q"], (H * self.dk, d)), WeightSpec(n["k"], (H * self.dk, d)),
                WeightSpec(n["v"], (H * self.dv, d)), WeightSpec(n["gate"], (H * self.dv, d)),
                WeightSpec(n["o"], (d, H * self.dv)),
                WeightSpec(n["out_norm"], (H * self.dv,), "gain"),
                WeightSpec(n["input_gate"], (H, d)), WeightSpec(n["input_gate_bias"], (H,), "gain"),
                WeightSpec(n["forget_gate"], (H, d)), WeightSpec(n["forget_gate_bias"], (H,), "gain")]

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((ops.mlstm_state_floats(self.H, self.dk, self.dv),))

    def bind(self, weights):
        n = self.names
        self.w_in = torch.cat([weights.pop(n[r]) for r in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.w_gates = torch.cat([weights.pop(n["input_gate"]), weights.pop(n["forget_gate"])],
                                 dim=0).contiguous()
        self.w_o = weights.pop(n["o"]).contiguous()
        self.out_gain = weights.pop(n["out_norm"]).to(torch.float32).contiguous()
        self.b_i = weights.pop(n["input_gate_bias"]).to(torch.float32).contiguous()
        self.b_f = weights.pop(n["forget_gate_bias"]).to(torch.float32).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm" if dtype == torch.float32 else "gemm_skinny", "layer_ops", "mlstm"]

    def _chunked(self) -> bool:
        return USE_CHUNKED and ops.mlstm_chunked_supports(self.H, self.dk, self.dv)

    def prepare_capture(self, ctx, cache) -> None:
        if not ctx.decode_only and self._chunked():
            step_chunks(ctx, ops.mlstm_chunk_tokens())

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        qk, vw = self.H * self.dk, self.H * self.dv
        products = 2.0 * n * self.hidden * (2 * qk + 2 * vw + 2 * self.H) + 2.0 * n * vw * self.hidden
        return products + 4.0 * n * self.H * self.dk * self.dv     # the state's update and read

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return 4.0 * ops.mlstm_state_floats(self.H, self.dk, self.dv)

    def forward(self, x, ctx, cache: LayerCache):
        H, dk, dv = self.H, self.dk, self.dv
        qk, vw = H * dk, H * dv
        x = ops.rows_of(x)
        z = ops.linear(x, self.w_in)
        q, k, v, gate = z[:, :qk], z[:, qk:2 * qk], z[:, 2 * qk:2 * qk + vw], z[:, 2 * qk + vw:]
        g = ops.linear(x, self.w_gates, out_dtype=torch.float32)       # [T, 2H]: input, forget
        o = torch.empty((x.shape[0], vw), dtype=torch.float32, device=x.device)
        args = (q, k, v, g[:, :H], g[:, H:], self.b_i, self.b_f, self.cap, self.q_scale, o,
                ctx.num_seqs, H, dk, dv, ctx.q_start, ctx.state_slots, cache.state)
        if not self._chunked():
            ops.mlstm(*args)             # a block per (request, head, columns), in order
        elif ctx.decode_only:
            ops.mlstm_chunked(*args)     # single tokens: the state streamed through once
        else:
            ops.mlstm_chunked(*args, *step_chunks(ctx, ops.mlstm_chunk_tokens()))
        y = torch.empty((x.shape[0], vw), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(o, gate, self.out_gain, y, H, self.eps, "sigmoid", False)
        return ops.linear(y, self.w_o, out_dtype=self.out_dtype)


MIXERS.register("mlstm", MLSTM)
