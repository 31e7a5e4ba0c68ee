"""Causal softmax attention over a compressed cache (the latent attention of DeepSeek-V2):
every token keeps ONE small row instead of keys and values per head.

    c_q = norm(W_dq x) * g_q                     the queries' latent (query_rank wide)
    q_h = W_uq,h c_q = [q_h,nope (head_dim), q_h,rope (rope_dim)]
    [c', r'] = W_dkv x;   c = norm(c') * g_kv    the latent (latent_rank wide)
                          r = rotated r'         one rotated key part for all heads (rope_dim)
    k_h,nope(j) = W_uk,h c(j),   v_h(j) = W_uv,h c(j)
    score_h(i, j) = (q_h,nope(i) . k_h,nope(j) + rotated q_h,rope(i) . r(j)) * scale,  j <= i
    out = W_o concat_h softmax_j(score_h(i, .)) v_h

The cache holds [c, r] per token, one plane, rows latent_rank + rope_dim wide. Keys and values
are never expanded: since q_nope . (W_uk c) = (W_uk^T q_nope) . c and sum_j w_j W_uv c(j) =
W_uv sum_j w_j c(j), the expansion matrices are applied to the query and to the attention's
result, a product per head, and the attention itself has one key/value head whose key is the
whole cached row and whose value is its first latent_rank channels. It runs in the kernels of
`sink_attention` (`parts/attention_sink.py`), which take such a row. Norms, rotation, scores
and softmax are float32. Tensor roles: q_down, q_down_norm, q_up, kv_down, kv_norm, k_up, v_up, o.
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .attention import step_tiles
from .attention_sink import sink_attention, tile_form
from .base import CacheNeed, LayerCache, Part


class LatentAttention(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.dn, self.dr = spec.num_heads, spec.head_dim, spec.rope_dim
        self.dv = spec.value_dim or spec.head_dim
        self.rank, self.q_rank = spec.latent_rank, spec.query_rank
        if min(self.H, self.dn, self.dv, self.rank, self.q_rank) <= 0 or self.dr < 0:
            raise ValueError("latent attention: heads, head_dim, value_dim, latent_rank and "
                             "query_rank must be positive")
        self.row = self.rank + self.dr               # what a token keeps in the cache
        self.eps = float(spec.norm_eps)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.dn + self.dr)
        pos = spec.position
        self.position = POSITIONS.get(pos.kind)(pos, self.dr, device) \
            if pos is not None and self.dr else None
        if self.position is not None and not hasattr(self.position, "table"):
            raise ValueError("latent attention: the rotation is done inside its kernels and needs "
                             "a position encoding that offers a table of cosines and sines")
        self.names = tensor_names(spec.tensors, prefix,
                                  ["q_down", "q_down_norm", "q_up", "kv_down", "kv_norm", "k_up",
                                   "v_up", "o"], "latent attention")
        self.w_dq = self.w_uq = self.w_dkv = self.w_uk_t = self.w_uv = self.w_o = None
        self.q_gain = self.kv_gain = None

    def weight_specs(self):
        n, d, H = self.names, self.hidden, self.H
        return [WeightSpec(n["q_down"], (self.q_rank, d)),
                WeightSpec(n["q_down_norm"], (self.q_rank,), "gain"),
                WeightSpec(n["q_up"], (H * (self.dn + self.dr), self.q_rank)),
                WeightSpec(n["kv_down"], (self.row, d)),
                WeightSpec(n["kv_norm"], (self.rank,), "gain"),
                WeightSpec(n["k_up"], (H * self.dn, self.rank)),
                WeightSpec(n["v_up"], (H * self.dv, self.rank)),
                WeightSpec(n["o"], (d, H * self.dv))]

    def cache_need(self):
        return CacheNeed("full", None, 1, (1, self.row))

    def state_need(self):
        return None

    def bind(self, weights):
        n, H = self.names, self.H
        self.w_dq = weights.pop(n["q_down"]).contiguous()
        self.w_uq = weights.pop(n["q_up"]).contiguous()
        self.w_dkv = weights.pop(n["kv_down"]).contiguous()
        # per head: W_uk,h^T [latent_rank, head_dim] (applied to the query) and W_uv,h
        # [value_dim, latent_rank] (applied to the attention's result)
        self.w_uk_t = weights.pop(n["k_up"]).reshape(H, self.dn, self.rank).transpose(1, 2).contiguous()
        self.w_uv = weights.pop(n["v_up"]).reshape(H, self.dv, self.rank).contiguous()
        self.w_o = weights.pop(n["o"]).contiguous()
        self.q_gain = weights.pop(n["q_down_norm"]).to(torch.float32).contiguous()
        self.kv_gain = weights.pop(n["kv_norm"]).to(torch.float32).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        names = ["sgemm" if dtype == torch.float32 else "gemm_skinny", "elementwise", "layer_ops",
                 "latent", "attention_generic"]
        if dtype == torch.bfloat16:
            names.append("attention_sink")
        return names

    def prepare_capture(self, ctx, cache) -> None:
        form, tokens = tile_form(self.H, 1, self.row, self.rank, self.row, ctx.act_dtype)
        if not ctx.decode_only and cache is not None and form is not None:
            step_tiles(ctx, tokens)

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n, H, d = sum(extents), self.H, self.hidden
        per_token = d * (self.q_rank + self.row) + self.q_rank * H * (self.dn + self.dr) + \
            H * self.dn * self.rank + H * self.dv * self.rank + H * self.dv * d
        keys = sum(extent * first + extent * (extent + 1) // 2
                   for first, extent in zip(first_positions, extents))
        return 2.0 * n * per_token + 2.0 * H * (self.row + self.rank) * keys

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return self.row * width * context_len

    def forward(self, x, ctx, cache: LayerCache):
        H, dn, dr, dv, rank, row = self.H, self.dn, self.dr, self.dv, self.rank, self.row
        x = ops.rows_of(x)
        T, dev = x.shape[0], x.device
        # the queries' latent: product in float32 rows, norm, then the up product
        cq_raw = ops.linear(x, self.w_dq, out_dtype=torch.float32)
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=dev)
        ops.gated_group_norm(cq_raw, None, self.q_gain, cq, 1, self.eps, None, False)
        q = ops.linear(cq, self.w_uq)                                   # [T, H (dn + dr)]
        kv = ops.linear(x, self.w_dkv)                                  # [T, rank + dr]
        table, rot, interleaved = None, 0, False
        if self.position is not None:
            table, rot = self.position.table(ctx), self.position.rotary_dim
            interleaved = getattr(self.position, "pairing", "half_split") == "interleaved"
        ops.latent_row_cache(kv, rank, dr, self.kv_gain, self.eps, table, rot, interleaved,
                             cache.slots, cache.k, cache.page_size)
        # the query as the cache sees it: [W_uk^T q_nope, rotated q_rope] per head
        qa = torch.empty((T, H * row), dtype=x.dtype, device=dev)
        ops.head_linear(q, dn + dr, self.w_uk_t, qa, row)
        if dr:
            ops.rope_slice(q, dn + dr, dn, qa, row, rank, H, dr, table, rot, interleaved)
        lat = torch.empty((T, H * rank), dtype=x.dtype, device=dev)
        sink_attention(qa, lat, H, 1, row, rank, cache, ctx, self.scale, 0, None, value_row=row)
        a = torch.empty((T, H * dv), dtype=x.dtype, device=dev)
        ops.head_linear(lat, rank, self.w_uv, a, dv)
        return ops.linear(a, self.w_o, out_dtype=self.out_dtype)


MIXERS.register("latent_attention", LatentAttention)
