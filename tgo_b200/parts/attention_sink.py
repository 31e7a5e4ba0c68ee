"""Grouped-query causal softmax attention over the paged cache, of the kind that has

  - keys `head_dim` wide and values `value_dim` wide (two cache planes with rows of their own);
  - `bias`: the q, k and v projections carry biases, added in float32;
  - a rotation of the first rotary_dim channels of q and k in either pairing (the position
    encoding says which);
  - `window`: a query reads itself and the window - 1 keys before it;
  - `sink`: one learned number per query head joins the softmax's denominator as exp(sink_h);
    the term stands for no token (nothing is read for it and nothing added to the output)
    and enters unscaled, a single time;
  - `qk_norm` with scope "row": q and k are RMS-normed over a token's whole projection row
    (all heads at once, gains as wide as the rows), before the heads are split and rotated;
  - `softcap` c: every scaled score goes through c tanh(score / c) before the softmax;
  - `conv_taps`: q, k and v each pass a causal convolution of that many taps over time (per
    channel, no bias), straight after their projections; the last taps - 1 projected rows of
    a request are its state;
  - `qk_unit_norm`: every q and k head is divided by its root mean square after the rotation;
  - `keep_first`: beside the window a query reads the first keep_first keys of its request;
  - `query_temperature` (coef, every): q at position p times 1 + coef ln(floor((p+1)/every) + 1);
  - `distance_bias_max` D: a learned table [rows, heads] adds table[bucket(i - j), h] to the
    scaled score, bucket(n) = n below rows/2, then min(rows - 1, rows/2 + floor(ln(n / (rows/2))
    / ln(D / (rows/2)) * (rows - rows/2))).

    score(i, j) = (q_i . k_j) * scale       for 0 <= i - j < window
    w(i, j)     = exp(score(i, j)) / (exp(sink_h) + sum_j' exp(score(i, j')))
    out_i       = Wo concat_h sum_j w_h(i, j) v_kv(h)(j)

Scores, softmax and sums are float32. Tensor roles: q, k, v, o and, with `bias`, q_bias, k_bias,
v_bias; with `sink`, sink; with the row norm, q_norm, k_norm; with the convolution, q_conv,
k_conv, v_conv ([channels, taps]); with the distance bias, distance_bias.
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .attention import decode_splits, step_tiles
from .base import CacheNeed, LayerCache, Part, StateNeed


def distance_bucket(n: int, rows: int, bias_max: int) -> int:
    """Row of a distance-bias table for the distance n >= 0."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half)
                                               * (rows - half))))


def bias_by_distance(table: torch.Tensor, bias_max: int) -> torch.Tensor:
    """[rows, heads] -> [n, heads] float32 with row i the bias at distance i; the last row
    stands for every larger distance (from bias_max on the bucket is the last one)."""
    rows = table.shape[0]
    if rows < 2 or bias_max <= rows // 2:
        raise ValueError(f"attention: a distance bias of {rows} rows up to distance {bias_max}; "
                         "the table needs two rows and a distance beyond its linear half")
    n = 1
    while distance_bucket(n - 1, rows, bias_max) < rows - 1:     # ends: bucket(bias_max) is the last
        n += 1
    idx = torch.tensor([distance_bucket(i, rows, bias_max) for i in range(n)], dtype=torch.long,
                       device=table.device)
    return table.to(torch.float32).index_select(0, idx).contiguous()


class SinkAttention(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.Hkv, self.dk = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.dv = spec.value_dim or spec.head_dim
        if self.H <= 0 or self.Hkv <= 0 or self.H % self.Hkv:
            raise ValueError(f"attention: {self.H} query heads do not group over {self.Hkv}")
        self.window = spec.window
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.dk)
        self.bias, self.sink = bool(spec.bias), bool(spec.sink)
        self.softcap = float(spec.softcap) if getattr(spec, "softcap", None) else 0.0
        self.row_norm = bool(spec.qk_norm)
        if self.row_norm and getattr(spec, "qk_norm_scope", "head") != "row":
            raise ValueError("attention: this mixer norms q and k over whole rows (qk_norm_scope "
                             "'row'); the per-head norm belongs to gqa_attention")
        if self.row_norm and self.bias:
            raise ValueError("attention: biased projections with a q/k norm are not offered")
        self.eps = float(spec.norm_eps)
        pos = spec.position
        self.position = POSITIONS.get(pos.kind)(pos, self.dk, device) if pos is not None else None
        if self.position is not None and not hasattr(self.position, "table"):
            raise ValueError("attention: this mixer rotates inside its own kernel and needs a "
                             "position encoding that offers a table of cosines and sines")
        self.taps = int(getattr(spec, "conv_taps", 0) or 0)
        self.unit_norm = bool(getattr(spec, "qk_unit_norm", False))
        self.keep_first = int(getattr(spec, "keep_first", 0) or 0)
        if self.keep_first and not self.window:
            raise ValueError("attention: keep_first belongs to a window")
        self.temperature = getattr(spec, "query_temperature", None)
        self.bias_max = getattr(spec, "distance_bias_max", None)
        if (self.taps or self.unit_norm) and (self.bias or self.row_norm):
            raise ValueError("attention: the convolution and the unit norm after the rotation are "
                             "not offered together with biases or the row norm")
        if self.temperature is not None and not self.row_norm:
            raise ValueError("attention: the query temperature is applied by the row norm's kernel")
        roles = ["q", "k", "v", "o"] + (["q_bias", "k_bias", "v_bias"] if self.bias else []) + \
            (["sink"] if self.sink else []) + (["q_norm", "k_norm"] if self.row_norm else []) + \
            (["q_conv", "k_conv", "v_conv"] if self.taps else []) + \
            (["distance_bias"] if self.bias_max is not None else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "attention")
        self.w_qkv = self.w_o = self.b_q = self.b_k = self.b_v = self.sinks = None
        self.q_gain = self.k_gain = self.conv = self.dist_bias = None

    def weight_specs(self):
        n, d = self.names, self.hidden
        qw, kw, vw = self.H * self.dk, self.Hkv * self.dk, self.Hkv * self.dv
        out = [WeightSpec(n["q"], (qw, d)), WeightSpec(n["k"], (kw, d)), WeightSpec(n["v"], (vw, d)),
               WeightSpec(n["o"], (d, self.H * self.dv))]
        if self.bias:
            out += [WeightSpec(n["q_bias"], (qw,), "gain"), WeightSpec(n["k_bias"], (kw,), "gain"),
                    WeightSpec(n["v_bias"], (vw,), "gain")]
        if self.sink:
            out.append(WeightSpec(n["sink"], (self.H,), "gain"))
        if self.row_norm:
            out += [WeightSpec(n["q_norm"], (qw,), "gain"), WeightSpec(n["k_norm"], (kw,), "gain")]
        if self.taps:
            out += [WeightSpec(n["q_conv"], (qw, self.taps), "constant"),
                    WeightSpec(n["k_conv"], (kw, self.taps), "constant"),
                    WeightSpec(n["v_conv"], (vw, self.taps), "constant")]
        if self.bias_max is not None:
            out.append(WeightSpec(n["distance_bias"], (-1, self.H), "constant"))   # rows: the tensor's
        return out

    def cache_need(self):
        return CacheNeed.keys_and_values_of(self.window, self.Hkv, self.dk, self.dv,
                                            keep_first=self.keep_first)

    def state_need(self):
        """The convolution's last taps - 1 projected rows (q, k, v side by side)."""
        if self.taps > 1:
            return StateNeed(((self.taps - 1) * (self.H * self.dk + self.Hkv * (self.dk + self.dv)),))
        return None

    def bind(self, weights):
        n = self.names
        self.w_qkv = torch.cat([weights.pop(n["q"]), weights.pop(n["k"]), weights.pop(n["v"])],
                               dim=0).contiguous()
        self.w_o = weights.pop(n["o"]).contiguous()
        if self.bias:
            self.b_q, self.b_k, self.b_v = (weights.pop(n[r]).to(torch.float32).contiguous()
                                            for r in ("q_bias", "k_bias", "v_bias"))
        if self.sink:
            self.sinks = weights.pop(n["sink"]).to(torch.float32).contiguous()
        if self.row_norm:
            self.q_gain = weights.pop(n["q_norm"]).to(torch.float32).contiguous()
            self.k_gain = weights.pop(n["k_norm"]).to(torch.float32).contiguous()
        if self.taps:
            self.conv = torch.cat([weights.pop(n[r]).to(torch.float32) for r in
                                   ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        if self.bias_max is not None:
            self.dist_bias = bias_by_distance(weights.pop(n["distance_bias"]), int(self.bias_max))

    def libraries(self, dtype, page_size) -> List[str]:
        names = ["sgemm" if dtype == torch.float32 else "gemm_skinny", "elementwise",
                 "attention_generic"]
        if dtype == torch.bfloat16:
            names.append("attention_sink")
        return names

    def prepare_capture(self, ctx, cache) -> None:
        if not ctx.decode_only and cache is not None and ctx.act_dtype == torch.bfloat16 and \
                USE_TILE_KERNELS and ops.attention_sink_supports(self.H, self.Hkv, self.dk, self.dv):
            step_tiles(ctx, ops.attention_sink_tile_tokens(self.H // self.Hkv))

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        qw, kw, vw = self.H * self.dk, self.Hkv * self.dk, self.H * self.dv
        total = 2.0 * n * self.hidden * (qw + kw + self.Hkv * self.dv) + 2.0 * n * vw * self.hidden
        keys = 0
        for first, extent in zip(first_positions, extents):
            if self.window:
                keys += sum(min(first + t + 1, self.window) for t in range(extent))
            else:
                keys += extent * first + extent * (extent + 1) // 2
        return total + (2.0 * qw + 2.0 * vw) * keys

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        reach = min(context_len, self.window) if self.window else context_len
        return self.Hkv * (self.dk + self.dv) * width * reach

    def forward(self, x, ctx, cache: LayerCache):
        H, Hkv, dk, dv = self.H, self.Hkv, self.dk, self.dv
        qw, kw = H * dk, Hkv * dk
        x = ops.rows_of(x)
        qkv = ops.linear(x, self.w_qkv)
        q, k, v = qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:]
        table, rot, interleaved = None, 0, False
        if self.position is not None:
            table, rot = self.position.table(ctx), self.position.rotary_dim
            interleaved = getattr(self.position, "pairing", "half_split") == "interleaved"
        if self.taps or self.unit_norm:
            q = torch.empty((x.shape[0], qw), dtype=qkv.dtype, device=qkv.device)
            ops.qkv_conv_rope_norm_cache(qkv, q, H, Hkv, dk, dv, self.conv, ctx.num_seqs, ctx.seq_ids,
                                         ctx.q_start, ctx.state_slots, cache.state, 0, table, rot,
                                         interleaved, self.unit_norm, self.eps, cache.slots, cache.k,
                                         cache.v, cache.page_size)
        elif self.row_norm:
            coef, every = self.temperature or (0.0, 0)
            ops.qk_rownorm_rope_cache(q, k, v, H, Hkv, dk, dv, self.q_gain, self.k_gain, self.eps,
                                      table, rot, interleaved, cache.slots, cache.k, cache.v,
                                      cache.page_size, ctx.positions, float(coef), int(every))
        else:
            ops.qkv_bias_rope_cache(q, k, v, H, Hkv, dk, dv, self.b_q, self.b_k, self.b_v, table,
                                    rot, interleaved, cache.slots, cache.k, cache.v, cache.page_size)
        a = torch.empty((x.shape[0], H * dv), dtype=q.dtype, device=q.device)
        sink_attention(q, a, H, Hkv, dk, dv, cache, ctx, self.scale, self.window or 0, self.sinks,
                       softcap=self.softcap, keep_first=self.keep_first, dist_bias=self.dist_bias)
        return ops.linear(a, self.w_o, out_dtype=self.out_dtype)


USE_TILE_KERNELS = True


def tile_form(H, Hkv, dk, dv, value_row, dtype):
    """Which tensor-core kernel takes an attention of these sizes, and how many tokens of one
    request a tile of its holds: ("tile", n) for key and value rows up to 128 wide, ("wide", n)
    for wider key rows whose first dv channels are the values (value_row == dk), else (None, 0)."""
    if not USE_TILE_KERNELS or dtype != torch.bfloat16 or value_row % 8:
        return None, 0
    if ops.attention_sink_supports(H, Hkv, dk, dv):
        return "tile", ops.attention_sink_tile_tokens(H // Hkv)
    if value_row == dk and ops.attention_sink_wide_supports(H, Hkv, dk, dv):
        return "wide", ops.attention_sink_wide_tile_tokens(H // Hkv)
    return None, 0


def sink_attention(q, out, H, Hkv, dk, dv, cache, ctx, scale, window, sinks, softcap=0.0,
                   value_row=0, keep_first=0, dist_bias=None) -> None:
    """`keep_first`: the first keys of a request that stay visible beside the window; `dist_bias`
    [n, H]: added to the scores by distance. `softcap` bounds the scores; `value_row` > 0 says that a value is the first dv channels
    of its key row, `value_row` wide (one cache plane serves as keys and values).
    Which kernel runs the attention of a step. bfloat16 at sizes a tensor-core kernel takes
    (`tile_form`): that kernel, over tiles of consecutive tokens for steps with prompt portions
    (single tokens beside them are tiles of one), a tile a token for steps of single tokens, whose
    keys may be cut over several blocks. float32,
    and other sizes: the generic kernel (a warp per token and head, keys in a fixed order)."""
    v_cache = cache.k if value_row else cache.v
    form, tokens = tile_form(H, Hkv, dk, dv, value_row, q.dtype)
    if form == "wide" and (keep_first or dist_bias is not None):
        form = None                     # the kernel for wide rows knows neither
    if form is not None and ops.attention_sink_takes(q, out):
        tok0, ntok = (None, None) if ctx.decode_only else step_tiles(ctx, tokens)
        if form == "wide":
            # one block a multiprocessor, tiles of rows several times as wide: by the sweep over
            # shares at batches 8 and 64, a start costs about one tile and the join two
            splits = decode_splits(ctx, Hkv, window, q.device, ctas_per_sm=1, start=1.0, join=2.0) \
                if ctx.decode_only else 1
            ops.attention_sink_wide(q, out, H, Hkv, dk, dv, cache.k, cache.page_size, cache.block_tables,
                                    ctx.seq_ids, ctx.positions, scale, window, sinks, tok0, ntok,
                                    n_splits=splits, softcap=softcap)
            return
        splits = decode_splits(ctx, Hkv, window, q.device) if ctx.decode_only else 1
        ops.attention_sink_tile(q, out, H, Hkv, dk, dv, cache.k, v_cache, cache.page_size,
                                cache.block_tables, ctx.seq_ids, ctx.positions, scale, window, sinks,
                                tok0, ntok, n_splits=splits, softcap=softcap, value_row=value_row,
                                keep_first=keep_first, dist_bias=dist_bias)
        return
    ops.attention_generic(q, out, H, Hkv, dk, cache.k, v_cache, cache.page_size,
                          cache.block_tables, ctx.seq_ids, ctx.positions, scale, window,
                          value_dim=dv, sinks=sinks, softcap=softcap, value_row=value_row,
                          keep_first=keep_first, dist_bias=dist_bias)


MIXERS.register("sink_attention", SinkAttention)
