"""Python face of the CUDA kernels: each function checks its tensors, then calls the
extern "C" entry point of the same name on the current CUDA stream.

Tensors are torch tensors on a CUDA device; nothing here computes with torch, and
nothing falls back to it. A refused size raises with the kernel's name in the message.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
E_BAD_ARG = 1000

c_int, c_ll, c_float, c_void = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void(0) if t is None else c_void(t.data_ptr())


def _stream():
    return c_void(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}. There is no CPU path.")


LAUNCHES = [0]        # kernels of this package launched so far (graph replays add theirs)


def _check(status: int, name: str, detail: str = "") -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status == E_BAD_ARG:
        raise KernelError(f"{name}: refused these sizes or types {detail}")
    raise KernelError(f"{name}: CUDA error {status} at launch {detail}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale, widened to float32. ids int32 [T]; out float32 [T, d]."""
    _need_cuda(table, ids, out)
    T, d = out.shape
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    lib = load_library("elementwise")
    _check(lib.tgo_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
                         c_int(T), c_int(d), c_int(table.shape[0]), c_float(scale), _stream()), "embed")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h += delta (if given, and rows is None), out = rmsnorm(h) * gain.
    With `rows` (int32 [n]): out[i] = rmsnorm(h[rows[i]] + delta[rows[i]]) * gain, h untouched."""
    _need_cuda(h, delta, gain, out, rows)
    n, d = out.shape
    assert h.dtype == torch.float32 and gain.dtype == torch.float32 and h.is_contiguous()
    assert gain.numel() == d and out.is_contiguous() and h.shape[1] == d
    if delta is not None:
        assert delta.shape == h.shape and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert h.shape[0] == n
    lib = load_library("elementwise")
    _check(lib.tgo_add_rmsnorm(_ptr(h), _ptr(delta),
                               c_int(dtype_code(delta.dtype) if delta is not None else 0),
                               _ptr(gain), c_float(eps), _ptr(out), c_int(dtype_code(out.dtype)),
                               _ptr(rows), c_int(n), c_int(d), _stream()), "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """h += delta, h float32."""
    _need_cuda(h, delta)
    assert h.dtype == torch.float32 and h.is_contiguous() and delta.is_contiguous()
    assert h.shape == delta.shape
    lib = load_library("elementwise")
    _check(lib.tgo_residual_add(_ptr(h), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                c_ll(h.numel()), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t, j] = silu(gate_j) * up_j; gate_up holds the gate columns then the up columns,
    or, `interleaved`, eight gate columns and the eight matching up columns in turn."""
    _need_cuda(gate_up, out)
    T, f = out.shape
    assert gate_up.shape == (T, 2 * f) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    lib = load_library("elementwise")
    _check(lib.tgo_swiglu(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T),
                          c_int(f), c_int(1 if interleaved else 0), _stream()), "swiglu",
           f"(T={T}, f={f})")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, mag: float = 1.0) -> torch.Tensor:
    """[T, 2 * half] float32: cos then sin of position * inv_freq, evaluated in float64, both
    multiplied by `mag`."""
    _need_cuda(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float64
    T, half = positions.numel(), inv_freq.numel()
    table = torch.empty((T, 2 * half), dtype=torch.float32, device=positions.device)
    lib = load_library("elementwise")
    _check(lib.tgo_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), c_int(T),
                              c_int(half), ctypes.c_double(mag), _stream()), "rope_table")
    return table


def qk_norm_rope_cache(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                       num_heads: int, num_kv_heads: int, head_dim: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       rope: Optional[torch.Tensor], rotary_dim: int,
                       slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], page_size: int) -> None:
    """Per-head RMSNorm of q and k (if gains are given), half-split rotation (if `rope`, a
    table from rope_table, is given), q written back in place, k and v stored at `slots` of
    the paged cache [page, kv_head, offset, head_dim]. q, k, v are 2-D views whose rows may
    be strided (columns of one joined projection output)."""
    _need_cuda(q, k, v, q_gain, k_gain, rope, slots, k_cache, v_cache)
    T = q.shape[0]
    for t in (q, k, v):
        if t is not None:
            assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim)
        assert rope.is_contiguous()
    if k_cache is not None:
        assert k_cache.dtype == q.dtype and k_cache.is_contiguous()
        assert (v is None and v_cache is None) or \
            (v_cache.dtype == q.dtype and v_cache.is_contiguous())
        assert slots.dtype == torch.int32 and slots.numel() == T
    lib = load_library("elementwise")
    _check(lib.tgo_qk_norm_rope_cache(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0) if k is not None else 0),
        _ptr(v), c_ll(v.stride(0) if v is not None else 0), c_int(dtype_code(q.dtype)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_gain), _ptr(k_gain),
        c_float(eps), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
        _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(page_size), _stream()),
        "qk_norm_rope_cache", f"(head_dim={head_dim}, rotary_dim={rotary_dim})")


def attention_generic(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                      block_tables: torch.Tensor, seq_ids: torch.Tensor, positions: torch.Tensor,
                      scale: float, window: int, value_dim: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, softcap: float = 0.0,
                      value_row: int = 0, keep_first: int = 0,
                      dist_bias: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention, one warp per (token, head). q is a 2-D view [T, >= H*dh]
    with unit column stride; out likewise. window 0 = every earlier key. `value_dim`: width
    of a value row where it differs from the keys'; `sinks`: float32 [H], a term exp(sink_h)
    in each head's softmax denominator that has no value; `softcap` c > 0: every scaled score
    goes through c tanh(s / c); `value_row`: elements from one value row to the next where
    that is not `value_dim` (values that are the first channels of their key rows: v_cache is
    k_cache and value_row the key rows' width); `keep_first`: with a window, the first keys of
    a request that every later query still reads; `dist_bias`: float32 [n, H], row
    min(distance, n - 1) is added to the scaled scores of the keys at that distance."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions, sinks, dist_bias)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and
                                 dist_bias.shape[1] == num_heads and dist_bias.is_contiguous())
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads and
                             sinks.is_contiguous())
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert block_tables.is_contiguous() and seq_ids.dtype == torch.int32
    assert positions.dtype == torch.int32
    lib = load_library("attention_generic")
    _check(lib.tgo_attention_generic(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), c_int(dtype_code(q.dtype)),
        c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(value_dim or head_dim), _ptr(k_cache),
        _ptr(v_cache), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(seq_ids), _ptr(positions), c_float(scale), c_int(window), _ptr(sinks),
        c_float(softcap or 0.0), c_int(value_row), c_int(keep_first if window else 0),
        _ptr(dist_bias), c_int(dist_bias.shape[0] if dist_bias is not None else 0), _stream()),
        "attention_generic", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")


def cast_rows(h: torch.Tensor, out: torch.Tensor) -> None:
    """out = h narrowed to the activation type (float32 stream -> bfloat16 rows)."""
    _need_cuda(h, out)
    assert h.dtype == torch.float32 and h.is_contiguous() and out.is_contiguous()
    assert h.shape == out.shape
    lib = load_library("layer_ops")
    _check(lib.tgo_cast_rows(_ptr(h), _ptr(out), c_int(dtype_code(out.dtype)), c_ll(h.numel()),
                             _stream()), "cast_rows")


def group_norm_scale_add(h: torch.Tensor, y: torch.Tensor, gain: torch.Tensor,
                         scale: Optional[torch.Tensor], eps: float, groups: int,
                         act: Optional[torch.Tensor] = None) -> None:
    """h += scale * gain * group_rmsnorm(y): y's rows are cut into `groups` equal consecutive
    parts, each divided by sqrt(mean of its squares + eps). h is the float32 stream; with
    `act` (bfloat16, h's shape) the new stream is also written there."""
    _need_cuda(h, y, gain, scale, act)
    T, d = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous() and y.is_contiguous()
    assert y.shape == h.shape and gain.dtype == torch.float32 and gain.numel() == d
    assert scale is None or (scale.dtype == torch.float32 and scale.numel() == d)
    assert act is None or (act.shape == h.shape and act.is_contiguous())
    lib = load_library("layer_ops")
    _check(lib.tgo_group_norm_scale_add(
        _ptr(h), _ptr(y), c_int(dtype_code(y.dtype)), _ptr(gain), _ptr(scale), c_float(eps),
        c_int(groups), _ptr(act), c_int(dtype_code(act.dtype) if act is not None else 0),
        c_int(T), c_int(d), _stream()), "group_norm_scale_add", f"(d={d}, groups={groups})")


def group_norm_rows(h: torch.Tensor, rows: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                    groups: int, out: torch.Tensor) -> None:
    """out[i] = gain * group_rmsnorm(h[rows[i]]) (rows None: every row)."""
    _need_cuda(h, rows, gain, out)
    n, d = out.shape
    assert h.dtype == torch.float32 and h.is_contiguous() and out.is_contiguous()
    assert h.shape[1] == d and gain.dtype == torch.float32 and gain.numel() == d
    assert (rows is None and h.shape[0] == n) or (rows.dtype == torch.int32 and rows.numel() == n)
    lib = load_library("layer_ops")
    _check(lib.tgo_group_norm_rows(_ptr(h), _ptr(rows), _ptr(gain), c_float(eps), c_int(groups),
                                   _ptr(out), c_int(dtype_code(out.dtype)), c_int(n), c_int(d),
                                   _stream()), "group_norm_rows", f"(d={d}, groups={groups})")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place, float32."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    lib = load_library("layer_ops")
    _check(lib.tgo_softcap(_ptr(x), c_ll(x.numel()), c_float(cap), _stream()), "softcap")


ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}
# activations of a feed-forward without a gate (and of routed experts): those, and relu squared
PLAIN_ACTIVATIONS = dict(ACTIVATIONS, relu_squared=3)


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool, activation: str,
              bias: Optional[torch.Tensor] = None) -> None:
    """out[t, j] = act(gate_j) * up_j, the columns laid out as for `swiglu`; `bias` (float32
    [2f], laid out like a row of gate_up) is added to both in float32 first."""
    _need_cuda(gate_up, out, bias)
    T, f = out.shape
    assert gate_up.shape == (T, 2 * f) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * f and
                            bias.is_contiguous())
    lib = load_library("layer_ops")
    _check(lib.tgo_gated_act(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T),
                             c_int(f), c_int(1 if interleaved else 0),
                             c_int(ACTIVATIONS[activation]), _ptr(bias), _stream()), "gated_act",
           f"(T={T}, f={f}, {activation})")


def scaled_add_norm(h: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor], alpha: float,
                    gain: torch.Tensor, eps: float, act: Optional[torch.Tensor] = None) -> None:
    """h <- gain * rmsnorm(alpha * h + y + bias), the float32 stream h in place; y float32 or
    bfloat16 [T, d]; bias float32 [d] or None; `act` (bfloat16) also gets the new stream."""
    _need_cuda(h, y, bias, gain, act)
    T, d = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous() and y.shape == h.shape
    assert y.is_contiguous() and gain.dtype == torch.float32 and gain.numel() == d
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == d)
    assert act is None or (act.dtype == torch.bfloat16 and act.shape == h.shape and
                           act.is_contiguous())
    lib = load_library("layer_ops")
    _check(lib.tgo_scaled_add_norm(_ptr(h), _ptr(y), c_int(dtype_code(y.dtype)), _ptr(bias),
                                   c_float(alpha), _ptr(gain), c_float(eps), _ptr(act), c_int(T),
                                   c_int(d), _stream()), "scaled_add_norm", f"(d={d})")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t] += bias, the sum in float32; y [T, d] in either storage type, bias float32 [d]."""
    _need_cuda(y, bias)
    T, d = y.shape
    assert y.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == d
    lib = load_library("layer_ops")
    _check(lib.tgo_add_bias(_ptr(y), c_int(dtype_code(y.dtype)), _ptr(bias), c_int(T), c_int(d),
                            _stream()), "add_bias")


def value_norm_share_cache(v: torch.Tensor, num_kv_heads: int, value_dim: int, norm: bool,
                           eps: float, blend: Optional[torch.Tensor],
                           shared: Optional[torch.Tensor], mode: int, slots: torch.Tensor,
                           v_cache: torch.Tensor, page_size: int) -> None:
    """Each head's value divided by its root mean square (if `norm`); mode 1 leaves the
    result in `shared` (float32 [T, Hkv * dv]), mode 2 blends it with that row by the device
    scalar `blend`: (1 - blend) v + blend shared; the result goes to `slots` of the paged
    plane [page, kv head, offset, dv]."""
    _need_cuda(v, blend, shared, slots, v_cache)
    T = v.shape[0]
    assert v.stride(1) == 1 and v_cache.dtype == v.dtype and v_cache.is_contiguous()
    assert slots.dtype == torch.int32 and slots.numel() == T
    if mode:
        assert shared.dtype == torch.float32 and shared.is_contiguous()
        assert shared.shape == (T, num_kv_heads * value_dim)
    if mode == 2:
        assert blend.dtype == torch.float32 and blend.numel() == 1
    lib = load_library("layer_ops")
    _check(lib.tgo_value_norm_share_cache(
        _ptr(v), c_ll(v.stride(0)), c_int(dtype_code(v.dtype)), c_int(T), c_int(num_kv_heads),
        c_int(value_dim), c_int(1 if norm else 0), c_float(eps), _ptr(blend), _ptr(shared),
        c_int(mode), _ptr(slots), _ptr(v_cache), c_int(page_size), _stream()),
        "value_norm_share_cache", f"(dv={value_dim}, mode={mode})")


def head_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, heads: int,
                   value_dim: int, eps: float) -> None:
    """out = o / rms(o over each head) * silu(gate): o float32 [T, heads * dv], gate a 2-D view
    in the activation type (None: no gate), out in the activation type."""
    _need_cuda(o, gate, out)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert o.shape == out.shape == (T, heads * value_dim)
    assert gate is None or (gate.stride(1) == 1 and gate.dtype == out.dtype)
    lib = load_library("layer_ops")
    _check(lib.tgo_head_norm_gate(_ptr(o), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0),
                                  _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(heads),
                                  c_int(value_dim), c_float(eps), _stream()), "head_norm_gate")


def weighted_sum(parts, scales, out: torch.Tensor) -> None:
    """out = sum_i scales[i] * parts[i], float32; the parts share a shape and a type."""
    _need_cuda(out, *parts)
    assert parts and len(parts) == len(scales) and out.dtype == torch.float32 and out.is_contiguous()
    for p in parts:
        assert p.shape == out.shape and p.is_contiguous() and p.dtype == parts[0].dtype
    lib = load_library("layer_ops")
    code = dtype_code(parts[0].dtype)
    if len(parts) == 1:
        _check(lib.tgo_scaled_sum(_ptr(parts[0]), c_float(scales[0]), _ptr(None), c_float(0.0),
                                  _ptr(out), c_int(code), c_ll(out.numel()), _stream()), "scaled_sum")
        return
    _check(lib.tgo_scaled_sum(_ptr(parts[0]), c_float(scales[0]), _ptr(parts[1]), c_float(scales[1]),
                              _ptr(out), c_int(code), c_ll(out.numel()), _stream()), "scaled_sum")
    for p, s in zip(parts[2:], scales[2:]):
        if p.dtype != torch.float32:
            raise KernelError("weighted_sum: more than two parts must be float32")
        _check(lib.tgo_scaled_sum(_ptr(p), c_float(s), _ptr(out), c_float(1.0), _ptr(out),
                                  c_int(code), c_ll(out.numel()), _stream()), "scaled_sum")


def attention_sink_supports(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core kernel of the windowed attention with a sink takes these sizes
    (bfloat16; widths that are multiples of 8 up to 128)."""
    return bool(load_library("attention_sink").tgo_attention_sink_supports(
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim)))


def attention_sink_tile_tokens(group: int) -> int:
    """Tokens of one request a tile of that kernel holds at most, for `group` query heads a
    kv head."""
    return max(1, int(load_library("attention_sink").tgo_attention_sink_tile_rows()) // group)


def attention_sink_takes(q: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether these views can be read 16 bytes at a time."""
    return q.dtype == torch.bfloat16 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and \
        out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0


def attention_sink_tile(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                        key_dim: int, value_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        page_size: int, block_tables: torch.Tensor, seq_ids: torch.Tensor,
                        positions: torch.Tensor, scale: float, window: int,
                        sinks: Optional[torch.Tensor], tile_tok0: Optional[torch.Tensor] = None,
                        tile_ntok: Optional[torch.Tensor] = None, n_splits: int = 1,
                        softcap: float = 0.0, value_row: int = 0, keep_first: int = 0,
                        dist_bias: Optional[torch.Tensor] = None) -> None:
    """`softcap`, `value_row`, `keep_first` and `dist_bias` as in `attention_generic`.
    Paged causal attention with keys `key_dim` and values `value_dim` wide, a window (0:
    none) and a sink per head (float32 [H] or None), bfloat16 on the tensor cores: a block per
    tile of consecutive tokens of one request (tile_tok0, tile_ntok: int32; None: every token
    is a tile of its own) and kv head. Without tile lists, `n_splits` > 1 cuts every token's
    keys over as many blocks and a second kernel joins their shares."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions, sinks, tile_tok0, tile_ntok,
               dist_bias)
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_tables.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and
                                 dist_bias.shape[1] == num_heads and dist_bias.is_contiguous())
    if tile_tok0 is not None:
        assert tile_tok0.dtype == torch.int32 and tile_ntok.dtype == torch.int32
        n_tiles = tile_tok0.numel()
    else:
        n_tiles = q.shape[0]
    part_o = part_ml = None
    if tile_tok0 is not None or value_dim % 2:
        n_splits = 1
    if n_splits > 1:
        part_o = torch.empty((n_tiles, num_heads, n_splits, value_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tiles, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_sink")
    _check(lib.tgo_attention_sink(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(positions),
        _ptr(seq_ids), _ptr(tile_tok0), _ptr(tile_ntok), c_int(n_tiles), c_int(num_heads),
        c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), c_float(scale), c_int(window),
        _ptr(sinks), c_int(n_splits), _ptr(part_o), _ptr(part_ml), c_float(softcap or 0.0),
        c_int(value_row), c_int(keep_first), _ptr(dist_bias),
        c_int(dist_bias.shape[0] if dist_bias is not None else 0), _stream()), "attention_sink",
        f"(heads={num_heads}/{num_kv_heads}, dk={key_dim}, dv={value_dim})")
    if n_splits > 1:
        LAUNCHES[0] += 1


def attention_sink_wide_supports(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core kernel for wide key rows whose first `value_dim` channels are the
    values takes these sizes (bfloat16; multiples of 8, keys up to 576, values up to 512)."""
    return bool(load_library("attention_sink").tgo_attention_sink_wide_supports(
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim)))


def attention_sink_wide_tile_tokens(group: int) -> int:
    """Tokens of one request a tile of that kernel holds at most, for `group` query heads a
    kv head."""
    return int(load_library("attention_sink").tgo_attention_sink_wide_tile_tokens(c_int(group)))


def attention_sink_wide(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                        key_dim: int, value_dim: int, k_cache: torch.Tensor, page_size: int,
                        block_tables: torch.Tensor, seq_ids: torch.Tensor, positions: torch.Tensor,
                        scale: float, window: int, sinks: Optional[torch.Tensor],
                        tile_tok0: Optional[torch.Tensor] = None,
                        tile_ntok: Optional[torch.Tensor] = None, n_splits: int = 1,
                        softcap: float = 0.0) -> None:
    """`attention_sink_tile` for key rows up to 576 wide of one cache plane [page, kv head,
    offset, key_dim] whose first `value_dim` channels are the values: a key tile is loaded
    once and serves both products."""
    _need_cuda(q, out, k_cache, block_tables, seq_ids, positions, sinks, tile_tok0, tile_ntok)
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous()
    assert k_cache.shape[-1] == key_dim and k_cache.shape[-2] == page_size
    assert block_tables.is_contiguous() and block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads)
    if tile_tok0 is not None:
        assert tile_tok0.dtype == torch.int32 and tile_ntok.dtype == torch.int32
        n_tiles = tile_tok0.numel()
        n_splits = 1
    else:
        n_tiles = q.shape[0]
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n_tiles, num_heads, n_splits, value_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tiles, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_sink")
    _check(lib.tgo_attention_sink_wide(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), c_int(page_size),
        _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(positions), _ptr(seq_ids),
        _ptr(tile_tok0), _ptr(tile_ntok), c_int(n_tiles), c_int(num_heads), c_int(num_kv_heads),
        c_int(key_dim), c_int(value_dim), c_float(scale), c_int(window), _ptr(sinks), c_int(n_splits),
        _ptr(part_o), _ptr(part_ml), c_float(softcap or 0.0), _stream()), "attention_sink_wide",
        f"(heads={num_heads}/{num_kv_heads}, dk={key_dim}, dv={value_dim})")
    if n_splits > 1:
        LAUNCHES[0] += 1


GATE_ACTIVATIONS = {None: 0, "silu": 1, "sigmoid": 2}


def gated_group_norm(o: torch.Tensor, gate: Optional[torch.Tensor], gain: Optional[torch.Tensor],
                     out: torch.Tensor, groups: int, eps: float, gate_activation: Optional[str],
                     gate_first: bool) -> None:
    """out = gain * group_rmsnorm(o) with a gate: o float32 [T, W] is cut into `groups` equal
    consecutive parts, each divided by its root mean square; the gate (a 2-D view in the
    activation type, through silu or the logistic function) multiplies the norm's input
    (`gate_first`) or its result. gain float32 [W] or None."""
    _need_cuda(o, gate, gain, out)
    T, W = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert out.shape == (T, W)
    assert gate is None or (gate.stride(1) == 1 and gate.dtype == out.dtype and gate.shape == (T, W))
    assert gain is None or (gain.dtype == torch.float32 and gain.numel() == W)
    lib = load_library("layer_ops")
    _check(lib.tgo_gated_group_norm(
        _ptr(o), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0), _ptr(gain), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(W), c_int(groups), c_float(eps),
        c_int(GATE_ACTIVATIONS[gate_activation] if gate is not None else 0),
        c_int(1 if gate_first else 0), _stream()), "gated_group_norm", f"(W={W}, groups={groups})")


def qkv_bias_rope_cache(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                        num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                        q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor],
                        v_bias: Optional[torch.Tensor], rope: Optional[torch.Tensor],
                        rotary_dim: int, interleaved: bool, slots: Optional[torch.Tensor],
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                        page_size: int) -> None:
    """Projection rows of an attention with biases, keys `key_dim` and values `value_dim`
    wide: bias added in float32, the first `rotary_dim` channels of q and k rotated by `rope`
    (a table from rope_table) with channel i paired with i + rotary_dim / 2 or, `interleaved`,
    2i with 2i + 1; q written back in place, k and v stored at `slots` of their cache planes
    [page, kv head, offset, width]. q, k, v are 2-D views with unit column stride."""
    _need_cuda(q, k, v, q_bias, k_bias, v_bias, rope, slots, k_cache, v_cache)
    T = q.shape[0]
    for t in (q, k, v):
        if t is not None:
            assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    for b, n in ((q_bias, num_heads * key_dim), (k_bias, num_kv_heads * key_dim),
                 (v_bias, num_kv_heads * value_dim)):
        assert b is None or (b.dtype == torch.float32 and b.numel() == n and b.is_contiguous())
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    if k is not None:
        assert k_cache is not None and k_cache.dtype == q.dtype and k_cache.is_contiguous()
        assert slots.dtype == torch.int32 and slots.numel() == T
    if v is not None:
        assert v_cache is not None and v_cache.dtype == q.dtype and v_cache.is_contiguous()
    lib = load_library("elementwise")
    _check(lib.tgo_qkv_bias_rope_cache(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0) if k is not None else 0),
        _ptr(v), c_ll(v.stride(0) if v is not None else 0), c_int(dtype_code(q.dtype)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), _ptr(q_bias),
        _ptr(k_bias), _ptr(v_bias), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
        c_int(1 if interleaved else 0), _ptr(slots), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _stream()), "qkv_bias_rope_cache",
        f"(dk={key_dim}, dv={value_dim}, rotary_dim={rotary_dim})")


def qk_rownorm_rope_cache(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                          num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                          q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                          rope: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                          slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], page_size: int,
                          positions: Optional[torch.Tensor] = None, temp_coef: float = 0.0,
                          temp_every: int = 0) -> None:
    """Projection rows of an attention whose q/k norm takes a token's WHOLE q row (all heads,
    num_heads * key_dim entries, a gain of that size) and whole k row at once: RMS norm in
    float32, then the first `rotary_dim` channels of every head rotated by `rope` (either
    pairing); q written back in place, k and v stored at `slots` of their cache planes
    [page, kv head, offset, width]. q, k, v are 2-D views with unit column stride. With
    `positions` (int32 [T]) and `temp_every` > 0 the normed q of a token at position p is also
    multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)."""
    _need_cuda(q, k, v, q_gain, k_gain, rope, slots, k_cache, v_cache, positions)
    assert positions is None or (positions.dtype == torch.int32 and positions.numel() == q.shape[0])
    T = q.shape[0]
    for t in (q, k, v):
        if t is not None:
            assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    for g, n in ((q_gain, num_heads * key_dim), (k_gain, num_kv_heads * key_dim)):
        assert g is None or (g.dtype == torch.float32 and g.numel() == n and g.is_contiguous())
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    if k is not None:
        assert k_cache is not None and k_cache.dtype == q.dtype and k_cache.is_contiguous()
        assert slots.dtype == torch.int32 and slots.numel() == T
    if v is not None:
        assert v_cache is not None and v_cache.dtype == q.dtype and v_cache.is_contiguous()
    lib = load_library("elementwise")
    _check(lib.tgo_qk_rownorm_rope_cache(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0) if k is not None else 0),
        _ptr(v), c_ll(v.stride(0) if v is not None else 0), c_int(dtype_code(q.dtype)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), _ptr(q_gain),
        _ptr(k_gain), c_float(eps), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
        c_int(1 if interleaved else 0), _ptr(slots), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _ptr(positions if temp_every > 0 else None), c_float(temp_coef),
        c_int(temp_every), _stream()), "qk_rownorm_rope_cache",
        f"(dk={key_dim}, dv={value_dim}, rotary_dim={rotary_dim})")


def qkv_conv_rope_norm_cache(qkv: torch.Tensor, q_out: torch.Tensor, num_heads: int,
                             num_kv_heads: int, key_dim: int, value_dim: int,
                             conv_w: Optional[torch.Tensor], num_seqs: int, seq_ids: torch.Tensor,
                             q_start: torch.Tensor, state_slots: torch.Tensor,
                             state: Optional[torch.Tensor], conv_offset: int,
                             rope: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                             unit_norm: bool, eps: float, slots: torch.Tensor, k_cache: torch.Tensor,
                             v_cache: torch.Tensor, page_size: int) -> None:
    """Projection rows [T, H dk + Hkv dk + Hkv dv] (q, k, v side by side) of an attention whose
    q, k and v each pass a short causal convolution over time (conv_w float32 [C, taps], the
    last column meets the current token; rows before a request's portion come from its state
    row, float32 [slots, n] with the last taps - 1 rows [taps - 1, C] at `conv_offset`, which
    is then moved on), then the first `rotary_dim` channels of q and k rotated by `rope`, then,
    `unit_norm`, every q and k head divided by sqrt(mean of its squares + eps). q goes to
    q_out [T, H dk]; k and v to `slots` of their cache planes [page, kv head, offset, width]."""
    _need_cuda(qkv, q_out, conv_w, seq_ids, q_start, state_slots, state, rope, slots, k_cache, v_cache)
    T = qkv.shape[0]
    C = num_heads * key_dim + num_kv_heads * (key_dim + value_dim)
    assert qkv.shape == (T, C) and qkv.stride(1) == 1 and q_out.stride(1) == 1
    assert q_out.shape == (T, num_heads * key_dim) and q_out.dtype == qkv.dtype
    assert k_cache.dtype == qkv.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert slots.dtype == torch.int32 and slots.numel() == T
    taps = 0
    if conv_w is not None:
        taps = conv_w.shape[1]
        assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == C
        assert seq_ids.dtype == q_start.dtype == state_slots.dtype == torch.int32
        assert q_start.numel() == num_seqs + 1 and state_slots.numel() == num_seqs
        if taps > 1:
            assert state is not None and state.dtype == torch.float32 and state.dim() == 2 and \
                state.stride(1) == 1
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    lib = load_library("elementwise")
    has_state = taps > 1
    _check(lib.tgo_qkv_conv_rope_norm_cache(
        _ptr(qkv), c_ll(qkv.stride(0)), _ptr(q_out), c_ll(q_out.stride(0)),
        c_int(dtype_code(qkv.dtype)), c_int(T), c_int(num_heads), c_int(num_kv_heads),
        c_int(key_dim), c_int(value_dim), _ptr(conv_w), c_int(taps), _ptr(seq_ids), _ptr(q_start),
        _ptr(state_slots), _ptr(state if has_state else None),
        c_ll(state.stride(0) if has_state else 0), c_ll(conv_offset), _ptr(rope),
        c_int(rotary_dim if rope is not None else 0), c_int(1 if interleaved else 0),
        c_int(1 if unit_norm else 0), c_float(eps), _ptr(slots), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _stream()), "qkv_conv_rope_norm_cache",
        f"(dk={key_dim}, dv={value_dim}, taps={taps}, rotary_dim={rotary_dim})")
    if has_state:
        _check(lib.tgo_conv_keep_rows(
            _ptr(qkv), c_ll(qkv.stride(0)), c_int(dtype_code(qkv.dtype)), c_int(num_seqs), c_int(C),
            c_int(taps), _ptr(q_start), _ptr(state_slots), _ptr(state), c_ll(state.stride(0)),
            c_ll(conv_offset), _stream()), "conv_keep_rows", f"(C={C}, taps={taps})")


MAX_STREAMS = 8          # residual streams a layer arrangement may keep (kernels' register budget)


def stream_spread(h: torch.Tensor, x: torch.Tensor) -> None:
    """x[s] = h for every stream s: x float32 [S, T, d], h float32 [T, d]."""
    _need_cuda(h, x)
    assert h.dtype == x.dtype == torch.float32 and h.is_contiguous() and x.is_contiguous()
    assert x.shape[1:] == h.shape
    lib = load_library("layer_ops")
    _check(lib.tgo_stream_spread(_ptr(h), _ptr(x), c_ll(h.numel()), c_int(x.shape[0]), _stream()),
           "stream_spread", f"(streams={x.shape[0]})")


def stream_read_norm(x: torch.Tensor, cin: torch.Tensor, gain: torch.Tensor, eps: float,
                     out: torch.Tensor) -> None:
    """out = gain * rmsnorm(sum_s cin[s] x[s]): what a sublayer reads of S residual streams
    (x float32 [S, T, d]; cin float32 [S]; out [T, d] in the activation type)."""
    _need_cuda(x, cin, gain, out)
    S, T, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == (T, d)
    assert cin.dtype == gain.dtype == torch.float32 and cin.numel() == S and gain.numel() == d
    lib = load_library("layer_ops")
    _check(lib.tgo_stream_read_norm(_ptr(x), c_int(S), c_int(T), c_int(d), _ptr(cin), _ptr(gain),
                                    c_float(eps), _ptr(out), c_int(dtype_code(out.dtype)), _stream()),
           "stream_read_norm", f"(streams={S}, d={d})")


def stream_write(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, cout: torch.Tensor,
                 eps: float = 0.0, next_in: Optional[torch.Tensor] = None,
                 next_gain: Optional[torch.Tensor] = None, next_out: Optional[torch.Tensor] = None,
                 sum_out: Optional[torch.Tensor] = None) -> None:
    """x[t] <- sum_s mix[s, t] x[s] + cout[t] * y for all streams t at once (x float32 [S, T, d],
    y [T, d], mix float32 [S, S] indexed [from, to], cout float32 [S]). With `next_out` the
    next sublayer's input gain * rmsnorm(sum_t next_in[t] x[t]) is made from the new streams in
    the same pass; with `sum_out` (float32 [T, d]) their plain sum."""
    _need_cuda(x, y, mix, cout, next_in, next_gain, next_out, sum_out)
    S, T, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == (T, d)
    assert mix.dtype == cout.dtype == torch.float32 and mix.numel() == S * S and mix.is_contiguous()
    assert cout.numel() == S
    if next_out is not None:
        assert next_out.shape == (T, d) and next_out.is_contiguous()
        assert next_in.dtype == next_gain.dtype == torch.float32
        assert next_in.numel() == S and next_gain.numel() == d
    assert sum_out is None or (sum_out.dtype == torch.float32 and sum_out.shape == (T, d) and
                               sum_out.is_contiguous())
    lib = load_library("layer_ops")
    _check(lib.tgo_stream_write(
        _ptr(x), c_int(S), c_int(T), c_int(d), _ptr(y), c_int(dtype_code(y.dtype)), _ptr(mix),
        _ptr(cout), _ptr(next_in), _ptr(next_gain), c_float(eps), _ptr(next_out),
        c_int(dtype_code(next_out.dtype) if next_out is not None else 0), _ptr(sum_out), _stream()),
        "stream_write", f"(streams={S}, d={d})")


def act_rows(x: torch.Tensor, activation: str) -> None:
    """x <- activation(x) in place: the hidden rows of a feed-forward without a gate."""
    _need_cuda(x)
    assert x.is_contiguous()
    lib = load_library("layer_ops")
    _check(lib.tgo_act_rows(_ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.numel()),
                            c_int(PLAIN_ACTIVATIONS[activation]), _stream()), "act_rows", activation)


def mlstm_state_floats(num_heads: int, key_dim: int, value_dim: int) -> int:
    """Floats of one request's state row: S [H, dk, dv], then n [H, dk], then m [H]."""
    return num_heads * key_dim * value_dim + num_heads * key_dim + num_heads


def mlstm(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate_i: torch.Tensor,
          gate_f: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
          q_scale: float, out: torch.Tensor, num_seqs: int, num_heads: int, key_dim: int,
          value_dim: int, q_start: torch.Tensor, state_slots: torch.Tensor,
          state: torch.Tensor) -> None:
    """The matrix memory with exponential gates over a step's tokens, request by request and
    in order, from and to `state` (float32 [slots, mlstm_state_floats]): q, k [T, H dk] and v
    [T, H dv] are 2-D views in the activation type; gate_i, gate_f float32 views [T, H] (the
    gate projections' rows, of one row stride) with their biases float32 [H]; log input gate
    cap tanh((a + b) / cap), log forget gate logsigmoid of the same form; q times q_scale;
    out float32 [T, H dv], the memory's read-out divided by its denominator."""
    _need_cuda(q, k, v, gate_i, gate_f, bias_i, bias_f, out, q_start, state_slots, state)
    T = q.shape[0]
    for t in (q, k, v):
        assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    assert gate_i.dtype == gate_f.dtype == torch.float32 and gate_i.shape == gate_f.shape == (T, num_heads)
    assert gate_i.stride(1) == gate_f.stride(1) == 1 and gate_i.stride(0) == gate_f.stride(0)
    assert bias_i.dtype == bias_f.dtype == torch.float32 and bias_i.numel() == bias_f.numel() == num_heads
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, num_heads * value_dim)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
    assert q_start.dtype == torch.int32 and state_slots.dtype == torch.int32
    rec = torch.empty((T, num_heads, 4), dtype=torch.float32, device=q.device)
    m_first = torch.empty((num_seqs, num_heads), dtype=torch.float32, device=q.device)
    lib = load_library("mlstm")
    _check(lib.tgo_mlstm(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)),
        c_int(dtype_code(q.dtype)), _ptr(gate_i), _ptr(gate_f), c_ll(gate_i.stride(0)), _ptr(bias_i),
        _ptr(bias_f), c_float(cap), c_float(q_scale), _ptr(out), c_int(num_seqs), c_int(num_heads),
        c_int(key_dim), c_int(value_dim), _ptr(q_start), _ptr(state_slots), _ptr(state),
        c_ll(state.shape[1]), _ptr(rec), _ptr(m_first), _stream()), "mlstm",
        f"(heads={num_heads}, dk={key_dim}, dv={value_dim})")
    LAUNCHES[0] += 1


def mlstm_chunk_tokens() -> int:
    """Tokens of one request a chunk of the chunked matrix-memory kernels holds at most."""
    return int(load_library("mlstm").tgo_mlstm_chunk_tokens())


def mlstm_chunked_supports(num_heads: int, key_dim: int, value_dim: int) -> bool:
    return bool(load_library("mlstm").tgo_mlstm_chunked_supports(
        c_int(num_heads), c_int(key_dim), c_int(value_dim)))


def mlstm_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate_i: torch.Tensor,
                  gate_f: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
                  q_scale: float, out: torch.Tensor, num_seqs: int, num_heads: int, key_dim: int,
                  value_dim: int, q_start: torch.Tensor, state_slots: torch.Tensor,
                  state: torch.Tensor, chunk_tok0: Optional[torch.Tensor] = None,
                  chunk_ntok: Optional[torch.Tensor] = None,
                  chunk_first: Optional[torch.Tensor] = None) -> None:
    """What `mlstm` computes, in parallel over chunks of a step's tokens: per chunk a summary
    of its keys and values under its own largest weight, a scan of the summaries through the
    state and its running maximum, then every chunk's outputs from the state before it (three
    launches; the scratch is made here). Without chunk lists every request brings one token:
    the state streamed through once, then n and m (two launches)."""
    _need_cuda(q, k, v, gate_i, gate_f, bias_i, bias_f, out, q_start, state_slots, state,
               chunk_tok0, chunk_ntok, chunk_first)
    T = q.shape[0]
    for t in (q, k, v):
        assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    assert gate_i.dtype == gate_f.dtype == torch.float32 and gate_i.shape == gate_f.shape == (T, num_heads)
    assert gate_i.stride(1) == gate_f.stride(1) == 1 and gate_i.stride(0) == gate_f.stride(0)
    assert bias_i.dtype == bias_f.dtype == torch.float32 and bias_i.numel() == bias_f.numel() == num_heads
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, num_heads * value_dim)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
    assert q_start.dtype == torch.int32 and q_start.numel() == num_seqs + 1
    assert state_slots.dtype == torch.int32 and state_slots.numel() == num_seqs
    single = chunk_tok0 is None
    scratch = m_last = None
    chunks = 0
    if single:
        assert T == num_seqs
    else:
        chunks = chunk_tok0.numel()
        assert chunk_tok0.dtype == chunk_ntok.dtype == chunk_first.dtype == torch.int32
        assert chunk_ntok.numel() == chunks and chunk_first.numel() == num_seqs
        scratch = torch.empty((chunks, num_heads, key_dim * value_dim + key_dim + 4),
                              dtype=torch.float32, device=q.device)
        m_last = torch.empty((num_seqs, num_heads), dtype=torch.float32, device=q.device)
    lib = load_library("mlstm")
    _check(lib.tgo_mlstm_chunked(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)),
        c_int(dtype_code(q.dtype)), _ptr(gate_i), _ptr(gate_f), c_ll(gate_i.stride(0)), _ptr(bias_i),
        _ptr(bias_f), c_float(cap), c_float(q_scale), _ptr(out), c_int(num_seqs), c_int(num_heads),
        c_int(key_dim), c_int(value_dim), _ptr(q_start), _ptr(state_slots), _ptr(state),
        c_ll(state.shape[1]), c_int(chunks), _ptr(chunk_tok0), _ptr(chunk_ntok), _ptr(chunk_first),
        _ptr(scratch), _ptr(m_last), c_int(1 if single else 0), _stream()), "mlstm_chunked",
        f"(heads={num_heads}, dk={key_dim}, dv={value_dim})")
    LAUNCHES[0] += 1 if single else 2


def latent_row_cache(kv: torch.Tensor, rank: int, width: int, gain: torch.Tensor, eps: float,
                     rope: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                     slots: torch.Tensor, cache: torch.Tensor, page_size: int) -> None:
    """The cache row of a latent attention: kv [T, rank + width] (a 2-D view): the first
    `rank` channels RMS-normed with `gain`, of the last `width` the first `rotary_dim` rotated
    by `rope`; stored at `slots` of the plane [page, 1, offset, rank + width]."""
    _need_cuda(kv, gain, rope, slots, cache)
    T = kv.shape[0]
    assert kv.stride(1) == 1 and kv.shape[1] == rank + width and cache.dtype == kv.dtype
    assert cache.is_contiguous() and cache.shape[-1] == rank + width and cache.shape[-2] == page_size
    assert cache.numel() == cache.shape[0] * page_size * (rank + width)
    assert gain.dtype == torch.float32 and gain.numel() == rank and slots.dtype == torch.int32
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    lib = load_library("latent")
    _check(lib.tgo_latent_row_cache(
        _ptr(kv), c_ll(kv.stride(0)), c_int(dtype_code(kv.dtype)), c_int(T), c_int(rank), c_int(width),
        _ptr(gain), c_float(eps), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
        c_int(1 if interleaved else 0), _ptr(slots), _ptr(cache), c_int(page_size), _stream()),
        "latent_row_cache", f"(rank={rank}, width={width})")


def rope_slice(src: torch.Tensor, src_head: int, src_off: int, dst: torch.Tensor, dst_head: int,
               dst_off: int, num_heads: int, width: int, rope: Optional[torch.Tensor],
               rotary_dim: int, interleaved: bool) -> None:
    """dst[t, h * dst_head + dst_off + i] = src[t, h * src_head + src_off + i] for i < width,
    the first `rotary_dim` of those channels rotated by `rope` (either pairing)."""
    _need_cuda(src, dst, rope)
    T = src.shape[0]
    assert src.stride(1) == 1 and dst.stride(1) == 1 and src.dtype == dst.dtype and dst.shape[0] == T
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    lib = load_library("latent")
    _check(lib.tgo_rope_slice(
        _ptr(src), c_ll(src.stride(0)), c_int(src_head), c_int(src_off), _ptr(dst),
        c_ll(dst.stride(0)), c_int(dst_head), c_int(dst_off), c_int(dtype_code(src.dtype)), c_int(T),
        c_int(num_heads), c_int(width), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
        c_int(1 if interleaved else 0), _stream()), "rope_slice")


HEAD_LINEAR_LIBRARY_ROWS = 65     # bfloat16 steps of this many rows or more: the library's
                                  # batched product


def head_linear(x: torch.Tensor, x_head: int, w: torch.Tensor, y: torch.Tensor, y_head: int) -> None:
    """A product per head: y[t, h * y_head + n] = sum_k x[t, h * x_head + k] w[h, n, k], with
    w [H, N, K]; x and y 2-D views with unit column stride. float32, and bfloat16 with few
    rows: this package's kernels (up to 16 rows and K up to 512: a warp an output, the lanes'
    partial sums joined in a fixed order; else tiles, k summed in order); bfloat16 with many
    rows: the library's batched product, where the dense products of as many rows take the
    library too."""
    _need_cuda(x, w, y)
    T = x.shape[0]
    H, N, K = w.shape
    assert w.is_contiguous() and x.stride(1) == 1 and y.stride(1) == 1
    assert x.dtype == w.dtype == y.dtype and y.shape[0] == T
    if x.dtype == torch.bfloat16 and T >= HEAD_LINEAR_LIBRARY_ROWS:
        xv = torch.as_strided(x, (H, T, K), (x_head, x.stride(0), 1))
        yv = torch.as_strided(y, (H, T, N), (y_head, y.stride(0), 1))
        yv.copy_(torch.bmm(xv, w.transpose(1, 2)))
        return
    lib = load_library("latent")
    _check(lib.tgo_head_linear(_ptr(x), c_ll(x.stride(0)), c_int(x_head), _ptr(w), _ptr(y),
                               c_ll(y.stride(0)), c_int(y_head), c_int(dtype_code(x.dtype)), c_int(T),
                               c_int(H), c_int(N), c_int(K), _stream()), "head_linear",
           f"(H={H}, N={N}, K={K})")


def causal_conv_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], y: torch.Tensor,
                    num_seqs: int, seq_ids: torch.Tensor, q_start: torch.Tensor,
                    state_slots: torch.Tensor, state: torch.Tensor, conv_offset: int) -> None:
    """y = silu(bias + causal convolution of x per channel): x a 2-D view [T, C] in the
    activation type, w float32 [C, taps] (the last column meets the current token), y float32
    [T, C]. The inputs before a request's portion come from its state row (float32
    [slots, n]; the last taps - 1 inputs [taps - 1, C] at `conv_offset`), which is then moved
    on by the step's inputs."""
    _need_cuda(x, w, bias, y, seq_ids, q_start, state_slots, state)
    T, C = x.shape
    taps = w.shape[1]
    assert x.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == C
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == C)
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, C)
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    assert seq_ids.dtype == q_start.dtype == state_slots.dtype == torch.int32
    assert q_start.numel() == num_seqs + 1 and state_slots.numel() == num_seqs
    lib = load_library("state_space")
    _check(lib.tgo_causal_conv_act(
        _ptr(x), c_ll(x.stride(0)), c_int(dtype_code(x.dtype)), _ptr(w), _ptr(bias), _ptr(y),
        c_int(T), c_int(num_seqs), c_int(C), c_int(taps), _ptr(seq_ids), _ptr(q_start),
        _ptr(state_slots), _ptr(state), c_ll(state.stride(0)), c_ll(conv_offset), _stream()),
        "causal_conv_act", f"(C={C}, taps={taps})")
    if taps > 1:
        LAUNCHES[0] += 1


def selective_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor],
                   a_log: torch.Tensor, d_skip: Optional[torch.Tensor], y: torch.Tensor,
                   num_seqs: int, heads: int, groups: int, state_dim: int, value_dim: int,
                   q_start: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor,
                   ssm_offset: int) -> None:
    """The scan of a selective state-space mixer over each request's tokens, from and into
    its state row (float32 [slots, n]; S [heads, state_dim, value_dim] at `ssm_offset`):
    dt = softplus(dt_raw + dt_bias), S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + D x.
    xbc float32 [T, heads * value_dim + 2 * groups * state_dim] holds x, then B, then C;
    dt_raw a 2-D view [T, heads] in the activation type; y float32 [T, heads * value_dim]."""
    _need_cuda(xbc, dt_raw, dt_bias, a_log, d_skip, y, q_start, state_slots, state)
    T, C = xbc.shape
    assert xbc.dtype == torch.float32 and xbc.is_contiguous()
    assert dt_raw.shape == (T, heads) and dt_raw.stride(1) == 1
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, heads * value_dim)
    for t in (dt_bias, a_log, d_skip):
        assert t is None or (t.dtype == torch.float32 and t.numel() == heads and t.is_contiguous())
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    assert q_start.dtype == state_slots.dtype == torch.int32
    assert q_start.numel() == num_seqs + 1 and state_slots.numel() == num_seqs
    lib = load_library("state_space")
    _check(lib.tgo_selective_scan(
        _ptr(xbc), c_int(C), _ptr(dt_raw), c_ll(dt_raw.stride(0)), c_int(dtype_code(dt_raw.dtype)),
        _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(y), c_int(num_seqs), c_int(heads),
        c_int(groups), c_int(state_dim), c_int(value_dim), _ptr(q_start), _ptr(state_slots),
        _ptr(state), c_ll(state.stride(0)), c_ll(ssm_offset), _stream()), "selective_scan",
        f"(heads={heads}, groups={groups}, state={state_dim}, vdim={value_dim})")


def moe_tile_rows() -> int:
    """Rows of one expert a tile of the routed products holds at most."""
    return int(load_library("moe").tgo_moe_tile_rows())


def moe_feed_forward(x: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor],
                     w_gate: Optional[torch.Tensor], w_up: torch.Tensor, w_down: torch.Tensor, top: int,
                     activation: str, extra: Optional[torch.Tensor] = None,
                     scores: str = "chosen", correction: Optional[torch.Tensor] = None,
                     identity: int = 0, extra_gated: bool = False) -> torch.Tensor:
    """A routed feed-forward: each row of x [T, d] goes to the `top` experts with the largest
    router scores (w_router float32 [E, d], b_router float32 [E]; float32 sums); expert e is
    w_down[e] (act(w_gate[e] x) * (w_up[e] x)), or, with w_gate None, w_down[e] act(w_up[e] x).
    w_gate, w_up [E, ff, d], w_down [E, d, ff] in x's type. `extra` float32 [T, d] is added (a shared
    expert's output). Returns float32 [T, d]. Nothing is read back to the host.

    `scores` "chosen": the choice is by the logits, the weights are the softmax over the chosen
    logits alone. "all": the scores are the softmax over every logit; the choice is by score +
    `correction` (float32, one per router output), the weights are the chosen scores divided by
    their sum. `identity`: the router has that many outputs after the E experts that stand for
    experts whose output is the row of x itself. `extra_gated`: w_router carries one more row,
    after all of those, whose logit through a logistic function multiplies `extra`."""
    _need_cuda(x, w_router, b_router, w_gate, w_up, w_down, extra, correction)
    T, d = x.shape
    E, ff = w_up.shape[0], w_up.shape[1]
    outputs = E + identity
    assert x.stride(1) == 1 and w_router.dtype == torch.float32 and w_router.is_contiguous()
    assert w_router.shape == (outputs + (1 if extra_gated else 0), d)
    assert b_router is None or (b_router.dtype == torch.float32 and b_router.numel() == outputs)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == outputs)
    assert w_up.shape == (E, ff, d) and w_down.shape == (E, d, ff)
    assert w_gate is None or w_gate.shape == w_up.shape
    for w in (w_gate, w_up, w_down):
        assert w is None or (w.dtype == x.dtype and w.is_contiguous())
    assert extra is None or (extra.shape == (T, d) and extra.is_contiguous() and
                             extra.dtype == torch.float32)
    assert not extra_gated or extra is not None
    assert 0 < top <= outputs and E > 0 and scores in ("chosen", "all")
    dev, pairs = x.device, T * top
    max_tiles = min(pairs, pairs // moe_tile_rows() + E)
    ints = torch.empty(3 * pairs + 3 * E + 2 + 3 * max_tiles, dtype=torch.int32, device=dev)
    ids, perm, place = ints[:pairs], ints[pairs:2 * pairs], ints[2 * pairs:3 * pairs]
    o = 3 * pairs
    counts, fill, offsets = ints[o:o + E], ints[o + E:o + 2 * E], ints[o + 2 * E:o + 3 * E + 1]
    tile_info = ints[o + 3 * E + 1:o + 3 * E + 2]
    tiles = ints[o + 3 * E + 2:]
    wts = torch.empty(pairs, dtype=torch.float32, device=dev)
    gate = torch.empty(T, dtype=torch.float32, device=dev) if extra_gated else None
    hidden = torch.empty((pairs, ff), dtype=x.dtype, device=dev)
    y = torch.empty((pairs, d), dtype=torch.float32, device=dev)
    out = torch.empty((T, d), dtype=torch.float32, device=dev)
    lib = load_library("moe")
    _check(lib.tgo_moe_route(
        _ptr(x), c_ll(x.stride(0)), c_int(dtype_code(x.dtype)), _ptr(w_router), _ptr(b_router),
        c_int(T), c_int(d), c_int(outputs), c_int(top), _ptr(ids), _ptr(wts), _ptr(counts), _ptr(fill),
        _ptr(offsets), _ptr(perm), _ptr(place), _ptr(tile_info), _ptr(tiles), c_int(max_tiles),
        c_int(1 if scores == "all" else 0), _ptr(correction), c_int(E), _ptr(gate),
        _stream()), "moe_route", f"(E={E}+{identity}, top={top})")
    _check(lib.tgo_moe_experts(
        _ptr(x), c_ll(x.stride(0)), c_int(dtype_code(x.dtype)), _ptr(w_gate), _ptr(w_up),
        _ptr(w_down), _ptr(hidden), _ptr(y), _ptr(wts), _ptr(extra), _ptr(out), c_int(T), c_int(d),
        c_int(ff), c_int(top), c_int(PLAIN_ACTIVATIONS[activation]), _ptr(perm), _ptr(tile_info),
        _ptr(tiles), c_int(max_tiles), _ptr(ids if identity else None), c_int(E), _ptr(gate),
        _stream()), "moe_experts", f"(d={d}, ff={ff})")
    LAUNCHES[0] += 4
    return out


def attention_mixed(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    key_dim: int, value_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    page_size: int, block_tables: torch.Tensor, seq_ids: torch.Tensor,
                    positions: torch.Tensor, mix: Optional[torch.Tensor], scale: float,
                    window: int) -> None:
    """Paged causal attention whose softmax weights are mixed across heads by `mix`
    (float32 [H, H]; None: not mixed) before they meet the values; keys are `key_dim` wide,
    values `value_dim`. One block per token, keys in a fixed order."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions, mix)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    assert v_cache.dtype == q.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert block_tables.is_contiguous() and seq_ids.dtype == torch.int32
    assert positions.dtype == torch.int32
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and
                           mix.shape == (num_heads, num_heads))
    lib = load_library("attention_mixed")
    _check(lib.tgo_attention_mixed(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), c_int(dtype_code(q.dtype)),
        c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim),
        _ptr(k_cache), _ptr(v_cache), c_int(page_size), _ptr(block_tables),
        c_int(block_tables.shape[1]), _ptr(seq_ids), _ptr(positions), _ptr(mix), c_float(scale),
        c_int(window), _stream()), "attention_mixed",
        f"(heads={num_heads}/{num_kv_heads}, dk={key_dim}, dv={value_dim})")


def attention_mixed_tile_supports(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                                  window: int) -> bool:
    """Whether the tensor-core tile kernel of the mixed-head attention takes these sizes."""
    lib = load_library("attention_mixed")
    return bool(lib.tgo_attention_mixed_tile_supports(c_int(num_heads), c_int(num_kv_heads),
                                                      c_int(key_dim), c_int(value_dim), c_int(window)))


def attention_mixed_tile(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         key_dim: int, value_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         page_size: int, block_tables: torch.Tensor, seq_ids: torch.Tensor,
                         positions: torch.Tensor, mix: Optional[torch.Tensor], scale: float,
                         tile_tok0: torch.Tensor, tile_ntok: torch.Tensor) -> None:
    """The mixed-head attention of `attention_mixed` for bfloat16 on the tensor cores, a block
    per tile of up to 16 consecutive tokens of one request (tile_tok0, tile_ntok: int32)."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions, mix, tile_tok0, tile_ntok)
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_tables.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert tile_tok0.dtype == torch.int32 and tile_ntok.dtype == torch.int32
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and
                           mix.shape == (num_heads, num_heads))
    lib = load_library("attention_mixed")
    _check(lib.tgo_attention_mixed_tile(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), c_int(tile_tok0.numel()),
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), _ptr(k_cache),
        _ptr(v_cache), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(seq_ids), _ptr(positions), _ptr(mix), c_float(scale), _ptr(tile_tok0),
        _ptr(tile_ntok), _stream()), "attention_mixed_tile",
        f"(heads={num_heads}/{num_kv_heads}, dk={key_dim}, dv={value_dim})")


def attention_mixed_decode_supports(num_heads: int, num_kv_heads: int, key_dim: int,
                                    value_dim: int, window: int) -> bool:
    """Whether the split-key decode kernels of the mixed-head attention take these sizes."""
    lib = load_library("attention_mixed")
    return bool(lib.tgo_attention_mixed_decode_supports(
        c_int(num_heads), c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), c_int(window)))


def attention_mixed_decode(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                           key_dim: int, value_dim: int, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, page_size: int, block_tables: torch.Tensor,
                           seq_ids: torch.Tensor, positions: torch.Tensor,
                           mix: Optional[torch.Tensor], scale: float, splits: int,
                           max_context: int) -> None:
    """The mixed-head attention for a step of single tokens, bfloat16: each token's keys cut
    into `splits` ranges, a block per (token, range), then a join; three launches. The
    scratch (scores, per-range maxima and sums, partial outputs) is made here."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions, mix)
    T = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and block_tables.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and
                           mix.shape == (num_heads, num_heads))
    stride = max(32, (max_context + 31) // 32 * 32)
    dev = q.device
    scores = torch.empty((T, num_heads, stride), dtype=torch.float32, device=dev)
    stats = torch.empty((T, splits, num_heads, 2), dtype=torch.float32, device=dev)
    partial = torch.empty((T, splits, num_heads * value_dim), dtype=torch.float32, device=dev)
    lib = load_library("attention_mixed")
    _check(lib.tgo_attention_mixed_decode(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(key_dim), c_int(value_dim), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(seq_ids),
        _ptr(positions), _ptr(mix), c_float(scale), c_int(splits), _ptr(scores), c_int(stride),
        _ptr(stats), _ptr(partial), _stream()), "attention_mixed_decode",
        f"(heads={num_heads}/{num_kv_heads}, dk={key_dim}, dv={value_dim}, splits={splits})")
    LAUNCHES[0] += 2


def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, num_seqs: int,
              num_heads: int, key_dim: int, value_dim: int, decay: torch.Tensor, k_scale: float,
              rope: Optional[torch.Tensor], rotary_dim: int, q_start: torch.Tensor,
              state_slots: torch.Tensor, state: torch.Tensor, *, act: int = 0) -> None:
    """Linear attention with a fixed decay per head over each request's tokens of the step,
    from and into the float32 state [slots, H, dk, dv]: S <- decay S + k v^T, o = S^T q,
    q and k rotated by `rope` first and k multiplied by k_scale. out float32 [T, H * dv].
    `act` 1: q, k and v go through SiLU (in float32) as they are read."""
    _need_cuda(q, k, v, out, decay, rope, q_start, state_slots, state)
    T = q.shape[0]
    for t in (q, k, v):
        assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    assert out.dtype == torch.float32 and out.is_contiguous()
    assert out.shape == (T, num_heads * value_dim)
    assert state.dtype == torch.float32 and state.is_contiguous()
    assert state.shape[1:] == (num_heads, key_dim, value_dim)
    assert decay.dtype == torch.float32 and decay.numel() == num_heads
    assert q_start.dtype == torch.int32 and q_start.numel() == num_seqs + 1
    assert state_slots.dtype == torch.int32 and state_slots.numel() == num_seqs
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    lib = load_library("retention")
    _check(lib.tgo_retention(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)),
        c_int(dtype_code(q.dtype)), _ptr(out), c_int(num_seqs), c_int(num_heads), c_int(key_dim),
        c_int(value_dim), _ptr(decay), c_float(k_scale), c_int(act), _ptr(rope),
        c_int(rotary_dim if rope is not None else 0), _ptr(q_start), _ptr(state_slots),
        _ptr(state), _stream()), "retention",
        f"(heads={num_heads}, dk={key_dim}, dv={value_dim})")


def retention_chunk_tokens() -> int:
    """Tokens of one request a chunk of the chunked retention kernels holds at most."""
    return int(load_library("retention").tgo_retention_chunk_tokens())


def retention_chunked_supports(num_heads: int, key_dim: int, value_dim: int) -> bool:
    return bool(load_library("retention").tgo_retention_chunked_supports(
        c_int(num_heads), c_int(key_dim), c_int(value_dim)))


def retention_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                      num_seqs: int, num_heads: int, key_dim: int, value_dim: int,
                      decay: torch.Tensor, k_scale: float, rope: Optional[torch.Tensor],
                      rotary_dim: int, q_start: torch.Tensor, state_slots: torch.Tensor,
                      state: torch.Tensor, chunk_tok0: Optional[torch.Tensor] = None,
                      chunk_ntok: Optional[torch.Tensor] = None,
                      chunk_first: Optional[torch.Tensor] = None, *, act: int = 0) -> None:
    """What `retention` computes, in parallel over chunks of a step's tokens: per chunk a
    summary of its keys and values, a scan of the summaries through the state, then every
    chunk's outputs from the state before it (three launches; the scratch for the summaries is
    made here). Without chunk lists every request brings one token: one launch that streams
    the state through once."""
    _need_cuda(q, k, v, out, decay, rope, q_start, state_slots, state, chunk_tok0, chunk_ntok,
               chunk_first)
    T = q.shape[0]
    for t in (q, k, v):
        assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    assert out.dtype == torch.float32 and out.is_contiguous()
    assert out.shape == (T, num_heads * value_dim)
    assert state.dtype == torch.float32 and state.is_contiguous()
    assert state.shape[1:] == (num_heads, key_dim, value_dim)
    assert decay.dtype == torch.float32 and decay.numel() == num_heads
    assert q_start.dtype == torch.int32 and q_start.numel() == num_seqs + 1
    assert state_slots.dtype == torch.int32 and state_slots.numel() == num_seqs
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim) and rope.is_contiguous()
    single = chunk_tok0 is None
    scratch, chunks = None, 0
    if single:
        assert T == num_seqs
    else:
        chunks = chunk_tok0.numel()
        assert chunk_tok0.dtype == chunk_ntok.dtype == chunk_first.dtype == torch.int32
        assert chunk_ntok.numel() == chunks and chunk_first.numel() == num_seqs
        scratch = torch.empty((chunks, num_heads, key_dim, value_dim), dtype=torch.float32,
                              device=q.device)
    lib = load_library("retention")
    _check(lib.tgo_retention_chunked(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)),
        c_int(dtype_code(q.dtype)), _ptr(out), c_int(num_seqs), c_int(num_heads), c_int(key_dim),
        c_int(value_dim), _ptr(decay), c_float(k_scale), c_int(act), _ptr(rope),
        c_int(rotary_dim if rope is not None else 0), _ptr(q_start), _ptr(state_slots),
        _ptr(state), c_int(chunks), _ptr(chunk_tok0), _ptr(chunk_ntok), _ptr(chunk_first),
        _ptr(scratch), c_int(1 if single else 0), _stream()), "retention_chunked",
        f"(heads={num_heads}, dk={key_dim}, dv={value_dim})")
    if not single:
        LAUNCHES[0] += 2


def sgemm_tn(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = x[M,K] . w[N,K]^T, all float32, plain FMA."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.dtype == w.dtype == out.dtype == torch.float32
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    lib = load_library("sgemm")
    _check(lib.tgo_sgemm_tn(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), _stream()),
           "sgemm_tn", f"(M={M}, N={N}, K={K})")


SKINNY_MAX_ROWS = 8

def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                gated: bool = False) -> None:
    """out = x . w^T for at most 64 rows, bfloat16 [M, K] by bfloat16 [N, K], the
    weight-streaming kernel. out: bfloat16 or float32 [M, N]; with `accumulate` (float32) the
    product is added to it; with `gated`, w is a gate/up matrix with rows interleaved in
    eights and out is silu(gate) * up, bfloat16 [M, N / 2]."""
    _need_cuda(x, w, out)
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    assert w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    assert x.shape[1] == K and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and N % 16 == 0
        omode = 3
    elif accumulate:
        assert out.dtype == torch.float32 and out.shape == (M, N)
        omode = 2
    else:
        assert out.dtype in (torch.bfloat16, torch.float32) and out.shape == (M, N)
        omode = 0 if out.dtype == torch.bfloat16 else 1
    lib = load_library("gemm_skinny")
    _check(lib.tgo_gemm_skinny(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                               c_int(omode), _stream()), "gemm_skinny", f"(M={M}, N={N}, K={K})")


class NormedRows:
    """RMSNorm(h) * gain for a few rows of the float32 stream, not computed yet: a
    weight-streaming product that takes it makes the rows while it stages them (one kernel
    fewer between two products of a decode step); anything else asks for `rows()`. Carries
    the shape, dtype and device of the rows it stands for."""

    def __init__(self, h: torch.Tensor, gain: torch.Tensor, eps: float, dtype: torch.dtype):
        self.h, self.gain, self.eps, self.dtype = h, gain, eps, dtype
        self.shape, self.device = h.shape, h.device
        self._rows: Optional[torch.Tensor] = None

    def rows(self) -> torch.Tensor:
        if self._rows is None:
            self._rows = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            add_rmsnorm(self.h, None, self.gain, self.eps, self._rows)
        return self._rows


def rows_of(x) -> torch.Tensor:
    """x itself, or the rows a NormedRows stands for."""
    return x.rows() if isinstance(x, NormedRows) else x


_folds = {}


def folds_norm(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming product of these sizes can take its rows as NormedRows."""
    key = (M, N, K)
    if key not in _folds:
        _folds[key] = bool(load_library("gemm_skinny").tgo_gemm_skinny_folds_norm(
            c_int(M), c_int(N), c_int(K)))
    return _folds[key]


def gemm_skinny_normed(x: NormedRows, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """gemm_skinny with RMSNorm(x.h) * x.gain as its rows (at most 8), the norm folded into
    the product: out bfloat16 or float32 [M, N], or, `gated`, silu(gate) * up [M, N / 2]."""
    _need_cuda(x.h, x.gain, w, out)
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    assert x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.shape[1] == K
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and out.is_contiguous()
    assert x.gain.dtype == torch.float32 and x.gain.numel() == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and N % 16 == 0
        omode = 3
    else:
        assert out.dtype in (torch.bfloat16, torch.float32) and out.shape == (M, N)
        omode = 0 if out.dtype == torch.bfloat16 else 1
    lib = load_library("gemm_skinny")
    _check(lib.tgo_gemm_skinny_normed(_ptr(x.h), _ptr(x.gain), c_float(x.eps), _ptr(w), _ptr(out),
                                      c_int(M), c_int(N), c_int(K), c_int(omode), _stream()),
           "gemm_skinny_normed", f"(M={M}, N={N}, K={K})")


def _skinny_ok(x, w) -> bool:
    dt = x.dtype
    return dt == torch.bfloat16 and w.dtype == torch.bfloat16 and \
        x.shape[0] <= SKINNY_MAX_ROWS and w.shape[1] % 8 == 0


# Which kernel multiplies, by the number of rows (measured on B200 with the 8B shapes,
# `python bench.py --only products`):
#   1..8      gemm_skinny (weight streaming, mma.sync)        8-16 % faster than the library
#   9..1024   the library product (cuBLASLt through torch.mm)  the tcgen05 kernel is behind it on
#             q/k/v, o and down here (at 1024 rows 43 / 32 / 101 us against 37 / 26 / 75: too few
#             tiles for 148 SMs)
#   1025..    gemm_tc (tcgen05 + TMEM + TMA)                   at 2048 rows q/k/v 81 us (library 71),
#             o 48 (49), down 145 (144), gate/up with the gate 286 (library and gate kernel 319)
TC_MIN_ROWS = 1025
TC_MIN_ROWS_GATED = 1024   # the gate/up product with the gate in its epilogue: from here on it beats
                           # the library product followed by the gate kernel (149.6 against 154.8 us
                           # at 1024 rows of the 8B shape, 286 against 319 at 2048)
USE_TC = True            # False: the library product for every size above 8 rows


def product_regime(rows: int) -> int:
    """Which of the three product kernels a bfloat16 product of this many rows takes
    (0 weight streaming, 1 the library, 2 tcgen05): an engine warms each one up once before
    it captures a graph that holds it."""
    return 0 if rows <= SKINNY_MAX_ROWS else 1 if rows < TC_MIN_ROWS else 2


def _tc_ok(x, w, min_rows: Optional[int] = None) -> bool:
    return USE_TC and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and \
        x.shape[0] >= (TC_MIN_ROWS if min_rows is None else min_rows) and w.shape[1] % 8 == 0 and \
        x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def _dense(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    M, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        sgemm_tn(x, w, y)
        return y
    if _tc_ok(x, w):
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_tc(x, w, y)
        return y
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return torch.mm(x, w.t()) if out_dtype == torch.bfloat16 else \
            torch.mm(x, w.t(), out_dtype=torch.float32)
    raise KernelError(f"linear: x is {x.dtype} and w is {w.dtype}")


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           residual: Optional[torch.Tensor] = None):
    """y = x . w^T with w stored [out, in]. residual: a float32 [M, N] tensor the product
    belongs to: either it is added there and None is returned, or the product is returned
    for the caller to add (the block hands it to the next norm).

    float32: this package's plain-FMA kernel. bfloat16 with few rows (a decode step): this
    package's weight-streaming kernel, which does the residual add in its epilogue.
    bfloat16 with many rows (TC_MIN_ROWS): this package's tcgen05 kernel (TMA-fed,
    accumulators in tensor memory); between them the library product. out_dtype float32
    keeps the accumulator's width (the logits).
    """
    out_dtype = out_dtype or x.dtype
    if isinstance(x, NormedRows):
        M, N = x.shape[0], w.shape[0]
        if residual is None and _skinny_ok(x, w) and folds_norm(M, N, w.shape[1]):
            out = torch.empty((M, N), dtype=out_dtype, device=x.device)
            gemm_skinny_normed(x, w, out)
            return out
        x = x.rows()
    if _skinny_ok(x, w):
        M, N = x.shape[0], w.shape[0]
        if residual is not None:
            gemm_skinny(x, w, residual, accumulate=True)
            return None
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_skinny(x, w, out)
        return out
    if residual is not None and x.dtype == torch.bfloat16:
        # more than a few rows: the library has no add into a float32 stream, and from the
        # tcgen05 product's epilogue a read-modify-write of the stream is slow (each thread
        # owns a row); hand the product back and let the next norm, which reads the stream
        # anyway, add it
        return _dense(x, w, out_dtype)
    y = _dense(x, w, out_dtype)
    if residual is not None:
        residual_add(residual, y)
        return None
    return y


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool,
                 activation: str = "silu", bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x . Wg^T) * (x . Wu^T) as [M, f] in x's dtype. w_gate_up is [2f, K]: the gate
    rows then the up rows, or (`interleaved`) eight gate rows and the eight matching up rows
    in turn, which lets the bfloat16 kernels apply the gate in their epilogue. The product
    kernels' epilogues know SiLU; another activation, or a `bias` (float32 [2f] in the rows'
    order), takes the product, then the gate kernel."""
    M, f = x.shape[0], w_gate_up.shape[0] // 2
    if activation != "silu" or bias is not None:
        x = rows_of(x)
        gu = linear(x, w_gate_up)
        out = torch.empty((M, f), dtype=x.dtype, device=x.device)
        gated_act(gu, out, interleaved, activation, bias)
        return out
    if isinstance(x, NormedRows):
        if interleaved and _skinny_ok(x, w_gate_up) and folds_norm(M, 2 * f, w_gate_up.shape[1]):
            out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
            gemm_skinny_normed(x, w_gate_up, out, gated=True)
            return out
        x = x.rows()
    if interleaved and _skinny_ok(x, w_gate_up):
        out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
        gemm_skinny(x, w_gate_up, out, gated=True)
        return out
    if interleaved and _tc_ok(x, w_gate_up, min(TC_MIN_ROWS, TC_MIN_ROWS_GATED)) and f % 8 == 0:
        out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
        gemm_tc(x, w_gate_up, out, gated=True)
        return out
    gu = _dense(x, w_gate_up, x.dtype)
    out = torch.empty((M, f), dtype=x.dtype, device=x.device)
    swiglu(gu, out, interleaved)
    return out


_num_sms = {}


def num_sms(device) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    key = torch.device(device).index or 0
    if key not in _num_sms:
        _num_sms[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _num_sms[key]


def flash_supports(head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernel has an instance for this head size and
    group (others go to the generic kernel)."""
    return bool(load_library("attention_flash").tgo_attention_flash_supports(
        c_int(head_dim), c_int(group)))


USE_TMA_DECODE = True       # decode attention with head size 128: cache pages by TMA


def attention_decode_tma_supports(head_dim: int, group: int, page_size: int) -> bool:
    if head_dim != 128:                  # do not build the library for models that cannot use it
        return False
    return bool(load_library("attention_decode_tma").tgo_attention_decode_tma_supports(
        c_int(head_dim), c_int(group), c_int(page_size)))


def attention_decode_tma_error() -> int:
    """1 if a wait of the TMA-fed decode attention kernel ever ran out, else 0. Synchronises."""
    value = ctypes.c_int(0)
    _check(load_library("attention_decode_tma").tgo_attention_decode_tma_error(ctypes.byref(value)),
           "attention_decode_tma_error")
    return int(value.value)


FUSE_DECODE_QK = True        # decode steps at head size 128: q/k-norm, rotation and cache write
                             # inside the attention kernel instead of in a kernel before it


def decode_attention_fuses(q: torch.Tensor, head_dim: int, group: int, page_size: int,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, rotary_dim: int) -> bool:
    """Whether attention_decode_fused takes this layer: bfloat16, the TMA decode kernel's
    shapes, and a rotation of the whole head or none."""
    return FUSE_DECODE_QK and USE_TMA_DECODE and q.dtype == torch.bfloat16 and \
        rotary_dim in (0, head_dim) and k_cache.dim() == 4 and k_cache.is_contiguous() and \
        v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16 and \
        attention_decode_tma_supports(head_dim, group, page_size)


def attention_decode_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                           num_heads: int, num_kv_heads: int, head_dim: int,
                           q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                           rope: Optional[torch.Tensor], slots: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, page_size: int, block_tables: torch.Tensor,
                           positions: torch.Tensor, seq_ids: torch.Tensor, scale: float, window: int,
                           n_splits: int = 1) -> None:
    """A decode step's qk_norm_rope_cache and attention_flash in one kernel (head size 128):
    q, k, v are the raw rows of the step's tokens, one a request; q and k are normed (gains, or
    None) and rotated (`rope` [T, 128] from rope_table, or None) as qk_norm_rope_cache does,
    bit for bit, k and v are stored at `slots` of the cache, and every token attends over its
    request's keys including its own. q is left as it came."""
    _need_cuda(q, k, v, out, q_gain, k_gain, rope, slots, k_cache, v_cache, block_tables, positions,
               seq_ids)
    T = q.shape[0]
    assert q.dtype == k.dtype == v.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and out.stride(1) == 1
    assert k.shape[0] == v.shape[0] == T and slots.dtype == torch.int32 and slots.numel() == T
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, head_dim) and rope.is_contiguous()
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T, num_heads, n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    _check(load_library("attention_decode_tma").tgo_attention_decode_tma_fused(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(positions), _ptr(seq_ids), c_int(T), c_int(num_heads), c_int(num_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits), _ptr(part_o), _ptr(part_ml),
        _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)), _ptr(q_gain), _ptr(k_gain),
        c_float(eps), _ptr(rope), _ptr(slots), _stream()),
        "attention_decode_tma_fused", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
    if n_splits > 1:
        _check(load_library("attention_flash").tgo_attention_flash_combine(
            _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T), c_int(num_heads),
            c_int(head_dim), c_int(n_splits), _stream()), "attention_flash_combine")


def attention_flash(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                    block_tables: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                    tile_tok0: Optional[torch.Tensor], tile_ntok: Optional[torch.Tensor],
                    scale: float, window: int, n_splits: int = 1,
                    tok_list: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention on the tensor cores (bfloat16). With tile arrays (int32,
    first token and token count of each tile, tokens of one request, at most
    flash_tile_rows() // group of them) any step; without them every token is a tile of its
    own (decode), and n_splits > 1 cuts each request's keys over that many CTAs and joins
    them. tok_list (int32, decode with head size 128 only): the tokens of the step to take,
    instead of all."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, positions, seq_ids, tile_tok0, tile_ntok,
               tok_list)
    T = q.shape[0] if tok_list is None else tok_list.numel()
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    n_tiles = T if tile_tok0 is None else tile_tok0.numel()
    tma = tile_tok0 is None and USE_TMA_DECODE and k_cache.dim() == 4 and k_cache.is_contiguous() and \
        v_cache.is_contiguous() and attention_decode_tma_supports(
            head_dim, num_heads // num_kv_heads, page_size)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T, num_heads, n_splits, head_dim), dtype=torch.float32,
                             device=q.device)
        part_ml = torch.empty((T, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_flash")
    if tma:
        # decode with the pages brought in by TMA
        _check(load_library("attention_decode_tma").tgo_attention_decode_tma(
            _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
            c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables),
            c_int(block_tables.shape[1]), _ptr(positions), _ptr(seq_ids), c_int(T), c_int(num_heads),
            c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits),
            _ptr(part_o), _ptr(part_ml), _ptr(tok_list), _stream()),
            "attention_decode_tma", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
        if n_splits > 1:
            _check(lib.tgo_attention_flash_combine_listed(
                _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T),
                c_int(num_heads), c_int(head_dim), c_int(n_splits), _ptr(tok_list), _stream()),
                "attention_flash_combine")
        return
    assert tok_list is None, "a token list is taken by the TMA decode kernel only"
    _check(lib.tgo_attention_flash(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(positions),
        _ptr(seq_ids), _ptr(tile_tok0), _ptr(tile_ntok), c_int(n_tiles), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        c_int(n_splits), _ptr(part_o), _ptr(part_ml), _stream()),
        "attention_flash", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
    if n_splits > 1:
        _check(lib.tgo_attention_flash_combine(
            _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T),
            c_int(num_heads), c_int(head_dim), c_int(n_splits), _stream()),
            "attention_flash_combine")


def attention_tc_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(load_library("attention_tc").tgo_attention_tc_supports(c_int(head_dim), c_int(group),
                                                                       c_int(page_size)))


def attention_tc_error() -> int:
    """The code a wait of the tcgen05 attention kernel left when it ran out (1 producer,
    2 issuer, 3 softmax), or 0. Synchronises with the device."""
    value = ctypes.c_int(0)
    _check(load_library("attention_tc").tgo_attention_tc_error(ctypes.byref(value)), "attention_tc_error")
    return int(value.value)


def attention_tc_prefill(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                         block_tables: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                         tile_tok0: torch.Tensor, tile_ntok: torch.Tensor, scale: float,
                         window: int) -> None:
    """Paged causal attention of prompt portions on the tcgen05 tensor cores (bfloat16, head
    size 128): tiles of 128 // group consecutive tokens of one request (tile_tok0, tile_ntok,
    int32); K and V pages [n_pages, kv_heads, page_size, 128] come in by TMA."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, positions, seq_ids, tile_tok0, tile_ntok)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape == v_cache.shape and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    lib = load_library("attention_tc")
    _check(lib.tgo_attention_tc_prefill(
        _ptr(q), c_ll(q.stride(0)), c_int(q.shape[0]), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(positions), _ptr(seq_ids), _ptr(tile_tok0), _ptr(tile_ntok), c_int(tile_tok0.numel()),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        _stream()), "attention_tc_prefill",
        f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads}, page_size={page_size})")


def flash_tile_rows() -> int:
    """Query rows (token x head of the group) one prefill tile of the attention kernel holds."""
    return int(load_library("attention_flash").tgo_attention_flash_tile_rows())


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, ties to the lowest id."""
    _need_cuda(logits, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert out.dtype == torch.int32 and out.numel() == n
    lib = load_library("sampling")
    part_v = torch.empty((n, 32), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((n, 32), dtype=torch.int32, device=logits.device)
    _check(lib.tgo_argmax(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V), _ptr(out),
                          _ptr(part_v), _ptr(part_i), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, draws: torch.Tensor, out: torch.Tensor,
           report: Optional[torch.Tensor] = None, logprob: Optional[torch.Tensor] = None,
           top_ids: Optional[torch.Tensor] = None, top_logprobs: Optional[torch.Tensor] = None
           ) -> None:
    """Per row: temperature 0 -> argmax; else the softmax of logits / temperature, cut to the
    top_k largest (0: no cut) and to the top_p nucleus (0: no cut), walked in ascending id
    order to draws[r] * total.

    With `report` (int32 per row; negative: nothing for this row), a row also writes ln of
    the drawn token's share of the distribution it was drawn from into logprob[r], and its
    report[r] most likely tokens, descending, into top_ids[r] and top_logprobs[r] (both
    [rows, at most 128]; a token the policy left no chance has -inf)."""
    _need_cuda(logits, temperature, top_k, top_p, draws, out, report, logprob, top_ids,
               top_logprobs)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert draws.dtype == torch.float32 and top_k.dtype == torch.int32 and out.dtype == torch.int32
    assert temperature.numel() == top_k.numel() == top_p.numel() == draws.numel() == n
    width = 0
    if report is not None:
        assert report.dtype == torch.int32 and report.numel() == n
        assert logprob is not None and logprob.dtype == torch.float32 and logprob.numel() == n
        if top_ids is not None:
            width = top_ids.shape[1]
            assert top_ids.dtype == torch.int32 and top_logprobs.dtype == torch.float32
            assert top_ids.shape == top_logprobs.shape == (n, width)
            assert top_ids.is_contiguous() and top_logprobs.is_contiguous()
    lib = load_library("sampling")
    _check(lib.tgo_sample(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(draws), _ptr(out),
                          _ptr(report), _ptr(logprob), _ptr(top_ids), _ptr(top_logprobs),
                          c_int(width), _stream()), "sample")


def logits_adjust(row: torch.Tensor, bias_ids: Optional[torch.Tensor],
                  bias: Optional[torch.Tensor], ids: Optional[torch.Tensor],
                  counts: Optional[torch.Tensor], repetition: float, presence: float,
                  frequency: float) -> None:
    """Edit one row of logits in place: add the biases, then apply the penalties to the
    distinct history tokens `ids` with their `counts`."""
    _need_cuda(row, bias_ids, bias, ids, counts)
    assert row.dtype == torch.float32 and row.dim() == 1 and row.is_contiguous()
    nb = 0 if bias_ids is None else bias_ids.numel()
    ni = 0 if ids is None else ids.numel()
    lib = load_library("sampling")
    _check(lib.tgo_logits_adjust(_ptr(row), _ptr(bias_ids), _ptr(bias), c_int(nb), _ptr(ids),
                                 _ptr(counts), c_int(ni), c_float(repetition), c_float(presence),
                                 c_float(frequency), c_int(row.numel()), _stream()),
           "logits_adjust")


_tc_err = {}


def gemm_tc_error_flag(device) -> torch.Tensor:
    """The int32 flag a tensor-core product sets if one of its waits ran out (0: none;
    1 producer, 2 issuer, 3 epilogue). One per device, made at first use."""
    key = torch.device(device).index or 0
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


_tc_tail = {}


def _tc_tail_buffers(device):
    """Per device: the float32 workspace and the zeroed flags through which the CTAs of a
    product's last round hand each other their parts of a tile (made at first use, outside
    any stream capture: the engine's first steps run uncaptured). One product at a time
    per device may use them."""
    key = torch.device(device).index or 0
    if key not in _tc_tail:
        lib = load_library("gemm_tc")
        lib.tgo_gemm_tc_tail_floats.restype = ctypes.c_longlong
        with torch.cuda.device(device):
            n, f = int(lib.tgo_gemm_tc_tail_floats()), int(lib.tgo_gemm_tc_tail_flags())
        _tc_tail[key] = (torch.empty(n, dtype=torch.float32, device=device),
                         torch.zeros(f, dtype=torch.int32, device=device))
    return _tc_tail[key]


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            gated: bool = False) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float32
    accumulation in tensor memory, TMA-fed); for many rows. out: bfloat16 or float32, or
    float32 that the product is added to. gated: w is a gate/up matrix with rows interleaved
    in eights and out is silu(gate) * up, bfloat16 [M, N / 2]. One thread at a time launches
    these (the forced tile and the last plan below are process-wide, the workspace of the
    last round's cut is one per device)."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    assert out.shape == ((M, N // 2) if gated else (M, N))
    if gated:
        assert out.dtype == torch.bfloat16 and N % 16 == 0
        omode = 4
    elif accumulate:
        assert out.dtype == torch.float32
        omode = 2
    else:
        omode = 0 if out.dtype == torch.bfloat16 else 1
        assert out.dtype in (torch.bfloat16, torch.float32)
    lib = load_library("gemm_tc")
    tail_ws, tail_flags = _tc_tail_buffers(x.device)
    _check(lib.tgo_gemm_tc(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(omode),
                           _ptr(tail_ws), _ptr(tail_flags), _ptr(gemm_tc_error_flag(x.device)),
                           _stream()), "gemm_tc", f"(M={M}, N={N}, K={K})")


def gemm_tc_force_tile(rows: int = 0, width: int = 0, cut_last_round: bool = True) -> None:
    """For tests and tuning: `gemm_tc` runs tiles of rows x width (rows 128
    or 256; width a multiple of 16 up to 256) instead of choosing; 0 gives the choice back.
    cut_last_round False: the tiles of the last round are not cut along K."""
    lib = load_library("gemm_tc")
    _check(lib.tgo_gemm_tc_force_tile(c_int(rows), c_int(width), c_int(0 if cut_last_round else 1)),
           "gemm_tc_force_tile", f"(rows={rows}, width={width})")


def gemm_tc_last_plan() -> tuple:
    """(rows, width, parts) of the last `gemm_tc`: its tile and into how many
    parts along K the tiles of its last round were cut (1: not cut)."""
    lib = load_library("gemm_tc")
    r, w, c = c_int(0), c_int(0), c_int(0)
    lib.tgo_gemm_tc_last_plan(ctypes.byref(r), ctypes.byref(w), ctypes.byref(c))
    return r.value, w.value, c.value


def kernel_wait_errors() -> dict:
    """Which kernels of this package gave up a wait (on an mbarrier or a grid barrier) since
    the process began: {kernel: code}, empty when none did. Their results are then not to be
    trusted. Looks only at libraries that are loaded; synchronises with the device."""
    from .build import _loaded
    out = {}
    if "attention_tc" in _loaded:
        code = attention_tc_error()
        if code:
            out["attention_tc"] = code
    if "attention_decode_tma" in _loaded:
        code = attention_decode_tma_error()
        if code:
            out["attention_decode_tma"] = code
    for key, flag in _tc_err.items():
        code = int(flag.item())
        if code:
            out[f"gemm_tc (device {key})"] = code
    return out
