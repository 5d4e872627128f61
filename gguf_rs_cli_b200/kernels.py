"""Typed Python faces of the CUDA entry points: tensors in, launch on the current
stream.  Nothing here computes; a missing or failing library raises NativeError.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .native import call, dtype_code, ptr, stream_ptr


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise native.NativeError("kernels take CUDA tensors only; there is no CPU path")


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t,:] = table[tokens[t],:] * scale in float32."""
    _cuda(table, tokens, out)
    V, E = table.shape
    T = tokens.numel()
    assert out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous() and tokens.dtype == torch.int32
    call("gb_embed", ptr(table), dtype_code(table), ptr(tokens), T, E, V, float(scale), ptr(out), stream_ptr())
    return out


def embed_shadow(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, xb: torch.Tensor, ssq: torch.Tensor,
                 scale: float = 1.0) -> None:
    """embed plus what a deferred norm needs: xb = bfloat16(out), ssq[t] = sum(out[t,:]^2)."""
    _cuda(table, tokens, out, xb, ssq)
    V, E = table.shape
    T = tokens.numel()
    assert out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous() and tokens.dtype == torch.int32
    assert xb.dtype == torch.bfloat16 and xb.shape == (T, E) and xb.is_contiguous() and ssq.dtype == torch.float32
    assert ssq.numel() >= T
    call("gb_embed_shadow", ptr(table), dtype_code(table), ptr(tokens), T, E, V, float(scale), ptr(out), ptr(xb), ptr(ssq),
         stream_ptr())


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x: float32 [T,E] residual stream.  delta: None, [T,E] or [S,T,E] terms still to be
    added to x.  rows: int32 row numbers to gather (then out has len(rows) rows)."""
    _cuda(x, delta, weight, out, rows)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.numel() == E
    n_delta, stride = 0, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, E)
        n_delta = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * E
    n_rows = T if rows is None else rows.numel()
    assert out.shape == (n_rows, E)
    call("gb_add_rmsnorm", ptr(x), ptr(delta), 0 if delta is None else dtype_code(delta), n_delta, stride, ptr(rows),
         n_rows, E, ptr(weight), dtype_code(weight), float(eps), ptr(out), dtype_code(out), int(write_x), stream_ptr())
    return out


def rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], n_heads: int, n_kv_heads: int,
                  head_dim: int, inv_freq: Optional[torch.Tensor], rotary_dim: int, pairing: int,
                  seq_of: torch.Tensor, pos: torch.Tensor, table: Optional[torch.Tensor], ring_pages: int,
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor]) -> None:
    """q, k, v: column slices [T, heads*head_dim] of one row-major buffer (equal row
    stride).  Rotates q in place; writes rotated k and v into the cache pages."""
    _cuda(q, k, v, inv_freq, seq_of, pos, table, kcache, vcache)
    T = q.shape[0]
    ld = q.stride(0)
    assert q.stride(1) == 1 and (k is None or (k.stride(0) == ld and v.stride(0) == ld and k.dtype == q.dtype))
    call("gb_rope_kv_write", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, T, n_heads, n_kv_heads, head_dim,
         rotary_dim, pairing, ptr(inv_freq), ptr(seq_of), ptr(pos), ptr(table),
         0 if table is None else table.shape[1], ring_pages, ptr(kcache), ptr(vcache),
         0 if kcache is None else dtype_code(kcache), stream_ptr())


def attention_generic(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, ring_pages: int,
                      kcache: torch.Tensor, vcache: Optional[torch.Tensor], window: int, scale: float,
                      v_dim: Optional[int] = None, keep_first: int = 0, head_pages: int = 0,
                      gate: Optional[torch.Tensor] = None, sink: bool = False, sink_values: Optional[torch.Tensor] = None,
                      chunk: int = 0) -> torch.Tensor:
    """v_dim: entries of a value when they differ from a key's head_dim.  vcache None: the values are the
    first v_dim entries of the key rows themselves (one latent row per position serves as key and value).
    keep_first: with a window, the sequence's first positions that stay visible behind it; their pages are the first
    head_pages entries of the page table, in front of the ring.  gate [T, heads*v_dim]: the result is multiplied by
    sigmoid(gate); a gate [T, heads] holds one number per head.  sink: the softmax's denominator counts one more key
    of score 0 that has no value, or of the score sink_values[head] (float32 [heads], not scaled).  chunk: instead of a
    window, a token sees the earlier tokens of its own chunk of that many positions, counted from the sequence's start."""
    _cuda(q, out, seq_of, pos, table, kcache, vcache, gate, sink_values)
    T = q.shape[0]
    per_head = _gate_per_head(gate, out, n_heads)
    assert sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == n_heads and sink_values.is_contiguous())
    v_dim = head_dim if v_dim is None else int(v_dim)
    v_row = head_dim if vcache is None else vcache.shape[-1]
    assert kcache.shape[-1] == head_dim and v_row >= v_dim and (vcache is None or vcache.dtype == kcache.dtype)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * v_dim)
    call("gb_attention_generic", ptr(q), dtype_code(q), q.stride(0), ptr(out), dtype_code(out), out.stride(0), T,
         n_heads, n_kv_heads, head_dim, v_dim, v_row, ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages,
         ptr(kcache), ptr(kcache if vcache is None else vcache), dtype_code(kcache), int(window or 0), float(scale),
         int(head_pages), int(keep_first or 0), ptr(gate), 0 if gate is None else dtype_code(gate),
         0 if gate is None else gate.stride(0), int(per_head), int(bool(sink) or sink_values is not None), ptr(sink_values),
         int(chunk or 0), stream_ptr())
    return out


def _gate_per_head(gate: Optional[torch.Tensor], out: torch.Tensor, n_heads: int) -> bool:
    """Whether a gate holds one number per head ([T, heads]) instead of one per entry of the result."""
    if gate is None:
        return False
    assert gate.stride(1) == 1 and gate.shape[0] == out.shape[0]
    if gate.shape[1] == n_heads and out.shape[1] != n_heads:
        return True
    assert gate.shape == out.shape
    return False


GATE_ACTS = {"silu": 1, "gelu_tanh": 2}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """gate_up: [T, 2F], gate in the first F columns; out[t,i] = act(gate)*up, act SiLU or GELU's tanh form."""
    _cuda(gate_up, out)
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.stride(1) == 1 and out.is_contiguous() and out.dtype == gate_up.dtype
    call("gb_swiglu", ptr(gate_up), gate_up.stride(0), ptr(out), T, F, dtype_code(out), GATE_ACTS[activation], stream_ptr())
    return out


def add_dyt(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor, alpha: float,
            out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """Dynamic tanh with the residual add in front of it: v = x + delta (32-bit, written back to x),
    out = tanh(alpha v) * weight + bias.  Arguments as add_rmsnorm."""
    _cuda(x, delta, weight, bias, out, rows)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert weight.numel() == E and bias.numel() == E and weight.dtype == bias.dtype
    n_delta, stride = 0, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, E)
        n_delta = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * E
    n_rows = T if rows is None else rows.numel()
    assert out.shape == (n_rows, E)
    call("gb_add_dyt", ptr(x), ptr(delta), 0 if delta is None else dtype_code(delta), n_delta, stride, ptr(rows), n_rows, E,
         ptr(weight), ptr(bias), dtype_code(weight), float(alpha), ptr(out), dtype_code(out), int(write_x), stream_ptr())
    return out


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x *= scale in place (float32, contiguous)."""
    _cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    call("gb_scale", ptr(x), x.numel(), float(scale), stream_ptr())
    return x


def short_conv_silu(xin: torch.Tensor, taps: torch.Tensor, state: Optional[torch.Tensor], ctx, out: torch.Tensor,
                    taps_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, c] = silu(sum_j taps[c, j] * xin[t - (K-1-j), c]) per sequence; rows before the step come from
    state [slots, K-1, C] (float32), which is then renewed with the sequence's last K-1 inputs.
    xin, out: [T, C] column slices (unit stride along c).  taps_t: the taps once more as bfloat16 [K, C]; with it,
    bfloat16 rows that start on 16 bytes are read and written 8 channels at a time."""
    _cuda(xin, taps, state, out, taps_t)
    assert taps_t is None or (taps_t.dtype == torch.bfloat16 and taps_t.shape == (taps.shape[1], taps.shape[0]) and taps_t.is_contiguous())
    T, C = xin.shape
    K = taps.shape[1]
    assert taps.shape == (C, K) and taps.is_contiguous() and xin.stride(1) == 1 and out.stride(1) == 1
    assert out.shape == (T, C) and out.dtype == xin.dtype
    assert state is None or (state.dtype == torch.float32 and state.shape[1:] == (K - 1, C) and state.is_contiguous())
    call("gb_short_conv_silu", ptr(xin), dtype_code(xin), xin.stride(0), T, ctx.B, C, K, ptr(taps), dtype_code(taps),
         ptr(taps_t), ptr(state), ptr(ctx.seq_of), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens), ptr(out), out.stride(0), stream_ptr())
    return out


def short_conv(xin: torch.Tensor, taps: torch.Tensor, state: Optional[torch.Tensor], ctx, out: torch.Tensor,
               taps_t: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> torch.Tensor:
    """short_conv_silu with its options open: bias [C] (of the taps' dtype) is added to the sum, activation None or "silu"."""
    _cuda(xin, taps, state, out, taps_t, bias)
    assert taps_t is None or (taps_t.dtype == torch.bfloat16 and taps_t.shape == (taps.shape[1], taps.shape[0]) and taps_t.is_contiguous())
    assert activation in (None, "silu")
    T, C = xin.shape
    K = taps.shape[1]
    assert taps.shape == (C, K) and taps.is_contiguous() and xin.stride(1) == 1 and out.stride(1) == 1
    assert out.shape == (T, C) and out.dtype == xin.dtype
    assert bias is None or (bias.shape == (C,) and bias.dtype == taps.dtype and bias.is_contiguous())
    assert state is None or (state.dtype == torch.float32 and state.shape[1:] == (K - 1, C) and state.is_contiguous())
    call("gb_short_conv", ptr(xin), dtype_code(xin), xin.stride(0), T, ctx.B, C, K, ptr(taps), dtype_code(taps), ptr(taps_t),
         ptr(bias), 1 if activation else 0, ptr(state), ptr(ctx.seq_of), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens), ptr(out),
         out.stride(0), stream_ptr())
    return out


def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, carried: torch.Tensor, ctx, out: torch.Tensor) -> torch.Tensor:
    """out[s, t, :] = h[t] + (h[t-1] - h[t]) * mu[s] for every blend s; the row before a sequence's first token of the
    step is carried [slots, E] (float32; zero when the sequence starts), which then receives the step's last row.
    out [S, T', E] with T' >= T: rows from T on are left as they are."""
    _cuda(h, mu, carried, out)
    T, E = h.shape
    S = mu.shape[0]
    assert h.stride(1) == 1 and mu.shape == (S, E) and mu.is_contiguous() and out.is_contiguous()
    assert out.dim() == 3 and out.shape[0] == S and out.shape[1] >= T and out.shape[2] == E
    assert out.dtype == h.dtype and carried.dtype == torch.float32 and carried.shape[1:] == (E,) and carried.is_contiguous()
    call("gb_token_shift_mix", ptr(h), dtype_code(h), h.stride(0), T, E, ptr(mu), dtype_code(mu), S, ptr(carried), ptr(ctx.seq_of),
         ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens), ptr(out), out.stride(0), stream_ptr())
    return out


def _walk_scratch(ctx, n_heads: int, dim: int, vdim: int):
    """Workspace of the walk over tokens that the mixers with a matrix state share: prepared rows, and room for the
    segments of long sequences."""
    lib = native.library()
    scratch = ctx.ws.get("walk.prepared", (lib.gb_linear_walk_scratch_floats(ctx.T, n_heads, dim, vdim),), torch.float32)
    seg = lib.gb_gla_segment_floats(ctx.B, ctx.max_qlen, n_heads, dim, vdim)
    return scratch, (ctx.ws.get("walk.segments", (seg,), torch.float32) if seg else None)


def wkv(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, w0: torch.Tensor, u: torch.Tensor,
        state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int, dim: int) -> torch.Tensor:
    """Per head, from and into state [slots, heads, dim, dim] (float32): out = (S + diag(u) k v^T)^T r, then
    S <- diag(w) S + k v^T with w = exp(-exp(a + w0)) per key channel.  r, k, v [T, heads*dim]; a [T, heads*dim] the
    decay's low-rank result; out float32 [T, heads*dim]."""
    _cuda(r, k, v, a, w0, u, state, out)
    T = r.shape[0]
    for t in (r, k, v, a):
        assert t.stride(1) == 1 and t.shape == (T, n_heads * dim)
    assert r.dtype == k.dtype == v.dtype and w0.dtype == u.dtype and w0.numel() == u.numel() == n_heads * dim
    assert w0.is_contiguous() and u.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (n_heads, dim, dim) and state.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, n_heads * dim) and out.stride(1) == 1
    scratch, seg = _walk_scratch(ctx, n_heads, dim, dim)
    call("gb_wkv", ptr(r), r.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0), dtype_code(r), ptr(a), dtype_code(a), a.stride(0),
         ptr(w0), ptr(u), dtype_code(w0), ptr(state), ptr(out), out.stride(0), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens),
         T, ctx.B, n_heads, dim, ptr(scratch), int(ctx.max_qlen), ptr(seg), stream_ptr())
    if seg is not None:
        native.count_launches(3)
    return out


def ssd(x: torch.Tensor, bm: torch.Tensor, cm: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
        skip: torch.Tensor, state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int, n_groups: int, n_state: int,
        vdim: int) -> torch.Tensor:
    """The selective state-space recurrence per head, from and into state [slots, heads, n_state, vdim] (float32):
    dt' = softplus(dt + dt_bias); S <- exp(-exp(a_log) dt') S + dt' B x^T; out = S^T C + skip x.  x [T, heads*vdim],
    bm, cm [T, groups*n_state]: column slices of one buffer; dt [T, heads]; out float32 [T, heads*vdim]."""
    _cuda(x, bm, cm, dt, dt_bias, a_log, skip, state, out)
    T, ld = x.shape[0], x.stride(0)
    assert bm.stride(0) == ld and cm.stride(0) == ld and x.dtype == bm.dtype == cm.dtype
    assert x.stride(1) == 1 and bm.stride(1) == 1 and cm.stride(1) == 1 and dt.stride(1) == 1
    assert x.shape == (T, n_heads * vdim) and bm.shape == cm.shape == (T, n_groups * n_state) and dt.shape == (T, n_heads)
    assert dt_bias.dtype == a_log.dtype == skip.dtype and dt_bias.numel() == a_log.numel() == skip.numel() == n_heads
    assert state.dtype == torch.float32 and state.shape[1:] == (n_heads, n_state, vdim) and state.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, n_heads * vdim) and out.stride(1) == 1
    scratch, seg = _walk_scratch(ctx, n_heads, n_state, vdim)
    call("gb_ssd", ptr(x), ptr(bm), ptr(cm), dtype_code(x), ld, ptr(dt), dtype_code(dt), dt.stride(0), ptr(dt_bias), ptr(a_log),
         ptr(skip), dtype_code(dt_bias), ptr(state), ptr(out), out.stride(0), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens),
         T, ctx.B, n_heads, n_groups, n_state, vdim, ptr(scratch), int(ctx.max_qlen), ptr(seg), stream_ptr())
    if seg is not None:
        native.count_launches(3)
    return out


def add_rmsnorm_pair(x: torch.Tensor, terms, weight: torch.Tensor, weight2: Optional[torch.Tensor], offset: float, eps: float,
                     out: torch.Tensor, out2: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                     write_x: bool = True) -> None:
    """x float32 [T,E] += the sum of up to three terms [T,E]; out = x / sqrt(mean(x^2) + eps) * (offset + weight), and
    out2 the same with weight2 when given.  rows: int32 row numbers to gather (then the results have len(rows) rows)."""
    _cuda(x, weight, weight2, out, out2, rows, *terms)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.numel() == E and len(terms) <= 3
    assert (weight2 is None) == (out2 is None) and (weight2 is None or (weight2.dtype == weight.dtype and weight2.numel() == E))
    n_rows = T if rows is None else rows.numel()
    assert out.shape == (n_rows, E) and (out2 is None or (out2.shape == out.shape and out2.dtype == out.dtype and out2.is_contiguous()))
    args = []
    for i in range(3):
        t = terms[i] if i < len(terms) else None
        assert t is None or (t.shape == (T, E) and t.is_contiguous())
        args += [ptr(t), 0 if t is None else dtype_code(t)]
    call("gb_add_rmsnorm_pair", ptr(x), *args, len(terms), ptr(rows), n_rows, E, ptr(weight), ptr(weight2), dtype_code(weight),
         float(offset), float(eps), ptr(out), ptr(out2), dtype_code(out), int(write_x), stream_ptr())


def embed_bigram(table: torch.Tensor, pairs: torch.Tensor, ctx, prev_token: torch.Tensor, buckets: int, mul_prev: int,
                 mul_cur: int, out: torch.Tensor, copy: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t,:] = table[token,:] * scale + pairs[row,:] in float32, row = (previous token * mul_prev + token * mul_cur)
    mod buckets, and row `buckets` for a sequence's first token.  prev_token int32 [slots]: the token before a step's
    first, renewed with the step's last.  copy receives the same rows once more."""
    _cuda(table, pairs, prev_token, out, copy)
    V, E = table.shape
    T = ctx.tokens.numel()
    assert pairs.shape == (buckets + 1, E) and table.is_contiguous() and pairs.is_contiguous()
    assert prev_token.dtype == torch.int32 and prev_token.dim() == 1 and prev_token.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous()
    assert copy is None or (copy.dtype == torch.float32 and copy.shape == (T, E) and copy.is_contiguous())
    call("gb_embed_bigram", ptr(table), dtype_code(table), ptr(pairs), dtype_code(pairs), ptr(ctx.tokens), ptr(ctx.pos),
         ptr(ctx.seq_of), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens), ptr(prev_token), T, E, V, int(buckets), int(mul_prev),
         int(mul_cur), float(scale), ptr(out), ptr(copy), stream_ptr())
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap tanh(x / cap) in place (float32)."""
    _cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    call("gb_softcap", ptr(x), x.numel(), float(cap), stream_ptr())
    return x


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, a: torch.Tensor,
               dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, out: torch.Tensor, ctx,
               n_heads: int, n_kv_heads: int, dim: int, vdim: int, q_scale: float) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over this step's tokens, from and into
    state [slots, heads, dim, vdim] (float32).  q, k [T, kv_heads*dim] and v [T, heads*vdim] are column slices
    of one buffer (after convolution and SiLU); beta [T, heads] and a [T, heads*dim] are the projections'
    outputs before sigmoid and softplus; out float32 [T, heads*vdim] is what the state gives for q.
    Two launches: what does not depend on the state for all tokens at once (into a workspace buffer), then the walk."""
    _cuda(q, k, v, beta, a, dt_bias, a_log, state, out)
    T = q.shape[0]
    ld = q.stride(0)
    assert k.stride(0) == ld and v.stride(0) == ld and q.dtype == k.dtype == v.dtype == beta.dtype == a.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and beta.stride(1) == 1 and a.stride(1) == 1
    assert state.dtype == torch.float32 and state.shape[1:] == (n_heads, dim, vdim) and state.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, n_heads * vdim) and out.stride(1) == 1
    assert dt_bias.dtype == a_log.dtype and dt_bias.numel() == n_heads * dim and a_log.numel() == n_heads
    need = native.library().gb_delta_rule_scratch_floats(T, n_heads, n_kv_heads, dim, vdim)
    scratch = ctx.ws.get("delta.prepared", (need,), torch.float32)
    call("gb_delta_rule", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, ptr(beta), beta.stride(0), ptr(a), a.stride(0),
         ptr(dt_bias), ptr(a_log), dtype_code(dt_bias), ptr(state), ptr(out), out.stride(0), ptr(ctx.cu), ptr(ctx.slots),
         ptr(ctx.qlens), T, ctx.B, n_heads, n_kv_heads, dim, vdim, float(q_scale), ptr(scratch), stream_ptr())
    return out


HEAD_GATES = {"sigmoid": 0, "silu": 1}


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                    n_heads: int, vdim: int, gate_function: str = "sigmoid", gate_first: bool = False) -> torch.Tensor:
    """out[t,h,:] = o[t,h,:] / sqrt(mean(o[t,h,:]^2) + eps) * weight * f(gate[t,h,:]); o float32; f the sigmoid or SiLU.
    weight: vdim entries that the heads share, or heads*vdim with a row per head.  gate_first: the gate comes before
    the norm, out = y / sqrt(mean(y^2) + eps) * weight with y = o f(gate)."""
    _cuda(o, gate, weight, out)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1
    assert o.shape == gate.shape == out.shape == (T, n_heads * vdim) and weight.numel() in (vdim, n_heads * vdim)
    assert weight.is_contiguous()
    per_head = weight.numel() == n_heads * vdim and n_heads > 1
    call("gb_gated_head_norm", ptr(o), o.stride(0), ptr(gate), dtype_code(gate), gate.stride(0), ptr(weight),
         dtype_code(weight), float(eps), ptr(out), dtype_code(out), out.stride(0), T, n_heads, vdim,
         HEAD_GATES[gate_function], int(per_head), int(bool(gate_first)), stream_ptr())
    return out


def gla(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, bias: torch.Tensor, tau: float, q_scale: float,
        state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Gated linear attention over this step's tokens, from and into state [slots, heads, dim, vdim] (float32):
    S <- diag(alpha) S + k v^T, out = S^T (q q_scale), alpha = sigmoid(a + bias)^(1/tau) per head and key channel.
    q, k [T, heads*dim] and v [T, heads*vdim] are column slices of one buffer; a [T, heads*dim] is the decay's
    projection; out float32 [T, heads*vdim].  Two launches: what does not depend on the state for all tokens at
    once (into a workspace buffer), then the walk; five where a sequence brings more than 256 tokens (its segments of 128
    are walked side by side, from zero, and again from the states that a short carry gives them)."""
    _cuda(q, k, v, a, bias, state, out)
    T, ld = q.shape[0], q.stride(0)
    assert k.stride(0) == ld and v.stride(0) == ld and q.dtype == k.dtype == v.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and a.stride(1) == 1
    assert q.shape[1] == n_heads * dim and v.shape[1] == n_heads * vdim and a.shape == (T, n_heads * dim)
    assert state.dtype == torch.float32 and state.shape[1:] == (n_heads, dim, vdim) and state.is_contiguous()
    assert out.dtype == torch.float32 and out.shape == (T, n_heads * vdim) and out.stride(1) == 1
    assert bias.numel() == n_heads * dim and bias.is_contiguous() and tau > 0
    need = native.library().gb_gla_scratch_floats(T, n_heads, dim, vdim)
    scratch = ctx.ws.get("gla.prepared", (need,), torch.float32)
    seg = native.library().gb_gla_segment_floats(ctx.B, ctx.max_qlen, n_heads, dim, vdim)
    seg_scratch = ctx.ws.get("gla.segments", (seg,), torch.float32) if seg else None
    call("gb_gla", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, ptr(a), dtype_code(a), a.stride(0), ptr(bias), dtype_code(bias),
         1.0 / float(tau), float(q_scale), ptr(state), ptr(out), out.stride(0), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens),
         T, ctx.B, n_heads, dim, vdim, ptr(scratch), int(ctx.max_qlen), ptr(seg_scratch), stream_ptr())
    if seg:
        native.count_launches(3)
    return out


def norm_residual_add(x: torch.Tensor, y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                      xb: Optional[torch.Tensor] = None) -> None:
    """x += y / sqrt(mean(y^2) + eps) * weight row by row (x float32, the sum in 32-bit); xb, when given, receives
    bfloat16(x).  y None: only the copy is made."""
    _cuda(x, y, weight, xb)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and (y is not None or xb is not None)
    assert y is None or (y.shape == (T, E) and y.stride(1) == 1 and weight.numel() == E)
    assert xb is None or (xb.dtype == torch.bfloat16 and xb.shape == (T, E) and xb.is_contiguous())
    call("gb_norm_residual_add", ptr(x), ptr(y), 0 if y is None else dtype_code(y), 0 if y is None else y.stride(0), T, E,
         ptr(weight), 0 if weight is None else dtype_code(weight), float(eps), ptr(xb), stream_ptr())


def head_prep_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, dim: int, vdim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rotary_dim: int, pairing: int, v_first: Optional[torch.Tensor],
                       mix: float, first_out: Optional[torch.Tensor], seq_of: torch.Tensor, pos: torch.Tensor,
                       table: torch.Tensor, ring_pages: int, head_pages: int, kcache: torch.Tensor, vcache: torch.Tensor) -> None:
    """q, k, v: column slices of one row-major buffer.  Per head: RMS norm with a weight of `dim` entries that all
    heads share (q_weight, k_weight; None: no norm), then the rotation of the first rotary_dim entries (inv_freq None:
    none); q in place, k into the cache.  v <- (1 - mix) v + mix v_first when v_first [T, kv_heads*vdim] is given,
    into the cache; first_out receives v as it came."""
    _cuda(q, k, v, q_weight, k_weight, inv_freq, v_first, first_out, seq_of, pos, table, kcache, vcache)
    T, ld = q.shape[0], q.stride(0)
    if k is None:                       # a layer that reads another layer's keys and values: its queries only
        assert v is None and v_first is None and first_out is None
        kcache = vcache = None
    else:
        assert q.stride(1) == 1 and k.stride(0) == ld and v.stride(0) == ld and k.dtype == q.dtype == v.dtype
        assert kcache.shape[-1] == dim and vcache.shape[-1] == vdim and kcache.dtype == vcache.dtype
    assert (q_weight is None) == (k_weight is None) and (q_weight is None or (q_weight.numel() == dim == k_weight.numel() and q_weight.dtype == k_weight.dtype))
    for t in (v_first, first_out):
        assert t is None or (t.shape == (T, n_kv_heads * vdim) and t.stride(1) == 1 and t.dtype == q.dtype)
    call("gb_head_prep_kv_write", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, T, n_heads, n_kv_heads, dim, vdim, ptr(q_weight),
         ptr(k_weight), 0 if q_weight is None else dtype_code(q_weight), float(eps), ptr(inv_freq), int(rotary_dim), int(pairing),
         ptr(v_first), 0 if v_first is None else v_first.stride(0), float(mix), ptr(first_out),
         0 if first_out is None else first_out.stride(0), ptr(seq_of), ptr(pos), ptr(table), table.shape[1], int(ring_pages),
         int(head_pages), ptr(kcache), ptr(vcache), 0 if kcache is None else dtype_code(kcache), stream_ptr())


def moe_route(logits: torch.Tensor, n_groups: int, keep: int, top: int, scale: float, ids: torch.Tensor,
              weights: torch.Tensor, softmax: bool = False, correction: Optional[torch.Tensor] = None) -> None:
    """Router logits float32 [T, experts] -> ids int32 [T, top] and weights float32 [T, top]: scores are sigmoids; the
    experts form n_groups equal groups of neighbours, a group's mark is the sum of its two largest scores, only the
    `keep` best groups' experts can be chosen; weights are the chosen scores over their sum, times scale."""
    _cuda(logits, ids, weights)
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and ids.dtype == torch.int32 and weights.dtype == torch.float32
    assert ids.shape == (T, top) and weights.shape == (T, top) and ids.is_contiguous() and weights.is_contiguous()
    _check_correction(correction, E)
    call("gb_moe_route", ptr(logits), T, E, int(n_groups), int(keep), int(top), float(scale), ptr(ids), ptr(weights),
         int(bool(softmax)), ptr(correction), stream_ptr())


def _check_correction(correction: Optional[torch.Tensor], n: int) -> None:
    assert correction is None or (correction.is_cuda and correction.dtype == torch.float32 and correction.numel() == n
                                  and correction.is_contiguous())


def moe_router(x: torch.Tensor, w: torch.Tensor, n_groups: int, keep: int, top: int, scale: float, ids: torch.Tensor,
               weights: torch.Tensor, softmax: bool = False, correction: Optional[torch.Tensor] = None) -> None:
    """The router's product x w^T (32-bit sums) and the choice of moe_route in one kernel; x [T, K], w [experts, K].
    softmax: scores are softmax over all experts instead of sigmoids; correction float32 [experts]: added to the scores
    for the choice, not for the weights."""
    _cuda(x, w, ids, weights)
    T, K = x.shape
    assert x.stride(1) == 1 and w.is_contiguous() and w.shape[1] == K and ids.dtype == torch.int32 and weights.dtype == torch.float32
    assert ids.shape == (T, top) and weights.shape == (T, top) and ids.is_contiguous() and weights.is_contiguous()
    _check_correction(correction, w.shape[0])
    call("gb_moe_router", ptr(x), dtype_code(x), x.stride(0), T, K, ptr(w), dtype_code(w), w.shape[0], int(n_groups), int(keep),
         int(top), float(scale), ptr(ids), ptr(weights), int(bool(softmax)), ptr(correction), stream_ptr())


def moe_gate_up(h: torch.Tensor, ids: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, limit: float,
                y: torch.Tensor, identity: int = 0) -> torch.Tensor:
    """y[t, r, :] = unit(W_gate[e] h_t, W_up[e] h_t), e = ids[t, r]; unit(g, u) = g' sigmoid(1.702 g') (u' + 1) with
    g' = min(g, limit), u' = clamp(u, -limit, limit).  w_gate, w_up [experts, F, K]; token by token on the CUDA cores."""
    _cuda(h, ids, w_gate, w_up, y)
    T, K = h.shape
    E, F, _ = w_gate.shape
    top = ids.shape[1]
    assert h.stride(1) == 1 and w_gate.is_contiguous() and w_up.is_contiguous() and w_gate.shape == w_up.shape == (E, F, K)
    assert w_gate.dtype == w_up.dtype and y.shape == (T, top, F) and y.is_contiguous() and ids.is_contiguous()
    call("gb_moe_gate_up", ptr(h), dtype_code(h), h.stride(0), T, K, F, top, ptr(ids), ptr(w_gate), ptr(w_up), dtype_code(w_gate),
         float(limit), ptr(y), dtype_code(y), E if identity else 0x7fffffff, stream_ptr())
    return y


def moe_down(y: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_down: torch.Tensor, out: torch.Tensor,
             accumulate: bool = False, ws=None, identity: int = 0, h: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] (+)= sum_r weights[t, r] W_down[ids[t, r]] y[t, r]; w_down [experts, N, F]; out float32 [T, N].  Every pair's
    row first (32-bit, in a buffer of the workspace `ws` when given), then the weighted sum per token: two launches."""
    _cuda(y, ids, weights, w_down, out)
    T, top, F = y.shape
    E, N, _ = w_down.shape
    assert y.is_contiguous() and w_down.is_contiguous() and w_down.shape == (E, N, F) and out.shape == (T, N)
    assert out.dtype == torch.float32 and out.is_contiguous() and ids.shape == (T, top) and weights.shape == (T, top)
    z = ws.get("moe.rows", (T * top, N), torch.float32) if ws is not None else torch.empty(T * top, N, dtype=torch.float32, device=y.device)
    # identity experts (ids from the number of matrices on, `identity` of them) give the token's own row h [T, N]
    assert not identity or (h is not None and h.shape == (T, N) and h.stride(1) == 1)
    own = h if identity else None
    call("gb_moe_down", ptr(y), dtype_code(y), T, F, N, top, ptr(ids), ptr(weights), ptr(w_down), dtype_code(w_down), ptr(z),
         ptr(out), int(bool(accumulate)), E, ptr(own), 0 if own is None else dtype_code(own), 0 if own is None else own.stride(0),
         stream_ptr())
    return out


def moe_grouped_supported(h: torch.Tensor, w_gate: torch.Tensor) -> bool:
    """Whether the tiled tensor-core kernels take these experts: bfloat16, K and F multiples of 8, aligned rows."""
    return h.dtype == torch.bfloat16 and w_gate.dtype == torch.bfloat16 and h.stride(1) == 1 and h.stride(0) % 8 == 0 \
        and h.data_ptr() % 16 == 0 and bool(native.library().gb_moe_grouped_supported(w_gate.shape[2], w_gate.shape[1]))


def moe_grouped(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, limit: float, out: torch.Tensor, ctx, accumulate: bool = False, identity: int = 0) -> torch.Tensor:
    """The routed experts of a step of many tokens on the tensor cores: the (token, choice) pairs sorted by expert on
    the device, gate and up with the clamped unit, down, and the weighted sum per token; what moe_gate_up and moe_down
    give, up to the rounding of bfloat16 unit outputs.  Four launches."""
    _cuda(h, ids, weights, w_gate, w_up, w_down, out)
    T, K = h.shape
    E, F, _ = w_gate.shape
    N, top = w_down.shape[1], ids.shape[1]
    assert w_gate.shape == w_up.shape == (E, F, K) and w_down.shape == (E, N, F) and out.shape == (T, N) and out.dtype == torch.float32
    assert w_gate.is_contiguous() and w_up.is_contiguous() and w_down.is_contiguous() and out.is_contiguous()
    assert ids.shape == weights.shape == (T, top) and ids.is_contiguous() and weights.is_contiguous()
    y = ctx.ws.get("moe.units", (T, top, F), torch.bfloat16)
    z = ctx.ws.get("moe.rows", (T * top, N), torch.float32)
    n_all = E + int(identity)                 # identity experts are numbered behind those with matrices
    scratch = ctx.ws.get("moe.sorted", (native.library().gb_moe_grouped_scratch_ints(T, top, n_all),), torch.int32)
    call("gb_moe_grouped", ptr(h), h.stride(0), T, K, F, N, n_all, top, ptr(ids), ptr(weights), ptr(w_gate), ptr(w_up), ptr(w_down),
         float(limit), ptr(y), ptr(z), ptr(scratch), ptr(out), int(bool(accumulate)), E, stream_ptr())
    return out


def moe_by_expert(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                  w_down: torch.Tensor, limit: float, out: torch.Tensor, ctx, accumulate: bool = False, identity: int = 0) -> torch.Tensor:
    """The routed experts of a step of very many tokens as ordinary products, expert by expert, on the tcgen05 product
    kernels: the pairs sorted by expert and the tokens' rows gathered in that order on the device; the experts' offsets
    read on the host (one wait per call: such steps are prompts, which no graph captures); per expert gate, up and down
    over its own rows; the clamped unit over all rows at once; the weighted sum per token in choice order."""
    _cuda(h, ids, weights, w_gate, w_up, w_down, out)
    T, K = h.shape
    E, F, _ = w_gate.shape
    N, top = w_down.shape[1], ids.shape[1]
    P = T * top
    assert h.dtype == torch.bfloat16 and w_gate.dtype == torch.bfloat16 and out.dtype == torch.float32 and out.shape == (T, N)
    lib = native.library()
    n_all = E + int(identity)                 # identity experts are sorted behind the others; their rows are never multiplied
    scratch = ctx.ws.get("moe.sorted", (lib.gb_moe_grouped_scratch_ints(T, top, n_all),), torch.int32)
    order = ctx.ws.get("moe.order", (n_all + 1 + 2 * P,), torch.int32)
    offsets, perm, place_of = order[:n_all + 1], order[n_all + 1:n_all + 1 + P], order[n_all + 1 + P:]
    call("gb_moe_sort", ptr(ids), T, top, n_all, ptr(offsets), ptr(perm), ptr(place_of), ptr(scratch), stream_ptr())
    rows = ctx.ws.get("moe.gathered", (P, K), torch.bfloat16)
    call("gb_moe_gather_rows", ptr(h), h.stride(0), T, K, top, ptr(perm), ptr(rows), stream_ptr())
    at = offsets.cpu().tolist()
    gu = ctx.ws.get("moe.gate_up", (P, 2 * F), torch.bfloat16)
    for e in range(E):
        a, b = at[e], at[e + 1]
        if b > a:
            gemm(rows[a:b], w_gate[e], None, gu[a:b, :F])
            gemm(rows[a:b], w_up[e], None, gu[a:b, F:])
    y = glu_clamped(gu, ctx.ws.get("moe.units", (P, F), torch.bfloat16), limit)
    z = ctx.ws.get("moe.rows", (P, N), torch.float32)
    for e in range(E):
        a, b = at[e], at[e + 1]
        if b > a:
            gemm(y[a:b], w_down[e], None, z[a:b])
    call("gb_moe_combine_sorted", ptr(z), ptr(place_of), ptr(weights), T, top, N, ptr(out), int(bool(accumulate)),
         ptr(ids) if identity else None, E, ptr(h), dtype_code(h), h.stride(0), stream_ptr())
    return out


UNARY_ACTS = {"silu": 1, "gelu_tanh": 2, "gelu": 3, "tanh": 4}


def unary_act_(x: torch.Tensor, activation: str) -> torch.Tensor:
    """x <- act(x) in place; gelu is the exact form 0.5 z (1 + erf(z / sqrt 2)).  x: contiguous, or a block of columns
    of a row-major buffer."""
    _cuda(x)
    if x.is_contiguous():
        call("gb_unary_act", ptr(x), dtype_code(x), x.numel(), UNARY_ACTS[activation], stream_ptr())
    else:
        assert x.dim() == 2 and x.stride(1) == 1
        call("gb_unary_act_rows", ptr(x), dtype_code(x), x.shape[0], x.shape[1], x.stride(0), UNARY_ACTS[activation], stream_ptr())
    return x


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float) -> torch.Tensor:
    """gate_up [T, 2F], gate in the first F columns; out[t, i] = g' sigmoid(1.702 g') (u' + 1) with the inputs clamped
    as in moe_gate_up."""
    _cuda(gate_up, out)
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.stride(1) == 1 and out.is_contiguous() and out.dtype == gate_up.dtype
    call("gb_glu_clamped", ptr(gate_up), gate_up.stride(0), ptr(out), T, F, dtype_code(out), float(limit), stream_ptr())
    return out


def qk_norm_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], n_heads: int, n_kv_heads: int,
                     dim: int, vdim: int, normalise: bool, eps: float, temp_coef: float, temp_every: int,
                     seq_of: torch.Tensor, pos: torch.Tensor, table: Optional[torch.Tensor], ring_pages: int,
                     kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor]) -> None:
    """q, k, v: column slices of one row-major buffer.  q heads are brought to unit root mean square and
    multiplied by 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1) in place; k heads normalised likewise
    and v heads as they are go into the cache pages (keys of `dim`, values of `vdim` entries)."""
    _cuda(q, k, v, seq_of, pos, table, kcache, vcache)
    T, ld = q.shape[0], q.stride(0)
    assert q.stride(1) == 1 and (k is None or (k.stride(0) == ld and v.stride(0) == ld and k.dtype == q.dtype == v.dtype))
    assert kcache is None or (kcache.shape[-1] == dim and vcache.shape[-1] == vdim and kcache.dtype == vcache.dtype)
    call("gb_qk_norm_kv_write", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, T, n_heads, n_kv_heads, dim, vdim,
         int(bool(normalise)), float(eps), float(temp_coef), int(temp_every), ptr(seq_of), ptr(pos), ptr(table),
         0 if table is None else table.shape[1], ring_pages, ptr(kcache), ptr(vcache),
         0 if kcache is None else dtype_code(kcache), stream_ptr())


def latent_prep(q: torch.Tensor, dkv: torch.Tensor, n_heads: int, dim: int, rot_dim: int, kv_rank: int, rot_dims: int,
                inv_freq: Optional[torch.Tensor], weight: torch.Tensor, eps: float, qa: Optional[torch.Tensor],
                seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, ring_pages: int, cache: torch.Tensor,
                row_out: Optional[torch.Tensor] = None, halves: bool = False) -> None:
    """Latent attention in front of the attention kernel: dkv [T, kv_rank + rot_dim] gives the cache row
    (RMS-normed latent, rotated shared key part; also copied to row_out [T, kv_rank + rot_dim] when given); the
    heads' rotated query parts go to qa [T, heads*(kv_rank + rot_dim)] behind the kv_rank entries that
    head_matmul fills, or, with qa None, are rotated in place in q."""
    _cuda(q, dkv, inv_freq, weight, qa, seq_of, pos, table, cache, row_out)
    T = q.shape[0]
    assert q.stride(1) == 1 and dkv.stride(1) == 1 and q.dtype == dkv.dtype
    assert q.shape[1] == n_heads * (dim + rot_dim) and dkv.shape[1] == kv_rank + rot_dim
    assert cache.shape[-1] == kv_rank + rot_dim and weight.numel() == kv_rank
    if qa is None:
        qa, stride, off = q, dim + rot_dim, dim
    else:
        stride, off = kv_rank + rot_dim, kv_rank
        assert qa.shape == (T, n_heads * (kv_rank + rot_dim)) and qa.stride(1) == 1 and qa.dtype == q.dtype
    assert row_out is None or (row_out.shape == (T, kv_rank + rot_dim) and row_out.is_contiguous() and row_out.dtype == q.dtype)
    call("gb_latent_prep", ptr(q), q.stride(0), ptr(dkv), dkv.stride(0), dtype_code(q), T, n_heads, dim, rot_dim, kv_rank,
         rot_dims, ptr(inv_freq), ptr(weight), dtype_code(weight), float(eps), ptr(qa), qa.stride(0), stride, off,
         ptr(row_out), ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages, ptr(cache), dtype_code(cache),
         int(bool(halves)), stream_ptr())


def pack_latent_heads(kv: torch.Tensor, row: torch.Tensor, n_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                      seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, k_pages: torch.Tensor,
                      v_pages: torch.Tensor) -> None:
    """Per-head keys [pages, heads, 64, dim + rot_dim] (the head's up-projected part, then the shared rotated part
    of `row`) and values [pages, heads, 64, vdim] of a prompt's tokens, at the pages `table` names."""
    _cuda(kv, row, seq_of, pos, table, k_pages, v_pages)
    T = kv.shape[0]
    assert kv.dtype == row.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16 and kv.stride(1) == 1 and row.is_contiguous()
    assert kv.shape[1] == n_heads * (dim + vdim) and row.shape == (T, kv_rank + rot_dim)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[1:] == (n_heads, 64, dim + rot_dim)
    assert v_pages.shape[1:] == (n_heads, 64, vdim) and table.dim() == 2
    call("gb_pack_latent_heads", ptr(kv), kv.stride(0), ptr(row), T, n_heads, dim, rot_dim, vdim, kv_rank, ptr(seq_of), ptr(pos),
         ptr(table), table.shape[1], ptr(k_pages), ptr(v_pages), stream_ptr())


def latent_decode_supported(n_heads: int, kv_rank: int, rot_dim: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and bool(native.library().gb_latent_decode_supported(n_heads, kv_rank, rot_dim, 1, 1))


def latent_decode_class(max_kv: int) -> int:
    """Class of a decode step for the latent decode kernel: half of the longest sequence's blocks of 32 keys, rounded
    down to one of a few values; steps of one class split their keys alike."""
    return _split_class(((max_kv + 31) // 32) // 2)


def latent_decode(qa: torch.Tensor, out: torch.Tensor, n_heads: int, kv_rank: int, rot_dim: int, ctx, table: torch.Tensor,
                  ring_pages: int, cache: torch.Tensor, scale: float, window: int = 0, sink_values: Optional[torch.Tensor] = None,
                  gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Latent attention of single tokens: qa [T, heads*(kv_rank + rot_dim)] (queries in the latent's space, then the
    rotated part), cache rows [kv_rank + rot_dim]; out [T, heads*kv_rank] is the mix of the rows' first kv_rank
    entries.  One pass over each token's rows serves all heads; the rows are split over CTAs (two blocks of 32 keys or
    more per split, while two CTAs per SM hold the step) and merged in order.  window: the last `window` positions only;
    sink_values float32 [heads]: one more key without a value of that score in the denominator; gate bfloat16 [T, heads]:
    a head's result times its sigmoid."""
    _cuda(qa, out, table, cache, sink_values, gate)
    assert sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == n_heads and sink_values.is_contiguous())
    assert gate is None or (gate.dtype == torch.bfloat16 and gate.shape == (qa.shape[0], n_heads) and gate.stride(1) == 1)
    T = qa.shape[0]
    assert qa.dtype == out.dtype == cache.dtype == torch.bfloat16 and qa.stride(1) == 1 and out.stride(1) == 1
    assert qa.shape[1] == n_heads * (kv_rank + rot_dim) and out.shape == (T, n_heads * kv_rank) and cache.shape[-1] == kv_rank + rot_dim
    lib = native.library()
    seen = min(ctx.max_kv, window + 31) if window else ctx.max_kv
    splits = max(1, min(latent_decode_class(seen), 64, (2 * tc_scratch(qa.device).sms) // max(T, 1)))
    scratch = ctx.ws.get("latent.partial", (lib.gb_latent_decode_scratch_floats(T, n_heads, kv_rank, splits),), torch.float32)
    call("gb_latent_decode", ptr(qa), qa.stride(0), ptr(out), out.stride(0), T, n_heads, kv_rank, rot_dim, ptr(ctx.seq_of),
         ptr(ctx.pos), ptr(table), table.shape[1], ring_pages, ptr(cache), float(scale), splits, ptr(scratch), int(window or 0),
         ptr(sink_values), ptr(gate), 0 if gate is None else gate.stride(0), stream_ptr())
    return out


def head_matmul(x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int) -> torch.Tensor:
    """out[t, h*out_head_stride + o] = sum_i x[t, h*x_head_stride + i] * w[h, i, o]; w [heads, in, out]."""
    _cuda(x, w, out)
    H, I, O = w.shape
    T = x.shape[0]
    assert w.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T
    assert x.shape[1] >= (H - 1) * x_head_stride + I and out.shape[1] >= (H - 1) * out_head_stride + O
    call("gb_head_matmul", ptr(x), dtype_code(x), x.stride(0), int(x_head_stride), ptr(w), dtype_code(w), H, I, O, ptr(out),
         dtype_code(out), out.stride(0), int(out_head_stride), T, stream_ptr())
    return out


def selective_scan(x: torch.Tensor, z: torch.Tensor, low: torch.Tensor, dt_rank: int, n_state: int, dt: torch.Tensor,
                   dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                   ctx) -> torch.Tensor:
    """The selective scan per channel c and state entry n, from and into state [slots, inner, n_state] (float32):
    dt' = softplus(dt + dt_bias); S[c, n] <- exp(-exp(a_log[c, n]) dt'_c) S[c, n] + dt'_c x_c B_n; y_c = sum_n S[c, n] C_n +
    skip_c x_c; out = y * silu(z).  x, z [T, inner]; low [T, dt_rank + 2 n_state] holds B and C behind its first
    dt_rank columns; dt float32 [T, inner]; dt_bias, skip [inner], a_log [inner, n_state] float32.  Prompts of more
    than 256 tokens run in segments of 128 side by side (three launches)."""
    _cuda(x, z, low, dt, dt_bias, a_log, skip, state, out)
    T, inner = x.shape
    assert z.shape == (T, inner) and x.dtype == z.dtype and x.stride(1) == 1 and z.stride(1) == 1
    assert low.shape == (T, dt_rank + 2 * n_state) and low.stride(1) == 1
    assert dt.dtype == torch.float32 and dt.shape == (T, inner) and dt.stride(1) == 1
    for t, shape in ((dt_bias, (inner,)), (a_log, (inner, n_state)), (skip, (inner,))):
        assert t.dtype == torch.float32 and t.shape == shape and t.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (inner, n_state) and state.is_contiguous()
    assert out.shape == (T, inner) and out.stride(1) == 1
    n = native.library().gb_selective_scan_segment_floats(ctx.B, int(ctx.max_qlen), inner, n_state)
    seg = ctx.ws.get("scan.segments", (n,), torch.float32) if n else None
    call("gb_selective_scan", ptr(x), x.stride(0), ptr(z), z.stride(0), dtype_code(x), ptr(low), dtype_code(low), low.stride(0), int(dt_rank),
         int(n_state), ptr(dt), dt.stride(0), ptr(dt_bias), ptr(a_log), ptr(skip), ptr(state), ptr(out), out.stride(0),
         dtype_code(out), ptr(ctx.cu), ptr(ctx.slots), ptr(ctx.qlens), T, ctx.B, inner, int(ctx.max_qlen), ptr(seg), stream_ptr())
    if seg is not None:
        native.count_launches(2)
    return out


def norm_sandwich(x: Optional[torch.Tensor], y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                  y2: Optional[torch.Tensor] = None, inner_weights=None, mix: float = 1.0,
                  next_weight: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None,
                  xb: Optional[torch.Tensor] = None, u_out: Optional[torch.Tensor] = None) -> None:
    """One pass over each row for a layer that norms what a sublayer reads and what it gives (rms(v) = sqrt(mean(v^2) +
    eps), 32-bit sums): u = y, or with y2 u = mix (y / rms(y) wy + y2 / rms(y2) wy2) for inner_weights (wy, wy2);
    x += u / rms(u) weight (x float32 [T, E]); then, each optional, h = x / rms(x) next_weight (the rows the next sublayer
    reads) and xb = bfloat16(x).  weight None: u itself goes to u_out (float32) and x is not touched.  y None: only h and xb."""
    wy, wy2 = inner_weights if inner_weights is not None else (None, None)
    _cuda(x, y, y2, weight, wy, wy2, next_weight, h, xb, u_out)
    ref = x if x is not None else y
    T, E = ref.shape
    ws = [w for w in (weight, wy, wy2, next_weight) if w is not None]
    assert ws and all(w.dtype == ws[0].dtype and w.numel() == E and w.is_contiguous() for w in ws)
    assert x is None or (x.dtype == torch.float32 and x.is_contiguous())
    for t in (y, y2):
        assert t is None or (t.shape == (T, E) and t.stride(1) == 1)
    assert h is None or (h.shape == (T, E) and h.is_contiguous())
    assert xb is None or (xb.dtype == torch.bfloat16 and xb.shape == (T, E) and xb.is_contiguous())
    assert u_out is None or (u_out.dtype == torch.float32 and u_out.shape == (T, E) and u_out.is_contiguous())
    call("gb_norm_sandwich", ptr(x), ptr(y), 0 if y is None else dtype_code(y), 0 if y is None else y.stride(0), ptr(y2),
         0 if y2 is None else dtype_code(y2), 0 if y2 is None else y2.stride(0), ptr(wy), ptr(wy2), float(mix), ptr(weight),
         ptr(next_weight), dtype_code(ws[0]), float(eps), ptr(h), 0 if h is None else dtype_code(h), ptr(xb), ptr(u_out), T, E,
         stream_ptr())


def token_side_gate(a: torch.Tensor, table: torch.Tensor, offset: int, tokens: torch.Tensor, out: torch.Tensor,
                    activation: str = "gelu_tanh") -> torch.Tensor:
    """out[t, j] = act(a[t, j]) * table[token_t, offset + j] for the dim = a.shape[1] columns of a layer's slice of a
    per-token table [vocabulary, all layers' columns]."""
    _cuda(a, table, tokens, out)
    T, dim = a.shape
    assert a.stride(1) == 1 and table.stride(1) == 1 and out.shape == (T, dim) and out.stride(1) == 1 and tokens.numel() == T
    call("gb_token_side_gate", ptr(a), dtype_code(a), a.stride(0), ptr(table), dtype_code(table), table.stride(0), int(offset),
         ptr(tokens), table.shape[0], T, dim, GATE_ACTS[activation], ptr(out), dtype_code(out), out.stride(0), stream_ptr())
    return out


def zero_rows(arena: torch.Tensor, table: torch.Tensor, slot: int) -> None:
    """Zeroes row `slot` of every region of a byte arena; table int64 [regions, 2] = (offset, bytes per row)."""
    _cuda(arena, table)
    assert arena.dtype == torch.uint8 and table.dtype == torch.int64 and table.is_contiguous()
    call("gb_zero_rows", ptr(arena), ptr(table), table.shape[0], int(slot), stream_ptr())


def gemm_generic(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[t,n] = sum_k x[t,k] w[n,k] + bias[n], 32-bit FMAs on the CUDA cores."""
    _cuda(x, w, bias, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    call("gb_gemm_generic", ptr(x), dtype_code(x), x.stride(0), ptr(w), dtype_code(w), w.stride(0), ptr(bias),
         0 if bias is None else dtype_code(bias), ptr(out), dtype_code(out), out.stride(0), T, N, K, stream_ptr())
    return out


def sample(logits: torch.Tensor, slots: torch.Tensor, seeds: torch.Tensor, temperature: float, top_k: int,
           top_p: float, rep_penalty: float, recent: torch.Tensor, count: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row of float32 logits [n, V].  The logits are the kernel's scratch: the repetition
    penalty is applied to them in place, and with a temperature they are left divided by it.
    recent [slots, 64] and count [slots] are the sequences' own state."""
    _cuda(logits, slots, seeds, recent, count, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and seeds.dtype == torch.int64
    assert slots.dtype == torch.int32 and recent.dtype == torch.int32 and count.dtype == torch.int32
    assert recent.shape[1] == 64 and recent.is_contiguous() and out.dtype == torch.int32 and out.numel() >= n
    call("gb_sample", ptr(logits), logits.stride(0), n, V, ptr(slots), ptr(seeds), float(temperature), int(top_k),
         float(top_p), float(rep_penalty), ptr(recent), ptr(count), ptr(out), stream_ptr())
    return out


class _TcScratch:
    """Scratch of the kernels that split their work and merge it (the tensor-core product's K split,
    decode attention's page split), per device: partial results and arrival counters (zero between
    launches).  Launches on one stream follow one another, so they can share it.

    It is allocated once, at the most any launch can need, and never again: a captured CUDA graph
    holds its address, so a buffer that grew would leave every graph captured before pointing at
    freed memory.  The product needs at most one partial tile per resident CTA (two CTAs per SM with
    tiles of up to 64 tokens, one with wider tiles: 2 * sms * 64 * 128 floats), decode attention
    (head_dim + 2) floats per head and split with no more CTAs than two per SM.  A launch that would
    need more (only a tuning override can ask for it) runs without splitting instead."""
    COUNTERS = 4096

    def __init__(self, device):
        self.device = device
        self.sms = native.library().gb_sm_count()
        self.capacity = 2 * max(self.sms, 1) * 256 * 128
        self.floats = torch.empty(self.capacity, dtype=torch.float32, device=device)
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)

    def fits(self, n_floats: int) -> bool:
        return n_floats <= self.capacity


_tc_scratch = {}


def tc_scratch(device) -> _TcScratch:
    key = torch.device(device).index or 0
    if key not in _tc_scratch:
        _tc_scratch[key] = _TcScratch(device)
    return _tc_scratch[key]


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    return bool(native.library().gb_gemm_tc_supported(ptr(x), x.stride(0), ptr(w), w.stride(0), x.shape[1]))


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2*64*ceil(F/64), K]: row 2f is gate row f, row 2f+1 is up row f, zero rows padding F to
    a multiple of 64: the layout gemm_tc's gated epilogue reads."""
    F, K = gate.shape
    pad = (F + 63) // 64 * 64 - F
    if pad:
        zeros = torch.zeros(pad, K, dtype=gate.dtype, device=gate.device)
        gate, up = torch.cat([gate, zeros]), torch.cat([up, zeros])
    return torch.stack([gate, up], dim=1).reshape(2 * (F + pad), K).contiguous()


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor],
            split_k: bool = True, swiglu_features: int = 0, row_ssq: Optional[torch.Tensor] = None, ssq_parts: int = 0,
            norm_size: int = 0, eps: float = 0.0, resid_x: Optional[torch.Tensor] = None,
            resid_xb: Optional[torch.Tensor] = None, ssq_out: Optional[torch.Tensor] = None,
            gate_activation: str = "silu") -> Optional[torch.Tensor]:
    """bf16 x bf16 -> f32 accumulate on tcgen05; out bf16 or f32.  Refuses what
    gemm_tc_supported refuses.  With swiglu_features = F, w is interleave_gate_up(gate, up)
    and out [T, F] = act(x gate^T) * (x up^T), act = gate_activation (GATE_ACTS).

    row_ssq [ssq_parts, T]: x holds rows whose RMS norm is deferred (its weight folded into w); each
    token's results are scaled by 1 / sqrt(sum_i row_ssq[i, t] / norm_size + eps).
    resid_x (f32 [T, N]): instead of writing `out`, resid_x += result in place, resid_xb gets the
    bfloat16 copy and ssq_out [ceil(N/128), T] the sums of squares per tile of 128 features."""
    _cuda(x, w, bias, out, row_ssq, resid_x, resid_xb, ssq_out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if resid_x is None:
        assert out.shape == (T, swiglu_features or N) and out.stride(1) == 1
    else:
        assert resid_x.shape == (T, N) and resid_x.dtype == torch.float32 and resid_x.stride(1) == 1
        assert resid_xb.shape == (T, N) and resid_xb.dtype == torch.bfloat16 and resid_xb.stride(0) == resid_x.stride(0)
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= ((N + 127) // 128) * T
    if row_ssq is not None:
        assert row_ssq.dtype == torch.float32 and row_ssq.numel() >= ssq_parts * T and ssq_parts > 0
    sc = tc_scratch(x.device)
    scratch = counters = None
    if split_k:
        need = native.library().gb_gemm_tc_scratch_floats(T, N, K, sc.sms)
        if need and sc.fits(need):
            scratch, counters = sc.floats, sc.counters
    call("gb_gemm_tc_fused", ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias), 0 if bias is None else dtype_code(bias),
         ptr(out), 1 if out is None else dtype_code(out), 0 if out is None else out.stride(0), T, N, K, ptr(scratch),
         ptr(counters), 0 if counters is None else counters.numel(), sc.sms, int(swiglu_features),
         GATE_ACTS[gate_activation], ptr(row_ssq),
         int(ssq_parts), int(norm_size), float(eps), ptr(resid_x), ptr(resid_xb), ptr(ssq_out),
         0 if resid_x is None else resid_x.stride(0), stream_ptr())
    return out


GROUPED_TILE = 256               # tokens of a tile of the kernel that pairs two SMs


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """G products of equal sizes as one launch on tcgen05: out[g] = x[g] @ w[g].T with x [G, R, K], w [G * N, K] (problem
    g's features from row g * N on) and out [G, R, N], all bfloat16, R a multiple of GROUPED_TILE.  Rows that a caller
    pads x with give rows of out that mean nothing.  For products too small to fill the device on their own."""
    _cuda(x, w, out)
    G, R, K = x.shape
    N = out.shape[2]
    assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and x.is_contiguous() and out.is_contiguous() and w.stride(1) == 1
    assert w.shape == (G * N, K) and out.shape == (G, R, N) and R % GROUPED_TILE == 0
    call("gb_gemm_tc_grouped", ptr(x), x.stride(1), ptr(w), w.stride(0), ptr(out), out.stride(1), G, R, N, K, tc_scratch(x.device).sms,
         stream_ptr())
    return out


def attention_decode_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_decode_supported(head_dim, dtype_code(kcache), dtype_code(q)))


SPLIT_CLASSES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128)


def _split_class(n: int) -> int:
    return max(c for c in SPLIT_CLASSES if c <= max(n, 1))


def decode_split_class(max_kv: int) -> int:
    """The class of a step whose longest sequence has max_kv positions: a quarter of its pages, rounded down
    to one of a few values.  Steps of one class split their sequences' pages in the same way (decode_splits),
    and a captured graph is made per class."""
    return _split_class(((max_kv + 63) // 64) // 4)


def decode_split_class_cuda(max_kv: int) -> int:
    """The same for the CUDA-core decode kernel, whose splits (decode_splits with mma False) follow an eighth of the pages."""
    return _split_class(((max_kv + 63) // 64) // 8)


def decode_split_class_exact(max_kv: int) -> int:
    """Class of a decode step of the normalised attention on the CUDA-core decode kernel: half of the pages."""
    return _split_class(((max_kv + 63) // 64) // 2)


def decode_splits_exact(T: int, n_heads: int, n_kv_heads: int, max_kv: int, sms: int) -> int:
    """Splits of each sequence's pages for that kernel: two pages or more per split while all CTAs fit the device at
    once with two per SM (the rule of decode_splits leaves a step of 8 sequences of 512 positions at 32 CTAs)."""
    group = n_heads // n_kv_heads
    tile = 8 if group >= 8 else 4 if group > 2 else group
    ctas = T * n_kv_heads * ((group + tile - 1) // tile)
    return max(1, min(decode_split_class_exact(max_kv), 32, (2 * sms) // ctas))


def decode_splits(T: int, n_heads: int, n_kv_heads: int, max_kv: int, sms: int, mma: bool) -> int:
    """Splits of each sequence's pages for a decode step; a function of the step's class (decode_split_class)
    and its CTAs, so that all steps of a captured graph split alike.

    The tensor-core kernels split only while the step keeps to one CTA per SM, where the kernel of twelve warps
    runs (measured against the kernels of many CTAs with more splits at 8 to 16 sequences of 1,000 to 8,000
    positions: 17.5 instead of 21.1 us, 26.9 instead of 31.1, 14.8 instead of 20.5).  Few CTAs (a quarter of the
    SMs or fewer) are bound by what one SM can read and spread out: splits of at least 4 pages, at most 8 of them.
    More CTAs pay more for merging than they gain below about 12 pages per split.  Sequences of less than 16 pages
    are never split.  The CUDA-core kernel splits into 8 pages or more per split while all CTAs fit the device at
    once with two per SM."""
    group = n_heads // n_kv_heads
    tile = 16 if mma else (8 if group >= 8 else 4 if group > 2 else group)
    ctas = T * n_kv_heads * ((group + tile - 1) // tile)
    pages = (max_kv + 63) // 64
    if not mma:
        return max(1, min(decode_split_class_cuda(max_kv), 32, (2 * sms) // ctas))
    cls = decode_split_class(max_kv)                       # a quarter of the pages, rounded down to a class
    if ctas > sms or cls < 4:
        return 1
    room = sms // ctas
    if 4 * ctas <= sms:
        return _split_class(min(room, 8, cls))
    return _split_class(min(room, cls // 3))


def attention_decode_mma_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_decode_mma_supported(head_dim, dtype_code(kcache), dtype_code(q)))


def attention_decode(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, ring_pages: int,
                     kcache: torch.Tensor, vcache: torch.Tensor, window: int, scale: float,
                     splits: Optional[int] = None, mma: Optional[bool] = None, max_kv: Optional[int] = None,
                     rope: Optional[tuple] = None, keep_first: int = 0, head_pages: int = 0,
                     gate: Optional[torch.Tensor] = None, sink: bool = False, sink_values: Optional[torch.Tensor] = None,
                     chunk: int = 0) -> torch.Tensor:
    """One token per sequence over the bf16 cache; all heads of a group share one pass over
    the keys and values.  mma: the tensor-core kernel (head sizes 64 and 128; the default
    where it fits) or the CUDA-core one (any head size that is a multiple of 16).
    rope = (k, v, inv_freq, rotary_dim, pairing), tensor-core kernel only: q, k and v are the
    unrotated projections; the kernel rotates q and k and writes k and v into the cache itself
    (k and v None: it reads another run's cache and only rotates q).
    keep_first, head_pages, gate, sink, sink_values, chunk (CUDA-core kernel only): as attention_generic."""
    _cuda(q, out, seq_of, pos, table, kcache, vcache, gate, sink_values)
    assert sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == n_heads and sink_values.is_contiguous())
    sink = bool(sink) or sink_values is not None
    kept = bool(keep_first or head_pages or gate is not None or sink or chunk)
    assert not kept or (mma is False and rope is None)
    assert gate is None or gate.dtype == torch.bfloat16
    per_head = _gate_per_head(gate, out, n_heads)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * head_dim)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    lib = native.library()
    sc = tc_scratch(q.device)
    if mma is None:
        mma = attention_decode_mma_supported(q, kcache, head_dim)
    entry = "gb_attention_decode_mma" if mma else "gb_attention_decode"
    if splits is None:
        splits = decode_splits(T, n_heads, n_kv_heads, max_kv if max_kv else table.shape[1] * 64, sc.sms, mma)
    need = lib.gb_attention_decode_scratch_floats(T, n_heads, head_dim, splits)
    scratch = counters = None
    if need:
        scratch, counters = sc.floats, sc.counters
        if T * n_heads > sc.COUNTERS or not sc.fits(need):
            splits, scratch, counters = 1, None, None
    if rope is not None:
        k, v, inv_freq, rotary_dim, pairing = rope
        _cuda(k, v, inv_freq)
        assert mma and (k is None or (k.stride(0) == q.stride(0) and v.stride(0) == q.stride(0) and k.dtype == q.dtype))
        call("gb_attention_decode_mma_rope", ptr(q), ptr(k), ptr(v), q.stride(0), ptr(out), out.stride(0), T, n_heads,
             n_kv_heads, head_dim, rotary_dim, pairing, ptr(inv_freq), ptr(seq_of), ptr(pos), ptr(table), table.shape[1],
             ring_pages, ptr(kcache), ptr(vcache), int(window or 0), float(scale), splits, ptr(scratch), ptr(counters),
             0 if counters is None else counters.numel(), stream_ptr())
        return out
    if kept:
        call("gb_attention_decode_kept", ptr(q), q.stride(0), ptr(out), out.stride(0), T, n_heads, n_kv_heads, head_dim,
             ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages, ptr(kcache), ptr(vcache), int(window or 0),
             float(scale), splits, ptr(scratch), ptr(counters), 0 if counters is None else counters.numel(), int(head_pages),
             int(keep_first or 0), ptr(gate), 0 if gate is None else gate.stride(0), int(per_head), int(bool(sink)),
             ptr(sink_values), int(chunk or 0), stream_ptr())
        return out
    call(entry, ptr(q), q.stride(0), ptr(out), out.stride(0), T, n_heads, n_kv_heads, head_dim,
         ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages, ptr(kcache), ptr(vcache), int(window or 0),
         float(scale), splits, ptr(scratch), ptr(counters), 0 if counters is None else counters.numel(), stream_ptr())
    return out


def attention_prefill_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_prefill_supported(head_dim, dtype_code(kcache), dtype_code(q)))


def attention_prefill_tiles(qlens) -> list:
    """(sequence row, first query) of every tile of queries, flat, for the step's sequences."""
    bm = native.library().gb_attention_prefill_tile()
    tiles = [(b, q0) for b, n in enumerate(qlens) for q0 in range(0, n, bm)]
    # the later queries of a sequence see more keys: their tiles start first, so that the last CTAs to
    # start are the short ones (the order changes no result)
    tiles.sort(key=lambda t: -t[1])
    flat = []
    for b, q0 in tiles:
        flat += [b, q0]
    return flat


def attention_prefill_tc_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_prefill_tc_supported(head_dim, dtype_code(kcache), dtype_code(q))) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0


def attention_prefill(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      tiles: torch.Tensor, cu: torch.Tensor, starts: torch.Tensor, qlens: torch.Tensor,
                      table: torch.Tensor, ring_pages: int, kcache: torch.Tensor, vcache: torch.Tensor, window: int,
                      scale: float, tc: Optional[bool] = None, exact: bool = False, keep_first: int = 0, head_pages: int = 0,
                      gate: Optional[torch.Tensor] = None, sink: bool = False, sink_values: Optional[torch.Tensor] = None,
                      chunk: int = 0) -> torch.Tensor:
    """Many tokens per sequence over the bf16 cache (which already holds their keys and
    values), flash style.  tc: both products on tcgen05 with S and PV in TMEM (the default where it
    fits), else on mma.sync; both take head sizes 64 and 128.  exact (mma.sync kernel only): the
    attention weights stay 32-bit, split into three bfloat16 terms for the product with the values.
    keep_first, head_pages, gate, sink, sink_values, chunk (mma.sync kernel only): as attention_generic."""
    _cuda(q, out, tiles, cu, starts, qlens, table, kcache, vcache, gate, sink_values)
    assert sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == n_heads and sink_values.is_contiguous())
    sink = bool(sink) or sink_values is not None
    assert gate is None or gate.dtype == torch.bfloat16
    per_head = _gate_per_head(gate, out, n_heads)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (q.shape[0], n_heads * head_dim)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    plain = not (exact or keep_first or head_pages or gate is not None or sink or chunk)
    if tc is None:
        tc = attention_prefill_tc_supported(q, kcache, head_dim) and plain
    assert not tc or plain
    if tc:
        assert kcache.is_contiguous() and vcache.is_contiguous()
        call("gb_attention_prefill_tc", ptr(q), q.stride(0), ptr(out), out.stride(0), q.shape[0], n_heads, n_kv_heads,
             head_dim, ptr(tiles), tiles.numel() // 2, ptr(cu), ptr(starts), ptr(qlens), ptr(table), table.shape[1],
             ring_pages, ptr(kcache), ptr(vcache), kcache.shape[0], int(window or 0), float(scale), stream_ptr())
        return out
    call("gb_attention_prefill", ptr(q), q.stride(0), ptr(out), out.stride(0), n_heads, n_kv_heads, head_dim, ptr(tiles),
         tiles.numel() // 2, ptr(cu), ptr(starts), ptr(qlens), ptr(table), table.shape[1], ring_pages, ptr(kcache),
         ptr(vcache), int(window or 0), float(scale), int(bool(exact)), int(head_pages), int(keep_first or 0), ptr(gate),
         0 if gate is None else gate.stride(0), int(per_head), int(bool(sink)), ptr(sink_values), int(chunk or 0), stream_ptr())
    return out


def tc_status() -> int:
    """Non-zero when a bounded wait inside a tensor-core kernel gave up (read after a
    synchronise)."""
    return native.library().gb_tc_status()


def check_tc_status() -> None:
    lib = native.library()
    code = tc_status()
    if code:
        lib.gb_tc_status_clear()
        for sc in _tc_scratch.values():              # a kernel that gave up may have left a tile's counter half counted
            sc.counters.zero_()
        raise native.NativeError(f"a tensor-core product gave up waiting (code {code}: 1 a stage never came free, "
                                 f"2 a load never arrived, 3/4 an accumulator never completed, 5 a CTA that shares a tile never arrived); "
                                 f"its output is invalid")
    code = lib.gb_attention_tc_status()
    if code:
        lib.gb_attention_tc_status_clear()
        raise native.NativeError(f"the tensor-core attention kernel gave up waiting (code {code}); its output is invalid")


# ------------------------------------------------------------------ dispatch
def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """The product path of every projection: the tensor-core kernel when dtype and sizes
    fit it, else the CUDA-core kernel."""
    if gemm_tc_supported(x, w):
        return gemm_tc(x, w, bias, out)
    return gemm_generic(x, w, bias, out)


def decode_rotates(ctx, q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    """Whether this step's attention kernel rotates q and k and writes the cache itself (a step of single
    tokens on the tensor-core decode kernel), so that no separate rotation kernel runs before it."""
    return bool(ctx.decode) and attention_decode_supported(q, kcache, head_dim) and \
        attention_decode_mma_supported(q, kcache, head_dim)


def attention(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, ctx, table: torch.Tensor,
              ring_pages: int, kcache: torch.Tensor, vcache: torch.Tensor, window: int, scale: float,
              rope: Optional[tuple] = None, tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one step over the cache; picks the kernel for the step's shape.  rope: see
    attention_decode; allowed where decode_rotates() says so (q, k and v then come unrotated).
    tiles: attention_prefill_tiles() of the step's sequences on the device (prompts on the tiled kernels)."""
    if rope is not None:
        assert decode_rotates(ctx, q, kcache, head_dim)
    if ctx.decode and attention_decode_supported(q, kcache, head_dim):
        return attention_decode(q, out, n_heads, n_kv_heads, head_dim, ctx.seq_of, ctx.pos, table, ring_pages, kcache,
                                vcache, window, scale, max_kv=min(ctx.max_kv, window) if window else ctx.max_kv,
                                mma=True if rope is not None else None, rope=rope)
    if not ctx.decode and tiles is not None and attention_prefill_supported(q, kcache, head_dim):
        return attention_prefill(q, out, n_heads, n_kv_heads, head_dim, tiles, ctx.cu, ctx.starts, ctx.qlens, table,
                                 ring_pages, kcache, vcache, window, scale)
    return attention_generic(q, out, n_heads, n_kv_heads, head_dim, ctx.seq_of, ctx.pos, table, ring_pages, kcache,
                             vcache, window, scale)
