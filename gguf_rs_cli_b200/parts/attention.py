"""Grouped-query causal attention over the cache, as the mixer of a layer:
q, k, v projections (+ biases before the rotation, src/model/llama.rs:364-369), rotation
of q and k and the cache write in one kernel (src/model/llama.rs:370-373), attention
over the cached positions (src/model/llama.rs:374-394), output projection
(src/model/llama.rs:395).  q, k and v are one matrix after loading.

A window (not in the reference) limits each token to the last `window` positions and
gives the layer a cache group of its own kind.  With `shares_kv`, the mixer has no k
and v of its own and reads the cache of the run its schedule entry names.

Three further options, none in the reference, for designs that bring positions in without a
rotation: values of another size than keys (`v_head_dim`); queries and keys divided by their
root mean square per head, without a weight (`qk_norm_eps`); and a query temperature that grows
with the position, q <- q (1 + coef ln(floor((p + 1) / every) + 1)) (`q_temp`).  With any of them
scores, softmax and the mix of values run in 32-bit in the general attention kernel.

Further options, for designs that norm and gate their heads (they go with a rotation, and also keep scores and
weights in 32-bit): an RMS norm per head on q and k with a weight of head_dim entries that all heads share, before
the rotation (`head_norm_eps`); the first positions of a sequence that stay visible behind the window
(`keep_first`; the cache keeps their pages in front of its ring); the heads' results multiplied by
sigmoid(W_g h) before the output projection (`out_gate`); and values mixed across layers (`v_mix`): the first
layer that says so ("gives") leaves its values of the step's tokens for the later ones ("takes"), which cache
v <- (1 - lambda) v + lambda v_first with a scalar lambda of their own.

And for designs that smooth their projections over time and let a head attend to nothing: a short causal convolution
per channel on q, k and v, directly behind the projection and before the rotation, without bias or activation (`conv`
taps; the last taps - 1 projected rows are per-sequence state); a softmax whose denominator counts one more key of
score 0 that has no value (`sink`); and a gate of one number per head instead of one per entry (`out_gate="head"`).

And for designs that cut the sequence into chunks or learn their sinks: keys in chunks of `chunk` positions counted from
the sequence's start, a token seeing the earlier tokens of its own chunk only (in a window's place; the cache keeps a
ring of that many positions); a sink whose score is a learned number per head, not scaled (`sink="learned"`, tensor
`sink` [heads]); `exact=True` asks for 32-bit scores and weights where nothing else does.  These paths also take q/k/v
biases and `shares_kv` (the layer then prepares its queries only and attends to the other run's keys and values).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..cache.cache import KVSpec
from ..weights.loader import TensorRequest, WeightStore
from .base import HostBatch, Part, RunView, StepContext
from .linear import Linear
from .registry import register_mixer


@register_mixer("attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window (None or W),
    bias (q/k/v biases), shares_kv (default False), v_head_dim (default head_dim),
    qk_norm_eps (default None: no normalisation), q_temp (default None, or {"coef", "every"}),
    head_norm_eps (default None), keep_first (default 0), out_gate (default False), v_mix (None, "gives" or "takes"),
    v_mix_optional (the folder may hold the scalar although nothing is mixed), conv (default None; taps of a short
    convolution on q, k and v), sink (default False; "learned": a score per head from the tensor `sink`), out_gate "head":
    one gate per head, chunk (None or C: chunks of C positions in a window's place), exact (default False), cache_span
    (when present: the positions the cache keeps, None for all, where runs with windows of their own share one cache).
    tensors: q [nh*hd, E], k [nkv*hd, E], v [nkv*vd, E], o [E, nh*vd], optional q_bias, k_bias, v_bias;
    with head_norm_eps q_norm, k_norm [hd]; with out_gate g [nh*vd, E] ("head": [nh, E]); with v_mix the scalar v_mix;
    with conv q_conv, k_conv, v_conv [channels, taps]."""

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.nh, self.nkv, self.hd = p["num_heads"], p["num_kv_heads"], p["head_dim"]
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} KV heads")
        self.scale = float(p.get("scale") or self.hd ** -0.5)
        self.window = p.get("window") or None
        self.shares_kv = bool(p.get("shares_kv", False))
        self.position = position
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.qk_norm_eps = p.get("qk_norm_eps")
        temp = p.get("q_temp") or None
        self.temp_coef, self.temp_every = (float(temp["coef"]), int(temp["every"])) if temp else (0.0, 1)
        if temp and self.temp_every <= 0:
            raise ValueError(f"attention: q_temp.every must be a positive whole number, got {temp['every']!r}")
        self.head_norm_eps = p.get("head_norm_eps")
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.out_gate = bool(p.get("out_gate", False))
        self.gate_per_head = p.get("out_gate") == "head"
        self.conv = int(p.get("conv") or 1)
        if not 1 <= self.conv <= 16:
            raise ValueError(f"attention: a convolution of {self.conv} taps is not supported (1..16)")
        self.sink = bool(p.get("sink", False))
        self.sink_learned = p.get("sink") == "learned"
        self.chunk = int(p.get("chunk") or 0)
        if self.chunk and (self.window or p.get("keep_first")):
            raise ValueError("attention: chunks go with neither a window nor kept first positions")
        self.v_mix = p.get("v_mix") or None
        if self.v_mix not in (None, "gives", "takes"):
            raise ValueError(f"attention: v_mix {self.v_mix!r} is not one of None, 'gives', 'takes'")
        # heads with a norm of their own, a gate, kept first positions or mixed values: prepared by one kernel
        # (norm, rotation, mixing, cache write) and attended to with 32-bit weights
        self.prepared = bool(self.head_norm_eps is not None or self.keep_first or self.out_gate or self.v_mix or self.conv > 1
                             or self.sink or self.chunk or p.get("exact"))
        # where the parts of the fused projection start: q, k, v and the gate, each at a multiple of 8 rows
        self.off, rows = {}, 0
        own = 0 if self.shares_kv else 1
        for n, size in (("q", self.nh * self.hd), ("k", own * self.nkv * self.hd), ("v", own * self.nkv * self.vd),
                        ("g", (self.nh if self.gate_per_head else self.nh * self.vd) if self.out_gate else 0)):
            self.off[n] = (rows + 7) // 8 * 8
            rows = self.off[n] + size
        self.gate_rows = rows - self.off["g"]
        self.conv_channels = self.off["v"] + own * self.nkv * self.vd      # q, k, v and the empty rows between them
        # normalised q and k, a query temperature or values of their own size: the exact path
        self.exact = self.prepared or self.vd != self.hd or self.qk_norm_eps is not None or self.temp_coef != 0.0
        if self.prepared and (self.qk_norm_eps is not None or self.temp_coef != 0.0):
            raise ValueError("attention: head_norm_eps, keep_first, out_gate, v_mix, conv, sink, chunk and exact go with neither "
                             "qk_norm_eps nor q_temp")
        if self.shares_kv and self.v_mix:
            raise ValueError("attention: a layer that reads another's keys and values has no values to mix")
        if self.exact and not self.prepared and (position is not None or self.shares_kv):
            raise ValueError("attention: qk_norm_eps, q_temp and v_head_dim go with neither a rotation nor shares_kv")

    def kv_spec(self) -> Optional[KVSpec]:
        return None if self.shares_kv else self.reads_kv_spec()

    def reads_kv_spec(self) -> KVSpec:
        """The kind of cache this mixer can read (its own, or another run's)."""
        # how many of the last positions the cache keeps: this layer's own reach, or `cache_span` where runs with other
        # windows read the same keys (None: all positions)
        span = self.p["cache_span"] if "cache_span" in self.p else (self.window or self.chunk or None)
        return KVSpec(self.nkv, self.hd, span, None if self.vd == self.hd else self.vd, self.keep_first)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"conv": ((self.conv - 1, self.conv_channels), "float32")} if self.conv > 1 else {}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t = self.p["hidden_size"], self.spec.tensors
        names = ["q"] + ([] if self.shares_kv else ["k", "v"])
        rows = {"q": self.nh * self.hd, "k": self.nkv * self.hd, "v": self.nkv * self.vd}
        req = [TensorRequest(t[n], (rows[n], E)) for n in names]
        req.append(TensorRequest(t["o"], (E, self.nh * self.vd)))
        if self.p.get("bias"):
            req += [TensorRequest(t[n + "_bias"], (rows[n],)) for n in names]
        if self.head_norm_eps is not None:
            req += [TensorRequest(t["q_norm"], (self.hd,), init="ones"), TensorRequest(t["k_norm"], (self.hd,), init="ones")]
        if self.out_gate:
            req.append(TensorRequest(t["g"], (self.gate_rows, E)))
        if self.conv > 1:
            req += [TensorRequest(t[n + "_conv"], (rows[n], self.conv), init="uniform:-0.6:0.6") for n in names]
        if self.sink_learned:
            req.append(TensorRequest(t["sink"], (self.nh,), init="uniform:-1:1"))
        if self.v_mix or self.p.get("v_mix_optional"):
            req.append(TensorRequest(t["v_mix"], (), optional=not self.v_mix, init="const:0.25" if self.v_mix else None))
        return req

    def load(self, store: WeightStore) -> None:
        req = {r.name: r for r in self.tensor_requests()}
        t = self.spec.tensors
        if self.prepared:
            return self._load_prepared(store, req)
        names = ["q"] + ([] if self.shares_kv else ["k", "v"])
        mats = [store.get(req[t[n]]) for n in names]
        dt = mats[0].dtype
        w = torch.cat([m.to(dt) for m in mats], dim=0) if len(mats) > 1 else mats[0]
        b = None
        if self.p.get("bias"):
            b = torch.cat([store.get(req[t[n + "_bias"]]).to(torch.float32) for n in names], dim=0)
        self.qkv = Linear(w, b, name="attn.qkv")
        self.o = Linear(store.get(req[t["o"]]), name="attn.o")

    def _load_prepared(self, store: WeightStore, req) -> None:
        """q, k, v and the gate as one matrix, each part starting at a multiple of 8 rows (zero rows between), so that
        one product reads h once and every slice of its result is aligned."""
        t = self.spec.tensors
        names = ["q"] + ([] if self.shares_kv else ["k", "v"]) + (["g"] if self.out_gate else [])
        mats = [store.get(req[t[n]]) for n in names]
        dt = mats[0].dtype
        total = (self.off["g"] + self.gate_rows + 7) // 8 * 8
        bias = None
        if self.p.get("bias"):
            bias = torch.zeros(total, dtype=torch.float32, device=mats[0].device)
            for n in names:
                if n != "g":
                    b = store.get(req[t[n + "_bias"]])
                    bias[self.off[n]:self.off[n] + b.numel()] = b.to(torch.float32)
        self.sink_values = store.get(req[t["sink"]]).to(torch.float32).contiguous() if self.sink_learned else None
        parts, rows = [], 0
        for n, m in zip(names, mats):
            pad = self.off[n] - rows
            if pad:
                parts.append(torch.zeros(pad, m.shape[1], dtype=dt, device=m.device))
            parts.append(m.to(dt))
            rows = self.off[n] + m.shape[0]
        pad = (rows + 7) // 8 * 8 - rows
        if pad:
            parts.append(torch.zeros(pad, mats[0].shape[1], dtype=dt, device=mats[0].device))
        self.qkv = Linear(torch.cat(parts, dim=0).contiguous(), bias, name="attn.qkvg")
        self.o = Linear(store.get(req[t["o"]]), name="attn.o")
        self.q_norm = self.k_norm = None
        if self.head_norm_eps is not None:
            self.q_norm, self.k_norm = store.get(req[t["q_norm"]]), store.get(req[t["k_norm"]])
            if self.q_norm.dtype != self.k_norm.dtype:
                self.k_norm = self.k_norm.to(self.q_norm.dtype)
        self.taps = self.taps_t = None
        if self.conv > 1:
            # one convolution over all columns of q, k and v; the empty rows between them have taps of zero
            self.taps = torch.zeros(self.conv_channels, self.conv, dtype=dt, device=mats[0].device)
            for n in (n for n in names if n != "g"):
                w = store.get(req[t[n + "_conv"]])
                self.taps[self.off[n]:self.off[n] + w.shape[0]] = w.to(dt)
            self.taps_t = self.taps.t().contiguous() if dt == torch.bfloat16 else None
        self.mix = 0.0
        if self.v_mix == "takes":
            lam = store.get(req[t["v_mix"]])
            self.mix = float(lam.float().item()) if lam.device.type != "meta" else 0.0

    accepts_residual = True

    # ---- planning on the host
    def plan_key(self):
        return ("attention", self.hd, self.vd, self.window, self.exact, self.prepared, self.keep_first, self.chunk, self.sink_learned)

    def plan(self, batch: HostBatch):
        """Prompts: the list of query tiles (sequence row, first query) that the prefill kernel's CTAs take."""
        if batch.decode or (self.exact and not self._exact_tiled()):
            return {}
        return {"tiles": kernels.attention_prefill_tiles(batch.qlens)}

    def _exact_tiled(self) -> bool:
        """Whether prompts of the exact path take the tiled kernel (bfloat16, keys and values of 64 or 128 entries
        both) with 32-bit attention weights; other sizes and the 32-bit mode take the general kernel."""
        return self.dtype == torch.bfloat16 and self.vd == self.hd and self.hd in (64, 128) and self._fast_masks()

    def _fast_masks(self) -> bool:
        """Whether the tiled and the decode kernel know this layer's mask and sink."""
        return True

    def _exact_decode(self) -> bool:
        """Whether single tokens of the exact path take the CUDA-core decode kernel (32-bit weights; bfloat16, keys
        and values of one size that is a multiple of 16 up to 256)."""
        return self.dtype == torch.bfloat16 and self.vd == self.hd and self.hd % 16 == 0 and self.hd <= 256 and self._fast_masks()

    def graph_class(self, batch: HostBatch):
        """The decode kernel splits each sequence's pages over CTAs by a rule of the longest sequence; steps
        of one class launch the same grid and may share a captured graph."""
        if self.exact:
            # the general kernel: one block per token and head, whatever the lengths; the CUDA-core decode kernel
            # splits each sequence's pages by a rule of the longest sequence
            return ("cuda", kernels.decode_split_class_exact(self._longest_seen(batch.max_kv))) if self._exact_decode() else ()
        return kernels.decode_split_class(min(batch.max_kv, self.window) if self.window else batch.max_kv)

    def _longest_seen(self, max_kv: int) -> int:
        """The most keys a token of a sequence of max_kv positions can see."""
        if self.window:
            return min(max_kv, self.window + self.keep_first)
        return min(max_kv, self.chunk) if self.chunk else max_kv

    def absorb_input_norm(self, weight: torch.Tensor) -> bool:
        """Multiplies the weight of the norm in front of this mixer into the q/k/v matrix, where
        the tensor-core product (which can apply the norm's per-token scale) will run it."""
        if not self.qkv.tensor_core():
            return False
        self.qkv.fold_input_scale(weight)
        return True

    V_FIRST = "attention.v_first"          # where the layer that gives its values leaves them for the step's later layers

    def _forward_prepared(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        """One product for q, k, v and the gate; one kernel for the heads' norm, the rotation, the mixing of values and
        the cache write; attention with 32-bit scores and weights behind the window and the kept first positions, its
        result gated; the output projection in 32-bit results."""
        nh, nkv, hd, vd, T = self.nh, self.nkv, self.hd, self.vd, h.shape[0]
        proj = self.qkv(h, ctx)
        ctx.mark("qkv")
        off = self.off
        gate = proj[:, off["g"]:off["g"] + self.gate_rows] if self.out_gate else None
        if self.conv > 1:
            conv = ctx.ws.get("attn.conv", (T, self.conv_channels), proj.dtype)
            kernels.short_conv(proj[:, :self.conv_channels], self.taps, ctx.state(f"run{run.index}.conv"), ctx, conv,
                               taps_t=self.taps_t)
            proj = conv
            ctx.mark("conv")
        q = proj[:, off["q"]:off["q"] + nh * hd]
        k = v = None                         # a layer that reads another run's cache prepares its queries only
        if not self.shares_kv:
            k, v = proj[:, off["k"]:off["k"] + nkv * hd], proj[:, off["v"]:off["v"] + nkv * vd]
        v_first = first_out = None
        if self.v_mix == "gives":
            first_out = ctx.shared[self.V_FIRST] = ctx.ws.get("attn.v_first", (T, nkv * vd), proj.dtype)
        elif self.v_mix == "takes":
            v_first = ctx.shared.get(self.V_FIRST)
            if v_first is None or v_first.shape != (T, nkv * vd):
                raise RuntimeError("attention: no earlier layer of this step has left values of this size to mix with")
        table, pos = ctx.tables[run.group], self.position
        kernels.head_prep_kv_write(q, k, v, nh, nkv, hd, vd, self.q_norm, self.k_norm, self.head_norm_eps or 1.0,
                                   None if pos is None else pos.inv_freq, 0 if pos is None else pos.rotary_dim,
                                   0 if pos is None else pos.pairing, v_first, self.mix, first_out, ctx.seq_of, ctx.pos, table,
                                   run.ring_pages, run.head_pages, run.k, run.v)
        ctx.mark("heads")
        out = ctx.ws.get("attn.out", (T, nh * vd), ctx.dtype)
        tiles = ctx.plan_of(self).get("tiles")
        kept = dict(keep_first=self.keep_first, head_pages=run.head_pages, gate=gate, sink=self.sink, sink_values=self.sink_values,
                    chunk=self.chunk)
        if not ctx.decode and tiles is not None and self._exact_tiled() and kernels.attention_prefill_supported(q, run.k, hd):
            # prompts, keys and values of 64 or 128 entries: the tiled kernel with 32-bit weights
            kernels.attention_prefill(q, out, nh, nkv, hd, tiles, ctx.cu, ctx.starts, ctx.qlens, table, run.ring_pages,
                                      run.k, run.v, self.window or 0, self.scale, tc=False, exact=True, **kept)
        elif ctx.decode and self._exact_decode() and kernels.attention_decode_supported(q, run.k, hd):
            # single tokens: one pass over a token's keys serves the heads of a group, 32-bit weights
            max_kv = self._longest_seen(ctx.max_kv)
            splits = kernels.decode_splits_exact(T, nh, nkv, max_kv, kernels.tc_scratch(q.device).sms)
            kernels.attention_decode(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                     self.window or 0, self.scale, mma=False, max_kv=max_kv, splits=splits, **kept)
        else:
            kernels.attention_generic(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                      self.window or 0, self.scale, v_dim=vd, **kept)
        ctx.mark("attention")
        term = self.o(out, ctx, out_dtype=torch.float32)
        ctx.mark("o")
        return term

    def forward(self, h, ctx: StepContext, run: RunView, residual=None) -> Optional[torch.Tensor]:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        if self.prepared:
            return self._forward_prepared(h, ctx, run)
        qkv = self.qkv(h, ctx)
        ctx.mark("qkv")
        if self.exact:
            return self._forward_exact(qkv, ctx, run, residual)
        q = qkv[:, :nh * hd]
        k = v = None
        if not self.shares_kv:
            k, v = qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
        table = ctx.tables[run.group]
        pos = self.position
        inv_freq = None if pos is None else pos.inv_freq
        rotary_dim, pairing = (0, 0) if pos is None else (pos.rotary_dim, pos.pairing)
        rope = None
        if kernels.decode_rotates(ctx, q, run.k, hd):
            rope = (k, v, inv_freq, rotary_dim, pairing)         # single tokens: the attention kernel rotates and writes
        else:
            kernels.rope_kv_write(q, k, v, nh, nkv, hd, inv_freq, rotary_dim, pairing, ctx.seq_of, ctx.pos, table,
                                  run.ring_pages, run.k if k is not None else None, run.v if k is not None else None)
        out = ctx.ws.get("attn.out", (h.shape[0], nh * hd), ctx.dtype)
        kernels.attention(q, out, nh, nkv, hd, ctx, table, run.ring_pages, run.k, run.v, self.window or 0, self.scale,
                          rope=rope, tiles=ctx.plan_of(self).get("tiles"))
        ctx.mark("attention")
        term = self.o(out, ctx, residual=residual)
        ctx.mark("o")
        return term

    def _forward_exact(self, qkv, ctx: StepContext, run: RunView, residual) -> Optional[torch.Tensor]:
        """q and k to unit root mean square, the query temperature and the cache write in one kernel, then
        attention with 32-bit scores and weights over keys of hd and values of vd entries."""
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
        table = ctx.tables[run.group]
        kernels.qk_norm_kv_write(q, k, v, nh, nkv, hd, vd, self.qk_norm_eps is not None, self.qk_norm_eps or 1.0,
                                 self.temp_coef, self.temp_every, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v)
        out = ctx.ws.get("attn.out", (qkv.shape[0], nh * vd), ctx.dtype)
        tiles = ctx.plan_of(self).get("tiles")
        if not ctx.decode and tiles is not None and self._exact_tiled() and kernels.attention_prefill_supported(q, run.k, hd):
            kernels.attention_prefill(q, out, nh, nkv, hd, tiles, ctx.cu, ctx.starts, ctx.qlens, table, run.ring_pages,
                                      run.k, run.v, self.window or 0, self.scale, tc=False, exact=True)
        elif ctx.decode and self._exact_decode() and kernels.attention_decode_supported(q, run.k, hd):
            max_kv = min(ctx.max_kv, self.window) if self.window else ctx.max_kv
            splits = kernels.decode_splits_exact(q.shape[0], nh, nkv, max_kv, kernels.tc_scratch(q.device).sms)
            kernels.attention_decode(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                     self.window or 0, self.scale, mma=False, max_kv=max_kv, splits=splits)
        else:
            kernels.attention_generic(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                      self.window or 0, self.scale, v_dim=vd)
        ctx.mark("attention")
        term = self.o(out, ctx, residual=residual)
        ctx.mark("o")
        return term
