"""Latent attention as the mixer of a layer: keys and values of all heads are products of one latent row
per position, c = rms_norm(W_dkv h)[:kv_rank] * w, plus one rotated key part of rot_dim entries that all
heads share; only these kv_rank + rot_dim numbers per position are cached.

Per head the score is (q_plain . W_uk c + q_rot . k_rot) * scale and the value W_uv c.  The products
with W_uk and W_uv are moved to the query's side: q' = W_uk^T q_plain lives in the latent's space, so a
head's score is [q', q_rot] . [c, k_rot], the mix of values is the mix of latent rows, and W_uv is applied
to that mix once per token.  The attention kernel then sees one key/value head of kv_rank + rot_dim entries
whose first kv_rank entries are also its values.  Scores, softmax and mix run in 32-bit.

Prompts that start their sequences take the other order where the sizes allow it (bfloat16, dim + rot_dim
= vdim = 64 or 128): the step's latent rows are multiplied with W_uk and W_uv in one tensor-core product,
the per-head keys [W_uk c, k_rot] and values are laid out as pages of the step's own, and the tiled
attention kernel runs over them with 32-bit weights; the cache still receives the latent rows only.

Options: a window of the last `window` positions (the cache then keeps a ring of pages); a sink, one more key without a
value in the softmax's denominator whose score is a learned number per head, not scaled (`sink="learned"`, tensor `sink`
[heads]); one sigmoid gate per head on the heads' results, from a projection of the mixer's input (`out_gate="head"`,
tensor `g` [heads, E]; a number per head commutes with W_uv, so it is applied to the mix of latent rows).  The rotation
pairs neighbours or halves, as the position table says.
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


@register_mixer("latent_attention")
class LatentAttention(Part):
    """params: hidden_size, heads, dim (unrotated q/k entries per head), rot_dim (rotated ones, behind them), vdim,
    kv_rank, scale, eps (of the latent's norm), window (default None), sink (default None; "learned"), out_gate (default
    None; "head").  position: a rotary table over the rot_dim part (its first rotary_dim entries are rotated, in the
    table's pairing).
    tensors: q [heads*(dim+rot_dim), E], dkv [kv_rank+rot_dim, E], dkv_norm [kv_rank], uk [heads*dim, kv_rank],
    uv [heads*vdim, kv_rank], o [E, heads*vdim]; with a sink `sink` [heads]; with a gate g [heads, E]."""

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.H, self.D, self.R, self.Dv, self.C = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
        self.position = position
        if self.R % 2:
            raise ValueError(f"latent_attention: rot_dim {self.R} must be even")
        if position is not None and position.rotary_dim > self.R:
            raise ValueError("latent_attention: the rotation must fit into rot_dim")
        self.halves = position is not None and position.pairing == 0
        self.window = p.get("window") or None
        if p.get("sink") not in (None, False, "learned") or p.get("out_gate") not in (None, False, "head"):
            raise ValueError("latent_attention: sink is None or 'learned', out_gate None or 'head'")
        self.sink, self.gated = p.get("sink") == "learned", p.get("out_gate") == "head"

    def kv_spec(self) -> Optional[KVSpec]:
        return KVSpec(1, self.C + self.R, self.window, 0)

    def reads_kv_spec(self) -> KVSpec:
        return self.kv_spec()

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t = self.p["hidden_size"], self.spec.tensors
        H, D, R, Dv, C = self.H, self.D, self.R, self.Dv, self.C
        req = [TensorRequest(t["q"], (H * (D + R), E)), TensorRequest(t["dkv"], (C + R, E)),
               TensorRequest(t["dkv_norm"], (C,), init="ones"), TensorRequest(t["uk"], (H * D, C)),
               TensorRequest(t["uv"], (H * Dv, C)), TensorRequest(t["o"], (E, H * Dv))]
        if self.sink:
            req.append(TensorRequest(t["sink"], (H,), init="uniform:-1:1"))
        if self.gated:
            req.append(TensorRequest(t["g"], (H, E)))
        return req

    def load(self, store: WeightStore) -> None:
        got = [store.get(r) for r in self.tensor_requests()]
        q, dkv, norm, uk, uv, o = got[:6]
        H, D, R, Dv, C = self.H, self.D, self.R, self.Dv, self.C
        self.sink_values = got[6].to(torch.float32).contiguous() if self.sink else None
        # q, the down-projection and the gate as one matrix, each part starting at a multiple of 8 rows
        parts, rows = [], 0
        self.off_dkv = self.off_g = 0
        for name, m in (("q", q), ("dkv", dkv)) + ((("g", got[-1]),) if self.gated else ()):
            at = (rows + 7) // 8 * 8
            if at > rows:
                parts.append(torch.zeros(at - rows, q.shape[1], dtype=q.dtype, device=q.device))
            if name == "dkv":
                self.off_dkv = at
            elif name == "g":
                self.off_g = at
            parts.append(m.to(q.dtype))
            rows = at + m.shape[0]
        if rows % 8:                      # rows of the result that start on 16 bytes, whatever the parts' sizes
            parts.append(torch.zeros(8 - rows % 8, q.shape[1], dtype=q.dtype, device=q.device))
        self.proj = Linear(torch.cat(parts, dim=0).contiguous(), name="latent.proj")
        self.norm_weight = norm
        self.uk = uk.reshape(H, D, C).contiguous()                           # q' = q_plain W_uk[h]: [in D, out C]
        self.uv_t = uv.reshape(H, Dv, C).transpose(1, 2).contiguous()        # value = mix W_uv[h]^T: [in C, out Dv]
        self.kv_up = Linear(torch.cat([uk, uv.to(uk.dtype)], dim=0).contiguous(), name="latent.kv") if self._tiled() else None
        self.o = Linear(o, name="latent.o")

    def _tiled(self) -> bool:
        """Whether prompts can take the tiled attention kernel over per-head keys and values."""
        return self.dtype == torch.bfloat16 and self.D + self.R == self.Dv and self.Dv in (64, 128)

    # ---- planning on the host
    def plan_key(self):
        return ("latent_attention", self.D, self.R, self.Dv, self._tiled(), self.window, self.sink, self.gated)

    def plan(self, batch: HostBatch):
        """Prompts that start their sequences, where the tiled kernel fits: its list of query tiles, and a page table
        of the step's own (sequence b's tokens lie in pages of their own, numbered from 0 on across the step)."""
        if batch.decode or not self._tiled() or any(batch.starts):
            return {}
        width = max((n + 63) // 64 for n in batch.qlens)
        table, base = [], 0
        for n in batch.qlens:
            pages = (n + 63) // 64
            table += list(range(base, base + pages)) + [0] * (width - pages)
            base += pages
        return {"tiles": kernels.attention_prefill_tiles(batch.qlens), "pages": table, "n_pages": [base]}

    accepts_residual = True

    def _fast_decode(self) -> bool:
        """Whether single tokens take the kernel that serves all heads from one pass over the latent rows."""
        return kernels.latent_decode_supported(self.H, self.C, self.R, self.dtype)

    def graph_class(self, batch: HostBatch):
        """The decode kernel splits each token's keys by a rule of the longest sequence; the general kernel launches one
        block per token and head whatever the lengths."""
        seen = min(batch.max_kv, self.window + 31) if self.window else batch.max_kv
        return ("latent", kernels.latent_decode_class(seen)) if self._fast_decode() else ()

    def forward(self, h, ctx: StepContext, run: RunView, residual=None) -> Optional[torch.Tensor]:
        H, D, R, Dv, C = self.H, self.D, self.R, self.Dv, self.C
        T = h.shape[0]
        proj = self.proj(h, ctx)
        ctx.mark("projections")
        q, dkv = proj[:, :H * (D + R)], proj[:, self.off_dkv:self.off_dkv + C + R]
        gate = proj[:, self.off_g:self.off_g + H] if self.gated else None
        more = dict(gate=gate, sink_values=self.sink_values)
        table = ctx.tables[run.group]
        pos = self.position
        plan = ctx.plan_of(self)
        if not ctx.decode and "pages" in plan and kernels.attention_prefill_supported(q, run.k, D + R):
            # per-head keys and values of this step's tokens as pages of the step's own
            row = ctx.ws.get("latent.row", (T, C + R), ctx.dtype)
            kernels.latent_prep(q, dkv, H, D, R, C, 0 if pos is None else pos.rotary_dim, None if pos is None else pos.inv_freq,
                                self.norm_weight, self.p["eps"], None, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k,
                                row_out=row, halves=self.halves)
            kv = self.kv_up(row[:, :C], ctx)
            own = plan["pages"].view(ctx.B, -1)
            n_pages = sum((n + 63) // 64 for n in ctx.host["qlens"])
            k_pages = ctx.ws.get("latent.k_pages", (n_pages, H, 64, D + R), ctx.dtype)
            v_pages = ctx.ws.get("latent.v_pages", (n_pages, H, 64, Dv), ctx.dtype)
            kernels.pack_latent_heads(kv, row, H, D, R, Dv, C, ctx.seq_of, ctx.pos, own, k_pages, v_pages)
            values = ctx.ws.get("latent.values", (T, H * Dv), ctx.dtype)
            kernels.attention_prefill(q, values, H, H, D + R, plan["tiles"], ctx.cu, ctx.starts, ctx.qlens, own, 1 << 20,
                                      k_pages, v_pages, self.window or 0, float(self.p["scale"]), tc=False, exact=True, **more)
            ctx.mark("attention")
            term = self.o(values, ctx, residual=residual)
            ctx.mark("o")
            return term
        qa = ctx.ws.get("latent.qa", (T, H * (C + R)), ctx.dtype)
        kernels.latent_prep(q, dkv, H, D, R, C, 0 if pos is None else pos.rotary_dim, None if pos is None else pos.inv_freq,
                            self.norm_weight, self.p["eps"], qa, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, halves=self.halves)
        kernels.head_matmul(q, D + R, self.uk, qa, C + R)
        mix = ctx.ws.get("latent.mix", (T, H * C), ctx.dtype)
        if ctx.decode and self._fast_decode():
            kernels.latent_decode(qa, mix, H, C, R, ctx, table, run.ring_pages, run.k, float(self.p["scale"]), window=self.window or 0,
                                  **more)
        else:
            kernels.attention_generic(qa, mix, H, 1, C + R, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, None,
                                      self.window or 0, float(self.p["scale"]), v_dim=C, **more)
        ctx.mark("attention")
        values = ctx.ws.get("latent.values", (T, H * Dv), ctx.dtype)
        kernels.head_matmul(mix, C, self.uv_t, values, Dv)
        term = self.o(values, ctx, residual=residual)
        ctx.mark("o")
        return term
