"""RMS norm: x / sqrt(mean(x^2) + eps) * w, sums in 32-bit (src/math/ops.rs:1-4,
src/gpu/rmsnorm.glsl:13-26), fused with the residual add that precedes it as the
reference's unused add_rmsnorm shader does (src/gpu/add_rmsnorm.glsl:1-32)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import FUSE_MAX_TOKENS, Blend, DeferredNorm, Part, StepContext, Stream
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    """params: size, eps, offset (default 0; 1 for a weight that is stored around zero: the rows are multiplied by
    offset + weight, the sum in 32-bit).  tensors: weight [size]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.offset = float(self.p.get("offset", 0.0))
        if self.offset:
            self.fold_weight = None               # a weight with an offset is not folded into a consumer's matrix

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.spec.tensors["weight"], (self.p["size"],), init="zeros" if self.offset else "ones")]

    def load(self, store: WeightStore) -> None:
        self.weight = store.get(self.tensor_requests()[0])
        self._ones = None

    graph_class = ()

    def fold_weight(self) -> torch.Tensor:
        """The weight, for a consumer that multiplies it into the columns of its own matrix."""
        return self.weight

    @staticmethod
    def _terms(stream: Stream) -> list:
        return ([stream.pending] if stream.pending is not None else []) + list(stream.more)

    def apply_pair(self, stream: Stream, other: "RMSNorm", ctx: StepContext, buffers=("normed", "normed2")):
        """This norm and `other` (same size, eps and offset, another weight) of the same x in one pass: adds everything
        that waits on the stream into x (32-bit) and returns both normalised copies."""
        if (other.p["size"], other.p["eps"], other.offset) != (self.p["size"], self.p["eps"], self.offset):
            raise ValueError("rmsnorm: two norms of one pass must agree in size, eps and offset")
        terms = self._terms(stream)
        shape = (stream.x.shape[0], self.p["size"])
        out1, out2 = ctx.ws.get(buffers[0], shape, ctx.dtype), ctx.ws.get(buffers[1], shape, ctx.dtype)
        w2 = other.weight if other.weight.dtype == self.weight.dtype else other.weight.to(self.weight.dtype)
        kernels.add_rmsnorm_pair(stream.x, terms, self.weight, w2, self.offset, self.p["eps"], out1, out2)
        if terms:
            stream.drop_shadow()
        stream.pending, stream.more = None, []
        return out1, out2

    def apply(self, stream: Stream, ctx: StepContext, rows: Optional[torch.Tensor] = None,
              buffer: str = "normed", absorbed: bool = False):
        """Adds the stream's pending term into x and returns the normalised rows.  With
        `rows`, only those rows are produced and x is left as it is.  absorbed: the consumer has
        this norm's weight in its matrix: it is left out here, and if the stream carries a valid
        shadow nothing is computed at all (a DeferredNorm is returned)."""
        if self.offset or stream.more:
            # weights around zero, or several terms waiting: the kernel that takes both
            terms = self._terms(stream)
            n = stream.x.shape[0] if rows is None else rows.numel()
            out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
            kernels.add_rmsnorm_pair(stream.x, terms, self.weight, None, self.offset, self.p["eps"], out, None, rows=rows,
                                     write_x=rows is None)
            if rows is None:
                if terms:
                    stream.drop_shadow()
                stream.pending, stream.more = None, []
            return out
        if absorbed and rows is None and stream.pending is None and stream.xb is not None and ctx.T <= FUSE_MAX_TOKENS:
            return DeferredNorm(stream.xb, stream.ssq, stream.ssq_parts, self.p["size"], self.p["eps"])
        weight = self.weight
        if absorbed:
            if self._ones is None:
                self._ones = torch.ones_like(self.weight)
            weight = self._ones
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
        kernels.add_rmsnorm(stream.x, stream.pending, weight, self.p["eps"], out, rows=rows, write_x=rows is None)
        if rows is None:
            if stream.pending is not None:
                stream.drop_shadow()              # x has changed
            stream.pending = None
        return out


    def add_normed(self, stream: Stream, term, ctx: StepContext, then: Optional["RMSNorm"] = None, buffer: str = "normed",
                   shadow: Optional[bool] = None):
        """x += term / sqrt(mean(term^2) + eps) * w: the norm of a sublayer's result on its way into the stream
        (32-bit).  In bfloat16 mode the stream's bfloat16 copy is renewed by the same kernel; sums of squares of x
        are not kept (a deferred norm in front of the next product would need them).

        For layers that norm a sublayer's input too: `then` is the norm in front of the next sublayer, whose rows
        (x / rms(x) * its weight, in the step's dtype) the same kernel writes and this call returns; term may be a
        Blend of two branches, finished in the same pass; shadow says whether the bfloat16 copy of x is wanted
        (default: in bfloat16 mode, as before)."""
        if stream.pending is not None or stream.more:
            raise RuntimeError("rmsnorm: a term is pending on the stream")
        if then is not None or isinstance(term, Blend) or shadow is not None:
            if self.offset or (then is not None and (then.offset or then.p["eps"] != self.p["eps"] or then.p["size"] != self.p["size"])):
                raise ValueError("rmsnorm: the norms of one pass must agree in size and eps and have plain weights")
            want = ctx.dtype == torch.bfloat16 if shadow is None else bool(shadow) and ctx.dtype == torch.bfloat16
            xb = ctx.ws.get("stream.xb", stream.x.shape, torch.bfloat16) if want else None
            h = ctx.ws.get(buffer, stream.x.shape, ctx.dtype) if then is not None else None
            nw = None if then is None else (then.weight if then.weight.dtype == self.weight.dtype else then.weight.to(self.weight.dtype))
            if isinstance(term, Blend):
                kernels.norm_sandwich(stream.x, term.a, self.weight, self.p["eps"], y2=term.b, inner_weights=term.weights,
                                      mix=term.mix, next_weight=nw, h=h, xb=xb)
            else:
                kernels.norm_sandwich(stream.x, term, self.weight, self.p["eps"], next_weight=nw, h=h, xb=xb)
            stream.xb, stream.ssq, stream.ssq_parts = xb, None, 0
            return h
        xb = ctx.ws.get("stream.xb", stream.x.shape, torch.bfloat16) if ctx.dtype == torch.bfloat16 else None
        kernels.norm_residual_add(stream.x, term, self.weight, self.p["eps"], xb=xb)
        stream.xb, stream.ssq, stream.ssq_parts = xb, None, 0


@register_norm("dyt")
class DynamicTanh(Part):
    """Dynamic tanh in a norm's place: tanh(alpha x) * weight + bias, no mean and no variance.
    params: size.  tensors: weight [size], bias [size], alpha [] (one scalar)."""

    def tensor_requests(self) -> List[TensorRequest]:
        t, n = self.spec.tensors, self.p["size"]
        return [TensorRequest(t["weight"], (n,), init="ones"), TensorRequest(t["bias"], (n,), init="zeros"),
                TensorRequest(t["alpha"], (), init="const:0.5")]

    def load(self, store: WeightStore) -> None:
        w, b, a = (store.get(r) for r in self.tensor_requests())
        self.weight, self.bias = w, b.to(w.dtype)
        self.alpha = float(a.float().item()) if a.device.type != "meta" else 0.0

    graph_class = ()

    def apply(self, stream: Stream, ctx: StepContext, rows: Optional[torch.Tensor] = None, buffer: str = "normed",
              absorbed: bool = False):
        """Adds the stream's pending term into x (32-bit) and returns tanh(alpha x) * weight + bias of all rows,
        or of `rows` only (x is then left as it is)."""
        if stream.more:
            raise RuntimeError("dyt: this norm adds one pending term only")
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
        kernels.add_dyt(stream.x, stream.pending, self.weight, self.bias, self.alpha, out, rows=rows, write_x=rows is None)
        if rows is None:
            if stream.pending is not None:
                stream.drop_shadow()
            stream.pending = None
        return out
