"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

import torch

from .. import kernels
from .base import RunView, StepContext, Stream
from .registry import register_block


@register_block("prenorm")
class PreNormBlock:
    """x += mixer(norm_m(x)); x += ff(norm_f(x)) (src/model/llama.rs:361-404).  The sums
    are not done here: each term is left pending on the stream and the next norm adds it
    in 32-bit while it normalises."""

    norm_names = ("mixer", "feed_forward")
    graph_class = ()

    def __init__(self, mixer, feed_forward, norms):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.absorbed = {"mixer": False, "feed_forward": False}

    def fuse(self) -> None:
        """After the weights are loaded: a part that can take the weight of the norm in front of it into
        its own matrix does so (then that norm costs no kernel when the stream carries a shadow)."""
        for name, part in (("mixer", self.mixer), ("feed_forward", self.feed_forward)):
            if part is None:
                continue
            give = getattr(self.norms[name], "fold_weight", None)
            take = getattr(part, "absorb_input_norm", None)
            if give and take and not self.absorbed[name]:
                self.absorbed[name] = bool(take(give()))

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        h = self._norm("mixer", stream, ctx)
        ctx.mark("norm")
        if getattr(self.mixer, "accepts_residual", False):
            term = self.mixer.forward(h, ctx, run, residual=stream)
        else:
            term = self.mixer.forward(h, ctx, run)
        self._add(stream, term)
        if self.feed_forward is None:
            return
        h = self._norm("feed_forward", stream, ctx)
        ctx.mark("ff_norm")
        if getattr(self.feed_forward, "accepts_residual", False):
            term = self.feed_forward.forward(h, ctx, residual=stream)
        else:
            term = self.feed_forward.forward(h, ctx)
        self._add(stream, term)

    def _norm(self, name: str, stream: Stream, ctx: StepContext):
        if self.absorbed[name]:
            return self.norms[name].apply(stream, ctx, absorbed=True)
        return self.norms[name].apply(stream, ctx)

    @staticmethod
    def _add(stream: Stream, term) -> None:
        """A part that has added its term to the stream itself returns None."""
        if term is not None:
            stream.pending = term
            stream.drop_shadow()


@register_block("outnorm")
class OutputNormBlock:
    """x += norm_m(mixer(x)); x += norm_f(ff(x)): the sublayers read the residual stream itself, and what they give
    is normed on its way into it.  The sums are 32-bit; in bfloat16 mode the products read a bfloat16 copy of x that
    the norm's kernel renews with every sum (`Stream.xb`)."""

    norm_names = ("mixer", "feed_forward")
    graph_class = ()

    def __init__(self, mixer, feed_forward, norms):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        for name in self.norm_names:
            if name in norms and not hasattr(norms[name], "add_normed"):
                raise ValueError(f"outnorm: the norm of kind {norms[name].spec.kind!r} cannot norm a sublayer's result into the stream")

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        term = self.mixer.forward(self._rows(stream, ctx), ctx, run)
        self.norms["mixer"].add_normed(stream, term, ctx)
        ctx.mark("mixer_norm")
        if self.feed_forward is None:
            return
        if getattr(self.feed_forward, "reads_stream", False):
            # a part that decides in 32-bit (a router) also gets the stream itself, not only its bfloat16 copy
            term = self.feed_forward.forward(self._rows(stream, ctx), ctx, x32=stream.x)
        else:
            term = self.feed_forward.forward(self._rows(stream, ctx), ctx)
        self.norms["feed_forward"].add_normed(stream, term, ctx)
        ctx.mark("ff_norm")

    @staticmethod
    def _rows(stream: Stream, ctx: StepContext):
        """x as the sublayers' products read it: x itself in 32-bit mode, else its bfloat16 copy."""
        if stream.pending is not None:
            raise RuntimeError("outnorm: a term is pending on the stream; this arrangement adds every term at once")
        if ctx.dtype == torch.float32:
            return stream.x
        if stream.xb is None:
            stream.xb = ctx.ws.get("stream.xb", stream.x.shape, torch.bfloat16)
            kernels.norm_residual_add(stream.x, None, None, 1.0, xb=stream.xb)
        return stream.xb


@register_block("parallel")
class ParallelBlock:
    """x += mixer(norm_m(x)) + ff(norm_f(x)): both sublayers read norms of the same x.  The two norms are one pass over
    the row (one root mean square, two weights); neither sum is done here: the mixer's term is left pending and the
    feed-forward's beside it, and the next norm adds them in 32-bit while it normalises."""

    norm_names = ("mixer", "feed_forward")
    graph_class = ()

    def __init__(self, mixer, feed_forward, norms):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        if feed_forward is not None and not hasattr(norms["mixer"], "apply_pair"):
            raise ValueError(f"parallel: the norm of kind {norms['mixer'].spec.kind!r} cannot give two norms of one row at once")

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        if self.feed_forward is None:
            h, h_ff = self.norms["mixer"].apply(stream, ctx), None
        else:
            h, h_ff = self.norms["mixer"].apply_pair(stream, self.norms["feed_forward"], ctx)
        ctx.mark("norm")
        term = self.mixer.forward(h, ctx, run)
        if term.dim() != 2 or term.dtype != torch.float32:
            raise RuntimeError("parallel: a mixer must give one 32-bit term [tokens, width]")
        stream.pending = term
        stream.drop_shadow()
        if self.feed_forward is not None:
            term = self.feed_forward.forward(h_ff, ctx)
            if term.dim() != 2:
                raise RuntimeError("parallel: a feed-forward must give one term [tokens, width]")
            stream.more.append(term)
            ctx.mark("ff")


@register_block("sandwich")
class SandwichBlock:
    """x += norm_mo(mixer(norm_m(x))); x += norm_fo(ff(norm_f(x))): every sublayer reads a norm of x and what it gives is
    normed again on its way into x.  One kernel per sublayer does both sides of the seam: it norms the result into x
    (32-bit) and writes the rows the next sublayer reads.  A mixer of two branches may hand over its branches unblended
    (`forward_blend`); the same kernel then norms and blends them first.  An extra part `side`, if the layer has one, adds
    an input of its own behind the feed-forward, normed in by `norms["side"]` (it reads x itself: the bfloat16 copy in
    bfloat16 mode).  norms: mixer, mixer_out, and with a feed-forward feed_forward, feed_forward_out."""

    norm_names = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")
    graph_class = ()

    def __init__(self, mixer, feed_forward, norms, extras=None):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.side = (extras or {}).get("side")
        need = ["mixer", "mixer_out"] + (["feed_forward", "feed_forward_out"] if feed_forward is not None else []) \
            + (["side"] if self.side is not None else [])
        for name in need:
            if name not in norms or not hasattr(norms[name], "add_normed"):
                raise ValueError(f"sandwich: the layer needs a norm {name!r} that can norm a result into the stream")

    def _last(self, norm, stream: Stream, term, ctx: StepContext, **kw) -> None:
        """The layer's last sum; its kernel also norms the rows for the next run's block where that block begins with a
        norm of the same kind."""
        then = stream.next_norm
        fits = then is not None and type(then) is type(norm) and not getattr(then, "offset", 0.0) \
            and (then.p["size"], then.p["eps"]) == (norm.p["size"], norm.p["eps"])
        h = norm.add_normed(stream, term, ctx, then=then if fits else None, buffer="normed", **kw)
        stream.normed = (then, h) if fits else None

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        norms = self.norms
        if stream.normed is not None and stream.normed[0] is norms["mixer"] and stream.pending is None and not stream.more:
            h = stream.normed[1]                      # the block in front has normed these rows already
        else:
            h = norms["mixer"].apply(stream, ctx)
        stream.normed = None
        ctx.mark("norm")
        give = getattr(self.mixer, "forward_blend", None) or self.mixer.forward
        term = give(h, ctx, run)
        bare, side = self.feed_forward is None, self.side is not None
        if bare and not side:
            self._last(norms["mixer_out"], stream, term, ctx, shadow=False)
        else:
            h = norms["mixer_out"].add_normed(stream, term, ctx, then=None if bare else norms["feed_forward"], buffer="normed2",
                                              shadow=bare and side)
        ctx.mark("mixer_norm")
        if not bare:
            term = self.feed_forward.forward(h, ctx)
            if side:
                norms["feed_forward_out"].add_normed(stream, term, ctx, shadow=True)
            else:
                self._last(norms["feed_forward_out"], stream, term, ctx, shadow=False)
            ctx.mark("ff_norm")
        if side:
            rows = stream.x if ctx.dtype == torch.float32 else stream.xb
            self._last(norms["side"], stream, self.side.forward(rows, ctx), ctx, shadow=False)
            ctx.mark("side")
