"""Dense gated feed-forward: down(act(gate(h)) * up(h)) with act = SiLU
(src/model/llama.rs:399-402, src/math/ops.rs:11), or GELU in its tanh form for designs that
ask for it.  gate and up are one matrix [2F, E] after loading, so one product reads h once."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from typing import Optional

from .base import DeferredNorm, Part, StepContext
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    """params: hidden_size, intermediate_size, activation ("silu" or "gelu_tanh"), term_f32 (default False: the down
    product's result, which is added to the residual stream, is kept in 32-bit also where the products run in bfloat16).
    tensors: gate [F, E], up [F, E], down [E, F]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.activation = self.p.get("activation", "silu")
        if self.activation not in kernels.GATE_ACTS:
            raise ValueError(f"gated_mlp: activation {self.activation!r} is not supported {sorted(kernels.GATE_ACTS)}")

    def tensor_requests(self) -> List[TensorRequest]:
        E, F, t = self.p["hidden_size"], self.p["intermediate_size"], self.spec.tensors
        return [TensorRequest(t["gate"], (F, E)), TensorRequest(t["up"], (F, E)), TensorRequest(t["down"], (E, F))]

    def load(self, store: WeightStore) -> None:
        g, u, d = (store.get(r) for r in self.tensor_requests())
        if g.dtype != u.dtype:
            u = u.to(g.dtype)
        # where the tensor-core product can take them, gate and up are interleaved tile by tile so
        # that its epilogue applies the activation; else they are stacked and a kernel follows
        self.fused = g.dtype == torch.bfloat16 and self.p["hidden_size"] % 8 == 0 and g.is_cuda
        if self.fused:
            self.gate_up_tiles = kernels.interleave_gate_up(g, u)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), name="ff.gate_up")
        self.down = Linear(d, name="ff.down")

    accepts_residual = True
    graph_class = ()              # the same launches every step

    def absorb_input_norm(self, weight: torch.Tensor) -> bool:
        """Multiplies the weight of the norm in front of this part into the gate/up matrix (only
        where the tensor-core product, which can apply the norm's per-token scale, runs it)."""
        if not self.fused:
            return False
        self.gate_up_tiles = (self.gate_up_tiles.float() * weight.float()[None, :]).to(torch.bfloat16).contiguous()
        return True

    def forward(self, h, ctx: StepContext, residual=None) -> Optional[torch.Tensor]:
        F = self.p["intermediate_size"]
        act = ctx.ws.get("ff.act", (h.shape[0], F), ctx.dtype)
        norm = dict(row_ssq=h.ssq, ssq_parts=h.parts, norm_size=h.size, eps=h.eps) if isinstance(h, DeferredNorm) else {}
        rows = h.xb if norm else h
        if self.fused and kernels.gemm_tc_supported(rows, self.gate_up_tiles):
            kernels.gemm_tc(rows, self.gate_up_tiles, None, act, swiglu_features=F, gate_activation=self.activation, **norm)
        elif self.fused:
            raise RuntimeError("gated_mlp: the activations given do not fit the fused product it was loaded for")
        else:
            kernels.swiglu(self.gate_up(h, ctx), act, self.activation)
        ctx.mark("gate_up")
        term = self.down(act, ctx, residual=residual, out_dtype=torch.float32 if self.p.get("term_f32") else None)
        ctx.mark("down")
        return term


@register_feed_forward("mlp")
class PlainMLP(Part):
    """down(act(up(h))): a feed-forward without a gate.  params: hidden_size, intermediate_size, activation ("gelu":
    the exact form with erf; "gelu_tanh"; "silu").  tensors: up [F, E], down [E, F]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.activation = self.p.get("activation", "gelu")
        if self.activation not in kernels.UNARY_ACTS:
            raise ValueError(f"mlp: activation {self.activation!r} is not supported {sorted(kernels.UNARY_ACTS)}")

    def tensor_requests(self) -> List[TensorRequest]:
        E, F, t = self.p["hidden_size"], self.p["intermediate_size"], self.spec.tensors
        return [TensorRequest(t["up"], (F, E)), TensorRequest(t["down"], (E, F))]

    def load(self, store: WeightStore) -> None:
        u, d = (store.get(r) for r in self.tensor_requests())
        self.up, self.down = Linear(u, name="ff.up"), Linear(d, name="ff.down")

    graph_class = ()

    def forward(self, h, ctx: StepContext) -> torch.Tensor:
        act = self.up(h, ctx, activation=self.activation)
        ctx.mark("up")
        term = self.down(act, ctx, out_dtype=torch.float32)
        ctx.mark("down")
        return term


@register_feed_forward("moe")
class RoutedExperts(Part):
    """A mixture of small gated feed-forwards of which each token uses a few, plus an optional one that all tokens
    use.  An expert is down(unit(gate(h), up(h))) with unit(g, u) = g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit),
    u' = clamp(u, -limit, limit); no biases.  The router (32-bit): scores sigmoid(W_r h); the experts form `groups`
    equal groups of neighbours, a group's mark is the sum of its two largest scores, and only experts of the `keep`
    best groups can be chosen; the `top` largest of those are, with weights score / (sum of the chosen scores + 1e-20)
    * scale.  The reference has no routed feed-forward (src/model/llama.rs:399-402 is its dense one).

    Options: scores that are a softmax over all experts instead of sigmoids (`score="softmax"`); a correction per expert
    that is added to the scores for the choice and left out of the weights (`correction=True`, tensor `correction`);
    `identity` experts without matrices, numbered behind the others, whose result is the token's own row h (the router's
    matrix and the correction then have experts + identity rows).

    params: hidden_size, experts, top, groups, keep, scale, expert_ff, limit, shared_ff, shared_limit (None: no shared
    expert), score ("sigmoid" or "softmax"), correction (default False), identity (default 0).  tensors: router
    [experts + identity, E]; experts: the prefix of the experts' names (<prefix><i>.gate [F, E], .up [F, E], .down [E, F]);
    shared: the prefix of the shared expert's (.gate, .up [Fs, E], .down [E, Fs]); correction [experts + identity]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = self.p
        self.n, self.top, self.F = int(p["experts"]), int(p["top"]), int(p["expert_ff"])
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or 1)
        self.shared_ff = p.get("shared_ff")
        self.identity = int(p.get("identity") or 0)
        self.n_all = self.n + self.identity
        self.score = p.get("score", "sigmoid")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"moe: score {self.score!r} is not one of 'sigmoid', 'softmax'")
        self.corrected = bool(p.get("correction", False))
        if self.identity and self.groups != 1:
            raise ValueError("moe: identity experts go with one group of experts")
        if self.n_all % self.groups or self.keep > self.groups or self.top > self.keep * (self.n_all // self.groups):
            raise ValueError(f"moe: {self.top} of {self.n} experts in {self.groups} groups of which {self.keep} are kept")

    def _names(self):
        t = self.spec.tensors
        return [(f"{t['experts']}{i}.{part}") for i in range(self.n) for part in ("gate", "up", "down")]

    def tensor_requests(self) -> List[TensorRequest]:
        E, F, t = self.p["hidden_size"], self.F, self.spec.tensors
        req = [TensorRequest(t["router"], (self.n_all, E))]
        for name in self._names():
            req.append(TensorRequest(name, (E, F) if name.endswith(".down") else (F, E)))
        if self.shared_ff:
            Fs = int(self.shared_ff)
            req += [TensorRequest(t["shared"] + ".gate", (Fs, E)), TensorRequest(t["shared"] + ".up", (Fs, E)),
                    TensorRequest(t["shared"] + ".down", (E, Fs))]
        if self.corrected:
            req.append(TensorRequest(t["correction"], (self.n_all,), init="zeros"))
        return req

    def load(self, store: WeightStore) -> None:
        req = self.tensor_requests()
        self.router = Linear(store.get(req[0]), name="moe.router")
        mats = [store.get(r) for r in req[1:1 + 3 * self.n]]
        dt = mats[0].dtype
        # the experts' matrices side by side: [experts, F, E] twice and [experts, E, F]
        self.w_gate = torch.stack([m.to(dt) for m in mats[0::3]]).contiguous()
        self.w_up = torch.stack([m.to(dt) for m in mats[1::3]]).contiguous()
        self.w_down = torch.stack([m.to(dt) for m in mats[2::3]]).contiguous()
        self.shared_gate_up = self.shared_down = None
        self.correction = store.get(req[-1]).to(torch.float32).contiguous() if self.corrected else None
        if self.shared_ff:
            g, u, d = (store.get(r) for r in req[1 + 3 * self.n:4 + 3 * self.n])
            self.shared_gate_up = Linear(torch.cat([g, u.to(g.dtype)], dim=0), name="moe.shared_gate_up")
            self.shared_down = Linear(d, name="moe.shared_down")

    TOKEN_BY_TOKEN = 16           # steps of at most this many tokens run every (token, choice) pair for itself
    BY_EXPERT = 128               # pairs per expert, on average, from which the experts run as ordinary products of their own
    BY_EXPERT_ENTRIES = 8 << 20   # ... where an expert's matrix has at least this many entries
    graph_class = ()              # grids depend on the number of tokens only
    reads_stream = True           # a block that has the rows in 32-bit gives them too (x32): the router reads those

    def forward(self, h, ctx: StepContext, x32: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, E, top = h.shape[0], self.p["hidden_size"], self.top
        # the router's product in 32-bit sums, from 32-bit rows where the block has them, and its choice
        ids = ctx.ws.get("moe.ids", (T, top), torch.int32)
        weights = ctx.ws.get("moe.weights", (T, top), torch.float32)
        kernels.moe_router(h if x32 is None else x32, self.router.weight, self.groups, self.keep, top,
                           float(self.p.get("scale", 1.0)), ids, weights, softmax=self.score == "softmax", correction=self.correction)
        ctx.mark("router")
        out = ctx.ws.get("moe.out", (T, E), torch.float32)
        if self.shared_ff:
            Fs = int(self.shared_ff)
            act = kernels.glu_clamped(self.shared_gate_up(h, ctx), ctx.ws.get("moe.shared_act", (T, Fs), ctx.dtype),
                                      float(self.p["shared_limit"]))
            self.shared_down(act, ctx, out_dtype=torch.float32, buffer="moe.out")
            ctx.mark("shared")
        if not ctx.decode and T * top >= self.BY_EXPERT * self.n and self.F * E >= self.BY_EXPERT_ENTRIES \
                and kernels.moe_grouped_supported(h, self.w_gate):
            # very many tokens (an expert gets 128 rows or more on average) and large experts: every expert's products on
            # the tcgen05 kernels (8,192 pairs, 16 experts of 3,584 x 4,096: 1.65 against 3.99 ms; of 2,048 x 2,048: 1.17
            # against 1.21 ms, the launches of small products fill a quarter of the device)
            kernels.moe_by_expert(h, ids, weights, self.w_gate, self.w_up, self.w_down, float(self.p["limit"]), out, ctx,
                                  accumulate=bool(self.shared_ff), identity=self.identity)
        elif T > self.TOKEN_BY_TOKEN and kernels.moe_grouped_supported(h, self.w_gate):
            # many tokens: pairs sorted by expert on the device, tiles of 64 pairs on the tensor cores
            kernels.moe_grouped(h, ids, weights, self.w_gate, self.w_up, self.w_down, float(self.p["limit"]), out, ctx,
                                accumulate=bool(self.shared_ff), identity=self.identity)
        else:
            y = ctx.ws.get("moe.units", (T, top, self.F), ctx.dtype)
            kernels.moe_gate_up(h, ids, self.w_gate, self.w_up, float(self.p["limit"]), y, identity=self.identity)
            kernels.moe_down(y, ids, weights, self.w_down, out, accumulate=bool(self.shared_ff), ws=ctx.ws, identity=self.identity,
                             h=h)
        ctx.mark("experts")
        return out
