"""Time mixing in the manner of RWKV with a decay per head and key channel that depends on the token, as the mixer
of a layer.

Every projection reads its own blend of the token's row h and the row h' of the token before it (zeros for a
sequence's first token): h + (h' - h) mu_s, s one of r, k, v, g, w.  Per head the mixer keeps a matrix S [dim, dim]
per sequence (32-bit) instead of keys and values:
    o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T
with r, k, v the projections of their blends, u a bonus that only the current token gets, and the decay
w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)).  What is read out is brought to unit root mean square per head,
multiplied by a weight (one per head and entry) and by SiLU(W_g blend_g), and projected back.  The rank of the
decay's low-rank pair is the files' own size.  The last row of h is per-sequence state beside S.  The reference has
no such mixer (src/model/llama.rs has attention only).

Steps of a few tokens run r, k, v, g and w1 as one product: the five blends stacked as rows against the five matrices
stacked as columns, of whose 25 blocks the five on the diagonal are used.  Such a step is bound by reading the
weights, which this does once and in one launch.  Long steps, bound by arithmetic, run r, k, v and g as four products
in one launch (kernels.gemm_tc_grouped: each alone has too few tiles to fill the device), the blends padded to whole
tiles of tokens; steps in between, and sizes that the grouped launch does not take, run a product per blend.

The recurrence is the walk that gated linear attention uses, reading the state before the token's own update
(csrc/wkv.cu, csrc/gla.cu).  Decays, their exponentials, the bonus and the state are 32-bit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..cache.cache import KVSpec
from ..weights.loader import TensorRequest, WeightStore
from .base import Part, RunView, StepContext
from .linear import Linear
from .registry import register_mixer

BLENDS = ("r", "k", "v", "g", "w")
STACK_MAX_TOKENS = 24            # 5 * 24 rows: still one tile of tokens for the tensor-core product
GROUPED_MIN_TOKENS = 512         # from here on, and where padding to whole tiles adds at most an eighth, one grouped launch


@register_mixer("wkv")
class TimeMix(Part):
    """params: hidden_size, heads, dim, eps (of the read-out's norm).
    tensors: mu_r, mu_k, mu_v, mu_g, mu_w [E]; r, k, v, g [heads*dim, E]; w1 [rank, E], w2 [heads*dim, rank], w0 [heads*dim];
    u [heads, dim]; norm [heads*dim]; o [E, heads*dim]."""

    NAMES = tuple("mu_" + s for s in BLENDS) + ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        self.H, self.D, self.E = self.p["heads"], self.p["dim"], self.p["hidden_size"]

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"S": ((self.H, self.D, self.D), "float32"), "prev": ((self.E,), "float32")}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t, n = self.E, self.spec.tensors, self.H * self.D
        rank = max(8, (E // 16 + 7) // 8 * 8)               # what random weights get where the files' own rank is missing
        return [TensorRequest(t["mu_" + s], (E,), init="uniform:0:1") for s in BLENDS] + \
               [TensorRequest(t[s], (n, E)) for s in ("r", "k", "v", "g")] + \
               [TensorRequest(t["w1"], (-1, E), init_shape=(rank, E)), TensorRequest(t["w2"], (n, -1), init_shape=(n, rank)),
                TensorRequest(t["w0"], (n,), init="uniform:-3:0"), TensorRequest(t["u"], (self.H, self.D), init="uniform:-0.5:0.5"),
                TensorRequest(t["norm"], (n,), init="ones"), TensorRequest(t["o"], (E, n))]

    def load(self, store: WeightStore) -> None:
        w = {local: store.get(r) for local, r in zip(self.NAMES, self.tensor_requests())}
        if w["w1"].shape[0] != w["w2"].shape[1]:
            raise ValueError(f"wkv: the low-rank pair does not fit: w1 {list(w['w1'].shape)} w2 {list(w['w2'].shape)}")
        dt = w["r"].dtype
        self.mu = torch.stack([w["mu_" + s].to(dt) for s in BLENDS]).contiguous()
        self.proj = {s: Linear(w[s], name="wkv." + s) for s in ("r", "k", "v", "g")}
        self.w1, self.w2 = Linear(w["w1"], name="wkv.w1"), Linear(w["w2"], name="wkv.w2")
        self.rank = w["w1"].shape[0]
        # all five matrices as one, each part starting at a multiple of 8 rows, for steps of a few tokens
        self.stack, self.off = None, {}
        if dt == torch.bfloat16 and self.E % 8 == 0 and w["r"].is_cuda:
            parts, rows = [], 0
            for s in ("r", "k", "v", "g", "w1"):
                pad = (rows + 7) // 8 * 8 - rows
                if pad:
                    parts.append(torch.zeros(pad, self.E, dtype=dt, device=w[s].device))
                self.off[s] = rows + pad
                parts.append(w[s].to(dt))
                rows = self.off[s] + w[s].shape[0]
            pad = (rows + 7) // 8 * 8 - rows
            if pad:
                parts.append(torch.zeros(pad, self.E, dtype=dt, device=w["r"].device))
            self.stack = Linear(torch.cat(parts, dim=0).contiguous(), name="wkv.stack")
        self.w0 = w["w0"].contiguous()
        self.u = w["u"].to(self.w0.dtype).contiguous()
        self.norm_weight = w["norm"].contiguous()
        self.o = Linear(w["o"], name="wkv.o")

    graph_class = ()              # grids depend on the batch size only

    def forward(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        H, D, T = self.H, self.D, h.shape[0]
        n = H * D
        padded = -(-T // kernels.GROUPED_TILE) * kernels.GROUPED_TILE
        grouped = (self.stack is not None and n % 8 == 0 and T >= GROUPED_MIN_TOKENS and (padded - T) * 8 <= T
                   and all(self.off[s] == i * n for i, s in enumerate(("r", "k", "v", "g"))))
        rows = padded if grouped else T
        blends = ctx.ws.get("wkv.blends", (len(BLENDS), rows, self.E), ctx.dtype)
        kernels.token_shift_mix(h, self.mu, ctx.state(f"run{run.index}.prev"), ctx, blends)
        ctx.mark("shift")
        if grouped:
            both = ctx.ws.get("wkv.rkvg", (4, rows, n), ctx.dtype)
            kernels.gemm_tc_grouped(blends[:4], self.stack.weight[:4 * n], both)
            r, k, v, g = (both[i, :T] for i in range(4))
            low = self.w1(blends[4, :T], ctx, activation="tanh")
        elif self.stack is not None and T <= STACK_MAX_TOKENS:
            both = self.stack(blends.view(len(BLENDS) * T, self.E), ctx)
            r, k, v, g = (both[i * T:(i + 1) * T, self.off[s]:self.off[s] + n] for i, s in enumerate(("r", "k", "v", "g")))
            low = kernels.unary_act_(both[4 * T:5 * T, self.off["w1"]:self.off["w1"] + self.rank], "tanh")
        else:
            r, k, v, g = (self.proj[s](blends[i, :T], ctx) for i, s in enumerate(("r", "k", "v", "g")))
            low = self.w1(blends[4, :T], ctx, activation="tanh")
        # the decay's second product keeps 32-bit results: their exponentials enter the recurrence
        a = self.w2(low, ctx, out_dtype=torch.float32)
        ctx.mark("projections")
        read = ctx.ws.get("wkv.read", (T, H * D), torch.float32)
        kernels.wkv(r, k, v, a, self.w0, self.u, ctx.state(f"run{run.index}.S"), read, ctx, H, D)
        ctx.mark("recurrence")
        normed = ctx.ws.get("wkv.normed", (T, H * D), ctx.dtype)
        kernels.gated_head_norm(read, g, self.norm_weight, self.p["eps"], normed, H, D, gate_function="silu")
        term = self.o(normed, ctx, out_dtype=torch.float32)
        ctx.mark("o")
        return term
