"""A selective state-space mixer in its state-space-duality form (one decay per head and token), as the mixer of a layer.

One projection gives [z | x | B | C | dt]: a gate z and inputs x of heads*vdim entries, B and C of groups*state entries
that the heads of a group share, and a step size per head.  x, B and C pass a short causal convolution per channel with a
bias, and SiLU.  Per head the mixer keeps a matrix S [state, vdim] per sequence (32-bit):
    dt' = softplus(dt + dt_bias);   S <- exp(-exp(A_log) dt') S + dt' B x^T;   y = S^T C + D x.
y times SiLU(z) is brought to unit root mean square in `norm_groups` equal parts (the gate comes before the norm),
multiplied by a weight and projected back.  The convolution's last inputs are per-sequence state beside S.  The
reference has no such mixer (src/model/llama.rs has attention only).

The recurrence is the walk that gated linear attention uses with the decay equal for all key channels (csrc/ssd.cu,
csrc/gla.cu).  Step sizes, decays with their softplus and exponentials, and the state are 32-bit; the step sizes'
rows of the projection are a product of their own that keeps 32-bit results.
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


@register_mixer("ssd")
class SelectiveStateSpace(Part):
    """params: hidden_size, heads, vdim, state, groups, conv (taps), norm_groups, eps (of the read-out's norm).
    tensors: in [2*heads*vdim + 2*groups*state + heads, E], conv [heads*vdim + 2*groups*state, taps], conv_bias, dt_bias,
    A_log, D [heads], norm [heads*vdim], o [E, heads*vdim]."""

    NAMES = ("in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o")

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.H, self.P, self.N, self.G, self.K, self.NG = p["heads"], p["vdim"], p["state"], p["groups"], p["conv"], p["norm_groups"]
        self.inner = self.H * self.P
        self.C = self.inner + 2 * self.G * self.N
        if self.H % self.G:
            raise ValueError(f"ssd: {self.H} heads are not a multiple of {self.G} groups")
        if self.inner % self.NG:
            raise ValueError(f"ssd: {self.inner} entries do not form {self.NG} equal parts for the norm")
        if not 1 <= self.K <= 16:
            raise ValueError(f"ssd: a convolution of {self.K} taps is not supported (1..16)")

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        spec = {"S": ((self.H, self.N, self.P), "float32")}
        if self.K > 1:
            spec["conv"] = ((self.K - 1, self.C), "float32")
        return spec

    def tensor_requests(self) -> List[TensorRequest]:
        E, t, H = self.p["hidden_size"], self.spec.tensors, self.H
        return [TensorRequest(t["in"], (self.inner + self.C + H, E)),
                TensorRequest(t["conv"], (self.C, self.K), init="uniform:-0.6:0.6"),
                TensorRequest(t["conv_bias"], (self.C,), init="uniform:-0.1:0.1"),
                TensorRequest(t["dt_bias"], (H,), init="uniform:-4:-1"), TensorRequest(t["A_log"], (H,), init="uniform:-1:1"),
                TensorRequest(t["D"], (H,), init="ones"), TensorRequest(t["norm"], (self.inner,), init="ones"),
                TensorRequest(t["o"], (E, self.inner))]

    def load(self, store: WeightStore) -> None:
        w = {local: store.get(r) for local, r in zip(self.NAMES, self.tensor_requests())}
        dt = w["in"].dtype
        main = self.inner + self.C                       # z, x, B, C: one product; the step sizes: another, 32-bit results
        self.proj = Linear(w["in"][:main].contiguous(), name="ssd.in")
        self.dt_proj = Linear(w["in"][main:].contiguous(), name="ssd.dt")
        self.taps = w["conv"].to(dt).contiguous()
        self.taps_t = self.taps.t().contiguous() if dt == torch.bfloat16 else None      # tap by tap, for 16-byte loads
        self.conv_bias = w["conv_bias"].to(dt).contiguous()
        self.dt_bias = w["dt_bias"].contiguous()
        self.a_log, self.skip = w["A_log"].to(self.dt_bias.dtype).contiguous(), w["D"].to(self.dt_bias.dtype).contiguous()
        self.norm_weight = w["norm"].contiguous()
        self.o = Linear(w["o"], name="ssd.o")

    graph_class = ()              # grids depend on the batch size only

    def forward(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        H, P, N, G, inner, C = self.H, self.P, self.N, self.G, self.inner, self.C
        T = h.shape[0]
        proj = self.proj(h, ctx)
        dt = self.dt_proj(h, ctx, out_dtype=torch.float32)
        ctx.mark("projections")
        conv = ctx.ws.get("ssd.conv", (T, C), ctx.dtype)
        carried = ctx.state(f"run{run.index}.conv") if self.K > 1 else None
        kernels.short_conv(proj[:, inner:inner + C], self.taps, carried, ctx, conv, taps_t=self.taps_t, bias=self.conv_bias,
                           activation="silu")
        ctx.mark("conv")
        read = ctx.ws.get("ssd.read", (T, inner), torch.float32)
        kernels.ssd(conv[:, :inner], conv[:, inner:inner + G * N], conv[:, inner + G * N:], dt, self.dt_bias, self.a_log, self.skip,
                    ctx.state(f"run{run.index}.S"), read, ctx, H, G, N, P)
        ctx.mark("recurrence")
        normed = ctx.ws.get("ssd.normed", (T, inner), ctx.dtype)
        kernels.gated_head_norm(read, proj[:, :inner], self.norm_weight, self.p["eps"], normed, self.NG, inner // self.NG,
                                gate_function="silu", gate_first=True)
        term = self.o(normed, ctx, out_dtype=torch.float32)
        ctx.mark("o")
        return term
