"""A selective state-space mixer whose decay differs per channel and per state entry (the selective scan of Mamba), as
the mixer of a layer.

W_in h is [x | z], inner entries each.  x passes a short causal convolution per channel with a bias, and SiLU.  W_x x is
[dt | B | C] with dt_rank, state and state entries; dt' = softplus(W_dt dt + dt_bias) is a step size per channel.  With
A = -exp(A_log) [inner, state], per channel c and state entry n
    S[c, n] <- exp(dt'_c A[c, n]) S[c, n] + dt'_c x_c B_n;    y_c = sum_n S[c, n] C_n + D_c x_c,
and the mixer gives W_o (y * SiLU(z)).  S (32-bit) and the convolution's last taps - 1 inputs are per-sequence state.
The projections run in the step's number format; the step sizes' product keeps 32-bit results, and step sizes with
their softplus, decays with their exponentials, the state and every sum of the recurrence are 32-bit
(csrc/selective_scan.cu).  The reference has no such mixer (src/model/llama.rs has attention only).
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


@register_mixer("selective_scan")
class SelectiveScan(Part):
    """params: hidden_size, inner, state, dt_rank, conv (taps).
    tensors: in [2*inner, E], conv [inner, taps], conv_bias [inner], x [dt_rank + 2*state, inner], dt [inner, dt_rank],
    dt_bias [inner], A_log [inner, state], D [inner], o [E, inner]."""

    NAMES = ("in", "conv", "conv_bias", "x", "dt", "dt_bias", "A_log", "D", "o")

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.inner, self.N, self.R, self.K = int(p["inner"]), int(p["state"]), int(p["dt_rank"]), int(p["conv"])
        if not 1 <= self.K <= 16:
            raise ValueError(f"selective_scan: a convolution of {self.K} taps is not supported (1..16)")
        if not 1 <= self.N <= 256:
            raise ValueError(f"selective_scan: a state of {self.N} entries per channel is not supported (1..256)")

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        spec = {"S": ((self.inner, self.N), "float32")}
        if self.K > 1:
            spec["conv"] = ((self.K - 1, self.inner), "float32")
        return spec

    def tensor_requests(self) -> List[TensorRequest]:
        E, t, I, N, R = self.p["hidden_size"], self.spec.tensors, self.inner, self.N, self.R
        return [TensorRequest(t["in"], (2 * I, E)), TensorRequest(t["conv"], (I, self.K), init="uniform:-0.6:0.6"),
                TensorRequest(t["conv_bias"], (I,), init="uniform:-0.1:0.1"), TensorRequest(t["x"], (R + 2 * N, I)),
                TensorRequest(t["dt"], (I, R), init="uniform:-0.3:0.3"), TensorRequest(t["dt_bias"], (I,), init="uniform:-4:-1"),
                TensorRequest(t["A_log"], (I, N), init="uniform:-1:1"), TensorRequest(t["D"], (I,), init="ones"),
                TensorRequest(t["o"], (E, I))]

    def load(self, store: WeightStore) -> None:
        w = {local: store.get(r) for local, r in zip(self.NAMES, self.tensor_requests())}
        dt = w["in"].dtype
        self.proj = Linear(w["in"], name="scan.in")
        self.taps = w["conv"].to(dt).contiguous()
        self.taps_t = self.taps.t().contiguous() if dt == torch.bfloat16 else None      # tap by tap, for 16-byte loads
        self.conv_bias = w["conv_bias"].to(dt).contiguous()
        self.low = Linear(w["x"], name="scan.low")
        self.dt_proj = Linear(w["dt"].to(dt).contiguous(), name="scan.dt")
        self.dt_bias = w["dt_bias"].to(torch.float32).contiguous()
        self.a_log = w["A_log"].to(torch.float32).contiguous()
        self.skip = w["D"].to(torch.float32).contiguous()
        self.o = Linear(w["o"], name="scan.o")

    graph_class = ()              # grids depend on the batch size only

    def forward(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        I, N, R = self.inner, self.N, self.R
        T = h.shape[0]
        proj = self.proj(h, ctx)
        ctx.mark("projections")
        x = ctx.ws.get("scan.conv", (T, I), ctx.dtype)
        carried = ctx.state(f"run{run.index}.conv") if self.K > 1 else None
        kernels.short_conv(proj[:, :I], self.taps, carried, ctx, x, taps_t=self.taps_t, bias=self.conv_bias, activation="silu")
        ctx.mark("conv")
        low = self.low(x, ctx)
        dt = self.dt_proj(low[:, :R], ctx, out_dtype=torch.float32)
        ctx.mark("low_rank")
        gated = ctx.ws.get("scan.gated", (T, I), ctx.dtype)
        kernels.selective_scan(x, proj[:, I:], low, R, N, dt, self.dt_bias, self.a_log, self.skip, ctx.state(f"run{run.index}.S"),
                               gated, ctx)
        ctx.mark("recurrence")
        term = self.o(gated, ctx, out_dtype=torch.float32)
        ctx.mark("o")
        return term
