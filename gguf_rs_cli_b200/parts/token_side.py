"""An input of a layer's own that depends on the token alone: a table with a row per token holds `dim` columns for
every layer; the layer's slice gates a low-rank view of the residual stream and is projected back,
    y = W_proj (act(W_gate x) * table[token, offset : offset + dim]),
which the block norms into the stream.  The reference has no such part (src/model/llama.rs adds nothing to the stream but
attention and the feed-forward).
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import Part, StepContext
from .linear import Linear
from .registry import register_extra


@register_extra("token_side")
class TokenSide(Part):
    """params: hidden_size, vocab_size, dim, columns (of the whole table: all layers' slices), offset (this layer's
    first column), activation ("gelu_tanh" or "silu").  tensors: table [vocab, columns] (one tensor for all layers),
    gate [dim, E], proj [E, dim]."""

    def tensor_requests(self) -> List[TensorRequest]:
        p, t = self.p, self.spec.tensors
        return [TensorRequest(t["table"], (p["vocab_size"], p["columns"])), TensorRequest(t["gate"], (p["dim"], p["hidden_size"])),
                TensorRequest(t["proj"], (p["hidden_size"], p["dim"]))]

    def load(self, store: WeightStore) -> None:
        table, gate, proj = (store.get(r) for r in self.tensor_requests())
        self.table = table
        self.gate, self.proj = Linear(gate, name="side.gate"), Linear(proj, name="side.proj")
        if not 0 <= self.p["offset"] <= self.p["columns"] - self.p["dim"]:
            raise ValueError(f"token_side: columns {self.p['offset']} .. of {self.p['columns']} do not hold {self.p['dim']}")

    graph_class = ()

    def forward(self, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """rows: x as products read it [T, E]; returns y float32 [T, E]."""
        a = self.gate(rows, ctx)
        g = ctx.ws.get("side.gated", a.shape, ctx.dtype)
        kernels.token_side_gate(a, self.table, self.p["offset"], ctx.tokens, g, self.p.get("activation", "gelu_tanh"))
        return self.proj(g, ctx, out_dtype=torch.float32)
