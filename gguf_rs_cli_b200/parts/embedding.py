"""Token embedding (a row gather, src/model/llama.rs:349) and the output head
(logits = W h, src/model/llama.rs:406-407), which falls back to the embedding table
when the folder has no matrix of its own (src/model/llama.rs:124)."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import FUSE_MAX_TOKENS, Part, StepContext, Stream
from .linear import Linear
from .registry import register_embedding, register_head


@register_embedding("embedding")
class Embedding(Part):
    """params: vocab_size, hidden_size, scale (default 1: the rows are multiplied by it in 32-bit).
    tensors: weight [V, E]."""

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.spec.tensors["weight"], (self.p["vocab_size"], self.p["hidden_size"]))]

    graph_class = ()

    def load(self, store: WeightStore) -> None:
        self.weight = store.get(self.tensor_requests()[0])

    def forward(self, tokens: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        x = ctx.ws.get("x", (tokens.numel(), self.p["hidden_size"]), torch.float32)
        return kernels.embed(self.weight, tokens, x, float(self.p.get("scale", 1.0)))

    def forward_stream(self, tokens: torch.Tensor, ctx: StepContext, copy: Optional[torch.Tensor] = None) -> Stream:
        """The residual stream of a step; in bfloat16 mode with the shadow (bfloat16 copy and sums of
        squares per token) that lets the first norm be deferred into the product after it.  copy: a second
        float32 buffer [T, E] that receives the same rows (for models that add them to the stream again)."""
        if copy is not None:
            kernels.embed(self.weight, tokens, copy, float(self.p.get("scale", 1.0)))
        if ctx.dtype != torch.bfloat16 or tokens.numel() > FUSE_MAX_TOKENS:
            return Stream(self.forward(tokens, ctx))
        T, E = tokens.numel(), self.p["hidden_size"]
        stream = Stream(ctx.ws.get("x", (T, E), torch.float32))
        stream.xb = ctx.ws.get("stream.xb", (T, E), torch.bfloat16)
        stream.ssq = ctx.ws.get("stream.ssq", ((E + 127) // 128, T), torch.float32)
        stream.ssq_parts = 1
        kernels.embed_shadow(self.weight, tokens, stream.x, stream.xb, stream.ssq, float(self.p.get("scale", 1.0)))
        return stream


@register_embedding("embedding_bigram")
class HashedPairEmbedding(Embedding):
    """The token's row plus a row of a second table that the pair (previous token, token) chooses by a hash:
    row (previous * mul_prev + token * mul_cur) mod buckets, and the table's last row (number `buckets`) for a
    sequence's first token.  The previous token of a step's first token is per-sequence state.
    params: vocab_size, hidden_size, buckets, mul_prev, mul_cur, scale (default 1, of the token's row only).
    tensors: weight [V, E], pairs [buckets + 1, E]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if int(self.p["buckets"]) <= 0:
            raise ValueError(f"embedding_bigram: buckets must be positive, got {self.p['buckets']!r}")

    def tensor_requests(self) -> List[TensorRequest]:
        return super().tensor_requests() + [TensorRequest(self.spec.tensors["pairs"], (self.p["buckets"] + 1, self.p["hidden_size"]))]

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"prev": ((), "int32")}

    def load(self, store: WeightStore) -> None:
        reqs = self.tensor_requests()
        self.weight, self.pairs = store.get(reqs[0]), store.get(reqs[1])

    def forward(self, tokens: torch.Tensor, ctx: StepContext, copy: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = ctx.ws.get("x", (tokens.numel(), self.p["hidden_size"]), torch.float32)
        return kernels.embed_bigram(self.weight, self.pairs, ctx, ctx.state("embed.prev"), self.p["buckets"], self.p["mul_prev"],
                                    self.p["mul_cur"], x, copy=copy, scale=float(self.p.get("scale", 1.0)))

    def forward_stream(self, tokens: torch.Tensor, ctx: StepContext, copy: Optional[torch.Tensor] = None) -> Stream:
        return Stream(self.forward(tokens, ctx, copy=copy))


@register_head("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied_to (the tensor that stands in when the folder has no
    head matrix of its own, or None), tied (the configuration says the head is the embedding: the
    random-weights mode then writes no matrix for it), logit_scale (default 1: the logits are multiplied by it),
    softcap (default None; c: the logits become c tanh(logits / c), after the scale).
    tensors: weight [V, E].  As in the reference, presence decides: a folder that has the matrix
    uses it, one that lacks it uses `tied_to` (src/model/llama.rs:124)."""

    def tensor_requests(self) -> List[TensorRequest]:
        shape = (self.p["vocab_size"], self.p["hidden_size"])
        init = None if self.p.get("tied") else "normal"
        if self.p.get("tied_to"):
            return [TensorRequest(self.spec.tensors["weight"], shape, optional=True, fallback=self.p["tied_to"], init=init)]
        return [TensorRequest(self.spec.tensors["weight"], shape, init=init)]

    graph_class = ()

    def load(self, store: WeightStore) -> None:
        self.proj = Linear(store.get(self.tensor_requests()[0]), name="logits")

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = self.proj(h, ctx, out_dtype=torch.float32)
        scale = float(self.p.get("logit_scale", 1.0))
        if scale != 1.0:
            kernels.scale_(logits, scale)
        cap = self.p.get("softcap")
        return kernels.softcap_(logits, float(cap)) if cap else logits
