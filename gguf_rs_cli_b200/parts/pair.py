"""Two mixers side by side as the mixer of a layer: both read the same rows, each result is brought to unit root mean
square over the model's width and multiplied by a weight of its own, and the mixer gives `mix` times their sum
(mix 0.5: their mean).  The branches are parts of the mixer registry; cache and state are theirs (at most one of them
may keep keys and values).  The reference has no such arrangement.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..cache.cache import KVSpec
from ..config.specs import PartSpec
from ..weights.loader import TensorRequest, WeightStore
from .base import Blend, HostBatch, Part, RunView, StepContext
from .registry import MIXERS, register_mixer


class _Prefixed:
    """A run as a branch sees it: its states are named <branch>.<name> in the layer's run."""

    def __init__(self, run: RunView, prefix: str):
        self._run, self._prefix = run, prefix

    def __getattr__(self, name):
        return getattr(self._run, name)

    @property
    def index(self):
        return f"{self._run.index}.{self._prefix}"


@register_mixer("pair")
class MixerPair(Part):
    """params: hidden_size, eps, mix (default 0.5), left, right (PartSpecs of two mixers), left_position (an object the
    decoder built, given through `position`).  tensors: left_out [E], right_out [E] (plain weights)."""

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.left = MIXERS.get(p["left"].kind)(p["left"], dtype, device, position=position)
        self.right = MIXERS.get(p["right"].kind)(p["right"], dtype, device, position=None)
        self.branches = (("left", self.left), ("right", self.right))
        self.mix = float(p.get("mix", 0.5))
        if sum(b.kv_spec() is not None for _, b in self.branches) > 1:
            raise ValueError("pair: at most one of two mixers side by side may keep keys and values")
        if p["left"].kind == p["right"].kind:
            raise ValueError("pair: two mixers of one kind would write their results into the same buffers of the step")
        if any(getattr(b, "shares_kv", False) for _, b in self.branches):
            raise ValueError("pair: a branch cannot read another run's keys and values")

    def kv_spec(self) -> Optional[KVSpec]:
        for _, b in self.branches:
            if b.kv_spec() is not None:
                return b.kv_spec()
        return None

    def reads_kv_spec(self) -> Optional[KVSpec]:
        return self.kv_spec()

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {f"{name}.{k}": v for name, b in self.branches for k, v in b.state_spec().items()}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t = self.p["hidden_size"], self.spec.tensors
        req = [r for _, b in self.branches for r in b.tensor_requests()]
        return req + [TensorRequest(t["left_out"], (E,), init="ones"), TensorRequest(t["right_out"], (E,), init="ones")]

    def load(self, store: WeightStore) -> None:
        for _, b in self.branches:
            b.load(store)
        wl, wr = (store.get(r) for r in self.tensor_requests()[-2:])
        self.weights = (wl, wr if wr.dtype == wl.dtype else wr.to(wl.dtype))

    # ---- planning and capture: the branches'
    def plan_key(self):
        from .base import plan_key_of
        return ("pair",) + tuple(plan_key_of(b) for _, b in self.branches)

    def plan(self, batch: HostBatch):
        out = {}
        for name, b in self.branches:
            if hasattr(b, "plan"):
                out.update({f"{name}.{k}": v for k, v in b.plan(batch).items()})
        return out

    def graph_class(self, batch: HostBatch):
        classes = []
        for _, b in self.branches:
            gc = getattr(b, "graph_class", None)
            c = gc(batch) if callable(gc) else gc
            if c is None:
                return None
            classes.append(c)
        return tuple(classes)

    def forward_blend(self, h, ctx: StepContext, run: RunView) -> Blend:
        terms = []
        for name, b in self.branches:
            if hasattr(b, "plan"):
                # the branch finds its own index arrays under its own key
                mine = {k[len(name) + 1:]: v for k, v in ctx.plan_of(self).items() if k.startswith(name + ".")}
                from .base import plan_key_of
                ctx.plans[plan_key_of(b)] = mine
            term = b.forward(h, ctx, _Prefixed(run, name))
            if term is None or term.dim() != 2:
                raise RuntimeError("pair: a branch must give one term [tokens, width]")
            terms.append(term)
        return Blend(terms[0], terms[1], self.weights, self.mix, float(self.p["eps"]))

    def forward(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        """The blended term itself, for arrangements that do not finish it in their own kernel."""
        b = self.forward_blend(h, ctx, run)
        out = ctx.ws.get("pair.out", b.a.shape, torch.float32)
        kernels.norm_sandwich(None, b.a, None, b.eps, y2=b.b, inner_weights=b.weights, mix=b.mix, u_out=out)
        return out
