"""Two mixers side by side: both read the same input, each output passes an RMS norm of its own (a plain weight over
the model width), and the result is half their sum.

    y = (norm_left(left(h)) + norm_right(right(h))) / 2

The branches are mixers of any kind; one may keep keys and values, one a per-sequence state (the block hands the
pair's needs on: the cache of whichever branch asks for one, the state likewise).  When both branches offer their
fused input projection (`input_weight()` and `forward(..., projected=...)`), the two projections run as one product.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import elementwise as K
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import KVNeed, LayerCache, Mixer, StateNeed, StepContext, register_mixer


class ParallelMixer(Mixer):
    def __init__(self, left: Mixer, right: Mixer, hidden: int, eps: float, left_norm: str, right_norm: str):
        """left_norm, right_norm: the names of the two norms' weights."""
        needs = [m.cache_need() for m in (left, right)]
        states = [m.state_need() for m in (left, right)]
        if all(n is not None for n in needs) or all(s is not None for s in states):
            raise ValueError("mixers side by side: at most one branch may keep keys and values, and one a state")
        self.left, self.right, self.hidden, self.eps = left, right, int(hidden), float(eps)
        self.left_norm, self.right_norm = left_norm, right_norm
        self.w_left = self.w_right = self.w_in = None

    def parts(self):
        return [self.left, self.right]

    def weight_specs(self) -> List[WeightSpec]:
        return (self.left.weight_specs() + self.right.weight_specs() +
                [WeightSpec(self.left_norm, (self.hidden,), init="one_plus_normal"),
                 WeightSpec(self.right_norm, (self.hidden,), init="one_plus_normal")])

    def bind(self, store: WeightStore) -> None:
        self.left.bind(store)
        self.right.bind(store)
        self.w_left, self.w_right = store.get(self.left_norm), store.get(self.right_norm)
        if self.w_left.dtype != self.w_right.dtype:
            self.w_left, self.w_right = self.w_left.float(), self.w_right.float()
        if all(hasattr(m, "input_weight") for m in (self.left, self.right)):
            a, b = self.left.input_weight(), self.right.input_weight()
            if a.dtype == b.dtype:
                self.w_in = torch.cat([a, b], dim=0).contiguous()       # one product for both branches
                self.left.w_qkv = self.w_in[:a.shape[0]]                # the branches keep views of it
                self.right.w_in = self.w_in[a.shape[0]:]

    def kernels(self) -> List[str]:
        return ["elementwise"] + self.left.kernels() + self.right.kernels()

    def cache_need(self) -> Optional[KVNeed]:
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.left.state_need() or self.right.state_need()

    def capturable(self) -> bool:
        return self.left.capturable() and self.right.capturable()

    def step_work(self, n_tokens, kv_tokens):
        return {}                # the branches are listed among the block's parts and say what they do themselves

    def forward_branches(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache):
        """The two branches' outputs before their norms, (a, w_left, b, w_right, eps), for a block whose norm on the
        mixer's output takes the branches' norms and their mean in its own pass."""
        if self.w_in is not None:
            proj = linear(xn, self.w_in, out_dtype=torch.float32)
            a = self.left.forward(xn, ctx, cache, projected=proj)
            b = self.right.forward(xn, ctx, cache, projected=proj, offset=self.left.input_weight().shape[0])
        else:
            a = self.left.forward(xn, ctx, cache)
            b = self.right.forward(xn, ctx, cache)
        return a, self.w_left, b, self.w_right, self.eps

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        a, wa, b, wb, eps = self.forward_branches(xn, ctx, cache)
        out = torch.empty((xn.shape[0], self.hidden), dtype=torch.float32, device=xn.device)
        return K.mean_of_norms(a, wa, b, wb, eps, out)


register_mixer("parallel", ParallelMixer)
