"""A per-layer token input: every layer adds to the residual stream a projection of its own slice of a second
embedding table, gated by the stream itself.

    e = table[token][col0 : col0 + dim]             (one table for the whole model, a slice per layer)
    g = act(W_gate x) * e                           (act: the tanh form of gelu by default)
    y = W_proj g
    x <- x + y / sqrt(mean(y^2) + eps) * w          (an RMS norm with a plain weight)

The gate's product, the activation and the projection run in the activation dtype with float32 sums; the norm and the
sum into the stream are float32.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import elementwise as K
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import Part, StepContext


class TokenSideInput(Part):
    def __init__(self, prefix: str, table_name: str, vocab: int, table_width: int, col0: int, dim: int, hidden: int,
                 eps: float, glu: K.Glu = K.GELU_TANH_GLU):
        if dim < 1 or col0 < 0 or col0 + dim > table_width:
            raise ValueError(f"token input '{prefix}': columns {col0}..{col0 + dim} of a table of {table_width}")
        self.prefix, self.table_name = prefix, table_name
        self.vocab, self.table_width, self.col0, self.dim = int(vocab), int(table_width), int(col0), int(dim)
        self.hidden, self.eps, self.glu = int(hidden), float(eps), glu
        self.table = self.w_gate = self.w_proj = self.w_norm = None

    def weight_specs(self) -> List[WeightSpec]:
        p = self.prefix
        return [WeightSpec(self.table_name, (self.vocab, self.table_width)), WeightSpec(p + "gate", (self.dim, self.hidden)),
                WeightSpec(p + "proj", (self.hidden, self.dim)), WeightSpec(p + "norm", (self.hidden,), init="one_plus_normal")]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        self.table = store.get(self.table_name)
        self.w_gate, self.w_proj, self.w_norm = store.get(p + "gate"), store.get(p + "proj"), store.get(p + "norm")

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        return {"matmul": (wb(self.w_gate) + wb(self.w_proj), 4.0 * n_tokens * self.hidden * self.dim)}

    def apply(self, x: torch.Tensor, ctx: StepContext, cast: Optional[torch.Tensor] = None, then=None):
        """x (float32 [T, hidden], the residual stream) is changed in place.  cast: x in the activation dtype, where
        the caller has it; then: a norm (weight, eps) that reads the new x next, taken in the same pass and returned
        (None where it was not)."""
        T, dev = x.shape[0], x.device
        exact = ctx.act_dtype == torch.float32
        h = x if exact else (cast if cast is not None else K.map_elements(x, torch.empty(x.shape, dtype=ctx.act_dtype, device=dev)))
        z = linear(h, self.w_gate, out_dtype=torch.float32)
        g = torch.empty((T, self.dim), dtype=ctx.act_dtype, device=dev)
        K.glu_table_rows(z, ctx.tokens, self.table, self.col0, g, self.glu)
        y = linear(g, self.w_proj, out_dtype=torch.float32)
        w = getattr(then, "weight", None)
        if w is not None and w.dtype == self.w_norm.dtype:
            out = torch.empty(x.shape, dtype=ctx.act_dtype, device=dev)
            K.add_rmsnorm(x, y, self.w_norm, self.eps, None, w, out, then.eps)
            return out
        K.add_rmsnorm(x, y, self.w_norm, self.eps)
        return None
