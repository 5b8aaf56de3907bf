"""RMSNorm: ss = sum(x^2)/n + eps; y = x * (1/sqrt(ss)) * w, the weight used as it is
(src/engine/tq_ops.c:1373-1410).  Reads the fp32 residual stream; statistics in fp32."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import elementwise as K
from ..weights.loader import WeightSpec, WeightStore
from .base import Norm, register_norm


class RMSNorm(Norm):
    def __init__(self, name: str, size: int, eps: float, around_zero: bool = False):
        """around_zero: the stored weight is the distance from one (y = x / rms * (1 + w)); the sum 1 + w is taken
        once, when the weights are bound, and kept in float32 (in bfloat16 it would lose the weight's low bits)."""
        if size < 1 or not eps > 0.0:
            raise ValueError(f"RMSNorm '{name}': size {size} and eps {eps} must be positive")
        self.name, self.size, self.eps, self.around_zero = name, int(size), float(eps), bool(around_zero)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), init="normal" if self.around_zero else "one_plus_normal")]

    def bind(self, store: WeightStore) -> None:
        self.weight = store.get(self.name)
        if self.around_zero:
            self.weight = (self.weight.float() + 1.0).contiguous()

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def forward(self, x, out_dtype, rows=None, add=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        return K.rmsnorm(x, self.weight, self.eps, out, add=add, rows=rows)

    def add_forward(self, x, y, out_dtype):
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        return K.rmsnorm(x, self.weight, self.eps, out, add=y)

    def add_normed(self, x, y, copy=None, then=None, then_dtype=None):
        """x += norm(y).  then (an RMSNorm of the same weight dtype): its norm of the new x is taken in the same pass
        and returned in then_dtype (None where the two weights' dtypes differ: the caller runs it by itself)."""
        if then is not None and isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype and \
                (copy is None or copy.dtype == then_dtype):
            out = torch.empty((x.shape[0], self.size), dtype=then_dtype, device=x.device)
            K.add_rmsnorm(x, y, self.weight, self.eps, copy, then.weight, out, then.eps)
            return out
        K.add_rmsnorm(x, y, self.weight, self.eps, copy)
        return None if then is not None else x


    def add_normed_pair(self, x, pair, copy=None, then=None, then_dtype=None):
        """x += norm(mean of two normed branches); pair = (a, wa, b, wb, eps) as a mixer of two branches leaves them
        (`forward_branches`).  Returns (done, normed): done False where the weights' dtypes differ and nothing was
        computed; normed: the norm `then` of the new x where it was taken along, else None."""
        a, wa, b, wb, pair_eps = pair
        if wa.dtype != self.weight.dtype or wb.dtype != self.weight.dtype:
            return False, None
        if then is not None and isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype and \
                (copy is None or copy.dtype == then_dtype):
            out = torch.empty((x.shape[0], self.size), dtype=then_dtype, device=x.device)
            K.add_rmsnorm_pair(x, a, wa, b, wb, pair_eps, self.weight, self.eps, copy, then.weight, out, then.eps)
            return True, out
        K.add_rmsnorm_pair(x, a, wa, b, wb, pair_eps, self.weight, self.eps, copy)
        return True, None

register_norm("rmsnorm", RMSNorm)


class DynamicTanh(Norm):
    """A norm without statistics: y = tanh(alpha * x) * w + b, with a learned scalar alpha (tensor `<name>.alpha`), a
    weight `<name>` and a bias `<name>.b`.  Reads the fp32 residual stream; computed in fp32.  The sums that other
    norms take along (`add`, `add_forward`) may carry a factor: x += scale * y.  `shifted()` mixes every token's
    output with that of the token before it (see there)."""

    def __init__(self, name: str, size: int):
        if size < 1:
            raise ValueError(f"DynamicTanh '{name}': size {size} must be positive")
        self.name, self.size = name, int(size)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha = 1.0

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), init="one_plus_normal"), WeightSpec(self.name + ".b", (self.size,)),
                WeightSpec(self.name + ".alpha", (), init="one_plus_normal")]

    def bind(self, store: WeightStore) -> None:
        self.weight, self.bias = store.get(self.name), store.get(self.name + ".b")
        if self.bias.dtype != self.weight.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()
        self.alpha = float(store.get(self.name + ".alpha").float().item())

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def forward(self, x, out_dtype, rows=None, add=None, add_scale: float = 1.0):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        return K.dyt(x, self.alpha, self.weight, self.bias, out, add=add, add_scale=add_scale, rows=rows)

    def add_forward(self, x, y, out_dtype, scale: float = 1.0):
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        return K.dyt(x, self.alpha, self.weight, self.bias, out, add=y, add_scale=scale)

    def shifted(self, x, out_dtype, shift: torch.Tensor, kept: torch.Tensor, ctx) -> torch.Tensor:
        """h_t + (h_(t-1) - h_t) * shift with h = this norm of x: h_(t-1) is the row above inside a sequence's run of
        new tokens and the sequence's kept row (kept [max_slots, size] float32, zero at its start) for the run's
        first token; the kept rows then take the runs' last outputs."""
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        if shift.dtype != self.weight.dtype:
            shift = shift.to(self.weight.dtype)
        return K.dyt(x, self.alpha, self.weight, self.bias, out, shift=shift, state=kept, seq_of_token=ctx.seq_of_token,
                     cu_seqlens=ctx.cu_seqlens, slots=ctx.slots, single_tokens=ctx.max_q_len == 1)


register_norm("dyt", DynamicTanh)
