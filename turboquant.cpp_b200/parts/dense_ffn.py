"""Dense SwiGLU feed-forward: down(silu(gate x) * (up x)) (src/engine/tq_transformer.c:2771-2806;
silu with exact exp, src/engine/tq_ops.c:1454-1478).  Gate and up are one fused product."""
from __future__ import annotations

from typing import List

import torch

from ..kernels import elementwise as K
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import FeedForward, StepContext, register_feed_forward


class SwiGLUFeedForward(FeedForward):
    def __init__(self, prefix: str, hidden: int, intermediate: int):
        if hidden < 1 or intermediate < 1:
            raise ValueError(f"feed-forward '{prefix}': sizes must be positive, got {hidden}, {intermediate}")
        self.prefix, self.hidden, self.intermediate = prefix, int(hidden), int(intermediate)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        p, H, I = self.prefix, self.hidden, self.intermediate
        return [WeightSpec(p + "gate_proj.weight", (I, H)), WeightSpec(p + "up_proj.weight", (I, H)),
                WeightSpec(p + "down_proj.weight", (H, I))]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        g, u = store.take(p + "gate_proj.weight"), store.take(p + "up_proj.weight")
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = store.get(p + "down_proj.weight")

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        return {"matmul": (wb(self.w_gate_up) + wb(self.w_down), 6.0 * n_tokens * self.hidden * self.intermediate)}

    def forward(self, xn: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(xn, self.w_gate_up, out_dtype=torch.float32)     # gate and up stay fp32 until the product
        h = torch.empty((xn.shape[0], self.intermediate), dtype=ctx.act_dtype, device=xn.device)
        K.silu_mul(gu, h)
        return linear(h, self.w_down, out_dtype=torch.float32)


register_feed_forward("swiglu", SwiGLUFeedForward)


class GluFeedForward(FeedForward):
    """down(glu(gate x, up x)) with a gated activation given by its constants (kernels.elementwise.Glu: caps on gate
    and up, the slope inside the sigmoid, an offset on up); the tensors' names are parameters.  Gate and up are
    one fused product whose float32 result the activation reads."""

    def __init__(self, prefix: str, hidden: int, intermediate: int, glu: K.Glu = K.SILU_GLU, gate_name: str = "gate",
                 up_name: str = "up", down_name: str = "down"):
        if hidden < 1 or intermediate < 1:
            raise ValueError(f"feed-forward '{prefix}': sizes must be positive, got {hidden}, {intermediate}")
        self.prefix, self.hidden, self.intermediate, self.glu = prefix, int(hidden), int(intermediate), glu
        self.names = (gate_name, up_name, down_name)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        p, H, I = self.prefix, self.hidden, self.intermediate
        return [WeightSpec(p + self.names[0], (I, H)), WeightSpec(p + self.names[1], (I, H)),
                WeightSpec(p + self.names[2], (H, I))]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        g, u = store.take(p + self.names[0]), store.take(p + self.names[1])
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = store.get(p + self.names[2])

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        return {"matmul": (wb(self.w_gate_up) + wb(self.w_down), 6.0 * n_tokens * self.hidden * self.intermediate)}

    def forward(self, xn: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(xn, self.w_gate_up, out_dtype=torch.float32)
        h = torch.empty((xn.shape[0], self.intermediate), dtype=ctx.act_dtype, device=xn.device)
        K.glu_mul(gu, h, self.glu)
        return linear(h, self.w_down, out_dtype=torch.float32)


register_feed_forward("glu", GluFeedForward)


class ReluSquaredFeedForward(FeedForward):
    """down(relu(up x)^2): one product up, the square of relu, one product down.  bias: both products have one
    (`<name>.b`); a block that adds this part's output to the stream may take the second bias into that sum
    (`forward(..., leave_bias=True)` and `down_bias`)."""

    def __init__(self, prefix: str, hidden: int, intermediate: int, up_name: str = "up", down_name: str = "down", bias: bool = False):
        if hidden < 1 or intermediate < 1:
            raise ValueError(f"feed-forward '{prefix}': sizes must be positive, got {hidden}, {intermediate}")
        self.prefix, self.hidden, self.intermediate = prefix, int(hidden), int(intermediate)
        self.up_name, self.down_name, self.has_bias = up_name, down_name, bool(bias)
        self.w_up = self.w_down = self.up_bias = self.down_bias = None

    def weight_specs(self) -> List[WeightSpec]:
        p = self.prefix
        specs = [WeightSpec(p + self.up_name, (self.intermediate, self.hidden)),
                 WeightSpec(p + self.down_name, (self.hidden, self.intermediate))]
        if self.has_bias:
            specs += [WeightSpec(p + self.up_name + ".b", (self.intermediate,)), WeightSpec(p + self.down_name + ".b", (self.hidden,))]
        return specs

    def bind(self, store: WeightStore) -> None:
        self.w_up, self.w_down = store.get(self.prefix + self.up_name), store.get(self.prefix + self.down_name)
        if self.has_bias:
            self.up_bias, self.down_bias = store.get(self.prefix + self.up_name + ".b"), store.get(self.prefix + self.down_name + ".b")

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        return {"matmul": (wb(self.w_up) + wb(self.w_down), 4.0 * n_tokens * self.hidden * self.intermediate)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, leave_bias: bool = False) -> torch.Tensor:
        u = linear(xn, self.w_up, out_dtype=torch.float32)          # fp32 until the activation has been taken
        h = torch.empty((xn.shape[0], self.intermediate), dtype=ctx.act_dtype, device=xn.device)
        if self.up_bias is not None:
            K.bias_map(u, self.up_bias, h, K.MAP_RELU_SQUARED)
        else:
            K.map_elements(u, h, K.MAP_RELU_SQUARED)
        y = linear(h, self.w_down, out_dtype=torch.float32)
        if self.down_bias is not None and not leave_bias:
            K.add_bias(y, self.down_bias)
        return y


register_feed_forward("relu2", ReluSquaredFeedForward)
