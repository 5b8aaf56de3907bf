"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/engine/tq_transformer.c:2494, 2268, 2685, 2701).

The residual sums are fused into the norm that follows them: a block receives the previous
sub-layer's output as `pending` and hands its own feed-forward output on the same way, so each
sum is one fp32 pass together with the next norm's statistics."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..kernels import elementwise as K
from ..weights.loader import WeightSpec, WeightStore
from .base import Block, FeedForward, KVNeed, LayerCache, Mixer, Norm, StateNeed, StepContext


class PreNormBlock(Block):
    """The feed-forward (and its norm) may be absent: the mixer's output is then what the block leaves open."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn: Optional[FeedForward] = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def cache_need(self) -> Optional[KVNeed]:
        return self.mixer.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.mixer.state_need()

    def capturable(self) -> bool:
        return self.mixer.capturable() and (self.ffn is None or self.ffn.capturable())

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def bind(self, store: WeightStore) -> None:
        for p in self.parts():
            p.bind(store)

    def kernels(self) -> List[str]:
        return [k for p in self.parts() for k in p.kernels()]

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, torch.Tensor]:
        if pending is None:
            xn = self.mixer_norm.forward(x, ctx.act_dtype)
        else:
            xn = self.mixer_norm.add_forward(x, pending, ctx.act_dtype)
        y = self.mixer.forward(xn, ctx, cache)
        if self.ffn is None:
            return x, y
        xn = self.ffn_norm.add_forward(x, y, ctx.act_dtype)
        return x, self.ffn.forward(xn, ctx)


class PostNormBlock(Block):
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the sub-layers read the residual stream itself and the
    norms sit on their outputs.  The feed-forward (and its norm) may be absent.  The stream stays float32; the
    sub-layers read it rounded to the activation dtype, and the first sum writes that copy for the second
    sub-layer in the same pass."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, ffn: Optional[FeedForward] = None, ffn_norm: Optional[Norm] = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def cache_need(self) -> Optional[KVNeed]:
        return self.mixer.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.mixer.state_need()

    def capturable(self) -> bool:
        return self.mixer.capturable() and (self.ffn is None or self.ffn.capturable())

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def bind(self, store: WeightStore) -> None:
        for p in self.parts():
            p.bind(store)

    def kernels(self) -> List[str]:
        return ["elementwise"] + [k for p in self.parts() for k in p.kernels()]

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        from ..kernels import elementwise as K
        if pending is not None:                      # a block of another kind ran before and left its sum open
            K.residual_add(x, pending)
        exact = ctx.act_dtype == torch.float32
        h = x if exact else K.map_elements(x, torch.empty(x.shape, dtype=ctx.act_dtype, device=x.device))
        y = self.mixer.forward(h, ctx, cache)
        if self.ffn is None:
            self.mixer_norm.add_normed(x, y)
            return x, None
        h = None if exact else torch.empty(x.shape, dtype=ctx.act_dtype, device=x.device)
        self.mixer_norm.add_normed(x, y, copy=h)
        y = self.ffn.forward(x if exact else h, ctx)
        self.ffn_norm.add_normed(x, y)
        return x, None


NORMED_STREAM = "normed_stream"       # StepContext.carry: the stream under the next block's first norm


class SandwichBlock(Block):
    """x += post_norm(mixer(pre_norm(x))); x += post_norm(feed_forward(pre_norm(x))): a norm before and one after each
    sub-layer.  The feed-forward (with its two norms) may be absent.  `after`: parts that change the stream once
    the sub-layers have run (`apply(x, ctx, cast, then)`, e.g. a per-layer token input).  The stream stays float32.
    `next_norm` (set by a model whose blocks run in a fixed order): the norm the next block starts with."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, mixer_post: Norm, ffn_norm: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None, ffn_post: Optional[Norm] = None, after=()):
        if len({ffn is None, ffn_norm is None, ffn_post is None}) != 1:
            raise ValueError("a feed-forward and its two norms come together")
        self.mixer_norm, self.mixer, self.mixer_post = mixer_norm, mixer, mixer_post
        self.ffn_norm, self.ffn, self.ffn_post = ffn_norm, ffn, ffn_post
        self.after = list(after)
        self.next_norm: Optional[Norm] = None        # the first norm of the block that runs next, if the model names it

    def parts(self):
        own = [self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post] + self.after
        out = []
        for p in own:
            if p is not None:
                out.append(p)
                out += p.parts() if hasattr(p, "parts") else []
        return out

    def _direct(self):
        return [p for p in [self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post] + self.after
                if p is not None]

    def cache_need(self) -> Optional[KVNeed]:
        return self.mixer.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.mixer.state_need()

    def capturable(self) -> bool:
        return self.mixer.capturable() and (self.ffn is None or self.ffn.capturable())

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self._direct() for s in p.weight_specs()]

    def bind(self, store: WeightStore) -> None:
        for p in self._direct():
            p.bind(store)

    def kernels(self) -> List[str]:
        return ["elementwise"] + [k for p in self._direct() for k in p.kernels()]

    @staticmethod
    def _add(norm: Norm, x, y, ctx, copy=None, then: Optional[Norm] = None):
        """x += norm(y); returns the norm `then` of the new x where it could be taken in the same pass, else None."""
        if then is None or not hasattr(norm, "weight"):
            norm.add_normed(x, y, copy)
            return None
        return norm.add_normed(x, y, copy, then=then, then_dtype=ctx.act_dtype)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        # the block before may have taken this block's first norm along with its last sum (`next_norm`)
        xn = ctx.carry.pop(NORMED_STREAM, None) if ctx.carry is not None else None
        if pending is not None:                      # a block of another kind ran before and left its sum open
            xn = self.mixer_norm.add_forward(x, pending, ctx.act_dtype)
        elif xn is None:
            xn = self.mixer_norm.forward(x, ctx.act_dtype)
        # every sum into the stream takes the norm that reads the stream next along: the feed-forward's, or, from
        # the block's last sum, the next block's first; the parts after the sub-layers get the stream in the
        # activation dtype from the sum before them
        exact = ctx.act_dtype == torch.float32
        n_after = len(self.after)
        cast = lambda wanted: torch.empty(x.shape, dtype=ctx.act_dtype, device=x.device) if wanted and not exact else None
        out_norm = self.next_norm if ctx.carry is not None else None
        last = self.ffn is None and not n_after
        h = cast(self.ffn is None and n_after)
        then = self.ffn_norm if self.ffn is not None else (out_norm if last else None)
        done = False
        if hasattr(self.mixer, "forward_branches") and hasattr(self.mixer_post, "add_normed_pair"):
            # a mixer of two normed branches: their norms and mean run inside the sum's pass
            pair = self.mixer.forward_branches(xn, ctx, cache)
            done, xn = self.mixer_post.add_normed_pair(x, pair, h, then=then, then_dtype=ctx.act_dtype)
            if not done:
                a, wa, b, wb, eps = pair
                xn = self._add(self.mixer_post, x, K.mean_of_norms(a, wa, b, wb, eps, torch.empty_like(a)), ctx, copy=h, then=then)
        else:
            xn = self._add(self.mixer_post, x, self.mixer.forward(xn, ctx, cache), ctx, copy=h, then=then)
        if self.ffn is not None:
            if xn is None:
                xn = self.ffn_norm.forward(x, ctx.act_dtype)
            h = cast(n_after)
            xn = self._add(self.ffn_post, x, self.ffn.forward(xn, ctx), ctx, copy=h, then=None if n_after else out_norm)
        for k, part in enumerate(self.after):
            xn = part.apply(x, ctx, cast=h if k == 0 else None, then=out_norm if k == n_after - 1 else None)
        if xn is not None and out_norm is not None:
            ctx.carry[NORMED_STREAM] = xn
        return x, None


KEPT_STREAMS = "kept_streams"       # StepContext.carry: the stream as the embedding and every layer so far left it


class DepthMixBlock(Block):
    """A pre-norm block with a factor on its sums, a token shift ahead of the mixer and a weighted sum over depth:

        h = shift(norm1(x));  y = x + r * mixer(h);  X = y + r * feed_forward(norm2(y))      (the second sum only with a
                                                                                              feed-forward)
        shift(h)_t = h_t + (h_(t-1) - h_t) * s       s: the tensor `shift_name`; h_(t-1) unshifted, zero before a sequence's
                                                     first token; a sequence keeps its last h (None: no shift)
        x <- sum_j depth[j] * X_j                    over the embedding's output X_0 and the results X_1 .. of all blocks
                                                     up to this one (`depth_name`: weights [index + 2]; None: x <- X)

    index: how many blocks of this kind ran before this one in the model (the blocks share the kept streams through
    the step's carry; `depth_total` of them, the embedding's output included, are kept).  The norms are DynamicTanh
    (`shifted`, `add_forward(scale=)`).  The stream stays float32.  The sequence's kept row of the shift lies ahead of
    the mixer's own state in the block's state row."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn: Optional[FeedForward] = None,
                 hidden: int = 0, residual_mult: float = 1.0, shift_name: Optional[str] = None,
                 depth_name: Optional[str] = None, index: int = 0, depth_total: int = 0):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        if hidden < 1 or index < 0 or (depth_name is not None and depth_total < index + 2):
            raise ValueError(f"block: width {hidden}, place {index} of {depth_total} kept streams")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.hidden, self.mult, self.shift_name, self.depth_name = int(hidden), float(residual_mult), shift_name, depth_name
        self.index, self.depth_total = int(index), int(depth_total)
        self.shift: Optional[torch.Tensor] = None
        self.depth: Optional[torch.Tensor] = None

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def cache_need(self) -> Optional[KVNeed]:
        return self.mixer.cache_need()

    def _own_state(self) -> int:
        return self.hidden if self.shift_name is not None else 0

    def state_need(self) -> Optional[StateNeed]:
        inner = self.mixer.state_need()
        if inner is not None and (inner.dtype != torch.float32 or len(inner.shape) != 1):
            raise ValueError("block: a mixer behind a token shift keeps its state as one float32 row")
        size = self._own_state() + (inner.shape[0] if inner is not None else 0)
        return StateNeed((size,), torch.float32) if size else None

    def capturable(self) -> bool:
        return self.mixer.capturable() and (self.ffn is None or self.ffn.capturable())

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self.parts() for s in p.weight_specs()]
        if self.shift_name is not None:
            specs.append(WeightSpec(self.shift_name, (self.hidden,)))
        if self.depth_name is not None:
            specs.append(WeightSpec(self.depth_name, (self.index + 2,), init="one_plus_normal"))
        return specs

    def bind(self, store: WeightStore) -> None:
        for p in self.parts():
            p.bind(store)
        if self.shift_name is not None:
            self.shift = store.get(self.shift_name)
        if self.depth_name is not None:
            self.depth = store.get(self.depth_name).float().contiguous()

    def kernels(self) -> List[str]:
        return ["elementwise"] + [k for p in self.parts() for k in p.kernels()]

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if pending is not None:                      # a block of another kind ran before and left its sum open
            K.residual_add(x, pending)
        hist = None
        if self.depth is not None:
            hist = ctx.carry.get(KEPT_STREAMS)
            if hist is None:
                hist = ctx.carry[KEPT_STREAMS] = torch.empty((self.depth_total,) + tuple(x.shape), dtype=torch.float32, device=x.device)
                hist[0].copy_(x)
        own = self._own_state()
        if own:
            h = self.mixer_norm.shifted(x, ctx.act_dtype, self.shift, cache.state[:, :own], ctx)
        else:
            h = self.mixer_norm.forward(x, ctx.act_dtype)
        inner = cache
        if cache.state is not None and own:
            inner = LayerCache(kv=cache.kv, page_table=cache.page_table, page_size=cache.page_size, writes=cache.writes,
                               state=cache.state[:, own:] if cache.state.shape[1] > own else None)
        y = self.mixer.forward(h, ctx, inner)
        f = bias = None
        if self.ffn is not None:
            xn = self.ffn_norm.add_forward(x, y, ctx.act_dtype, scale=self.mult)          # x += r * y on the way
            bias = getattr(self.ffn, "down_bias", None)
            f = self.ffn.forward(xn, ctx, leave_bias=True) if bias is not None else self.ffn.forward(xn, ctx)
        else:
            f = y
        if hist is None:
            K.residual_add(x, f if self.mult == 1.0 and bias is None else _scaled(f, self.mult, bias))
            return x, None
        K.depth_mix(hist, self.index + 1, x, self.depth, x, add=f, add_scale=self.mult, bias=bias)
        return x, None


def _scaled(f: torch.Tensor, mult: float, bias: Optional[torch.Tensor]) -> torch.Tensor:
    f = f.float() if f.dtype != torch.float32 else f
    return K.scale_bias_cols(f, mult, None if bias is None else (bias.float() * mult).contiguous())
