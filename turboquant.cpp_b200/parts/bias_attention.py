"""Attention with a learned distance bias, a window that keeps a sequence's first positions, a sink in the softmax
and values mixed across layers.  No rotation: positions enter through the bias and the mask only.

With h the mixer's input, H query heads on G key/value heads (head a reads a // (H / G)), key size dk, value size dv:

    q = W_q h, k = W_k h, v = W_v h                                    (one fused product, float32 result)
    score(i, j) = q_i . k_j * scale + rel[bucket(i - j)][a]
    bucket(n)   = n                                                    for n < B / 2           (B rows in rel)
                = min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(far / (B/2)) * (B - B/2)))   otherwise
    i sees j    iff j <= i and (i - j < window or j < keep_first)
    p_j         = exp(score_j) / (1 + sum of exp(score_j) over the visible j)
    out_i       = W_o concat_a sum_j p_j v_j

The bucket depends on the distance alone, so the table is spread out per distance once, when the weights are bound
(distances from `far` on share the last row), and the kernels add row min(i - j, far).  The one in the denominator
is a sink of score 0: the kernels take a sink per head, here zeros.  Value mixing (`mix_values`): the first mixer of
a model that mixes keeps its values under a name in the step's `carry`; every later one turns its own into
(1 - lambda) v + lambda v_first before they are cached, lambda being the layer's scalar tensor `vmix`.
A position's cache row is [k | v] per key/value head (one plane).

Options other designs use: a rotation of queries and keys (`position`: an encoding that gives float32 frequencies, the
first `dims` elements of each head), a unit norm on every query and key head after it (`unit_eps` > 0: the head divided
by sqrt(mean(head^2) + unit_eps), no weight), a cap on the scaled score (`softcap` > 0: s <- softcap * tanh(s / softcap),
before any bias), and a learned sink per head (`sink_name`: the tensor's name below the prefix) instead of the zero one.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..kernels import bias_attention as KB
from ..kernels import gemv as KG
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import KVNeed, LayerCache, Mixer, StepContext, register_mixer


def distance_buckets(rows: int, far: int) -> List[int]:
    """bucket(n) for n = 0 .. far (every distance beyond `far` falls into the last row, as `far` itself does)."""
    half = rows // 2
    out = []
    for n in range(far + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


def paged_attention(q: torch.Tensor, cache: LayerCache, ctx: StepContext, heads: int, kv_heads: int, dim: int, vdim: int,
                    scale: float, window: int = 0, keep_first: int = 0, bias: Optional[torch.Tensor] = None,
                    bias_t: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    cell: int = 0, runs_min: int = 16) -> torch.Tensor:
    """Softmax attention of the step's queries q [T, heads, dim] over the rows [k | v] of a paged cache, [T, heads *
    vdim] in the activation dtype: the kernel for runs of new tokens where the step has a run of runs_min tokens and
    the shape is one it is built for, else one of the token forms with the visible keys cut into ranges.  The mask
    is a window (with a sequence's first positions kept) or, with cell > 0, the query's own cell of positions."""
    T, act, dev = q.shape[0], ctx.act_dtype, q.device
    o = torch.empty((T, heads * vdim), dtype=act, device=dev)
    if ctx.max_q_len >= runs_min and KB.runs_usable(act, dim, vdim, cache.page_size):
        return KB.attention_runs(q, cache.kv, bias_t, sink, ctx.cu_seqlens, ctx.seq_start, cache.page_table, cache.page_size,
                                 window, keep_first, scale, o, ctx.n_seqs, ctx.max_q_len, heads, kv_heads, dim, vdim,
                                 softcap=softcap, cell=cell)
    if cell:
        longest = min(cell, ctx.max_kv_len)
    else:
        longest = min(window + keep_first, ctx.max_kv_len) if window else ctx.max_kv_len
    per_kv = heads // kv_heads
    gc = KB.group_heads(act, dim, vdim, per_kv)
    blocks = kv_heads * -(-per_kv // gc) if gc else heads
    unit = 8
    if KB.heads_form(act, dim, vdim, per_kv, cache.page_size):
        blocks, unit = kv_heads * -(-per_kv // 16), 16
    return KB.attention(q, cache.kv, bias, sink, ctx.positions, ctx.seq_of_token, cache.page_table, cache.page_size,
                        window, keep_first, scale, o, heads, kv_heads, dim, vdim,
                        n_splits=KB.splits_for(T, blocks, longest, dev, unit), bias_t=bias_t, softcap=softcap, cell=cell)


class BiasedWindowAttentionMixer(Mixer):
    RUNS_MIN = 16             # steps whose longest run of new tokens is at least this take the kernel for runs

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int = 0, keep_first: int = 0, bias_rows: int = 0, bias_far: int = 0, sink: bool = True,
                 mix_values: Optional[str] = None, mix_first: bool = False, position=None, unit_eps: float = 0.0,
                 softcap: float = 0.0, sink_name: Optional[str] = None):
        """bias_rows: rows of the bias table `rel` (0: no bias; -1: as many as the stored tensor has); bias_far: the
        distance from which all share the last row.  mix_values: the name under which the model's mixing layers share values in a step's carry (None: this
        layer does not mix); mix_first: this layer is the one that provides them."""
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"attention '{prefix}': {heads} heads are not a multiple of {kv_heads} key/value heads")
        if not (1 <= dim <= KB.MAX_DIM and 1 <= vdim <= KB.MAX_DIM):
            raise ValueError(f"attention '{prefix}': key size {dim} and value size {vdim} must be in 1..{KB.MAX_DIM}")
        if unit_eps < 0.0 or softcap < 0.0:
            raise ValueError(f"attention '{prefix}': the unit norm's eps {unit_eps} and the cap {softcap} must not be negative")
        if position is not None and (not hasattr(position, "freq") or position.dims > dim):
            raise ValueError(f"attention '{prefix}': the position encoding must give frequencies for at most {dim} elements")
        if (position is not None or unit_eps > 0.0) and mix_values is not None:
            raise ValueError(f"attention '{prefix}': mixed values come without rotation and unit norm")
        self.position, self.unit_eps, self.softcap, self.sink_name = position, float(unit_eps), float(softcap), sink_name
        if window < 0 or keep_first < 0:
            raise ValueError(f"attention '{prefix}': negative window {window} or kept positions {keep_first}")
        if bias_rows > 0:
            self._check_bias(prefix, bias_rows, bias_far)
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.window, self.keep_first = float(scale), int(window), int(keep_first) if window else 0
        self.bias_rows, self.bias_far, self.has_sink = int(bias_rows), int(bias_far), bool(sink) or sink_name is not None
        self.mix_values, self.mix_first = mix_values, bool(mix_first)
        self.q_size, self.k_size, self.v_size = heads * dim, kv_heads * dim, kv_heads * vdim
        self.w_qkv = self.w_o = self.bias = self.bias_t = self.sink = None
        self.mix = 0.0

    @staticmethod
    def _check_bias(prefix: str, rows: int, far: int) -> None:
        if rows < 2 or far <= rows // 2:
            raise ValueError(f"attention '{prefix}': a bias table of {rows} rows needs a far distance beyond "
                             f"{rows // 2}, got {far}")

    def weight_specs(self) -> List[WeightSpec]:
        p, W = self.prefix, self.hidden
        specs = [WeightSpec(p + "q", (self.q_size, W)), WeightSpec(p + "k", (self.k_size, W)),
                 WeightSpec(p + "v", (self.v_size, W)), WeightSpec(p + "o", (W, self.heads * self.vdim))]
        if self.bias_rows:
            specs.append(WeightSpec(p + "rel", (self.bias_rows, self.heads)))
        if self.mix_values is not None:
            specs.append(WeightSpec(p + "vmix", ()))
        if self.sink_name is not None:
            specs.append(WeightSpec(p + self.sink_name, (self.heads,)))
        return specs

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        ws = [store.take(p + n) for n in "qkv"]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()      # one product for q, k and v
        self.w_o = store.get(p + "o")
        if self.bias_rows:
            rel = store.get(p + "rel").float()
            self._check_bias(p, rel.shape[0], self.bias_far)
            self.bias_rows = rel.shape[0]
            index = torch.tensor(distance_buckets(rel.shape[0], self.bias_far), dtype=torch.long, device=rel.device)
            self.bias = rel[index].contiguous()                                  # [far + 1, heads], a row per distance
            self.bias_t = self.bias.t().contiguous()                             # [heads, far + 1] for the kernel for runs
        if self.sink_name is not None:
            self.sink = store.get(p + self.sink_name).float().contiguous()
        elif self.has_sink:
            self.sink = torch.zeros(self.heads, dtype=torch.float32, device=store.device)
        if self.position is not None:
            self.position.prepare(store.device)
        if self.mix_values is not None:
            self.mix = float(store.get(p + "vmix").float().item())

    def kernels(self) -> List[str]:
        return ["bias_attention"] + (["gemv"] if getattr(self, "run_dtype", None) == torch.bfloat16 else [])

    def cache_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, self.dim + self.vdim, self.window, planes=1, keep_first=self.keep_first)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        proj = self.hidden * (self.q_size + self.k_size + self.v_size) + self.heads * self.vdim * self.hidden
        el = 2 if getattr(self, "run_dtype", None) == torch.bfloat16 else 4
        seen = min(kv_tokens, n_tokens * (self.window + self.keep_first)) if self.window else kv_tokens
        return {"matmul": (wb(self.w_qkv) + wb(self.w_o), 2.0 * n_tokens * proj),
                "attn": (float((self.k_size + self.v_size) * el * seen), 2.0 * self.heads * (self.dim + self.vdim) * seen)}

    def input_weight(self) -> torch.Tensor:
        """The fused input projection's weight [q | k | v rows, hidden]: a mixer that runs this one beside another
        on the same input may compute both projections as one product and hand the rows over (`projected`)."""
        return self.w_qkv

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache, projected: Optional[torch.Tensor] = None) -> torch.Tensor:
        """projected: float32 rows that begin with this mixer's [q | k | v] (the rows may be longer); needs the rotating writer."""
        T, act, dev = xn.shape[0], ctx.act_dtype, xn.device
        if projected is not None and self.position is None and self.unit_eps == 0.0:
            raise ValueError(f"attention '{self.prefix}': rows of a wider projection need the rotating writer")
        qkv = projected if projected is not None else linear(xn, self.w_qkv, out_dtype=torch.float32)
        q = torch.empty((T, self.heads, self.dim), dtype=act, device=dev)
        keep = other = None
        if self.mix_values is not None:
            if self.mix_first:
                keep = ctx.carry[self.mix_values] = torch.empty((T, self.v_size), dtype=torch.float32, device=dev)
            else:
                other = ctx.carry.get(self.mix_values)
                if other is None or other.shape != (T, self.v_size):
                    raise RuntimeError(f"attention '{self.prefix}': no values of {self.v_size} elements to mix with "
                                       f"were handed on by an earlier layer of this step")
        if self.position is not None or self.unit_eps > 0.0:
            pe = self.position
            KB.kv_write_rot(qkv, q, cache.kv if cache.writes else None, pe.freq if pe is not None and pe.dims else None,
                            pe.dims if pe is not None else 0, pe is not None and pe.halves, self.unit_eps, ctx.positions,
                            ctx.seq_of_token, cache.page_table, cache.page_size, self.heads, self.kv_heads, self.dim, self.vdim)
        else:
            KB.kv_write(qkv, q, cache.kv if cache.writes else None, keep, other, self.mix, ctx.positions, ctx.seq_of_token,
                        cache.page_table, cache.page_size, self.heads, self.kv_heads, self.dim, self.vdim)
        o = paged_attention(q, cache, ctx, self.heads, self.kv_heads, self.dim, self.vdim, self.scale, window=self.window,
                            keep_first=self.keep_first, bias=self.bias, bias_t=self.bias_t, sink=self.sink,
                            softcap=self.softcap, runs_min=self.RUNS_MIN)
        if KG.pays(o, self.w_o):                   # a few tokens: the output projection as a stream of its weights
            return KG.gemv(o, self.w_o, torch.empty((T, self.hidden), dtype=torch.float32, device=dev))
        return linear(o, self.w_o, out_dtype=torch.float32)


register_mixer("window_bias_attention", BiasedWindowAttentionMixer)
