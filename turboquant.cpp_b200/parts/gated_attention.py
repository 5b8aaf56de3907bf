"""Two gated softmax attentions over the paged cache of rows [k | v] (the kernels of `bias_attention`).

`RotatedValueAttentionMixer` (mixer `rotated_value_attention`): H query heads on G key/value heads, causal.

    q = W_q h, k = W_k h, v = W_v h, z = W_g h                 (one fused product, float32 result; z: one logit a head)
    q, k <- rms(q) * w_q, rms(k) * w_k per head                 (weights of one head's size shared by the heads;
                                                                 rms(x) = x / sqrt(mean(x^2) + eps)), then rotated
                                                                 by the position (`position`: frequencies, pairing,
                                                                 a factor on cos and sin)
    v_j <- R(j) v_j                                             every pair of a value turned by j * value_base^(-2m/dv),
                                                                 cached so
    s_ij = cap * tanh(q_i . k_j * scale / cap)                  (cap 0: uncapped); softmax over j <= i
    o_i = R(-i) sum_j p_ij v_j                                  turned back by the query's own position: what is summed
                                                                 depends on i - j only
    out = W_o concat_a sigmoid(z_a) o_a

`DifferentialAttentionMixer` (mixer `differential_attention`): two softmax maps per head over the same values.

    q = W_q h [H, 2, dk], k = W_k h [G, 2, dk], v = W_v h [G, dv], z = W_g h [H * dv]
    a_m = softmax_j(q_m . k_m * scale) v        for m = 1, 2; j <= i, and with `cell` only j of i's own cell of
                                                  positions (i // cell == j // cell)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    o = rms(a_1 - lambda a_2) * (1 - diff)       per head, no weight
    out = W_o (concat_a o_a * sigmoid(z))

The cache keeps the two maps' keys as two key heads that share one value head (the value is stored with each), and
the query rows are ordered so that the maps of a key/value head's queries lie side by side; the attention kernels
then see 2H query heads on 2G key heads.  A layer built with own_cache=False has no key and value projections: it
reads the rows another layer cached (the model names that layer in its schedule) with its own queries and mask.
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
from .bias_attention import paged_attention


def _fuse(ws: List[torch.Tensor]) -> torch.Tensor:
    dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
    return torch.cat([w.to(dt) for w in ws], dim=0).contiguous()


def _output(o: torch.Tensor, w_o: torch.Tensor, hidden: int) -> torch.Tensor:
    if KG.pays(o, w_o):                   # a few tokens: the output projection as a stream of its weights
        return KG.gemv(o, w_o, torch.empty((o.shape[0], hidden), dtype=torch.float32, device=o.device))
    return linear(o, w_o, out_dtype=torch.float32)


class RotatedValueAttentionMixer(Mixer):
    RUNS_MIN = 16

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 position=None, value_base: Optional[float] = None, softcap: float = 0.0, head_norm: bool = True,
                 window: int = 0):
        """position: an encoding with float32 frequencies (`freq`, `dims`, `halves`, `mag`) or None; value_base: the
        base of the values' rotation over all of vdim in the position's pairing (None: values are not turned);
        head_norm: the weighted RMS norm of every query and key head ahead of the rotation."""
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"attention '{prefix}': {heads} heads are not a multiple of {kv_heads} key/value heads")
        if not (1 <= dim <= KB.MAX_DIM and 1 <= vdim <= KB.MAX_DIM):
            raise ValueError(f"attention '{prefix}': key size {dim} and value size {vdim} must be in 1..{KB.MAX_DIM}")
        if position is not None and (not hasattr(position, "freq") or position.dims > dim):
            raise ValueError(f"attention '{prefix}': the position encoding must give frequencies for at most {dim} elements")
        if value_base is not None and (vdim % 2 or not value_base > 0):
            raise ValueError(f"attention '{prefix}': values of {vdim} elements cannot be turned in pairs with base {value_base}")
        if softcap < 0.0 or window < 0 or not eps > 0.0:
            raise ValueError(f"attention '{prefix}': cap {softcap}, window {window} and eps {eps}")
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.softcap, self.window = float(scale), float(eps), float(softcap), int(window)
        self.position, self.value_base, self.head_norm = position, value_base, bool(head_norm)
        self.gate_off = self.heads * self.dim + self.kv_heads * (self.dim + self.vdim)
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.v_freq = None

    def weight_specs(self) -> List[WeightSpec]:
        p, W = self.prefix, self.hidden
        specs = [WeightSpec(p + "q", (self.heads * self.dim, W)), WeightSpec(p + "k", (self.kv_heads * self.dim, W)),
                 WeightSpec(p + "v", (self.kv_heads * self.vdim, W)), WeightSpec(p + "g", (self.heads, W)),
                 WeightSpec(p + "o", (W, self.heads * self.vdim))]
        if self.head_norm:
            specs += [WeightSpec(p + "q.norm", (self.dim,), init="one_plus_normal"),
                      WeightSpec(p + "k.norm", (self.dim,), init="one_plus_normal")]
        return specs

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        self.w_in = _fuse([store.take(p + n) for n in ("q", "k", "v", "g")])       # one product for q, k, v and the gates
        self.w_o = store.get(p + "o")
        if self.head_norm:
            self.q_norm = store.get(p + "q.norm").float().contiguous()
            self.k_norm = store.get(p + "k.norm").float().contiguous()
        if self.position is not None:
            self.position.prepare(store.device)
        if self.value_base is not None:
            m = torch.arange(self.vdim // 2, dtype=torch.float64)
            f = torch.pow(torch.tensor(self.value_base, dtype=torch.float64), -2.0 * m / self.vdim)
            self.v_freq = f.to(torch.float32).to(store.device).contiguous()

    def kernels(self) -> List[str]:
        return ["bias_attention"] + (["gemv"] if getattr(self, "run_dtype", None) == torch.bfloat16 else [])

    def cache_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, self.dim + self.vdim, self.window, planes=1)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        proj = self.hidden * (self.gate_off + self.heads) + self.heads * self.vdim * self.hidden
        el = 2 if getattr(self, "run_dtype", None) == torch.bfloat16 else 4
        seen = min(kv_tokens, n_tokens * self.window) if self.window else kv_tokens
        return {"matmul": (wb(self.w_in) + wb(self.w_o), 2.0 * n_tokens * proj),
                "attn": (float(self.kv_heads * (self.dim + self.vdim) * el * seen), 2.0 * self.heads * (self.dim + self.vdim) * seen)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T, act, dev = xn.shape[0], ctx.act_dtype, xn.device
        rows = linear(xn, self.w_in, out_dtype=torch.float32)                   # [q | k | v | gate logits]
        q = torch.empty((T, self.heads, self.dim), dtype=act, device=dev)
        pe = self.position
        halves = pe.halves if pe is not None else True
        KB.kv_write_rot(rows, q, cache.kv if cache.writes else None, pe.freq if pe is not None and pe.dims else None,
                        pe.dims if pe is not None else 0, halves, 0.0, ctx.positions, ctx.seq_of_token, cache.page_table,
                        cache.page_size, self.heads, self.kv_heads, self.dim, self.vdim, mag=getattr(pe, "mag", 1.0),
                        q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.eps, v_freq=self.v_freq)
        o = paged_attention(q, cache, ctx, self.heads, self.kv_heads, self.dim, self.vdim, self.scale, window=self.window,
                            softcap=self.softcap, runs_min=self.RUNS_MIN)
        KB.heads_unrotate_gate(o, rows, self.gate_off, self.v_freq, halves, ctx.positions, o, self.heads, self.vdim)
        return _output(o, self.w_o, self.hidden)


register_mixer("rotated_value_attention", RotatedValueAttentionMixer)


class DifferentialAttentionMixer(Mixer):
    RUNS_MIN = 16

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float,
                 diff: float, cell: int = 0, own_cache: bool = True, keep: Optional[int] = None):
        """cell: the size of the cells of positions a query stays inside (0: every earlier position is seen).
        own_cache False: the layer has no key and value projections and reads another layer's rows.  keep: how many
        of the latest positions the cache must keep (None: `cell`; a layer whose rows others read with wider masks
        is told so by the model; 0: all)."""
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"attention '{prefix}': {heads} heads are not a multiple of {kv_heads} key/value heads")
        if not (1 <= dim <= KB.MAX_DIM and 1 <= vdim <= KB.MAX_DIM):
            raise ValueError(f"attention '{prefix}': key size {dim} and value size {vdim} must be in 1..{KB.MAX_DIM}")
        if cell < 0 or not eps > 0.0:
            raise ValueError(f"attention '{prefix}': cells of {cell} positions, eps {eps}")
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.diff, self.cell, self.own_cache = float(scale), float(eps), float(diff), int(cell), bool(own_cache)
        self.keep = self.cell if keep is None else int(keep)
        self.q_size = 2 * self.heads * self.dim
        self.kv_size = self.kv_heads * (2 * self.dim + self.vdim) if self.own_cache else 0
        self.w_in = self.w_o = None
        self.lam = 0.0

    def weight_specs(self) -> List[WeightSpec]:
        p, W = self.prefix, self.hidden
        specs = [WeightSpec(p + "q", (self.q_size, W)), WeightSpec(p + "g", (self.heads * self.vdim, W)),
                 WeightSpec(p + "o", (W, self.heads * self.vdim))]
        specs += [WeightSpec(p + n, (self.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")]
        if self.own_cache:
            specs += [WeightSpec(p + "k", (2 * self.kv_heads * self.dim, W)), WeightSpec(p + "v", (self.kv_heads * self.vdim, W))]
        return specs

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        # query rows [head][map][dim] -> [kv head][map][head of the group][dim]: the two maps of a group's heads side by side
        per = self.heads // self.kv_heads
        wq = store.take(p + "q")
        wq = wq.view(self.kv_heads, per, 2, self.dim, self.hidden).permute(0, 2, 1, 3, 4).reshape(self.q_size, self.hidden)
        parts = [wq] + ([store.take(p + "k"), store.take(p + "v")] if self.own_cache else []) + [store.take(p + "g")]
        self.w_in = _fuse(parts)
        self.w_o = store.get(p + "o")
        l = {n: store.get(p + n).double() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((l["lq1"] * l["lk1"]).sum())) - math.exp(float((l["lq2"] * l["lk2"]).sum())) + self.diff

    def kernels(self) -> List[str]:
        return ["bias_attention"] + (["gemv"] if getattr(self, "run_dtype", None) == torch.bfloat16 else [])

    def cache_need(self) -> KVNeed:
        return KVNeed(2 * self.kv_heads, self.dim + self.vdim, self.keep, planes=1)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        proj = self.hidden * (self.q_size + self.kv_size + 2 * self.heads * self.vdim)
        el = 2 if getattr(self, "run_dtype", None) == torch.bfloat16 else 4
        seen = min(kv_tokens, n_tokens * self.cell) if self.cell else kv_tokens
        return {"matmul": (wb(self.w_in) + wb(self.w_o), 2.0 * n_tokens * proj),
                "attn": (float(2 * self.kv_heads * (self.dim + self.vdim) * el * seen),
                         4.0 * self.heads * (self.dim + self.vdim) * seen)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T, act, dev = xn.shape[0], ctx.act_dtype, xn.device
        if cache.writes != self.own_cache:
            raise RuntimeError(f"attention '{self.prefix}': the layer {'keeps' if self.own_cache else 'reads'} a cache, "
                               f"the model's schedule says otherwise")
        rows = linear(xn, self.w_in, out_dtype=torch.float32)                   # [q | k | v | gate logits] or [q | gate logits]
        H2, G2 = 2 * self.heads, 2 * self.kv_heads
        q = torch.empty((T, H2, self.dim), dtype=act, device=dev)
        KB.kv_write_rot(rows, q, cache.kv if cache.writes else None, None, 0, True, 0.0, ctx.positions, ctx.seq_of_token,
                        cache.page_table, cache.page_size, H2, G2, self.dim, self.vdim, v_share=2)
        maps = paged_attention(q, cache, ctx, H2, G2, self.dim, self.vdim, self.scale, cell=self.cell, runs_min=self.RUNS_MIN)
        o = torch.empty((T, self.heads * self.vdim), dtype=act, device=dev)
        KB.diff_combine(maps, rows, self.q_size + self.kv_size, self.lam, self.eps, 1.0 - self.diff, o, self.heads,
                        self.kv_heads, self.vdim)
        return _output(o, self.w_o, self.hidden)


register_mixer("differential_attention", DifferentialAttentionMixer)
