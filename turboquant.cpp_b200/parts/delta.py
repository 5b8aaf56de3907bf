"""A delta-rule mixer with a decay per key channel.

With H value heads on G query/key heads (head a reads a // (H / G)), key size dk, value size dv, h the input:

    q = silu(conv(W_q h)), k = silu(conv(W_k h)) [G, dk], v = silu(conv(W_v h)) [H, dv]
                                      conv: a causal convolution per channel over `taps` tokens, the last tap on the
                                      current token, zeros before a sequence's start, no bias
    q <- q / sqrt(sum(q^2) + 1e-6) * dk^-1/2,  k <- k / sqrt(sum(k^2) + 1e-6)          per head
    beta = sigmoid(W_b h) [H]
    g = exp(-exp(A_log_a) * softplus(W_a2 (W_a1 h) + dt_bias)) [H, dk]                  a decay per key channel
    per head:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q       S [dk, dv], zero at the start
    out = W_o concat_a (o_a / sqrt(mean(o_a^2) + eps) * w * sigmoid(W_g2 (W_g1 h))_a)   w [dv] shared by the heads

A sequence's state is S of every head (stored column by column, [dv, dk]) and the convolution's last taps-1 inputs,
both float32, in one row of the cache's state area.  The fused input projection [q | k | v | beta | a1 | g1] leaves
the library's product as float32; the two second products of the low-rank pairs read their slices of it; everything
behind the projections is float32 up to the gated norm's output.
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import gemv as KG
from ..kernels import ssm as KS
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import LayerCache, Mixer, StateNeed, StepContext, register_mixer

UNIT_EPS = 1e-6          # inside the root of the unit vectors of q and k


class ChannelDeltaMixer(Mixer):
    RUNS_MIN = 16             # steps whose longest run of new tokens is at least this take the two-launch form

    def __init__(self, prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: int = -1, gate_rank: int = -1):
        """decay_rank, gate_rank: the inner sizes of the two low-rank pairs; -1: read from the stored tensors (a model
        drawn at random needs them)."""
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"delta mixer '{prefix}': {heads} heads are not a multiple of {kv_heads} query/key heads")
        if not 1 <= dim <= KS.MAX_STATE or vdim < 1 or not 1 <= taps <= KS.MAX_TAPS:
            raise ValueError(f"delta mixer '{prefix}': keys of {dim} (1..{KS.MAX_STATE}), values of {vdim}, {taps} taps (1..{KS.MAX_TAPS})")
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = int(heads), int(kv_heads), int(dim), int(vdim), int(taps), float(eps)
        self.qk_size, self.inner = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk_size + self.inner                         # what the convolution sees: q | k | v
        self.decays = self.heads * self.dim
        self.kept_size = (self.taps - 1) * self.channels
        self.rank_a, self.rank_g = int(decay_rank), int(gate_rank)            # -1: read from the stored tensors
        self.w_in = self.w_conv = self.w_a2 = self.w_g2 = self.dt_bias = self.a_log = self.w_norm = self.w_o = None

    def weight_specs(self) -> List[WeightSpec]:
        p, W = self.prefix, self.hidden
        specs = [WeightSpec(p + "q", (self.qk_size, W)), WeightSpec(p + "k", (self.qk_size, W)), WeightSpec(p + "v", (self.inner, W)),
                 WeightSpec(p + "q.conv", (self.qk_size, self.taps)), WeightSpec(p + "k.conv", (self.qk_size, self.taps)),
                 WeightSpec(p + "v.conv", (self.inner, self.taps)), WeightSpec(p + "b", (self.heads, W)),
                 WeightSpec(p + "A_log", (self.heads,)), WeightSpec(p + "dt_bias", (self.decays,)),
                 WeightSpec(p + "a1", (self.rank_a, W)), WeightSpec(p + "a2", (self.decays, self.rank_a)),
                 WeightSpec(p + "g1", (self.rank_g, W)), WeightSpec(p + "g2", (self.inner, self.rank_g)),
                 WeightSpec(p + "norm", (self.vdim,), init="one_plus_normal"), WeightSpec(p + "o", (W, self.inner))]
        return specs

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        ws = [store.take(p + n) for n in ("q", "k", "v", "b", "a1", "g1")]
        self.rank_a, self.rank_g = ws[4].shape[0], ws[5].shape[0]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_a2, self.w_g2 = store.get(p + "a2"), store.get(p + "g2")
        if self.w_a2.shape[1] != self.rank_a or self.w_g2.shape[1] != self.rank_g:
            raise ValueError(f"delta mixer '{p}': the low-rank pairs' inner sizes differ "
                             f"({self.rank_a} / {self.w_a2.shape[1]}, {self.rank_g} / {self.w_g2.shape[1]})")
        cs = [store.take(p + n + ".conv") for n in "qkv"]
        self.w_conv = torch.cat([c.to(cs[0].dtype) for c in cs], dim=0).contiguous()
        # what enters the recurrence is float32
        self.dt_bias, self.a_log = (store.get(p + n).float().contiguous() for n in ("dt_bias", "A_log"))
        self.w_norm = store.get(p + "norm").repeat(self.heads).contiguous()      # one weight per element of a row
        self.w_o = store.get(p + "o")
        self.b_off = self.channels
        self.a1_off = self.b_off + self.heads
        self.g1_off = self.a1_off + self.rank_a

    def kernels(self) -> List[str]:
        return ["ssm"] + (["gemv"] if getattr(self, "run_dtype", None) == torch.bfloat16 else [])

    def state_need(self) -> StateNeed:
        return StateNeed((self.kept_size + self.heads * self.vdim * self.dim,), torch.float32)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        state = 4.0 * self.heads * self.dim * self.vdim
        flops = 2.0 * n_tokens * (self.hidden * (self.w_in.shape[0] if self.w_in is not None else 0) + self.rank_a * self.decays
                                  + self.rank_g * self.inner + self.inner * self.hidden)
        return {"matmul": (wb(self.w_in) + wb(self.w_a2) + wb(self.w_g2) + wb(self.w_o), flops),
                "other": (2.0 * state, 7.0 * n_tokens * self.heads * self.dim * self.vdim)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T, dev = xn.shape[0], xn.device
        st = cache.state                                                       # [max_slots, kept | S]
        kept = st[:, :self.kept_size].unflatten(1, (self.taps - 1, self.channels))
        S = st[:, self.kept_size:self.kept_size + self.heads * self.vdim * self.dim].unflatten(1, (self.heads, self.vdim, self.dim))
        proj = linear(xn, self.w_in, out_dtype=torch.float32)                  # [T, q | k | v | beta | a1 | g1]
        qkv = torch.empty((T, self.channels), dtype=torch.float32, device=dev)
        KS.conv_silu(proj, 0, self.w_conv, None, kept, qkv, ctx.seq_of_token, ctx.cu_seqlens, ctx.slots)
        raw = linear(proj[:, self.a1_off:self.a1_off + self.rank_a], self.w_a2, out_dtype=torch.float32)      # raw decays
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        # runs of many tokens: the recurrence's inputs prepared side by side first; single tokens: one launch
        scan = KS.delta_scan_runs if ctx.max_q_len >= self.RUNS_MIN else KS.delta_scan
        scan(qkv, 0, self.qk_size, 2 * self.qk_size, proj, self.b_off, raw, 0, self.dt_bias, self.a_log, S, y,
             self.heads, self.kv_heads, self.dim, self.vdim, UNIT_EPS, self.dim ** -0.5, ctx.cu_seqlens, ctx.slots)
        gate = linear(proj[:, self.g1_off:self.g1_off + self.rank_g], self.w_g2, out_dtype=torch.float32)
        o = torch.empty((T, self.inner), dtype=ctx.act_dtype, device=dev)
        KS.gated_group_norm(y, gate, 0, self.w_norm, self.heads, self.eps, o, gate_after=True, sigmoid_gate=True)
        if KG.pays(o, self.w_o):
            return KG.gemv(o, self.w_o, torch.empty((T, self.hidden), dtype=torch.float32, device=dev))
        return linear(o, self.w_o, out_dtype=torch.float32)


register_mixer("channel_delta", ChannelDeltaMixer)
