"""Retention: linear attention with a fixed decay per head and no softmax.

With h the mixer's input, H heads, key size dk, value size dv:

    q = W_q h, k = W_k h, v = W_v h, g = W_g h             (one fused product, float32 result)
    q, k <- rotate(q), rotate(k) * k_scale                  (`position`: frequencies, pairing, rotated elements)
    S  <- decay_a S + k v^T                                 S is [dk, dv] per head a, zero at a sequence's start
    o   = S^T q
    out = W_o (unit(o) * silu(g))                           unit: each head divided by sqrt(mean(o^2) + eps)

A sequence's state is S of every head (stored column by column, [dv, dk]) in float32, one row of the cache's state
area.  Rotation, the recurrence and the unit norm are float32; the recurrence is the state-space mixer's kernel with a
constant decay, a step size of one and one group per head (B = k, C = q, x = v).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from ..kernels import ssm as KS
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import LayerCache, Mixer, StateNeed, StepContext, register_mixer


class RetentionMixer(Mixer):
    def __init__(self, prefix: str, hidden: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 position=None, k_scale: Optional[float] = None):
        """decay: one number per head; k_scale: the factor on the rotated keys (default dim^(-1/2))."""
        if heads < 1 or vdim < 1 or not 1 <= dim <= min(KS.MAX_STATE, KS.MAX_ROTATED_HEAD):
            raise ValueError(f"retention '{prefix}': {heads} heads of key size {dim} (1..{min(KS.MAX_STATE, KS.MAX_ROTATED_HEAD)}) "
                             f"and value size {vdim}")
        if len(decay) != heads:
            raise ValueError(f"retention '{prefix}': {len(decay)} decays for {heads} heads")
        if position is not None and (not hasattr(position, "freq") or position.dims > dim):
            raise ValueError(f"retention '{prefix}': the position encoding must give frequencies for at most {dim} elements")
        self.prefix, self.hidden = prefix, int(hidden)
        self.heads, self.dim, self.vdim, self.eps = int(heads), int(dim), int(vdim), float(eps)
        self.decay_values = [float(d) for d in decay]
        self.position = position
        self.k_scale = float(k_scale) if k_scale is not None else float(dim) ** -0.5
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.w_in = self.w_o = self.decay = None
        self._sm_count: Optional[int] = None

    # rows of the fused input projection: [q | k | v | g]
    @property
    def proj_rows(self) -> int:
        return 2 * self.qk + 2 * self.inner

    def weight_specs(self) -> List[WeightSpec]:
        p, W = self.prefix, self.hidden
        return [WeightSpec(p + "q", (self.qk, W)), WeightSpec(p + "k", (self.qk, W)), WeightSpec(p + "v", (self.inner, W)),
                WeightSpec(p + "g", (self.inner, W)), WeightSpec(p + "o", (W, self.inner))]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        ws = [store.take(p + n) for n in "qkvg"]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_in = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_o = store.get(p + "o")
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(store.device)
        if self.position is not None:
            self.position.prepare(store.device)

    def kernels(self) -> List[str]:
        return ["ssm"]

    def state_need(self) -> StateNeed:
        return StateNeed((self.heads * self.vdim * self.dim,), torch.float32)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        state = 4.0 * self.heads * self.dim * self.vdim
        return {"matmul": (wb(self.w_in) + wb(self.w_o), 2.0 * n_tokens * self.hidden * (self.proj_rows + self.inner)),
                "other": (2.0 * state, 4.0 * n_tokens * self.heads * self.dim * self.vdim)}

    def input_weight(self) -> torch.Tensor:
        """The fused input projection's weight ([q | k | v | g] rows): see `forward(projected=...)`."""
        return self.w_in

    MIN_CHUNK = 64           # the shortest chunk worth cutting a run into
    # decode steps with at least this many (sequence, head) pairs take the one-launch form (TQ_RETENTION_STEP_MIN_BLOCKS)
    STEP_MIN_BLOCKS = int(os.environ.get("TQ_RETENTION_STEP_MIN_BLOCKS", "0"))

    def _chunks(self, ctx: StepContext):
        """None, or how this step's runs are cut into chunks for the recurrence: (token offsets of the chunks
        [chunks + 1], chunk numbers [chunks], each sequence's chunks [sequences + 1]) on the device.  The recurrence
        kernel walks a run token by token with a warp per four columns of a head's state; where those warps fill
        less than half of the GPU and a run is long, cutting the runs fills it, at the price of walking them once
        more for the states alone (half the work of a walk with outputs).  The plan depends on the step's runs and
        on heads and vdim only, and is kept for the step's other layers."""
        lens = list(ctx.host_q_lens)
        if not lens or len(lens) != ctx.n_seqs or max(lens) < 2 * self.MIN_CHUNK:
            return None
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(ctx.device).multi_processor_count
        cuts = self._sm_count * KS.SCAN_WARPS_PER_SM // KS.scan_warps(len(lens), self.heads, self.vdim)
        if cuts < 2:
            return None
        size = max(self.MIN_CHUNK, -(-max(lens) // cuts))
        size = -(-size // 16) * 16
        if max(lens) < 2 * size:
            return None
        key = f"retention_chunks_{size}"
        plan = ctx.carry.get(key) if ctx.carry is not None else None
        if plan is None:
            cu, seq_chunks, at = [0], [0], 0
            for n in lens:
                for c0 in range(0, n, size):
                    cu.append(at + min(n, c0 + size))
                at += n
                seq_chunks.append(len(cu) - 1)
            i32 = lambda v: torch.tensor(v, dtype=torch.int32).to(ctx.device, non_blocking=True)
            plan = (i32(cu), torch.arange(len(cu) - 1, dtype=torch.int32, device=ctx.device), i32(seq_chunks))
            if ctx.carry is not None:
                ctx.carry[key] = plan
        return plan

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache, projected: Optional[torch.Tensor] = None,
                offset: int = 0) -> torch.Tensor:
        """projected: float32 rows of a wider product that hold this mixer's [q | k | v | g] from column `offset`."""
        T, dev = xn.shape[0], xn.device
        proj = projected if projected is not None else linear(xn, self.w_in, out_dtype=torch.float32)
        S = cache.state.unflatten(1, (self.heads, self.vdim, self.dim))          # column by column
        pe = self.position
        if ctx.max_q_len == 1 and ctx.n_seqs == T and T * self.heads >= self.STEP_MIN_BLOCKS:
            # every sequence brings one token: rotation, the state's update and read-out, unit norm and gate in one launch
            g = torch.empty((T, self.inner), dtype=ctx.act_dtype, device=dev)
            KS.retention_step(proj, offset, offset + self.qk, offset + 2 * self.qk, offset + 2 * self.qk + self.inner,
                              pe.freq if pe is not None and pe.dims else None, pe.dims if pe is not None else 0,
                              pe is not None and pe.halves, self.k_scale, ctx.positions, S, ctx.slots, self.decay, g,
                              self.heads, self.dim, self.vdim, self.eps)
            return linear(g, self.w_o, out_dtype=torch.float32)
        xbc = torch.empty((T, self.inner + 2 * self.qk), dtype=torch.float32, device=dev)
        KS.retention_prepare(proj, offset, offset + self.qk, offset + 2 * self.qk, xbc,
                             pe.freq if pe is not None and pe.dims else None, pe.dims if pe is not None else 0,
                             pe is not None and pe.halves, self.k_scale, ctx.positions, self.heads, self.dim, self.vdim)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        plan = self._chunks(ctx)
        if plan is None:
            KS.ssm_scan(xbc, None, 0, None, None, None, S, y, self.heads, self.vdim, self.dim, self.heads, ctx.cu_seqlens,
                        ctx.slots, fixed_decay=self.decay)
        else:
            # long runs on few blocks: the chunks of a run side by side from zero states, the states they should have
            # started from out of the states they reached, and the chunks once more from those for the outputs
            cu_chunks, chunk_ids, seq_chunks = plan
            n_chunks = chunk_ids.shape[0]
            ends = torch.zeros((n_chunks,) + tuple(S.shape[1:]), dtype=torch.float32, device=dev)
            starts = torch.empty_like(ends)
            scan = lambda st, out: KS.ssm_scan(xbc, None, 0, None, None, None, st, out, self.heads, self.vdim, self.dim, self.heads,
                                               cu_chunks, chunk_ids, fixed_decay=self.decay)
            scan(ends, None)                     # the states alone: half the work of a walk with outputs
            KS.retention_combine(S, ctx.slots, ends, starts, seq_chunks, cu_chunks, self.decay)
            scan(starts, y)
        g = torch.empty((T, self.inner), dtype=ctx.act_dtype, device=dev)
        KS.gated_group_norm(y, proj, offset + 2 * self.qk + self.inner, None, self.heads, self.eps, g, gate_after=True)
        return linear(g, self.w_o, out_dtype=torch.float32)


register_mixer("retention", RetentionMixer)
