"""Launchers of csrc/bias_attention.cu: attention with a distance bias, a window that keeps a sequence's first
positions and a sink in the softmax, over cache rows that hold a key and a value of different sizes."""
from __future__ import annotations

from ctypes import c_float, c_int
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32

_LIB = "bias_attention"
MAX_DIM = 256        # csrc/bias_attention.cu BA_MAX_DIM: the most elements of a key or of a value


def kv_write(qkv: torch.Tensor, q_out: torch.Tensor, cache: Optional[torch.Tensor], v_keep: Optional[torch.Tensor],
             v_other: Optional[torch.Tensor], mix: float, positions: torch.Tensor, seq_of_token: torch.Tensor,
             page_table: torch.Tensor, page_size: int, heads: int, kv_heads: int, dk: int, dv: int) -> None:
    """qkv float32 [T, heads * dk + kv_heads * (dk + dv)], the fused projection [q | k | v]: queries go to q_out
    [T, heads, dk] (activation dtype), keys and values to the token's place in cache [pages, 1, kv_heads, page_size,
    dk + dv].  v_other float32 [T, kv_heads * dv]: the values become (1 - mix) v + mix v_other first; v_keep (same
    shape) receives the values as they are cached."""
    want_f32(qkv, "the fused projection")
    T = qkv.shape[0]
    if qkv.shape[1] != heads * dk + kv_heads * (dk + dv):
        raise KernelError("kv_write: the projection's width does not fit the heads")
    for t in (v_keep, v_other):
        if t is not None:
            want_f32(t, "values handed between layers")
            if t.shape != (T, kv_heads * dv):
                raise KernelError("kv_write: values handed between layers must be [T, kv_heads * dv]")
    if cache is not None and (cache.dtype != q_out.dtype or cache.shape[1] != 1 or cache.shape[2] != kv_heads
                              or cache.shape[4] != dk + dv):
        raise KernelError("kv_write: the cache does not fit the heads")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_bias_kv_write(
        ptr(qkv), ptr(q_out), ptr(cache), c_int(code(q_out.dtype)), ptr(v_keep), ptr(v_other), c_float(mix),
        ptr(positions), ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), c_int(T),
        c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), c_int(page_table.shape[0]),
        c_int(cache.shape[0] if cache is not None else 0), stream()))


def kv_write_rot(qkv: torch.Tensor, q_out: torch.Tensor, cache: Optional[torch.Tensor], freq: Optional[torch.Tensor],
                 rot_dims: int, halves: bool, unit_eps: float, positions: torch.Tensor, seq_of_token: torch.Tensor,
                 page_table: torch.Tensor, page_size: int, heads: int, kv_heads: int, dk: int, dv: int, mag: float = 1.0,
                 q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                 v_freq: Optional[torch.Tensor] = None, v_share: int = 1) -> None:
    """The split of `kv_write` with norms and rotations on the way.  qkv float32 [T, >= heads*dk + kv_heads*dk +
    (kv_heads / v_share)*dv]: rows that begin with [q | k | v] (they may hold more behind).  Per query and key head:
    with q_norm / k_norm (float32 [dk], shared by the heads) the head becomes x / sqrt(mean(x^2) + norm_eps) * weight;
    then the first rot_dims elements turn by position * freq[i] (freq float32 [rot_dims / 2]; pairs (2i, 2i+1), or
    (i, i + rot_dims/2) with `halves`), cos and sin multiplied by `mag`; then, with unit_eps > 0, each head is divided
    by sqrt(mean(head^2) + unit_eps).  Queries go to q_out [T, heads, dk], keys and values to the token's place in
    cache [pages, 1, kv_heads, page_size, dk + dv]; key head g keeps value head g // v_share of the row, turned by
    position * v_freq[m] over all dv elements in the same pairing where v_freq (float32 [dv / 2]) is given.  Without a
    cache the rows need to hold the queries only."""
    want_f32(qkv, "the fused projection")
    want_int32(positions, "positions")
    T = qkv.shape[0]
    if v_share < 1 or kv_heads % v_share or \
            qkv.shape[1] < heads * dk + (kv_heads * dk + kv_heads // v_share * dv if cache is not None else 0):
        raise KernelError("kv_write_rot: the projection's width does not hold the heads")
    if freq is not None:
        want_f32(freq, "frequencies")
        if 2 * freq.numel() != rot_dims:
            raise KernelError("kv_write_rot: one frequency per rotated pair")
    for w in (q_norm, k_norm):
        if w is not None:
            want_f32(w, "a head norm's weight")
            if w.numel() != dk:
                raise KernelError("kv_write_rot: a head norm's weight has one element per element of a head")
    if v_freq is not None:
        want_f32(v_freq, "the values' frequencies")
        if 2 * v_freq.numel() != dv:
            raise KernelError("kv_write_rot: one frequency per pair of a value")
    if cache is not None and (cache.dtype != q_out.dtype or cache.shape[1] != 1 or cache.shape[2] != kv_heads
                              or cache.shape[4] != dk + dv):
        raise KernelError("kv_write_rot: the cache does not fit the heads")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_bias_kv_write_rot(
        ptr(qkv), c_int(qkv.shape[1]), ptr(q_out), ptr(cache), c_int(code(q_out.dtype)), ptr(freq), c_int(rot_dims),
        c_int(1 if halves else 0), c_float(mag), c_float(unit_eps), ptr(q_norm), ptr(k_norm), c_float(norm_eps), ptr(v_freq),
        c_int(v_share), ptr(positions), ptr(seq_of_token), ptr(page_table),
        c_int(page_table.shape[1]), c_int(page_size), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
        c_int(page_table.shape[0]), c_int(cache.shape[0] if cache is not None else 0), stream()))


def heads_unrotate_gate(o: torch.Tensor, gates: torch.Tensor, gate_off: int, v_freq: Optional[torch.Tensor], halves: bool,
                        positions: torch.Tensor, out: torch.Tensor, heads: int, dv: int) -> torch.Tensor:
    """out[t, h] = unrotate(o[t, h]) * sigmoid(gates[t, gate_off + h]): each head's dv values turned back by the token's
    position (pair m by -position * v_freq[m]; v_freq None: not turned) and scaled by the head's gate.  o, out
    [T, heads * dv] in the activation dtype (they may be the same tensor); gates float32 rows."""
    want_f32(gates, "the gates")
    want_int32(positions, "positions")
    if v_freq is not None:
        want_f32(v_freq, "the values' frequencies")
        if 2 * v_freq.numel() != dv:
            raise KernelError("heads_unrotate_gate: one frequency per pair of a value")
    T = o.shape[0]
    if o.shape != (T, heads * dv) or out.shape != o.shape or out.dtype != o.dtype:
        raise KernelError("heads_unrotate_gate: input and output must be [T, heads * dv] of one dtype")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_heads_unrotate_gate(ptr(o), c_int(code(o.dtype)), ptr(gates), c_int(gates.shape[1]), c_int(gate_off),
                                           ptr(v_freq), c_int(1 if halves else 0), ptr(positions), ptr(out), c_int(T),
                                           c_int(heads), c_int(dv), stream()))
    return out


def diff_combine(o: torch.Tensor, gates: torch.Tensor, gate_off: int, lam: float, eps: float, out_scale: float,
                 out: torch.Tensor, heads: int, kv_heads: int, dv: int) -> torch.Tensor:
    """Two attention maps per head over the same values, o [T, 2 * heads * dv] with the maps of a key/value head's
    queries side by side (head (g, map, j) at g * 2 * per + map * per + j, per = heads // kv_heads), into
    out[t, h] = unit(a1 - lam * a2) * out_scale * sigmoid(gates[t, gate_off + h * dv + e]), unit(v) = v / sqrt(mean(v^2) + eps)."""
    want_f32(gates, "the gates")
    T = o.shape[0]
    if o.shape != (T, 2 * heads * dv) or out.shape != (T, heads * dv) or out.dtype != o.dtype:
        raise KernelError("diff_combine: the maps must be [T, 2 * heads * dv] and the output [T, heads * dv] of one dtype")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_diff_combine(ptr(o), c_int(code(o.dtype)), ptr(gates), c_int(gates.shape[1]), c_int(gate_off),
                                    c_float(lam), c_float(eps), c_float(out_scale), ptr(out), c_int(T), c_int(heads),
                                    c_int(kv_heads), c_int(dv), stream()))
    return out


RUN_SIZES = (32, 64, 128)      # key and value sizes the tensor-core kernel for runs is built for


def runs_usable(dtype: torch.dtype, dk: int, dv: int, page_size: int) -> bool:
    """Whether the tensor-core kernel for runs of new tokens takes this shape: bfloat16, key and value sizes of 32,
    64 or 128, pages of 64 positions (TQ_BIAS_NO_MMA=1 switches it off)."""
    import os
    return (dtype == torch.bfloat16 and dk in RUN_SIZES and dv in RUN_SIZES and page_size == 64
            and os.environ.get("TQ_BIAS_NO_MMA", "") in ("", "0"))


def attention_runs(q: torch.Tensor, cache: torch.Tensor, bias_t: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                   cu_seqlens: torch.Tensor, seq_start: torch.Tensor, page_table: torch.Tensor, page_size: int,
                   window: int, keep_first: int, scale: float, out: torch.Tensor, n_seqs: int, max_run: int,
                   heads: int, kv_heads: int, dk: int, dv: int, softcap: float = 0.0, cell: int = 0) -> torch.Tensor:
    """The same attention for steps with runs of new tokens (prompts), bfloat16 on tensor cores: blocks of 64
    queries of a (sequence, head) walk the pages they can see.  bias_t float32 [heads, far + 1]: the bias per head
    and distance (the transpose of what `attention` takes).  softcap > 0: the scaled score s becomes
    softcap * tanh(s / softcap) before the bias.  cell > 0: instead of the window, position i sees
    j <= i of its own cell only (i // cell == j // cell)."""
    far = 0
    if bias_t is not None:
        want_f32(bias_t, "the distance bias")
        if bias_t.dim() != 2 or bias_t.shape[0] != heads:
            raise KernelError("attention_runs: the distance bias must be [heads, distances]")
        far = bias_t.shape[1] - 1
    if sink is not None:
        want_f32(sink, "the sink")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_bias_attention_runs(
        ptr(q), ptr(cache), c_int(code(q.dtype)), ptr(bias_t), c_int(far), ptr(sink), ptr(cu_seqlens), ptr(seq_start),
        ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), c_int(window), c_int(keep_first), c_int(cell), c_float(scale),
        c_float(softcap), ptr(out), c_int(n_seqs), c_int(max_run), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
        c_int(cache.shape[0]), stream()))
    return out


def group_heads(dtype: torch.dtype, dk: int, dv: int, per_kv: int) -> int:
    """Query heads of one key/value head that a block of the grouped token form keeps (it reads every cached row
    once for all of them); 0: this shape takes the form with a block per head (float32, sizes other than 32, 64,
    128; TQ_BIAS_NO_GROUP=1)."""
    import os
    if dtype != torch.bfloat16 or os.environ.get("TQ_BIAS_NO_GROUP", "") not in ("", "0"):
        return 0
    return int(load_kernel(_LIB).tq_bias_attention_group_heads(c_int(dk), c_int(dv), c_int(per_kv)))


def heads_form(dtype: torch.dtype, dk: int, dv: int, per_kv: int, page_size: int) -> bool:
    """Whether steps of single tokens take the tensor-core token form (up to sixteen heads of a key/value head are the
    rows of a tile): bfloat16, sizes of 32, 64 or 128, pages that are multiples of 16, and at least HEADS_FORM_MIN
    query heads per key/value head (TQ_BIAS_TOKEN_FORM=group|heads forces one)."""
    import os
    if dtype != torch.bfloat16 or dk not in RUN_SIZES or dv not in RUN_SIZES or page_size % 16:
        return False
    how = os.environ.get("TQ_BIAS_TOKEN_FORM", "")
    if how in ("group", "heads"):
        return how == "heads"
    return per_kv >= HEADS_FORM_MIN


HEADS_FORM_MIN = 2


def splits_for(n_tokens: int, blocks_per_token: int, longest: int, device, unit: int = 8) -> int:
    """Ranges the visible keys of a token are cut into.  A block's four warps walk its range in units of `unit` keys
    (16 in the tensor-core form); three blocks run on an SM at once.  The count that gives the fewest rounds of
    blocks times units per warp, a block's fixed cost (its queries, the merge) counted as two units, and never fewer
    than a unit per warp: a step of few tokens is cut until it fills the GPU, a large batch so that its last round
    of blocks is full.  (Measured on B200 at 64 tokens x 4 key/value heads x 1,028 keys of 128 + 128, tensor-core
    form: one range 45.2 us, 2 ranges 50.2 + 3.4 us for the merge, 3: 41.9 + 4.6, 5: 44.7 + 5.1, 7: 53.3 + 6.5, 13: 64.4 + 8.1.)  The ranges are joined in range order, so a launch shape always gives the same bits; logits
    agree across shapes to rounding."""
    import os
    forced = os.environ.get("TQ_BIAS_SPLITS", "")
    if forced:
        return max(1, min(64, int(forced)))
    slots = 3 * torch.cuda.get_device_properties(device).multi_processor_count
    units = -(-max(1, longest) // unit)
    best, best_cost = 1, float("inf")
    for s in range(1, min(64, max(1, units // 4)) + 1):
        per_block = -(-(-(-units // s)) // 4) + 2
        rounds = -(-(n_tokens * blocks_per_token * s) // slots)
        cost = rounds * per_block + 0.05 * s
        if cost < best_cost:
            best, best_cost = s, cost
    return best


def attention(q: torch.Tensor, cache: torch.Tensor, bias: Optional[torch.Tensor], sink: Optional[torch.Tensor],
              positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int,
              window: int, keep_first: int, scale: float, out: torch.Tensor, heads: int, kv_heads: int, dk: int,
              dv: int, n_splits: int = 1, bias_t: Optional[torch.Tensor] = None, softcap: float = 0.0, cell: int = 0) -> torch.Tensor:
    """Every (token, head) on its own over its sequence's cache; with bias_t (the bias as [heads, far + 1]) given or
    no bias at all, and a shape the grouped form is built for, a block per (token, key/value head) instead.  q [T, heads, dk]; out [T, heads * dv]; bias float32
    [far + 1, heads], row min(distance, far) added to the scaled score (None: no bias); sink float32 [heads]: exp(sink)
    joins the softmax's denominator (None: an ordinary softmax); window 0: every earlier position is seen, else the
    last `window` and the first `keep_first`; softcap > 0: the scaled score s becomes softcap * tanh(s / softcap)
    before the bias is added; cell > 0: instead of the window, position i sees j <= i of its own cell only
    (i // cell == j // cell)."""
    T = q.shape[0]
    want_int32(positions, "positions")
    want_int32(page_table, "page table")
    far = 0
    if bias is not None:
        want_f32(bias, "the distance bias")
        if bias.dim() != 2 or bias.shape[1] != heads:
            raise KernelError("attention: the distance bias must be [distances, heads]")
        far = bias.shape[0] - 1
    if sink is not None:
        want_f32(sink, "the sink")
    partial = torch.empty(T * heads * n_splits * (dv + 2), dtype=torch.float32, device=q.device) if n_splits > 1 else None
    lib = load_kernel(_LIB)
    if (bias is None or bias_t is not None) and heads_form(q.dtype, dk, dv, heads // kv_heads, page_size):
        check(_LIB, lib.tq_bias_attention_heads(
            ptr(q), ptr(cache), ptr(bias_t), c_int(far), ptr(sink), ptr(positions), ptr(seq_of_token), ptr(page_table),
            c_int(page_table.shape[1]), c_int(page_size), c_int(window), c_int(keep_first), c_int(cell), c_float(scale), c_float(softcap), ptr(out),
            ptr(partial), c_int(n_splits), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
            c_int(page_table.shape[0]), c_int(cache.shape[0]), stream()), kernels=2 if n_splits > 1 else 1)
        return out
    if (bias is None or bias_t is not None) and page_size % 8 == 0 and group_heads(q.dtype, dk, dv, heads // kv_heads):
        check(_LIB, lib.tq_bias_attention_group(
            ptr(q), ptr(cache), ptr(bias_t), c_int(far), ptr(sink), ptr(positions), ptr(seq_of_token), ptr(page_table),
            c_int(page_table.shape[1]), c_int(page_size), c_int(window), c_int(keep_first), c_int(cell), c_float(scale), c_float(softcap), ptr(out),
            ptr(partial), c_int(n_splits), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
            c_int(page_table.shape[0]), c_int(cache.shape[0]), stream()), kernels=2 if n_splits > 1 else 1)
        return out
    check(_LIB, lib.tq_bias_attention(
        ptr(q), ptr(cache), c_int(code(q.dtype)), ptr(bias), c_int(far), ptr(sink), ptr(positions), ptr(seq_of_token),
        ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), c_int(window), c_int(keep_first), c_int(cell), c_float(scale),
        c_float(softcap), ptr(out), ptr(partial), c_int(n_splits), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
        c_int(page_table.shape[0]), c_int(cache.shape[0]), stream()), kernels=2 if n_splits > 1 else 1)
    return out
