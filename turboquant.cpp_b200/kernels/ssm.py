"""Launchers of csrc/ssm.cu: the short causal convolution and the recurrence of a state-space mixer."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32
from .elementwise import ctypes_ptr

_LIB = "ssm"
MAX_STATE = 256      # csrc/ssm.cu SSM_MAX_STATE
MAX_TAPS = 8         # csrc/ssm.cu SSM_MAX_TAPS


def conv_silu(proj: torch.Tensor, off: int, weight: torch.Tensor, bias: Optional[torch.Tensor], kept: torch.Tensor,
              out: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """out[t, c] = silu(bias[c] + sum_k weight[c, k] * u[t - (taps-1-k), c]) with u = proj[:, off:off+C] inside a
    sequence and zeros before its start.  kept float32 [max_slots, taps-1, C] (rows may be strided): every
    sequence's last taps-1 inputs, read for a run's first tokens and renewed after the convolution."""
    want_f32(proj, "the projection")
    want_f32(out, "the convolution's output")
    want_f32(kept, "the kept inputs")
    T, C = out.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or kept.shape[1:] != (taps - 1, C) or kept.stride(2) != 1 or kept.stride(1) != C:
        raise KernelError("conv_silu: weight, kept inputs and output do not fit together")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_conv_silu(ptr(proj), c_int(proj.shape[1]), c_int(off), ptr(weight), ptr(bias), c_int(code(weight.dtype)),
                                 ctypes_ptr(kept), c_longlong(kept.stride(0)), ptr(out), c_int(T), c_int(C), c_int(taps),
                                 ptr(seq_of_token), ptr(cu_seqlens), ptr(slots), c_int(cu_seqlens.shape[0] - 1), stream()),
          kernels=2 if taps > 1 else 1)
    return out


def ssm_scan(xbc: torch.Tensor, proj: Optional[torch.Tensor], dt_off: int, dt_bias: Optional[torch.Tensor],
             a_log: Optional[torch.Tensor], d_skip: Optional[torch.Tensor], state: torch.Tensor, y: Optional[torch.Tensor], heads: int,
             vdim: int, n_state: int, groups: int, cu_seqlens: torch.Tensor, slots: torch.Tensor,
             fixed_decay: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence over every sequence's run of new tokens.  xbc float32 [T, heads*vdim + 2*groups*n_state]
    (x | B | C after convolution and silu); the raw step sizes are proj[:, dt_off:dt_off+heads];
    state float32 [max_slots, heads, vdim, n_state] (a head's state column by column; rows may be strided); y float32 [T, heads*vdim],
    or None: the states are walked on and no output is written.
    fixed_decay float32 [heads]: S <- fixed_decay[h] S + B x^T, y = S^T C instead (a constant decay per head, a step
    size of one, no skip term); proj and the per-head tensors are then not read and may be None."""
    for t, what in ((xbc, "x, B and C"), (state, "the state")) + (((y, "the output"),) if y is not None else ()):
        want_f32(t, what)
    if fixed_decay is not None:
        want_f32(fixed_decay, "the decays")
        if fixed_decay.numel() != heads:
            raise KernelError("ssm_scan: one decay per head")
        lib = load_kernel(_LIB)
        if tuple(state.shape[1:]) != (heads, vdim, n_state) or not state[0].is_contiguous():
            raise KernelError("ssm_scan: the state must be [slots, heads, vdim, state] with dense rows")
        check(_LIB, lib.tq_ssm_scan(ptr(xbc), c_int(xbc.shape[1]), None, c_int(0), c_int(0), None, None, None, c_int(0),
                                    ctypes_ptr(state), c_longlong(state.stride(0)), ptr(y), c_int(cu_seqlens.shape[0] - 1),
                                    c_int(heads), c_int(vdim), c_int(n_state), c_int(groups), ptr(cu_seqlens), ptr(slots),
                                    ptr(fixed_decay), stream()))
        return y
    want_f32(proj, "the projection")
    if not (dt_bias.dtype == a_log.dtype == d_skip.dtype):
        raise KernelError("ssm_scan: the per-head constants must share a dtype")
    if tuple(state.shape[1:]) != (heads, vdim, n_state) or not state[0].is_contiguous():
        raise KernelError("ssm_scan: the state must be [slots, heads, vdim, state] with dense rows")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_ssm_scan(ptr(xbc), c_int(xbc.shape[1]), ptr(proj), c_int(proj.shape[1]), c_int(dt_off), ptr(dt_bias),
                                ptr(a_log), ptr(d_skip), c_int(code(dt_bias.dtype)), ctypes_ptr(state),
                                c_longlong(state.stride(0)), ptr(y), c_int(cu_seqlens.shape[0] - 1), c_int(heads), c_int(vdim),
                                c_int(n_state), c_int(groups), ptr(cu_seqlens), ptr(slots), None, stream()))
    return y


MAX_ROTATED_HEAD = 256      # csrc/ssm.cu RET_MAX_DIM
SCAN_WARPS_PER_SM = 16      # warps of the recurrence kernel an SM holds: two blocks of eight (128 registers a thread)


def scan_warps(n_seqs: int, heads: int, vdim: int) -> int:
    """Warps that `ssm_scan` launches for this many sequences (a warp owns four columns of a head's state and walks
    its sequence's run token by token)."""
    return int(load_kernel(_LIB).tq_ssm_scan_warps(c_int(n_seqs), c_int(heads), c_int(vdim)))


def retention_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, out: torch.Tensor,
                      freq: Optional[torch.Tensor], rot_dims: int, halves: bool, k_scale: float, positions: torch.Tensor,
                      heads: int, dk: int, dv: int) -> torch.Tensor:
    """out[t] = [v | rotate(k) * k_scale | rotate(q)] (float32 [T, heads*dv + 2*heads*dk]) from a fused projection's
    float32 rows: the input of `ssm_scan` with one group per head (x = v, B = k, C = q).  The first rot_dims elements
    of each head of q and k turn by position * freq[i] (float32 [rot_dims / 2]), pairs of neighbours or of halves."""
    want_f32(proj, "the projection")
    want_f32(out, "the recurrence's input")
    want_int32(positions, "positions")
    if freq is not None:
        want_f32(freq, "frequencies")
    T = proj.shape[0]
    if out.shape != (T, heads * dv + 2 * heads * dk):
        raise KernelError("retention_prepare: the output must be [T, heads*dv + 2*heads*dk]")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_retention_prepare(ptr(proj), c_int(proj.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off), ptr(out),
                                         ptr(freq), c_int(rot_dims), c_int(1 if halves else 0), c_float(k_scale),
                                         ptr(positions), c_int(T), c_int(heads), c_int(dk), c_int(dv), stream()))
    return out


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, z_off: int, weight: Optional[torch.Tensor], norm_groups: int,
                     eps: float, out: torch.Tensor, gate_after: bool = False, sigmoid_gate: bool = False) -> torch.Tensor:
    """out = rms_in_groups(y * silu(z)) * weight with z = proj[:, z_off:z_off+inner]: the gate first, then each of
    the norm_groups equal parts of a row divided by its own root mean square.  gate_after: the norm first, then the
    gate: rms_in_groups(y) * weight * silu(z).  weight None: no weight.  sigmoid_gate: sigmoid(z) where silu(z) stands."""
    want_f32(y, "the recurrence's output")
    want_f32(proj, "the projection")
    T, inner = y.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gated_group_norm(ptr(y), ptr(proj), c_int(proj.shape[1]), c_int(z_off), ptr(weight),
                                        c_int(code(weight.dtype) if weight is not None else 0), ptr(out),
                                        c_int(code(out.dtype)), c_int(T), c_int(inner), c_int(norm_groups), c_float(eps),
                                        c_int(1 if gate_after else 0), c_int(1 if sigmoid_gate else 0), stream()))
    return out


def retention_combine(state: torch.Tensor, slots: torch.Tensor, ends: torch.Tensor, starts: torch.Tensor,
                      seq_chunks: torch.Tensor, cu_chunks: torch.Tensor, decay: torch.Tensor) -> None:
    """Chunks of long runs that `ssm_scan(fixed_decay=)` walked side by side from zero states: from the states they
    reached (ends [chunks, heads, vdim, n]) and the sequences' kept states (state [slots, heads, vdim, n], rows by
    `slots`), the states each chunk should have started from (starts, like ends) and the sequences' new kept states.
    Sequence s owns chunks seq_chunks[s]..seq_chunks[s+1]; chunk c the tokens cu_chunks[c]..cu_chunks[c+1]."""
    for t, what in ((state, "the state"), (ends, "the chunks' states"), (starts, "the chunks' starts"), (decay, "the decays")):
        want_f32(t, what)
    for t, what in ((slots, "slots"), (seq_chunks, "the sequences' chunks"), (cu_chunks, "the chunks' tokens")):
        want_int32(t, what)
    heads = state.shape[1]
    if ends.shape != starts.shape or ends.shape[1:] != state.shape[1:] or not (ends.is_contiguous() and starts.is_contiguous()) \
            or not state[0].is_contiguous() or decay.numel() != heads or cu_chunks.numel() != ends.shape[0] + 1:
        raise KernelError("retention_combine: the chunks' states must be dense and shaped like the kept state's rows")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_retention_combine(ctypes_ptr(state), c_longlong(state.stride(0)), ptr(slots), ptr(ends), ptr(starts),
                                         ptr(seq_chunks), ptr(cu_chunks), ptr(decay), c_int(seq_chunks.shape[0] - 1),
                                         c_int(heads), c_int(state[0, 0].numel()), stream()))


def retention_step(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, g_off: int, freq: Optional[torch.Tensor],
                   rot_dims: int, halves: bool, k_scale: float, positions: torch.Tensor, state: torch.Tensor,
                   slots: torch.Tensor, decay: torch.Tensor, out: torch.Tensor, heads: int, dk: int, dv: int, eps: float) -> torch.Tensor:
    """One token of every sequence through retention in one launch (token t is sequence t, its state the row
    slots[t]): `retention_prepare`, `ssm_scan(fixed_decay=)` and `gated_group_norm(gate_after=True)` without a weight,
    for rows of the fused projection proj float32 [T, P] that hold q, k (heads x dk) and v, g (heads x dv) from the
    given columns.  state float32 [slots, heads, dv, dk]; out [T, heads*dv]."""
    want_f32(proj, "the projection")
    want_f32(state, "the state")
    want_f32(decay, "the decays")
    want_int32(positions, "positions")
    want_int32(slots, "slots")
    T = proj.shape[0]
    if tuple(state.shape[1:]) != (heads, dv, dk) or not state[0].is_contiguous() or out.shape != (T, heads * dv) \
            or slots.numel() != T or positions.numel() != T or decay.numel() != heads:
        raise KernelError("retention_step: the state must be [slots, heads, vdim, dim] with dense rows, one slot and position a token")
    if freq is not None:
        want_f32(freq, "frequencies")
        if 2 * freq.numel() != rot_dims:
            raise KernelError("retention_step: one frequency per rotated pair")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_retention_step(ptr(proj), c_int(proj.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off), c_int(g_off),
                                      ptr(freq), c_int(rot_dims), c_int(1 if halves else 0), c_float(k_scale), ptr(positions),
                                      ctypes_ptr(state), c_longlong(state.stride(0)), ptr(slots), ptr(decay), ptr(out),
                                      c_int(code(out.dtype)), c_int(T), c_int(heads), c_int(dk), c_int(dv), c_float(eps), stream()))
    return out


def delta_scan(xqkv: torch.Tensor, q_off: int, k_off: int, v_off: int, proj: torch.Tensor, b_off: int, a_raw: torch.Tensor,
               a_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, y: torch.Tensor, heads: int,
               kv_heads: int, dk: int, dv: int, unit_eps: float, q_scale: float, cu_seqlens: torch.Tensor,
               slots: torch.Tensor) -> torch.Tensor:
    """The delta rule with a decay per key channel over every sequence's run of new tokens:
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; y = S^T q, with k and q made unit vectors
    (x / sqrt(sum(x^2) + unit_eps), q times q_scale), beta = sigmoid(proj[:, b_off + a]) and
    g = exp(-exp(a_log[a]) * softplus(a_raw[:, a_off + a*dk : ...] + dt_bias[a])).  xqkv float32 [T, C] holds q, k
    (kv_heads x dk) and v (heads x dv) from the given columns; state float32 [max_slots, heads, dv, dk] (a head's
    state column by column; rows may be strided); y float32 [T, heads*dv]."""
    for t, what in ((xqkv, "q, k and v"), (proj, "the projection"), (a_raw, "the raw decays"), (dt_bias, "the decays' bias"),
                    (a_log, "the decay rates"), (state, "the state"), (y, "the output")):
        want_f32(t, what)
    want_int32(cu_seqlens, "the sequences' bounds")
    want_int32(slots, "slots")
    if tuple(state.shape[1:]) != (heads, dv, dk) or not state[0].is_contiguous():
        raise KernelError("delta_scan: the state must be [slots, heads, vdim, dim] with dense rows")
    if dt_bias.numel() != heads * dk or a_log.numel() != heads or y.shape != (xqkv.shape[0], heads * dv):
        raise KernelError("delta_scan: one decay bias per head and key channel, one rate per head, an output of heads*dv")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_delta_scan(ptr(xqkv), c_int(xqkv.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off), ptr(proj),
                                  c_int(proj.shape[1]), c_int(b_off), ptr(a_raw), c_int(a_raw.shape[1]), c_int(a_off),
                                  ptr(dt_bias), ptr(a_log), ctypes_ptr(state), c_longlong(state.stride(0)), ptr(y),
                                  c_int(cu_seqlens.shape[0] - 1), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
                                  c_float(unit_eps), c_float(q_scale), ptr(cu_seqlens), ptr(slots), stream()))
    return y


def delta_scan_runs(xqkv: torch.Tensor, q_off: int, k_off: int, v_off: int, proj: torch.Tensor, b_off: int, a_raw: torch.Tensor,
                    a_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, y: torch.Tensor, heads: int,
                    kv_heads: int, dk: int, dv: int, unit_eps: float, q_scale: float, cu_seqlens: torch.Tensor,
                    slots: torch.Tensor) -> torch.Tensor:
    """`delta_scan` for steps with runs of many tokens, in two launches: the unit vectors, decays and betas of all
    tokens side by side into rows of scratch, then the recurrence over those rows (a chunk of rows copied into shared
    memory while the chunk before is computed).  Arguments and result as for `delta_scan`; the sums are the same
    up to their order."""
    for t, what in ((xqkv, "q, k and v"), (proj, "the projection"), (a_raw, "the raw decays"), (dt_bias, "the decays' bias"),
                    (a_log, "the decay rates"), (state, "the state"), (y, "the output")):
        want_f32(t, what)
    want_int32(cu_seqlens, "the sequences' bounds")
    want_int32(slots, "slots")
    if tuple(state.shape[1:]) != (heads, dv, dk) or not state[0].is_contiguous():
        raise KernelError("delta_scan_runs: the state must be [slots, heads, vdim, dim] with dense rows")
    if dt_bias.numel() != heads * dk or a_log.numel() != heads or y.shape != (xqkv.shape[0], heads * dv):
        raise KernelError("delta_scan_runs: one decay bias per head and key channel, one rate per head, an output of heads*dv")
    lib = load_kernel(_LIB)
    T = xqkv.shape[0]
    rows = torch.empty((T, int(lib.tq_delta_rows_width(c_int(heads), c_int(kv_heads), c_int(dk)))), dtype=torch.float32, device=xqkv.device)
    check(_LIB, lib.tq_delta_scan_runs(ptr(xqkv), c_int(xqkv.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off), ptr(proj),
                                       c_int(proj.shape[1]), c_int(b_off), ptr(a_raw), c_int(a_raw.shape[1]), c_int(a_off),
                                       ptr(dt_bias), ptr(a_log), ptr(rows), ctypes_ptr(state), c_longlong(state.stride(0)), ptr(y),
                                       c_int(T), c_int(cu_seqlens.shape[0] - 1), c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv),
                                       c_float(unit_eps), c_float(q_scale), ptr(cu_seqlens), ptr(slots), stream()), kernels=2)
    return y
