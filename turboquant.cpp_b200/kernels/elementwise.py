"""Row-wise kernels (csrc/elementwise.cu): embedding rows, RMSNorm, SiLU*up, row gather."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32

_LIB = "elementwise"


def embed_rows(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32.  tokens int32 [T]; table [V, H]; out float32 [T, H]."""
    want_int32(tokens, "tokens")
    want_f32(out, "the residual stream")
    T, H = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_embed_rows(ptr(tokens), ptr(table), c_int(code(table.dtype)), ptr(out),
                                  c_int(T), c_int(H), c_int(table.shape[0]), stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            add: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of rows of the float32 residual stream x [T, H] into out [R, H].

    add:  the norm is taken of x + add (summed in float32).
    rows: out[r] = norm of row rows[r] and x is left alone; without rows, R = T and the sum
          x + add is written back into x."""
    want_f32(x, "the residual stream")
    R, H = out.shape
    if rows is not None:
        want_int32(rows, "rows")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_rmsnorm(ptr(x), ptr(add), c_int(code(add.dtype) if add is not None else 0), ptr(rows),
                               ptr(weight), c_int(code(weight.dtype)), ptr(out), c_int(code(out.dtype)),
                               c_int(R), c_int(H), c_float(eps), stream()))
    return out


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y with x float32."""
    want_f32(x, "the residual stream")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_residual_add(ptr(x), ptr(y), c_int(code(y.dtype)), c_longlong(x.numel()), stream()))
    return x


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[t, :] += bias, in place, summed in float32.  x [T, N]; bias [N] (any of the two dtypes)."""
    T, N = x.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_add_bias(ptr(x), c_int(code(x.dtype)), ptr(bias), c_int(code(bias.dtype)), c_int(T), c_int(N),
                                stream()))
    return x


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    T, I = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_silu_mul(ptr(gate_up), c_int(code(gate_up.dtype)), ptr(out), c_int(code(out.dtype)),
                                c_int(T), c_int(I), stream()))
    return out


GLU_SIGMOID, GLU_GELU_TANH = 0, 1       # csrc/common.cuh TQ_GLU_SIGMOID, TQ_GLU_GELU_TANH


class Glu:
    """A gated activation: g = min(gate, limit), u = clamp(up, -limit, limit); act(g) * (u + offset) with
    act(g) = g * sigmoid(slope * g) (kind GLU_SIGMOID), or the tanh form of gelu (kind GLU_GELU_TANH; the slope is not
    used).  limit 0 means no caps; (0, 1, 0) is silu(gate) * up.  The fused epilogues of the expert products know
    the sigmoid kind only."""

    def __init__(self, limit: float = 0.0, slope: float = 1.0, offset: float = 0.0, kind: int = GLU_SIGMOID):
        if limit < 0.0:
            raise ValueError(f"a gated activation's caps must not be negative, got {limit}")
        if kind not in (GLU_SIGMOID, GLU_GELU_TANH):
            raise ValueError(f"a gated activation's kind must be GLU_SIGMOID or GLU_GELU_TANH, got {kind}")
        self.limit, self.slope, self.offset, self.kind = float(limit), float(slope), float(offset), int(kind)

    def __repr__(self):
        return f"Glu(limit={self.limit}, slope={self.slope}, offset={self.offset}, kind={self.kind})"


SILU_GLU = Glu()
GELU_TANH_GLU = Glu(kind=GLU_GELU_TANH)


def glu_mul(gate_up: torch.Tensor, out: torch.Tensor, glu: Glu = SILU_GLU) -> torch.Tensor:
    """out[t, i] = glu(gate_up[t, i], gate_up[t, I + i]), computed in float32."""
    T, I = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_glu_mul(ptr(gate_up), c_int(code(gate_up.dtype)), ptr(out), c_int(code(out.dtype)),
                               c_int(T), c_int(I), c_float(glu.limit), c_float(glu.slope), c_float(glu.offset),
                               c_int(glu.kind), stream()))
    return out


def mean_of_norms(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float,
                  out: torch.Tensor) -> torch.Tensor:
    """out = (a / rms(a) * wa + b / rms(b) * wb) / 2 row by row in float32: two branches, each under an RMS norm of its
    own, averaged.  a, b, out float32 [R, H]."""
    for t, what in ((a, "the first branch"), (b, "the second branch"), (out, "the mean")):
        want_f32(t, what)
    if a.shape != b.shape or out.shape != a.shape or wa.dtype != wb.dtype:
        raise KernelError("mean_of_norms: the branches, their weights and the output must agree")
    R, H = a.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_mean_of_norms(ptr(a), ptr(wa), ptr(b), ptr(wb), c_int(code(wa.dtype)), ptr(out), c_int(R), c_int(H),
                                     c_float(eps), stream()))
    return out


def glu_table_rows(z: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, col0: int, out: torch.Tensor,
                   glu: Glu = SILU_GLU) -> torch.Tensor:
    """out[t, j] = glu(z[t, j], table[tokens[t], col0 + j]): a gated activation whose second operand is a slice of
    each token's row of a table.  z float32 [T, D]; out [T, D]."""
    want_f32(z, "the gate")
    want_int32(tokens, "tokens")
    T, D = z.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_glu_table_rows(ptr(z), ptr(tokens), ptr(table), c_int(code(table.dtype)), c_int(table.shape[1]),
                                      c_int(col0), ptr(out), c_int(code(out.dtype)), c_int(T), c_int(D),
                                      c_int(table.shape[0]), c_float(glu.limit), c_float(glu.slope), c_float(glu.offset),
                                      c_int(glu.kind), stream()))
    return out


def scale_bias_cols(x: torch.Tensor, scale: float = 1.0, bias: Optional[torch.Tensor] = None,
                    cols: Optional[int] = None) -> torch.Tensor:
    """x[t, j] = x[t, j] * scale + bias[j] in place for the first `cols` columns (all by default) of float32 rows."""
    want_f32(x, "the rows")
    T, S = x.shape
    N = S if cols is None else int(cols)
    if bias is not None:
        want_f32(bias, "the bias")
        if bias.numel() != N:
            raise KernelError("scale_bias_cols: one bias per column")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_scale_bias_cols(ptr(x), ptr(bias), c_float(scale), c_int(T), c_int(N), c_int(S), stream()))
    return x


def gather_rows(src: torch.Tensor, index: torch.Tensor, divisor: int, out: torch.Tensor) -> torch.Tensor:
    """out[r] = src[index[r] // divisor]."""
    want_int32(index, "index")
    R, H = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gather_rows(ptr(src), ptr(index), c_int(divisor), ptr(out), c_int(code(out.dtype)),
                                   c_int(R), c_int(H), c_int(src.shape[0]), stream()))
    return out


def embed_pair_rows(tokens: torch.Tensor, table: torch.Tensor, pair: Optional[torch.Tensor], scale: float,
                    buckets: int, mul_prev: int, mul_cur: int, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor,
                    seq_start: torch.Tensor, slots: torch.Tensor, last_token: Optional[torch.Tensor],
                    out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tok] * scale + pair[(prev * mul_prev + tok * mul_cur) mod buckets] as float32; a sequence's
    first token takes row `buckets` of the pair table.  last_token int32 [max_slots]: each sequence's last token
    so far, read for a step's first token and renewed by the same launch."""
    want_int32(tokens, "tokens")
    want_f32(out, "the residual stream")
    if pair is not None:
        want_int32(last_token, "the last tokens")
        if pair.dtype != table.dtype:
            raise KernelError("the pair table must have the embedding table's dtype")
    T, H = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_embed_pair_rows(ptr(tokens), ptr(table), ptr(pair), c_int(code(table.dtype)), ptr(out), c_int(T),
                                       c_int(H), c_int(table.shape[0]), c_float(scale), c_int(buckets),
                                       c_longlong(mul_prev), c_longlong(mul_cur), ptr(seq_of_token), ptr(cu_seqlens),
                                       ptr(seq_start), ptr(slots), ptr(last_token), c_int(cu_seqlens.shape[0] - 1),
                                       stream()))
    return out


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                copy: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None,
                next_out: Optional[torch.Tensor] = None, next_eps: Optional[float] = None) -> torch.Tensor:
    """x += y / sqrt(mean(y^2) + eps) * weight, row by row in float32 (the norm sits on the sub-layer's output);
    `copy` receives the new x in its own dtype.  next_weight, next_out: the norm that reads the new x next is taken
    in the same pass, next_out = x / sqrt(mean(x^2) + next_eps) * next_weight (next_weight in weight's dtype,
    next_out in copy's if both are given)."""
    want_f32(x, "the residual stream")
    R, H = x.shape
    if next_out is not None:
        if next_weight is None or next_weight.dtype != weight.dtype or (copy is not None and copy.dtype != next_out.dtype):
            raise KernelError("add_rmsnorm: the following norm's weight and output must share the dtypes of weight and copy")
    side = copy if copy is not None else next_out
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_add_rmsnorm(ptr(x), ptr(y), c_int(code(y.dtype)), ptr(weight), c_int(code(weight.dtype)),
                                   ptr(copy), c_int(code(side.dtype) if side is not None else 0), c_int(R), c_int(H),
                                   c_float(eps), ptr(next_weight if next_out is not None else None), ptr(next_out),
                                   c_float(eps if next_eps is None else next_eps), stream()))
    return x


def add_rmsnorm_pair(x: torch.Tensor, a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, pair_eps: float,
                     weight: torch.Tensor, eps: float, copy: Optional[torch.Tensor] = None,
                     next_weight: Optional[torch.Tensor] = None, next_out: Optional[torch.Tensor] = None,
                     next_eps: Optional[float] = None) -> torch.Tensor:
    """`mean_of_norms(a, wa, b, wb, pair_eps)` under `add_rmsnorm(x, ., weight, eps, copy, next...)` in one pass:
    x += m / sqrt(mean(m^2) + eps) * weight with m the mean of the two normed branches.  a, b float32 [R, H]; the four
    weights share a dtype."""
    want_f32(x, "the residual stream")
    want_f32(a, "the first branch")
    want_f32(b, "the second branch")
    R, H = x.shape
    if a.shape != x.shape or b.shape != x.shape:
        raise KernelError("add_rmsnorm_pair: the branches and the stream must agree in shape")
    ws = [wa, wb, weight] + ([next_weight] if next_out is not None else [])
    if any(w is None or w.dtype != weight.dtype for w in ws):
        raise KernelError("add_rmsnorm_pair: the norms' weights must share a dtype")
    if next_out is not None and copy is not None and copy.dtype != next_out.dtype:
        raise KernelError("add_rmsnorm_pair: copy and the following norm's output must share a dtype")
    side = copy if copy is not None else next_out
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_add_rmsnorm_pair(ptr(x), ptr(a), ptr(wa), ptr(b), ptr(wb), c_float(pair_eps), ptr(weight),
                                        c_int(code(weight.dtype)), ptr(copy), c_int(code(side.dtype) if side is not None else 0),
                                        c_int(R), c_int(H), c_float(eps), ptr(next_weight if next_out is not None else None),
                                        ptr(next_out), c_float(eps if next_eps is None else next_eps), stream()))
    return x


MAP_COPY, MAP_RELU_SQUARED = 0, 1


def map_elements(src: torch.Tensor, out: torch.Tensor, function: int = MAP_COPY) -> torch.Tensor:
    """out = f(src) element by element, computed in float32 and rounded to out's dtype."""
    if src.numel() != out.numel():
        raise KernelError("map_elements: sizes differ")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_map(ptr(src), c_int(code(src.dtype)), ptr(out), c_int(code(out.dtype)), c_longlong(src.numel()),
                           c_int(function), stream()))
    return out


def rotate_pairs(x: torch.Tensor, freq: torch.Tensor, positions: torch.Tensor, mag: float, offset: int = 0) -> None:
    """Turns the pairs (2i, 2i+1), i < len(freq), from element `offset` of every head of x [T, heads, d] in place
    by angle position * freq[i] (float32); cos and sin carry the factor `mag`.  x may be a view whose last
    dimension is dense."""
    want_f32(freq, "frequencies")
    want_int32(positions, "positions")
    T, heads, d = x.shape
    if x.stride(2) != 1 or offset + 2 * freq.shape[0] > d:
        raise KernelError("rotate_pairs: heads must be dense and hold the rotated pairs")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_rotate_pairs(ctypes_ptr(x), c_int(code(x.dtype)), ptr(freq), ptr(positions), c_int(T), c_int(heads),
                                    c_int(x.stride(1)), c_longlong(x.stride(0)), c_int(offset), c_int(freq.shape[0]),
                                    c_float(mag), stream()))


def ctypes_ptr(t: torch.Tensor):
    """Pointer to the first element of a CUDA tensor that may be a strided view."""
    import ctypes
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors; there is no CPU path")
    return ctypes.c_void_p(t.data_ptr())


def dyt(x: torch.Tensor, alpha: float, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor,
        add: Optional[torch.Tensor] = None, add_scale: float = 1.0, rows: Optional[torch.Tensor] = None,
        shift: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, seq_of_token: Optional[torch.Tensor] = None,
        cu_seqlens: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None, single_tokens: bool = False) -> torch.Tensor:
    """out = tanh(alpha * v) * weight + bias for the rows v of x float32 [T, H] (`rows`: those rows only), or of
    x + add_scale * add, which x then holds (without `rows`).  shift [H]: the output h_t becomes
    h_t + (h_(t-1) - h_t) * shift, h_(t-1) the unshifted output of the sequence's token before: the row above inside a
    run, else the sequence's kept row state[slots[s]] (float32 [max_slots, H], rows may be strided; zero at a
    sequence's start), which afterwards holds the run's last unshifted output.  single_tokens: every sequence brings
    one token (the kept rows are renewed in the same launch)."""
    want_f32(x, "the residual stream")
    R = x.shape[0] if rows is None else rows.shape[0]
    H = x.shape[1]
    if weight.dtype != bias.dtype or (shift is not None and shift.dtype != weight.dtype):
        raise KernelError("dyt: weight, bias and shift must share a dtype")
    n_seqs = 0
    if shift is not None:
        if add is not None or rows is not None or state is None:
            raise KernelError("dyt: the shift wants whole steps, the sequences' kept rows and no sum on the way")
        want_f32(state, "the kept rows")
        if state.shape[1] != H or state.stride(1) != 1:
            raise KernelError("dyt: kept rows of the stream's width")
        n_seqs = cu_seqlens.shape[0] - 1
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_dyt(ptr(x), ptr(add), c_int(code(add.dtype) if add is not None else 0), c_float(add_scale), ptr(rows),
                           c_float(alpha), ptr(weight), ptr(bias), c_int(code(weight.dtype)), ptr(out), c_int(code(out.dtype)),
                           c_int(R), c_int(H), ptr(shift), ctypes_ptr(state) if state is not None else None,
                           c_longlong(state.stride(0) if state is not None else 0), ptr(seq_of_token), ptr(cu_seqlens),
                           ptr(slots), c_int(n_seqs), c_int(1 if single_tokens else 0), stream()),
          kernels=2 if shift is not None and not single_tokens else 1)
    return out


def depth_mix(hist: torch.Tensor, at: int, x: torch.Tensor, weights: torch.Tensor, out: torch.Tensor,
              add: Optional[torch.Tensor] = None, add_scale: float = 1.0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """hist float32 [n, T, H]: hist[at] = x + add_scale * (add + bias), then out = sum over j <= at of weights[j] *
    hist[j].  weights float32 [>= at + 1]; x and out float32 [T, H] (they may be one tensor); add [T, H], bias [H]."""
    for t, what in ((hist, "the kept streams"), (x, "the stream"), (weights, "the weights"), (out, "the output")):
        want_f32(t, what)
    if hist.shape[1:] != x.shape or out.shape != x.shape or not 0 <= at < hist.shape[0] or weights.numel() <= at:
        raise KernelError("depth_mix: kept streams, stream, output and weights do not fit together")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_depth_mix(ptr(hist), c_int(at), c_longlong(x.numel()), ptr(x), ptr(add),
                                 c_int(code(add.dtype) if add is not None else 0), ptr(bias),
                                 c_int(code(bias.dtype) if bias is not None else 0), c_int(x.shape[1]), c_float(add_scale),
                                 ptr(weights), ptr(out), stream()))
    return out


def bias_map(src: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, function: int = MAP_COPY) -> torch.Tensor:
    """out[t, i] = f(src[t, i] + bias[i]) for float32 rows src [T, N], rounded to out's dtype."""
    want_f32(src, "the rows")
    T, N = src.shape
    if bias.numel() != N or out.shape != src.shape:
        raise KernelError("bias_map: one bias per column, an output of the input's shape")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_bias_map(ptr(src), ptr(bias), c_int(code(bias.dtype)), ptr(out), c_int(code(out.dtype)), c_int(T),
                                c_int(N), c_int(function), stream()))
    return out
