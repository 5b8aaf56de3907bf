"""Rotary position encoding: for pair index i < hd/2, freq_i = theta^(-2i/hd), angle = pos*freq_i,
(a, b) <- (a cos - b sin, a sin + b cos) (src/engine/tq_ops.c:1418-1448).

pairing "half" rotates (x[i], x[i+hd/2]), the layout of safetensors checkpoints of this family;
"interleaved" rotates (x[2i], x[2i+1]) as the reference does.  The reference recomputes
powf/cosf/sinf for every head of every token; here cos and sin are float32 tables over positions,
built once (angles in float64, rounded once to float32)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_position: int, pairing: str = "half"):
        if head_dim % 2:
            raise ValueError(f"rotary: head size {head_dim} must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary: pairing must be 'half' or 'interleaved', got '{pairing}'")
        if not theta > 0 or max_position < 1:
            raise ValueError(f"rotary: theta {theta} and max_position {max_position} must be positive")
        self.head_dim, self.theta, self.max_position, self.pairing = int(head_dim), float(theta), int(max_position), pairing
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        if self.cos is not None and self.cos.device == torch.device(device):
            return
        i = torch.arange(self.head_dim // 2, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.head_dim)
        ang = torch.arange(self.max_position, dtype=torch.float64)[:, None] * freq[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(device).contiguous()

    def tables(self):
        return self.cos, self.sin, self.pairing


register_position_encoding("rotary", RotaryEncoding)


class ScaledRotaryEncoding(PositionEncoding):
    """Rotation of interleaved pairs (2i, 2i+1), i < dims/2, with frequencies stretched for contexts longer than
    the one trained on: with f_i = base^(-2i/dims) and, for a number of turns t over the original context,
    pair(t) = dims * ln(original / (2 pi t)) / (2 ln base), the pairs below lo = max(floor(pair(fast)), 0) keep
    f_i, the pairs above hi = min(ceil(pair(slow)), dims - 1) take f_i / factor, and between them the two are
    mixed by ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1).  cos and sin are multiplied by
    0.1 ln(factor) + 1.  Without a factor it is the plain interleaved rotation.

    There is no table over positions and so no longest position: kernels compute angle = position * frequency
    in float32 from the frequencies (`freq`, float32 [dims/2] on the device) and the factor `mag`."""

    def __init__(self, dims: int, base: float, factor: Optional[float] = None, original: float = 0.0,
                 fast: float = 0.0, slow: float = 0.0, pairing: str = "neighbours"):
        """pairing: 'neighbours' rotates (2i, 2i+1), 'halves' (i, i + dims/2); kernels that rotate from `freq`
        ask `halves`, `apply()` knows neighbours only."""
        if dims % 2 or dims < 0:
            raise ValueError(f"rotary: {dims} rotated dimensions must be even")
        if pairing not in ("neighbours", "halves"):
            raise ValueError(f"rotary: pairing must be 'neighbours' or 'halves', got '{pairing}'")
        self.pairing = pairing
        if not base > 0:
            raise ValueError(f"rotary: base {base} must be positive")
        self.dims, self.base = int(dims), float(base)
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / max(self.dims, 1))
        self.mag = 1.0
        if factor is not None:
            if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
                raise ValueError("rotary: factor, original, fast and slow must be positive")
            pair = lambda turns: self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(pair(fast)), 0)
            hi = min(math.ceil(pair(slow)), self.dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.mag = 0.1 * math.log(factor) + 1.0
        self._freq64 = f
        self.freq: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        if self.freq is None or self.freq.device != torch.device(device):
            self.freq = self._freq64.to(torch.float32).to(device).contiguous()

    def kernels(self):
        return ["elementwise"]

    @property
    def halves(self) -> bool:
        return self.pairing == "halves"

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        from ..kernels import elementwise as K
        if self.dims == 0:
            return
        if self.halves:
            raise NotImplementedError("rotary: pairs of halves are rotated by the kernels that read `freq`")
        K.rotate_pairs(q, self.freq, positions, self.mag)
        if k is not None:
            K.rotate_pairs(k, self.freq, positions, self.mag)


register_position_encoding("rotary_scaled", ScaledRotaryEncoding)


class BandRotaryEncoding(PositionEncoding):
    """Rotation of the first `dims` elements of a head by angle = position * f_i, f_i = base^(-2i/dims), over pairs of
    neighbours (2i, 2i+1) or of halves (i, i + dims/2).  With `factor`, frequencies are stretched by wavelength bands:
    with l = 2 pi / f and the wavelengths `original / high` and `original / low`, short waves (l below the first)
    keep f, long waves (l above the second) take f / factor, and between the two the blend
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).

    There is no table over positions and so no longest position: kernels compute the angle in float32 from
    `freq` (float32 [dims/2] on the device after prepare())."""

    def __init__(self, dims: int, base: float, pairing: str = "neighbours", factor: Optional[float] = None,
                 low: float = 0.0, high: float = 0.0, original: float = 0.0):
        if dims % 2 or dims < 0:
            raise ValueError(f"rotary: {dims} rotated dimensions must be even")
        if pairing not in ("neighbours", "halves"):
            raise ValueError(f"rotary: pairing must be 'neighbours' or 'halves', got '{pairing}'")
        if not base > 0:
            raise ValueError(f"rotary: base {base} must be positive")
        self.dims, self.base, self.pairing = int(dims), float(base), pairing
        f = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        if factor is not None:
            if not (factor > 0 and original > 0 and high > low >= 0):
                raise ValueError("rotary: factor and original must be positive and high above low")
            for i, fi in enumerate(f):
                wave = 2.0 * math.pi / fi
                if low > 0 and wave > original / low:
                    f[i] = fi / factor
                elif wave >= original / high:
                    s = (original / wave - low) / (high - low)
                    f[i] = (1.0 - s) * fi / factor + s * fi
        self._freq64 = torch.tensor(f, dtype=torch.float64)
        self.freq: Optional[torch.Tensor] = None

    @property
    def halves(self) -> bool:
        return self.pairing == "halves"

    def prepare(self, device) -> None:
        if self.freq is None or self.freq.device != torch.device(device):
            self.freq = self._freq64.to(torch.float32).to(device).contiguous()


register_position_encoding("rotary_bands", BandRotaryEncoding)
