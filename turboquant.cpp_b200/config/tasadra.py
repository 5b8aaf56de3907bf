"""Typed configuration of the Tasadra decoder.

config.json of this design is nested: ``vocab``, ``width``, ``norm`` (eps), ``residual_mult`` and ``layers``, a list
in which every entry names its mixer (``type``: attention, channel_delta or attention_2), the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``, or null for none; ``kind`` dense).  The order of the layers and
all sizes are data: two models of the design may differ in all of it.  Every size and constant is read here; the parts
get them as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .lumevik import _sub
from .reader import ConfigError, KeyReader

ARCHITECTURE = "Tasadra"
# limits of the kernels the design's parts launch (csrc/bias_attention.cu BA_MAX_DIM, csrc/ssm.cu SSM_MAX_STATE and
# SSM_MAX_TAPS), checked when the configuration is read
MAX_HEAD_SIZE = 256
MAX_TAPS = 8


@dataclass(frozen=True)
class ScaledRotation:
    dims: int                      # rotated elements of a head (the first ones); 0: none
    base: float
    factor: Optional[float]        # None: frequencies as they are
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotatedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                 # 0: scores are not capped
    rot: Optional[ScaledRotation]


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int                # -1: read from the stored tensors
    gate_rank: int


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    cell: int                      # 0: every earlier position is seen
    kv_from: Optional[int]         # the layer whose keys and values this one reads; None: its own


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class TasadraLayer:
    type: str
    mixer: Any                     # one of the three mixer configurations
    mlp: Optional[DenseMlpConfig]


LAYER_TYPES = ("attention", "channel_delta", "attention_2")


@dataclass(frozen=True)
class TasadraConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[TasadraLayer, ...]
    raw: Dict[str, Any]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ARCHITECTURE
    # the design has no longest sequence of its own (angles are computed from the position)
    max_position_embeddings: int = 1 << 30

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "TasadraConfig":
        r = KeyReader(raw, where)
        width = r.integer("width", minimum=1)
        r.seen.add("layers")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(layers_raw):
            lw = f"{where}: layers[{i}]"
            lr = KeyReader(item, lw)
            kind = lr.string("type")
            m = _sub(lr, "mixer")
            if kind == "attention":
                mixer = _rotated_attention(m)
            elif kind == "channel_delta":
                mixer = _channel_delta(m)
            elif kind == "attention_2":
                mixer = _differential(m, i, layers)
            else:
                raise ConfigError(f"{lw}: unknown layer type '{kind}' (known: {', '.join(LAYER_TYPES)})")
            ml = _sub(lr, "mlp", required=False)
            layers.append(TasadraLayer(kind, mixer, None if ml is None else _mlp(ml)))
        return cls(vocab=r.integer("vocab", minimum=1), width=width, eps=_sub(r, "norm").real("eps", positive=True),
                   residual_mult=r.real("residual_mult", default=1.0), layers=tuple(layers), raw=dict(raw),
                   eos_token_ids=tuple(r.token_ids("eos_token_id")))


def _heads(m: KeyReader) -> Tuple[int, int, int, int]:
    heads = m.integer("heads", minimum=1)
    kv_heads = m.integer("kv_heads", default=heads, minimum=1)
    dim = m.integer("dim", minimum=1)
    vdim = m.integer("vdim", default=dim, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{m.where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads, dim, vdim


def _rotation(m: KeyReader, dim: int) -> Optional[ScaledRotation]:
    rot = _sub(m, "rot", required=False)
    if rot is None:
        return None
    dims = rot.integer("dims", minimum=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{rot.where}: dims ({dims}) must be even and at most the head's size ({dim})")
    sc = _sub(rot, "scaling", required=False)
    if sc is None:
        return ScaledRotation(dims, rot.real("base", positive=True), None, 0.0, 0.0, 0.0)
    return ScaledRotation(dims, rot.real("base", positive=True), sc.real("factor", positive=True),
                          sc.real("original", positive=True), sc.real("fast", positive=True), sc.real("slow", positive=True))


def _rotated_attention(m: KeyReader) -> RotatedAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(m)
    cfg = RotatedAttentionConfig(heads, kv_heads, dim, vdim, scale=m.real("scale"), softcap=m.real("softcap", default=0.0),
                                 rot=_rotation(m, dim))
    if max(dim, vdim) > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({dim}) and vdim ({vdim}) may not exceed the {MAX_HEAD_SIZE} elements the "
                          f"attention kernels take per key or value")
    if cfg.softcap < 0.0:
        raise ConfigError(f"{m.where}: softcap ({cfg.softcap}) must not be negative")
    if cfg.rot is not None and vdim % 2:
        raise ConfigError(f"{m.where}: vdim ({vdim}) must be even: the values are turned in pairs")
    return cfg


def _channel_delta(m: KeyReader) -> ChannelDeltaConfig:
    heads, kv_heads, dim, vdim = _heads(m)
    cfg = ChannelDeltaConfig(heads, kv_heads, dim, vdim, taps=m.integer("conv", minimum=1),
                             decay_rank=m.integer("decay_rank", default=-1), gate_rank=m.integer("gate_rank", default=-1))
    if dim > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({dim}) may not exceed the {MAX_HEAD_SIZE} rows the recurrence keeps per state column")
    if cfg.taps > MAX_TAPS:
        raise ConfigError(f"{m.where}: conv ({cfg.taps}) may not exceed the {MAX_TAPS} taps the convolution kernel holds")
    return cfg


def _differential(m: KeyReader, index: int, before) -> DifferentialAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(m)
    mask = _sub(m, "mask", required=False)
    m.seen.add("kv_from")
    src = m.raw.get("kv_from")
    cfg = DifferentialAttentionConfig(heads, kv_heads, dim, vdim, scale=m.real("scale"), diff=m.real("diff"),
                                      cell=mask.integer("size", minimum=1) if mask is not None else 0,
                                      kv_from=None if src is None else m.integer("kv_from", minimum=0))
    if max(dim, vdim) > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({dim}) and vdim ({vdim}) may not exceed the {MAX_HEAD_SIZE} elements the "
                          f"attention kernels take per key or value")
    if cfg.kv_from is not None:
        j = cfg.kv_from
        if j >= index or before[j].type != "attention_2" or before[j].mixer.kv_from is not None:
            raise ConfigError(f"{m.where}: kv_from ({j}) must name an earlier attention_2 layer with keys and values of its own")
        o = before[j].mixer
        if (o.kv_heads, o.dim, o.vdim) != (kv_heads, dim, vdim):
            raise ConfigError(f"{m.where}: kv_from ({j}) names a layer with other key/value heads or sizes")
    return cfg


def _mlp(ml: KeyReader) -> DenseMlpConfig:
    kind = ml.string("kind", default="dense")
    if kind != "dense":
        raise ConfigError(f"{ml.where}: unknown feed-forward kind '{kind}' (known: dense)")
    return DenseMlpConfig(ml.integer("ff", minimum=1))
