"""Typed configuration of the Sisepel decoder.

config.json of this design is nested: ``vocab``, ``width``, ``norm`` (eps), ``logit_scale``, ``token_side`` (dim: the
width of every layer's slice of the second embedding table; absent: no such input) and ``layers``, a list in which
every entry names its kind (``type``: parallel), the sizes and constants of its two mixers (``mixer.left``: windowed
softmax attention, ``mixer.right``: retention) and its feed-forward (``mlp``, or null for none; ``kind`` dense or moe).
The order of the layers and all sizes are data: two models of the design may differ in all of it.  Every size and
constant is read here; the parts get them as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .lumevik import _sub
from .reader import ConfigError, KeyReader

ARCHITECTURE = "Sisepel"
# limits of the kernels the design's parts launch (csrc/bias_attention.cu BA_MAX_DIM, csrc/ssm.cu SSM_MAX_STATE and
# RET_MAX_DIM), checked when the configuration is read
MAX_HEAD_SIZE = 256


@dataclass(frozen=True)
class RotationConfig:
    dims: int                      # rotated elements of a head (the first ones); 0: none
    base: float
    factor: Optional[float]        # None: frequencies as they are
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                 # 0: scores are not capped
    window: int                    # 0: every earlier position is seen
    rot: Optional[RotationConfig]


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[RotationConfig]


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: RetentionConfig


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int                 # 0: no shared expert


@dataclass(frozen=True)
class SisepelLayer:
    type: str
    mixer: ParallelMixerConfig
    mlp: Any                       # DenseMlpConfig, MoeMlpConfig or None


@dataclass(frozen=True)
class SisepelConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    side_dim: int                  # 0: no per-layer token input
    layers: Tuple[SisepelLayer, ...]
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
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "SisepelConfig":
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
            if kind != "parallel":
                raise ConfigError(f"{lw}: unknown layer type '{kind}' (known: parallel)")
            m = _sub(lr, "mixer")
            mixer = ParallelMixerConfig(_window_attention(_sub(m, "left")), _retention(_sub(m, "right")))
            ml = _sub(lr, "mlp", required=False)
            layers.append(SisepelLayer(kind, mixer, None if ml is None else _mlp(ml)))
        side = _sub(r, "token_side", required=False)
        return cls(vocab=r.integer("vocab", minimum=1), width=width, eps=_sub(r, "norm").real("eps", positive=True),
                   logit_scale=r.real("logit_scale", default=1.0),
                   side_dim=side.integer("dim", minimum=1) if side is not None else 0,
                   layers=tuple(layers), raw=dict(raw), eos_token_ids=tuple(r.token_ids("eos_token_id")))


def _rotation(m: KeyReader, dim: int) -> Optional[RotationConfig]:
    rot = _sub(m, "rot", required=False)
    if rot is None:
        return None
    dims = rot.integer("dims", minimum=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{rot.where}: dims ({dims}) must be even and at most the head's size ({dim})")
    sc = _sub(rot, "scaling", required=False)
    cfg = RotationConfig(dims=dims, base=rot.real("base", positive=True),
                         factor=sc.real("factor", positive=True) if sc is not None else None,
                         low=sc.real("low") if sc is not None else 0.0, high=sc.real("high") if sc is not None else 0.0,
                         original=sc.real("original", positive=True) if sc is not None else 0.0)
    if sc is not None and not cfg.high > cfg.low >= 0.0:
        raise ConfigError(f"{sc.where}: high ({cfg.high}) must lie above low ({cfg.low}), and low must not be negative")
    return cfg


def _window_attention(m: KeyReader) -> WindowAttentionConfig:
    heads = m.integer("heads", minimum=1)
    dim = m.integer("dim", minimum=1)
    mask = _sub(m, "mask", required=False)
    cfg = WindowAttentionConfig(
        heads=heads, kv_heads=m.integer("kv_heads", default=heads, minimum=1), dim=dim, vdim=m.integer("vdim", default=dim, minimum=1),
        scale=m.real("scale"), softcap=m.real("softcap", default=0.0),
        window=mask.integer("size", minimum=1) if mask is not None else 0, rot=_rotation(m, dim))
    if cfg.heads % cfg.kv_heads:
        raise ConfigError(f"{m.where}: heads ({cfg.heads}) must be a multiple of kv_heads ({cfg.kv_heads})")
    if max(cfg.dim, cfg.vdim) > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({cfg.dim}) and vdim ({cfg.vdim}) may not exceed the {MAX_HEAD_SIZE} elements "
                          f"the attention kernels take per key or value")
    if cfg.softcap < 0.0:
        raise ConfigError(f"{m.where}: softcap ({cfg.softcap}) must not be negative")
    return cfg


def _retention(m: KeyReader) -> RetentionConfig:
    heads = m.integer("heads", minimum=1)
    dim = m.integer("dim", minimum=1)
    m.seen.add("decay")
    decay = m.raw.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
        raise ConfigError(f"{m.where}: 'decay' must list one number per head ({heads})")
    if dim > MAX_HEAD_SIZE:
        raise ConfigError(f"{m.where}: dim ({dim}) may not exceed the {MAX_HEAD_SIZE} rows the recurrence keeps per state column")
    return RetentionConfig(heads=heads, dim=dim, vdim=m.integer("vdim", default=dim, minimum=1),
                           decay=tuple(float(d) for d in decay), rot=_rotation(m, dim))


def _mlp(ml: KeyReader):
    kind = ml.string("kind", default="dense")
    if kind == "dense":
        return DenseMlpConfig(ml.integer("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{ml.where}: unknown feed-forward kind '{kind}' (known: dense, moe)")
    ex, ro = _sub(ml, "expert"), _sub(ml, "router")
    sh = _sub(ml, "shared", required=False)
    cfg = MoeMlpConfig(experts=ro.integer("experts", minimum=1), top=ro.integer("top", minimum=1),
                       ff=ex.integer("ff", minimum=1), shared_ff=sh.integer("ff", minimum=1) if sh is not None else 0)
    if cfg.top > cfg.experts:
        raise ConfigError(f"{ro.where}: top ({cfg.top}) exceeds experts ({cfg.experts})")
    return cfg
