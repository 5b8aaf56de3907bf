"""The Tasadra decoder as a list of parts.

Plain embedding; layers in the order config.json lists them, each a `DepthMixBlock`: dynamic-tanh norms, a token shift
ahead of the mixer, a factor on both sums and a weighted sum over the embedding's output and all layers' results
behind it.  Three mixers: softmax attention with normed and rotated queries and keys, rotated values and a gate per
head; a delta rule with a decay per key channel; differential attention inside cells of positions, which may read an
earlier such layer's cached rows.  Dense feed-forward with the square of relu and biases.  Final norm, a head of its own.
Tensors: embed, l<i>.norm1|norm2 (+ .b, .alpha), l<i>.shift, l<i>.dwa, l<i>.mix.<name>, l<i>.mlp.up|down (+ .b),
final.norm (+ .b, .alpha), head.
"""
from __future__ import annotations

import torch

from ..config.registry import register_architecture
from ..config.tasadra import ARCHITECTURE, TasadraConfig
from ..parts import DepthMixBlock, make_feed_forward, make_mixer, make_norm, make_position_encoding
from .decoder import DecoderModel, Embedding, LMHead, ScheduleEntry


def _position(rot):
    if rot is None:
        return None
    return make_position_encoding("rotary_scaled", dims=rot.dims, base=rot.base, factor=rot.factor, original=rot.original,
                                  fast=rot.fast, slow=rot.slow, pairing="halves")


class TasadraModel(DecoderModel):
    def __init__(self, cfg: TasadraConfig, dtype: torch.dtype):
        W, L = cfg.width, len(cfg.layers)
        norm = lambda name: make_norm("dyt", name=name, size=W)
        # a layer whose rows later layers read keeps them for the widest of the masks (all of them if one sees everything)
        keep = {}
        for i, layer in enumerate(cfg.layers):
            if layer.type == "attention_2":
                src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
                cells = keep.setdefault(src, [])
                cells.append(layer.mixer.cell)
        blocks, schedule = [], []
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            cache_of = None
            if layer.type == "attention":
                mixer = make_mixer("rotated_value_attention", prefix=p + "mix.", hidden=W, heads=m.heads, kv_heads=m.kv_heads,
                                   dim=m.dim, vdim=m.vdim, scale=m.scale, eps=cfg.eps, position=_position(m.rot),
                                   value_base=m.rot.base if m.rot is not None else None, softcap=m.softcap)
            elif layer.type == "channel_delta":
                mixer = make_mixer("channel_delta", prefix=p + "mix.", hidden=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                                   vdim=m.vdim, taps=m.taps, eps=cfg.eps, decay_rank=m.decay_rank, gate_rank=m.gate_rank)
            else:
                src = i if m.kv_from is None else m.kv_from
                cells = keep[src]
                mixer = make_mixer("differential_attention", prefix=p + "mix.", hidden=W, heads=m.heads, kv_heads=m.kv_heads,
                                   dim=m.dim, vdim=m.vdim, scale=m.scale, eps=cfg.eps, diff=m.diff, cell=m.cell,
                                   own_cache=m.kv_from is None, keep=0 if 0 in cells else max(cells))
                cache_of = m.kv_from
            ffn = ffn_norm = None
            if layer.mlp is not None:
                ffn_norm = norm(p + "norm2")
                ffn = make_feed_forward("relu2", prefix=p + "mlp.", hidden=W, intermediate=layer.mlp.ff, bias=True)
            blocks.append(DepthMixBlock(norm(p + "norm1"), mixer, ffn_norm, ffn, hidden=W, residual_mult=cfg.residual_mult,
                                        shift_name=p + "shift", depth_name=p + "dwa", index=i, depth_total=L + 1))
            schedule.append(ScheduleEntry(i, cache_of=cache_of))
        super().__init__(cfg, dtype, embedding=Embedding("embed", cfg.vocab, W), blocks=blocks, schedule=schedule,
                         final_norm=norm("final.norm"), head=LMHead("head", cfg.vocab, W))


register_architecture(ARCHITECTURE, TasadraConfig, TasadraModel)
