"""The Sisepel decoder as a list of parts.

Plain embedding; layers in the order config.json lists them, each a pair of mixers side by side (windowed softmax
attention with rotated, unit-length queries and keys, capped scores and a learned sink; retention with a fixed decay
per head) and an optional feed-forward (dense with the tanh form of gelu, or routed experts with a bias on the
router's logits and a shared expert), a norm before and one after each sub-layer; after a layer's sub-layers a token
input of its own from a second embedding table; final norm; a head of its own whose logits are scaled.
Tensors: embed, side.embed, l<i>.norm1|norm1b|norm2|norm2b, l<i>.mix.left.<name>, l<i>.mix.right.<name>,
l<i>.mix.left.out|right.out, l<i>.mlp.<name>, l<i>.side.gate|proj|norm, final.norm, head.
"""
from __future__ import annotations

import torch

from ..config.registry import register_architecture
from ..config.sisepel import ARCHITECTURE, DenseMlpConfig, RotationConfig, SisepelConfig
from ..kernels.elementwise import GELU_TANH_GLU
from ..parts import SandwichBlock, TokenSideInput, make_feed_forward, make_mixer, make_norm, make_position_encoding
from .decoder import DecoderModel, Embedding, LMHead, ScheduleEntry

MOE_NAMES = {"router": "router", "router_bias": "router.b", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down",
             "shared": "shared."}
SIDE_TABLE = "side.embed"


def _position(rot: RotationConfig, pairing: str):
    if rot is None or rot.dims == 0:
        return None
    return make_position_encoding("rotary_bands", dims=rot.dims, base=rot.base, pairing=pairing, factor=rot.factor,
                                  low=rot.low, high=rot.high, original=rot.original)


class SisepelModel(DecoderModel):
    def __init__(self, cfg: SisepelConfig, dtype: torch.dtype):
        W = cfg.width
        norm = lambda name: make_norm("rmsnorm", name=name, size=W, eps=cfg.eps)
        blocks = []
        for i, layer in enumerate(cfg.layers):
            p = f"l{i}."
            a, r = layer.mixer.left, layer.mixer.right
            left = make_mixer("window_bias_attention", prefix=p + "mix.left.", hidden=W, heads=a.heads, kv_heads=a.kv_heads,
                              dim=a.dim, vdim=a.vdim, scale=a.scale, window=a.window, bias_rows=0, sink=True,
                              sink_name="sink", position=_position(a.rot, "neighbours"), unit_eps=cfg.eps, softcap=a.softcap)
            right = make_mixer("retention", prefix=p + "mix.right.", hidden=W, heads=r.heads, dim=r.dim, vdim=r.vdim,
                               decay=r.decay, eps=cfg.eps, position=_position(r.rot, "halves"))
            mixer = make_mixer("parallel", left=left, right=right, hidden=W, eps=cfg.eps,
                               left_norm=p + "mix.left.out", right_norm=p + "mix.right.out")
            ffn = ffn_norm = ffn_post = None
            if layer.mlp is not None:
                ffn_norm, ffn_post = norm(p + "norm2"), norm(p + "norm2b")
                if isinstance(layer.mlp, DenseMlpConfig):
                    ffn = make_feed_forward("glu", prefix=p + "mlp.", hidden=W, intermediate=layer.mlp.ff, glu=GELU_TANH_GLU)
                else:
                    e = layer.mlp
                    ffn = make_feed_forward("moe", prefix=p + "mlp.", hidden=W, n_experts=e.experts, top_k=e.top,
                                            intermediate=e.ff, norm_topk=True, shared_intermediate=e.shared_ff,
                                            shared_gate=False, router_bias=True, names=MOE_NAMES)
            after = []
            if cfg.side_dim:
                after.append(TokenSideInput(p + "side.", SIDE_TABLE, cfg.vocab, cfg.side_dim * len(cfg.layers),
                                            i * cfg.side_dim, cfg.side_dim, W, cfg.eps))
            blocks.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b"), ffn_norm, ffn, ffn_post, after))
        for b, nxt in zip(blocks, blocks[1:]):               # the layers run in the listed order, each once
            b.next_norm = nxt.mixer_norm
        super().__init__(cfg, dtype, embedding=Embedding("embed", cfg.vocab, W), blocks=blocks,
                         schedule=[ScheduleEntry(i) for i in range(len(blocks))],
                         final_norm=norm("final.norm"), head=LMHead("head", cfg.vocab, W, scale=cfg.logit_scale))


register_architecture(ARCHITECTURE, SisepelConfig, SisepelModel)
