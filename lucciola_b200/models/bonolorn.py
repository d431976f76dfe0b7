"""The Bonolorn decoder, composed from parts.

    x = embed[token] + sinusoid(position)
    each layer:  x += m * ln1(mixer(x));  x += m * ln2(ffn(x))                   (PostNormBlock)
        mixer(x) = a * attention(x) + b * decay_attention(x)                       (SideBySideMixer)
        ffn: gated gelu, or routed clamped-swish experts with one every token uses
    logits = embed . ln(x)

Tensor names: embed, final.norm and, for layer i, l<i>.norm1, l<i>.norm2, l<i>.mix.left.{q,k,v,g,o,q.norm,k.norm},
l<i>.mix.right.{q,k,v,g,o,norm}, l<i>.mlp.{gate,up,down} or l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}.
The attention keeps pages of keys and values (a sliding window gives pages back as it passes), the decay attention a
32-bit state slot.
"""
from __future__ import annotations

import torch

from ..config.bonolorn_config import MOE, BonolornConfig
from ..config.registry import register_architecture
from ..parts.attention import GatedBiasAttention, distance_slopes
from ..parts.base import Runtime
from ..parts.block import PostNormBlock
from ..parts.decay_attention import DecayLinearAttention
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.experts import RoutedExperts
from ..parts.mlp import GatedFeedForward
from ..parts.norm import LayerNorm
from ..parts.side_by_side import SideBySideMixer
from .decoder import DecoderModel, LayerCall

SINUSOID_BASE = 10000.0
SLOPE_EXPONENT = 8.0            # head h's distance slope is 2^(-8 (h + 1) / heads)


def build_bonolorn(cfg: BonolornConfig, rt: Runtime) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    embedding = TokenEmbedding(rt, "embed", cfg.vocab, W, sinusoid_base=SINUSOID_BASE)
    blocks = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        a, r = l.left, l.right
        left = GatedBiasAttention(rt, f"{p}.mix.left", W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, eps,
                                  distance_slopes(a.heads, SLOPE_EXPONENT))
        right = DecayLinearAttention(rt, f"{p}.mix.right", W, r.heads, r.dim, r.vdim, r.decay, eps)
        mixer = SideBySideMixer(rt, W, left, right, l.left_scale, l.right_scale)
        f = l.mlp
        if f is None:
            ffn = None
        elif f.kind == MOE:
            shared = None
            if f.shared_ff:
                shared = GatedFeedForward(rt, f"{p}.mlp.shared.gate", f"{p}.mlp.shared.up", f"{p}.mlp.shared.down", W, f.shared_ff,
                                          act="clamped_swish", limit=f.shared_limit)
            ffn = RoutedExperts(rt, f"{p}.mlp", W, f.experts, f.top, f.ff, "clamped_swish", f.limit, f.router_scale, f.groups, f.keep,
                                shared=shared, out_dtype=torch.float32)
        else:
            ffn = GatedFeedForward(rt, f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down", W, f.ff, act="gelu_tanh", out_dtype=torch.float32)
        blocks.append(PostNormBlock(mixer, ffn, LayerNorm(rt, f"{p}.norm1", W, eps),
                                    LayerNorm(rt, f"{p}.norm2", W, eps) if ffn is not None else None, cfg.residual_mult, rt.act_dtype))
    calls = [LayerCall(i, i) for i in range(len(blocks))]
    final_norm = LayerNorm(rt, "final.norm", W, eps)
    head = OutputHead(rt, "lm_head", cfg.vocab, W, embedding)
    # positions have no limit of their own (max_positions 0): the engine's options or its pool of pages set one
    unused = [f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.mlp is None]      # the norm of a feed-forward that is not there
    return DecoderModel(rt, embedding, blocks, calls, final_norm, head, cfg.vocab, 0, cfg.eos_token_ids, ignored_names=unused)


register_architecture(BonolornConfig.ARCHITECTURE, BonolornConfig.from_dict, build_bonolorn, replace=True)
