"""The Riruzen decoder, composed from parts.

    x = embed[token] + pos[position]
    each layer:  h = group_rmsnorm(x);  x += mixer(h + taps(h)) + ffn(h)        (ParallelBlock)
    logits = (embed . group_rmsnorm(x)) * logit_scale

Tensor names: embed, pos, final.norm and, for layer i, l<i>.norm1, l<i>.canon1, l<i>.mix.* (the mixer's), l<i>.mlp.{gate,up,down}.
The mixers are LatentAttention (pages of latents) and GatedLinearRecurrence (a state slot); every layer also keeps the
last inputs of its causal taps in a state slot.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.riruzen_config import HGRN2, LATENT_ATTENTION, RiruzenConfig
from ..parts.base import Runtime
from ..parts.block import ParallelBlock
from ..parts.causal_taps import CausalTaps
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.gated_recurrence import GatedLinearRecurrence
from ..parts.latent_attention import LatentAttention
from ..parts.mlp import GatedFeedForward
from ..parts.norm import GroupRMSNorm
from .decoder import DecoderModel, LayerCall


def build_riruzen(cfg: RiruzenConfig, rt: Runtime) -> DecoderModel:
    W = cfg.width
    embedding = TokenEmbedding(rt, "embed", cfg.vocab, W, positions_name="pos", max_positions=cfg.max_positions)
    blocks = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        if l.type == LATENT_ATTENTION:
            mixer = LatentAttention(rt, f"{p}.mix", W, l.heads, l.dim, l.vdim, l.q_rank, l.kv_rank, l.scale, cfg.norm_eps)
        elif l.type == HGRN2:
            mixer = GatedLinearRecurrence(rt, f"{p}.mix", W, l.heads, l.dim, l.vdim, cfg.norm_eps)
        else:
            raise ValueError(f"layer {i}: unknown type {l.type!r}")
        ffn = GatedFeedForward(rt, f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down", W, l.ff, act="relu") if l.ff is not None else None
        blocks.append(ParallelBlock(mixer, ffn, GroupRMSNorm(rt, f"{p}.norm1", W, cfg.norm_groups, cfg.norm_eps), rt.act_dtype,
                                    input_taps=CausalTaps(rt, f"{p}.canon1", W, cfg.taps)))
    calls = [LayerCall(i, i) for i in range(len(blocks))]
    final_norm = GroupRMSNorm(rt, "final.norm", W, cfg.norm_groups, cfg.norm_eps)
    head = OutputHead(rt, "lm_head", cfg.vocab, W, embedding, scale=cfg.logit_scale)
    return DecoderModel(rt, embedding, blocks, calls, final_norm, head, cfg.vocab, cfg.max_positions, cfg.eos_token_ids)


register_architecture(RiruzenConfig.ARCHITECTURE, RiruzenConfig.from_dict, build_riruzen, replace=True)
