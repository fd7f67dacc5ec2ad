"""The Gugalorn decoder put together from parts.

Token embeddings times a factor; pre-norm layers whose mixer reads its normed input through a short causal convolution
(x + conv(x)); the mixer is a state-space layer (a scalar decay a head) or two mixers side by side (softmax attention
with whole-projection q/k norms, partial rotation, a sink in the denominator and an output gate, beside gated linear
attention), a layer may have a silu-gated feed-forward or none; a last RMS norm and a head tied to the embedding table.
Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``.
Every layer remembers several things (the convolution's last inputs, pages of keys and values, states of fixed size):
its schedule entry names one cache for each.
"""
from __future__ import annotations

from ..config.gugalorn import GugalornConfig
from ..parts.attention import GatedAttentionMixer
from ..parts.base import LayerCall
from ..parts.block import PreNormBlock
from ..parts.conv import ShortConv
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.feedforward import SwiGLUFeedForward
from ..parts.norm import RMSNorm
from ..parts.position import RotaryEmbedding
from ..parts.recurrent import GatedLinearMixer, ParallelMixer, StateSpaceMixer
from ..registry import register_architecture
from .spec import ModelSpec


def _mixer(prefix: str, c: GugalornConfig, layer):
    m = layer.mixer
    if layer.type == "mamba2":
        return StateSpaceMixer(prefix, c.width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, c.eps)
    a, g = m.left, m.right
    left = GatedAttentionMixer(f"{prefix}.left", c.width, a.heads, a.kv_heads, a.dim, a.vdim,
                               RotaryEmbedding(a.dim, a.rot_base, rotary_dim=a.rot_dims), a.scale, whole_norm_eps=c.eps,
                               sink=True, gate=True)
    right = GatedLinearMixer(f"{prefix}.right", c.width, g.heads, g.dim, g.vdim, c.eps, out_name="mixer_out_right")
    return ParallelMixer(left, right, m.left_scale, m.right_scale)


def build_gugalorn(config: GugalornConfig) -> ModelSpec:
    c = config
    embedding = TokenEmbedding("embed", c.vocab, c.width, scale=c.embedding_scale)
    blocks, schedule, next_cache = [], [], 0
    for i, layer in enumerate(c.layers):
        p = f"l{i}"
        canon = ShortConv(f"{p}.canon1", c.width, c.canon_taps, residual=True) if c.canon_taps > 0 else None
        ffn = SwiGLUFeedForward(f"{p}.mlp", c.width, layer.ff, activation="silu", names=("gate", "up", "down")) if layer.ff else None
        block = PreNormBlock(RMSNorm(f"{p}.norm1", c.width, c.eps), _mixer(f"{p}.mix", c, layer),
                             RMSNorm(f"{p}.norm2", c.width, c.eps) if ffn is not None else None, ffn, input_conv=canon)
        blocks.append(block)
        ids = tuple(range(next_cache, next_cache + len(block.cache_specs())))
        next_cache += len(ids)
        schedule.append(LayerCall(i, ids))
    spec = ModelSpec(config=c, embedding=embedding, blocks=blocks, schedule=schedule,
                     final_norm=RMSNorm("final.norm", c.width, c.eps), head=OutputHead(c.vocab, c.width, tied_to=embedding),
                     vocab_size=c.vocab, eos_token_ids=tuple(c.eos_token_id))
    spec.check_schedule()
    return spec


register_architecture("Gugalorn", GugalornConfig, build_gugalorn, model_types=("gugalorn",))
