"""The Resolorn decoder put together from parts.

Token embedding plus a learned position vector; every layer one RMS norm whose rows feed a latent-attention mixer
and a feed-forward side by side (dense with the tanh form of GELU, or routed experts with silu and a shared
expert, or none), their sum times the model's factor added to the stream; a last RMS norm and an output head of
its own.  Tensors: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
A layer whose mixer names ``kv_from`` reads the latents another layer cached: its schedule entry names that layer's
cache, which is kept as long as the widest window among its readers asks.
"""
from __future__ import annotations

from ..config.resolorn import ResolornConfig
from ..parts.base import LayerCall
from ..parts.block import ParallelBlock
from ..parts.embedding import OutputHead, PositionedEmbedding
from ..parts.feedforward import SwiGLUFeedForward
from ..parts.latent_attention import LatentAttentionMixer
from ..parts.norm import RMSNorm
from ..parts.routed import RoutedFeedForward
from ..registry import register_architecture
from .spec import ModelSpec

_NAMES = ("gate", "up", "down")


def _feed_forward(prefix: str, width: int, f):
    if f is None:
        return None
    if f.kind == "dense":
        return SwiGLUFeedForward(prefix, width, f.ff, activation="gelu_tanh", names=_NAMES)
    shared = SwiGLUFeedForward(f"{prefix}.shared", width, f.shared_ff, activation="silu", names=_NAMES) if f.shared_ff else None
    return RoutedFeedForward(prefix, width, f.ff, f.experts, f.top, activation="silu", shared=shared, names=_NAMES)


def build_resolorn(config: ResolornConfig) -> ModelSpec:
    c = config
    embedding = PositionedEmbedding("embed", c.vocab, c.width, "pos", c.max_positions)
    keep = c.cache_windows()
    blocks, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        owner = i if m.kv_from is None else m.kv_from
        mixer = LatentAttentionMixer(f"l{i}.mix", c.width, m.heads, m.dim, m.vdim, m.q_rank, m.kv_rank, c.eps, scale=m.scale,
                                     window=m.window, cache_window=keep[owner], own_latent=m.kv_from is None)
        blocks.append(ParallelBlock(RMSNorm(f"l{i}.norm1", c.width, c.eps), mixer,
                                    _feed_forward(f"l{i}.mlp", c.width, layer.mlp), factor=c.residual_mult))
        schedule.append(LayerCall(i, owner))
    spec = ModelSpec(config=c, embedding=embedding, blocks=blocks, schedule=schedule,
                     final_norm=RMSNorm("final.norm", c.width, c.eps),
                     head=OutputHead(c.vocab, c.width, name="head"), vocab_size=c.vocab,
                     eos_token_ids=tuple(c.eos_token_id))
    spec.check_schedule()
    return spec


register_architecture("Resolorn", ResolornConfig, build_resolorn, model_types=("resolorn",))
