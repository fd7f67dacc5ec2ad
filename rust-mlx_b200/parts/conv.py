"""A short causal convolution over time on each channel, with the last taps - 1 inputs of every request as its state.

out_t = act(bias + sum_j w[:, j] * x_(t - taps + 1 + j)) (+ x_t with ``residual``); inputs before a sequence's first
token are zero.  The weight is [channels, taps] in a checkpoint (its last column is the current token's), held transposed in float32; sums are
formed in float and rounded once.  The state is a ring [taps - 1, channels] in the compute dtype, input p at row
p % (taps - 1), so a step reads what lies before its tokens and stores its last ones without moving anything.
"""
from __future__ import annotations

from .base import CacheSpec, ParamSpec, Part


class ShortConv(Part):
    graph_safe = True

    def __init__(self, name: str, channels: int, taps: int, bias_name: str | None = None, activation: str | None = None,
                 residual: bool = False):
        if activation not in (None, "silu"):
            raise ValueError(f"unknown activation {activation!r}")
        self.name, self.channels, self.taps = name, int(channels), int(taps)
        self.bias_name, self.activation, self.residual = bias_name, activation, bool(residual)
        self.weight = self.bias = None

    def cache_spec(self):
        return CacheSpec("state", state_shape=(max(self.taps - 1, 1), self.channels), state_dtype="compute")

    def cache_specs(self):
        return [self.cache_spec()]

    def param_specs(self):
        specs = [ParamSpec(self.name, (self.channels, self.taps), "linear", "float32")]
        if self.bias_name:
            specs.append(ParamSpec(self.bias_name, (self.channels,), "linear", "float32"))
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].t().contiguous()      # taps-major, as the kernel reads it
        self.bias = tensors[self.bias_name].contiguous() if self.bias_name else None

    def forward(self, x, batch, cache, out):
        """``x`` and ``out``: [tokens, channels], either may be some columns of wider rows."""
        self.ctx.ops.short_conv(x, self.weight, self.bias, out, cache.state, batch, cache.slots, self.activation, self.residual)
        return out
