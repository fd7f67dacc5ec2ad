"""A routed feed-forward (mixture of experts) with an optional shared expert.

    z = W_router x                      in float32, whatever the activations' type
    E(x) = the ``top`` experts with the largest z; weight_e = softmax over those z alone
    y = sum over e in E(x) of weight_e * expert_e(x)  (+ shared(x))
    expert(x) = down(act(gate x) * (up x)), no biases

The experts' weights are kept stacked, [experts, 2 * inner, width] (gate rows, then up rows) and
[experts, width, inner].  A step sorts its (row, choice) pairs by expert on the device and the experts'
products run over their runs of rows (``csrc/kernels/moe.cu``); nothing waits for the host, so decode
steps can be captured in graphs.  The shared expert is a gated feed-forward like any other.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec


class RoutedFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, width: int, inner: int, n_experts: int, top: int, activation: str = "silu",
                 shared: FeedForward | None = None, router_name: str = "router", expert_name: str = "e{index}",
                 names: tuple = ("gate", "up", "down")):
        if not 0 < top <= n_experts:
            raise ValueError(f"a row cannot take {top} of {n_experts} experts")
        if top > 32:
            raise ValueError("at most 32 experts a row")
        self.prefix, self.width, self.inner = prefix, int(width), int(inner)
        self.n_experts, self.top, self.activation = int(n_experts), int(top), activation
        self.shared = shared
        self.router = f"{prefix}.{router_name}"
        self.expert_names = [tuple(f"{prefix}.{expert_name.format(index=e)}.{n}" for n in names) for e in range(self.n_experts)]
        self.w_router = self.w_gate_up = self.w_down = None

    def children(self):
        return [self.shared] if self.shared is not None else []

    def param_specs(self):
        specs = [ParamSpec(self.router, (self.n_experts, self.width), "linear", "float32")]
        for gate, up, down in self.expert_names:
            specs += [ParamSpec(gate, (self.inner, self.width)), ParamSpec(up, (self.inner, self.width)),
                      ParamSpec(down, (self.width, self.inner))]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.w_router = tensors[self.router].contiguous()
        gu, down = [], []
        for gate, up, d in self.expert_names:
            gu.append(torch.cat([tensors.pop(gate), tensors.pop(up)], dim=0))
            down.append(tensors.pop(d))
        self.w_gate_up = torch.stack(gu).contiguous()      # [experts, 2 * inner, width]
        self.w_down = torch.stack(down).contiguous()       # [experts, width, inner]

    def forward(self, x, batch=None):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, top, e = x.shape[0], self.top, self.n_experts
        ids = ws.get("moe_ids", (n, top), torch.int32)
        weights = ws.get("moe_weights", (n, top), torch.float32)
        ops.moe_route(x, self.w_router, top, ids, weights)
        tap = self.ctx.tap
        if tap is not None:
            tap("moe_ids", ids)
            tap("moe_weights", weights)
        offsets = ws.get("moe_offsets", (e + 1,), torch.int32)
        pairs = ws.get("moe_sorted", (n * top,), torch.int32)
        where = ws.get("moe_where", (n * top,), torch.int32)
        ops.moe_sort(ids, e, offsets, pairs, where)
        if tap is not None:
            tap("moe_sorted", pairs)
        gu = ws.get("moe_gate_up", (n * top, 2 * self.inner), dt)
        ops.moe_gemm(x, self.w_gate_up, gu, offsets, sorted_pairs=pairs, top=top)
        if tap is not None:
            tap("moe_gate_up", gu)
        act = ws.get("moe_act", (n * top, self.inner), dt)
        ops.swiglu(gu, act, 0, self.activation)
        if tap is not None:
            tap("moe_act", act)
        y = ws.get("moe_expert_out", (n * top, self.width), dt)
        ops.moe_gemm(act, self.w_down, y, offsets)
        if tap is not None:
            tap("moe_expert_out", y)
        shared = self.shared.forward(x, batch, out_name="ffn_shared_out") if self.shared is not None else None
        if tap is not None and shared is not None:
            tap("moe_shared_out", shared)
        out = ws.get("ffn_out", (n, self.width), dt)
        ops.moe_combine(y, where, weights, shared, out)
        return out
