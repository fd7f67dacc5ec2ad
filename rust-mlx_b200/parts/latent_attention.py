"""Attention through a cached latent, without positions.

    c_q = RMSNorm(W_dq x)          q_h = W_uq,h c_q                      (heads h, ``dim`` numbers each)
    c   = RMSNorm(W_dkv x)         k_h = W_uk,h c,   v_h = W_uv,h c      (``vdim`` numbers a value)
    s_h[i, j] = scale * q_h[i] . k_h[j]      over the keys j <= i of the window (i - j < window; 0: all)
    o_h = softmax(s_h) v_h * sigmoid(W_g x)_h        y = W_o [o_1 .. o_H]

Only c is kept per token (``kv_rank`` numbers in one pool of pages: ``CacheSpec(values=False)``).  Keys and
values are never formed: since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, the query is carried into the latent's space
(one small product a head), attention runs there with c as key and as value of every head (one kv head of
size kv_rank: the framework's attention kernels, with the same pool as keys and values), and W_uv,h is applied
to the result.  A step's work then follows the latents it reads, not heads * head size.

The three products that read x (W_dq, W_dkv, W_g) are one product over the stacked weights.  A mixer built with
``own_latent=False`` has no W_dkv: its schedule entry names the cache of the layer whose latents it reads, with its
own W_uk, W_uv, queries and window.
"""
from __future__ import annotations

import torch

from .base import CacheSpec, Mixer, ParamSpec


class LatentAttentionMixer(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, eps: float,
                 scale: float | None = None, window: int = 0, cache_window: int | None = None, own_latent: bool = True,
                 gated: bool = True):
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale is not None else self.dim ** -0.5
        self.window = int(window)
        # how long the cache keeps a latent: the widest window of the layers that read it (0: for ever)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.own_latent, self.gated = bool(own_latent), bool(gated)

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=1, head_dim=self.kv_rank, window=self.cache_window, values=False)

    def heads_a_call(self) -> int:
        """How many heads one attention launch takes: all of them share the one latent "kv head", and the kernels take
        groups of up to 16 query heads (the tensor-core kernels by their tiles; the FMA kernel runs a warp a head and
        has registers for 16 of them in a block).  More heads go in several launches over the same latents."""
        return min(self.heads, 16)

    def graph_key(self, shape):
        return (self.ctx.ops.decode_attention_splits(shape.n_seqs, 1, self.kv_rank, self.heads_a_call(), shape.max_seq_len,
                                                     self.ctx.dtype),)

    def param_specs(self):
        p = self.prefix
        specs = [ParamSpec(f"{p}.dq", (self.q_rank, self.width)),
                 ParamSpec(f"{p}.dq.norm", (self.q_rank,), "norm", "float32"),
                 ParamSpec(f"{p}.uq", (self.heads * self.dim, self.q_rank))]
        if self.own_latent:
            specs += [ParamSpec(f"{p}.dkv", (self.kv_rank, self.width)),
                      ParamSpec(f"{p}.dkv.norm", (self.kv_rank,), "norm", "float32")]
        specs += [ParamSpec(f"{p}.uk", (self.heads * self.dim, self.kv_rank)),
                  ParamSpec(f"{p}.uv", (self.heads * self.vdim, self.kv_rank))]
        if self.gated:
            specs.append(ParamSpec(f"{p}.g", (self.heads, self.width)))
        specs.append(ParamSpec(f"{p}.o", (self.width, self.heads * self.vdim)))
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        p = self.prefix
        down = [tensors.pop(f"{p}.dq")]
        if self.own_latent:
            down.append(tensors.pop(f"{p}.dkv"))
            self.kv_norm = tensors[f"{p}.dkv.norm"].contiguous()
        else:
            self.kv_norm = None
        if self.gated:
            down.append(tensors.pop(f"{p}.g"))
        self.w_down = torch.cat(down, dim=0).contiguous()          # rows: [query latent | key/value latent | gates]
        self.q_norm = tensors[f"{p}.dq.norm"].contiguous()
        self.w_uq = tensors[f"{p}.uq"].contiguous()
        # W_uk,h^T: [heads, kv_rank, dim], the matrix that carries head h's query into the latent's space
        self.w_uk_t = tensors.pop(f"{p}.uk").view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors.pop(f"{p}.uv").view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()

    def linear_weights(self):
        return [self.w_down, self.w_uq, self.w_o]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n, H, r = x.shape[0], self.heads, self.kv_rank
        tap = self.ctx.tap
        kv = r if self.own_latent else 0
        proj = ws.get("latent_down", (n, self.w_down.shape[0]), dt)
        ops.linear(x, self.w_down, proj, ws, batch.status)
        if tap is not None:
            tap("latent_down", proj)
        cq = ws.get("latent_q", (n, self.q_rank), dt)
        write = self.own_latent and not cache.read_only
        ops.latent_norms(proj, self.q_rank, kv, self.q_norm, self.kv_norm, self.eps, cq, cache.k_pool if write else None,
                         batch.positions, batch.seq_index, cache.block_table, cache.page_size, batch.status)
        if tap is not None:
            tap("latent_q", cq)
        q = ws.get("q_heads", (n, H * self.dim), dt)
        ops.linear(cq, self.w_uq, q, ws, batch.status)
        if tap is not None:
            tap("q_heads", q)
        q_lat = ws.get("q_rot", (n, H * r), dt)
        ops.linear_heads(q.view(n, H, self.dim), self.w_uk_t, q_lat.view(n, H, r))
        if tap is not None:
            tap("q_latent", q_lat)
        o_lat = ws.get("attn_out", (n, H * r), dt)
        step = self.heads_a_call()
        if step >= H:
            ops.attention(q_lat, cache.k_pool, cache.k_pool, batch, cache.block_table, cache.page_size, o_lat, H, 1, r,
                          self.window, self.scale, ws)
        else:
            for h0 in range(0, H, step):
                hc = min(step, H - h0)
                q_part = ws.get("q_rot_part", (n, hc * r), dt)
                o_part = ws.get("attn_out_part", (n, hc * r), dt)
                q_part.view(n, hc, r).copy_(q_lat.view(n, H, r)[:, h0:h0 + hc])
                ops.attention(q_part, cache.k_pool, cache.k_pool, batch, cache.block_table, cache.page_size, o_part, hc, 1, r,
                              self.window, self.scale, ws)
                o_lat.view(n, H, r)[:, h0:h0 + hc].copy_(o_part.view(n, hc, r))
        if tap is not None:
            tap("attn_out", o_lat)
        o = ws.get("attn_heads", (n, H * self.vdim), dt)
        ops.linear_heads(o_lat.view(n, H, r), self.w_uv, o.view(n, H, self.vdim))
        if tap is not None:
            tap("attn_values", o)
        if self.gated:
            ops.gate_heads(o, proj[:, self.q_rank + kv:], H, self.vdim)
        if tap is not None:
            tap("attn_heads", o)
        y = ws.get("mixer_out", (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        return y
