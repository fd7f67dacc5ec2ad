"""A plain, slow implementation of the Gugalorn decoder: float64, whole sequences, no cache, one function a mechanism.

It shares no code with the package.  ``config`` is the nested dictionary of config.json, ``tensors`` maps checkpoint
names to torch tensors.  Notation: T tokens, rows are tokens; W applied as ``h @ W.T``.

    layer:      x += mixer(h + conv(h)), h = norm1(x);   x += ff(norm2(x)) where the layer has a feed-forward
    mamba2:     per head S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t
    parallel:   cl * attention(h) + cr * hgrn2(h)
    hgrn2:      per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(h, w, bias=None):
    """out[t, c] = sum_j w[c, j] * h[t - taps + 1 + j, c] (+ bias[c]); rows before the first are zero."""
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        shift = taps - 1 - j
        if shift == 0:
            out += h * w[:, j]
        elif shift < h.shape[0]:
            out[shift:] += h[:-shift] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def rotate(x, positions, dims, base):
    """x [T, heads, size]: the first ``dims`` numbers of every head turn, number i paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_attention(q, k, v, scale, window=0):
    """q [T, H, d], k [T, G, d], v [T, G, e]; causal; weights exp(s_j) / (1 + sum_j exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    idx = torch.arange(T)
    mask = idx[None, :] <= idx[:, None]
    if window:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = torch.where(mask, s, torch.full_like(s, -math.inf))
        m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))
        out[:, h] = p @ v[:, g]
    return out


def gated_attention(h, positions, t, p, m, eps):
    """The softmax side: whole-projection norms of q and k, rotation, a sink in the denominator, an output gate."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ t[f"{p}.q"].T, eps) * t[f"{p}.q.norm"]
    k = rms(h @ t[f"{p}.k"].T, eps) * t[f"{p}.k.norm"]
    v = h @ t[f"{p}.v"].T
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    q = rotate(q.view(T, H, d), positions, dims, base)
    k = rotate(k.view(T, G, d), positions, dims, base)
    o = sink_attention(q, k, v.view(T, G, e), m["scale"]).reshape(T, H * e)
    o = o * torch.sigmoid(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


def hgrn2(h, t, p, m, eps, state=None):
    """The linear side: the forget gate f also decides what is written (1 - f)."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ t[f"{p}.q"].T).view(T, H, d)
    v = (h @ t[f"{p}.v"].T).view(T, H, e)
    low = t[f"{p}.lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ t[f"{p}.f"].T + t[f"{p}.f.b"])).view(T, H, d)
    S = torch.zeros(H, d, e, dtype=F64) if state is None else state
    out = torch.zeros(T, H, e, dtype=F64)
    for i in range(T):
        S = f[i][:, :, None] * S + (1.0 - f[i])[:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hde,hd->he", S, q[i])
    out = rms(out, eps) * t[f"{p}.norm"]
    return out.reshape(T, H * e) @ t[f"{p}.o"].T


def parallel_mixer(h, positions, t, p, m, eps):
    left = gated_attention(h, positions, t, f"{p}.left", m["left"], eps)
    right = hgrn2(h, t, f"{p}.right", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mamba2(h, t, p, m, eps):
    T = h.shape[0]
    H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * e
    proj = h @ t[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[f"{p}.conv"], t[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(T, H, e)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + t[f"{p}.dt_bias"])
    decay = torch.exp(-torch.exp(t[f"{p}.A_log"]) * dt)           # [T, H]
    per = H // G
    S = torch.zeros(H, N, e, dtype=F64)
    y = torch.zeros(T, H, e, dtype=F64)
    for i in range(T):
        Bh = B[i].repeat_interleave(per, dim=0)                    # [H, N]
        Ch = C[i].repeat_interleave(per, dim=0)
        S = decay[i][:, None, None] * S + dt[i][:, None, None] * Bh[:, :, None] * x[i][:, None, :]
        y[i] = torch.einsum("hne,hn->he", S, Ch) + t[f"{p}.D"][:, None] * x[i]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * t[f"{p}.norm"]
    return y @ t[f"{p}.o"].T


def feed_forward(h, t, p):
    return (silu(h @ t[f"{p}.gate"].T) * (h @ t[f"{p}.up"].T)) @ t[f"{p}.down"].T


def forward(config, tensors, tokens, layers_out=None):
    """Logits [T, vocab] (float64) of one sequence from position 0.  ``layers_out``: a list that receives the residual
    stream after every layer."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = t["embed"][ids] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        h = rms(x, eps) * t[f"{p}.norm1"]
        if config.get("canon"):                      # (a model without the key has no input convolution)
            h = h + causal_conv(h, t[f"{p}.canon1"])
        if layer["type"] == "mamba2":
            x = x + mamba2(h, t, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, positions, t, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown mixer {layer['type']!r}")
        if layer.get("mlp") is not None:
            x = x + feed_forward(rms(x, eps) * t[f"{p}.norm2"], t, f"{p}.mlp")
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * t["final.norm"]) @ t["embed"].T
