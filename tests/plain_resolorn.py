"""A plain, slow implementation of the Resolorn decoder: float64, whole sequences, no cache.

One function per mechanism, written from the design's equations in this file's own notation; it shares
no code with the package.  ``config`` is the dictionary of a config.json, ``w`` maps tensor names to
float64 tensors.  With ``bf16=True`` the places where the serving path rounds (products' results and
activations) are rounded to bfloat16 too, so that two bfloat16 evaluations can be compared.

Notation: T tokens, D width, H heads, d query/key size, dv value size, r latent size.
"""
import math

import torch


def rnd(x, bf16):
    return x.to(torch.bfloat16).to(torch.float64) if bf16 else x


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def gated_unit(x, gate, up, down, act, bf16=False):
    """down . (act(gate . x) * (up . x)), row by row."""
    g = rnd(x @ gate.T, bf16)
    u = rnd(x @ up.T, bf16)
    return rnd(rnd(act(g) * u, bf16) @ down.T, bf16)


def routed_experts(x, w, prefix, mlp, bf16=False):
    """Each row goes to the ``top`` experts with the largest router logits; their weights are the softmax over the
    chosen logits alone; a shared expert, where the layer has one, is added for every row."""
    n_experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = x @ w[f"{prefix}.router"].T                       # [T, E]
    chosen = torch.topk(logits, top, dim=-1)
    weights = torch.softmax(chosen.values, dim=-1)               # over the chosen only
    out = torch.zeros_like(x)
    for e in range(n_experts):
        rows, slot = torch.nonzero(chosen.indices == e, as_tuple=True)
        if rows.numel() == 0:
            continue
        y = gated_unit(x[rows], w[f"{prefix}.e{e}.gate"], w[f"{prefix}.e{e}.up"], w[f"{prefix}.e{e}.down"], silu, bf16)
        out[rows] += weights[rows, slot].unsqueeze(-1) * y
    if mlp.get("shared"):
        out = out + gated_unit(x, w[f"{prefix}.shared.gate"], w[f"{prefix}.shared.up"], w[f"{prefix}.shared.down"], silu, bf16)
    return rnd(out, bf16)


def feed_forward(x, w, prefix, mlp, bf16=False):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return gated_unit(x, w[f"{prefix}.gate"], w[f"{prefix}.up"], w[f"{prefix}.down"], gelu_tanh, bf16)
    if mlp["kind"] == "moe":
        return routed_experts(x, w, prefix, mlp, bf16)
    raise ValueError(mlp["kind"])


def latent(x, w, prefix, eps, bf16=False):
    """The cached quantity: RMS norm of the down-projected row."""
    return rnd(rms_norm(rnd(x @ w[f"{prefix}.dkv"].T, bf16), w[f"{prefix}.dkv.norm"], eps), bf16)


def visible(T, window):
    """[T, T] bool: query i sees key j iff 0 <= i - j < window (window None: every key up to i)."""
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


def latent_attention(x, c, w, prefix, m, eps, bf16=False):
    """x [T, D]: the mixer's input; c [T, r]: the latents it attends over (its own, or another layer's)."""
    T = x.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rnd(rms_norm(rnd(x @ w[f"{prefix}.dq"].T, bf16), w[f"{prefix}.dq.norm"], eps), bf16)
    q = rnd(cq @ w[f"{prefix}.uq"].T, bf16).view(T, H, d)
    k = rnd(c @ w[f"{prefix}.uk"].T, bf16).view(T, H, d)
    v = rnd(c @ w[f"{prefix}.uv"].T, bf16).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    window = (m.get("mask") or {}).get("size")
    scores = scores.masked_fill(~visible(T, window), -math.inf)
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v)                        # [T, H, dv]
    gate = torch.sigmoid(x @ w[f"{prefix}.g"].T)                  # [T, H]
    o = rnd(o * gate.unsqueeze(-1), bf16).reshape(T, H * dv)
    return rnd(o @ w[f"{prefix}.o"].T, bf16)


def forward(config, w, tokens, bf16=False, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer."""
    eps = config["norm"]["eps"]
    mult = config["residual_mult"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    x = w["embed"][ids] + w["pos"][:T]
    latents = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        m = layer["mixer"]
        h = rnd(rms_norm(x, w[f"{p}.norm1"], eps), bf16)
        src = m.get("kv_from")
        if src is None:
            latents[i] = latent(h, w, f"{p}.mix", eps, bf16)
            c = latents[i]
        else:
            c = latents[src]
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        total = latent_attention(h, c, w, f"{p}.mix", m, eps, bf16)
        f = feed_forward(h, w, f"{p}.mlp", layer.get("mlp"), bf16)
        if f is not None:
            total = total + f
        x = x + mult * total
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(rms_norm(x, w["final.norm"], eps), bf16)
    return x @ w["head"].T
