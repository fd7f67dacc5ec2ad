"""Tiny Resolorn configurations and helpers for the tests.

R1: dense feed-forwards and a layer without one; a layer that reads another layer's latents with a wider window
than that layer's own; a layer without a window; odd sizes (vdim != dim, a vocabulary that is no multiple of 4).
R2: routed feed-forwards: top 2 of 6 with a shared expert, top == experts without one, top 1 of 5; latents of 96
and 64 numbers; 3 and 8 heads.  R3: a latent of 128 numbers and 8 heads, pages of 64 (the bfloat16 replay then
runs the tensor-core attention kernels that serve such sizes), one layer reading the other's latents.
"""
import json
import os

import torch


def _mixer(heads, dim, vdim, q_rank, kv_rank, window=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _moe(ff, experts, top, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


R1 = {"architecture": "Resolorn", "vocab": 211, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5},
      "residual_mult": 0.5,
      "layers": [_layer(_mixer(2, 16, 24, 24, 32, window=20), {"kind": "dense", "ff": 96}),
                 _layer(_mixer(2, 16, 8, 20, 32, window=33, kv_from=0, scale=0.31), None),
                 _layer(_mixer(4, 8, 8, 16, 64), {"kind": "dense", "ff": 40})]}
PAGE_R1 = 16

R2 = {"architecture": "Resolorn", "vocab": 300, "width": 96, "max_positions": 640, "norm": {"eps": 1e-6},
      "residual_mult": 1.0,
      "layers": [_layer(_mixer(3, 32, 16, 40, 96, window=70), _moe(48, 6, 2, shared=32)),
                 _layer(_mixer(3, 16, 16, 24, 96, window=70, kv_from=0), _moe(24, 4, 4)),
                 _layer(_mixer(8, 16, 16, 48, 64, window=129), _moe(40, 5, 1, shared=64))]}
PAGE_R2 = 32

R3 = {"architecture": "Resolorn", "vocab": 320, "width": 128, "max_positions": 1024, "norm": {"eps": 1e-6},
      "residual_mult": 0.7,
      "layers": [_layer(_mixer(8, 32, 32, 64, 128, window=100), {"kind": "dense", "ff": 192}),
                 _layer(_mixer(8, 16, 32, 48, 128, kv_from=0), _moe(64, 4, 2, shared=64))]}
PAGE_R3 = 64

# R4: more heads than an attention launch takes (20 over a latent of 64: 16 + 4; 40 over one of 24: 16 + 16 + 8), top 1 of 1
R4 = {"architecture": "Resolorn", "vocab": 150, "width": 80, "max_positions": 256, "norm": {"eps": 1e-6},
      "residual_mult": 0.4,
      "layers": [_layer(_mixer(20, 8, 8, 24, 64, window=40), _moe(16, 1, 1)),
                 _layer(_mixer(40, 4, 4, 16, 24), {"kind": "dense", "ff": 56})]}
PAGE_R4 = 16

# R5: sizes that are multiples of nothing much (width 90, vocabulary 97, heads of 6 and 10 numbers, latents of 40 and 18):
# the kernels' plain arrangements in both dtypes, a window shorter than a page, a factor above 1, a larger eps
R5 = {"architecture": "Resolorn", "vocab": 97, "width": 90, "max_positions": 200, "norm": {"eps": 1e-4},
      "residual_mult": 1.3,
      "layers": [_layer(_mixer(3, 6, 10, 30, 40, window=7, scale=0.5), _moe(20, 3, 2, shared=14)),
                 _layer(_mixer(5, 10, 6, 22, 18), {"kind": "dense", "ff": 36}),
                 _layer(_mixer(2, 14, 14, 10, 40, window=50, kv_from=0), None)]}
PAGE_R5 = 16

CONFIGS = {"R1": (R1, PAGE_R1), "R2": (R2, PAGE_R2), "R3": (R3, PAGE_R3), "R4": (R4, PAGE_R4), "R5": (R5, PAGE_R5)}


def make_folder(tmp_path, raw: dict, seed: int = 0, sharp: float = 8.0, out_boost: float = 20.0) -> str:
    """A model folder from the engine's random-weights mode, its query and key up-projections multiplied by
    ``sharp``: with N(0, 0.02) weights every score is near zero and attention an average over all keys, so that a
    key that is missing, stale or read from the wrong page hides in the tolerance; scaled, a few keys carry most of
    the weight and any wrong key shows.  The mixers' output projections are multiplied by ``out_boost``: otherwise
    what a mixer adds is a few percent of the embedding it is added to, and a wrong mixer changes the logits little."""
    from safetensors.torch import load_file, save_file
    from rust_mlx_b200.config import ResolornConfig
    from rust_mlx_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"resolorn_{abs(hash(json.dumps(raw, sort_keys=True))) % 10**8}_{seed}_{sharp}_{out_boost}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(ResolornConfig.from_dict(raw), folder, seed=seed, store_dtype="bfloat16")
        t = load_file(os.path.join(folder, "model.safetensors"))
        for k in t:
            if k.endswith(".mix.uq") or k.endswith(".mix.uk"):
                t[k] = (t[k].float() * sharp).to(t[k].dtype)
            if k.endswith(".mix.o"):
                t[k] = (t[k].float() * out_boost).to(t[k].dtype)
        save_file(t, os.path.join(folder, "model.safetensors"))
    return folder


def weights(folder: str) -> dict:
    from safetensors.torch import load_file
    return {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def row_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (means taken off) over that of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-12)
