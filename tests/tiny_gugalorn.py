"""Tiny Gugalorn configurations and helpers for the tests.

G1: both mixers twice, layers with and without a feed-forward, one kv head for four query heads, no rotation in one
layer, value heads wider and narrower than key heads, groups of one and of several heads in the state-space layers,
convolutions of 2, 3 and 4 taps.  G2: heads of 64 and 128 with pages of 64 (the bfloat16 replay then runs the
tensor-core attention kernels that serve such sizes), states of 64 rows.  G3: sizes that are multiples of nothing much
(width 90, vocabulary 97, a state of 7 and of 40 rows a head, value heads of 6 and 10 numbers), no input convolution at
all, an inner convolution of one tap, a side of the parallel mixer switched off by its factor, factors of 1.
"""
import json
import os

import torch


def ssm(heads, vdim, state, groups, conv, norm_groups, ff=0):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def par(left, right, left_scale=1.0, right_scale=1.0, ff=0):
    h, g, d, e, dims, base, scale = left
    rh, rd, re = right
    return {"type": "parallel",
            "mixer": {"left": {"heads": h, "kv_heads": g, "dim": d, "vdim": e, "rot": {"dims": dims, "base": base}, "scale": scale},
                      "right": {"heads": rh, "dim": rd, "vdim": re}, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(vocab, width, taps, layers, eps=1e-5, scale=1.0):
    raw = {"architecture": "Gugalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "layers": layers}
    if taps:
        raw["canon"] = {"taps": taps}
    return raw


G1 = model(211, 64, 3, [ssm(4, 8, 16, 1, 2, 1, ff=48),
                        par((4, 1, 16, 16, 8, 10000.0, 0.25), (2, 8, 12), 0.7, 1.3),
                        ssm(6, 4, 24, 3, 4, 3),
                        par((2, 2, 8, 24, 0, 10000.0, 0.4), (3, 20, 8), 1.1, 0.6, ff=40)], scale=0.5)
G2 = model(320, 128, 4, [par((8, 2, 64, 64, 32, 1e6, 0.125), (4, 32, 32), 1.2, 0.5, ff=96),
                         ssm(8, 16, 64, 2, 4, 2),
                         par((4, 4, 128, 128, 128, 5e5, 0.09), (2, 64, 16), 0.8, 0.9)], eps=1e-6, scale=2.0)
G3 = model(97, 90, 0, [par((6, 3, 12, 20, 4, 100.0, 0.3), (1, 7, 10), 1.0, 1.0, ff=36),
                       ssm(5, 6, 40, 5, 1, 1, ff=20),
                       par((3, 1, 10, 6, 10, 50.0, 0.5), (5, 5, 6), 0.0, 1.0),
                       ssm(2, 10, 7, 1, 3, 2)], eps=1e-4, scale=1.0)
CONFIGS = {"G1": (G1, 16), "G2": (G2, 64), "G3": (G3, 16)}


def make_folder(tmp_path, raw: dict, seed: int = 0, sharp: float = 8.0, out_boost: float = 12.0) -> str:
    """A model folder from the engine's random-weights mode, with the tensors whose useful range is not N(0, 0.02) drawn
    anew: lower bounds of the forget gate in (0.05, 0.95), its bias N(0, 1), A_log in (-1.5, 0.5), dt_bias in (-3, 0.5),
    D near 1, convolution taps of some size; the q and k projections times ``sharp`` and their norm weights spread (a
    few keys carry most of a row's weight, so a lost or stale key shows); output projections times ``out_boost`` (what a
    mixer adds to the stream is comparable to the stream)."""
    from safetensors.torch import load_file, save_file
    from rust_mlx_b200.config import GugalornConfig
    from rust_mlx_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"gugalorn_{abs(hash(json.dumps(raw, sort_keys=True))) % 10**8}_{seed}_{sharp}_{out_boost}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(GugalornConfig.from_dict(raw), folder, seed=seed, store_dtype="bfloat16")
        t = load_file(os.path.join(folder, "model.safetensors"))
        g = torch.Generator().manual_seed(1000 + seed)
        rnd = lambda like: torch.rand(like.shape, generator=g)          # noqa: E731
        nrm = lambda like: torch.randn(like.shape, generator=g)         # noqa: E731
        bf = lambda x: x.to(torch.bfloat16).float()                     # noqa: E731  (what a bfloat16 checkpoint can hold)
        for k in list(t):
            v = t[k]
            if k.endswith(".lower"):
                t[k] = bf(0.05 + 0.9 * rnd(v))
            elif k.endswith(".f.b"):
                t[k] = bf(nrm(v))
            elif k.endswith(".right.f") or k.endswith(".mix.in"):
                t[k] = (v.float() * 6.0).to(v.dtype)
            elif k.endswith(".A_log"):
                t[k] = bf(-1.5 + 2.0 * rnd(v))
            elif k.endswith(".dt_bias"):
                t[k] = bf(-3.0 + 3.5 * rnd(v))
            elif k.endswith(".D"):
                t[k] = bf(1.0 + 0.3 * nrm(v))
            elif k.endswith(".conv") or k.endswith(".canon1"):
                t[k] = bf(0.4 * nrm(v))
            elif k.endswith(".conv.b"):
                t[k] = bf(0.2 * nrm(v))
            elif k.endswith(".left.q") or k.endswith(".left.k"):
                t[k] = (v.float() * sharp).to(v.dtype)
            elif k.endswith(".q.norm") or k.endswith(".k.norm"):
                t[k] = bf(2.5 * (1.0 + 0.5 * nrm(v)))
            elif k.endswith(".o"):
                t[k] = (v.float() * out_boost).to(v.dtype)
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
