"""Configuration of the Resolorn decoder.

config.json of this family is nested:

    architecture      "Resolorn"
    vocab, width, max_positions (rows of the learned position table)
    norm.eps          the eps of every RMS norm
    residual_mult     what a layer adds to the stream is multiplied by this
    layers[]          one entry a layer, in order:
        type          which mixer: "latent_attention"
        mixer         heads, dim (query/key numbers a head), vdim (value numbers a head), q_rank, kv_rank (sizes of
                      the query and the key/value latent), scale (of the scores), mask.size (a query sees itself
                      and the mask.size - 1 tokens before it; absent: every token before it), kv_from (the layer
                      whose cached latents this layer reads instead of making its own)
        mlp           null, or kind "dense" with ff, or kind "moe" with expert.ff, router.experts, router.top and
                      an optional shared.ff

Every size and constant is read from here; every problem of a file is reported in one ``ConfigError``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .base import ConfigError, ModelConfig

MIXERS = ("latent_attention",)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int = 0             # 0: no window
    kv_from: Optional[int] = None

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
               "vdim": self.vdim}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int                     # inner size (of every expert, for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class ResolornLayer:
    type: str
    mixer: LatentAttentionConfig
    mlp: Optional[FeedForwardConfig]

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None, "type": self.type}


def _int(problems, where, node, key, minimum=1, required=True, default=0):
    v = node.get(key) if isinstance(node, dict) else None
    if v is None:
        if required:
            problems.append(f"{where}: missing '{key}'")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        problems.append(f"{where}: '{key}' must be an integer, got {v!r}")
        return default
    if int(v) < minimum:
        problems.append(f"{where}: '{key}' must be at least {minimum}, got {v!r}")
        return default
    return int(v)


def _float(problems, where, node, key, required=True, default=0.0):
    v = node.get(key) if isinstance(node, dict) else None
    if v is None:
        if required:
            problems.append(f"{where}: missing '{key}'")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        problems.append(f"{where}: '{key}' must be a number, got {v!r}")
        return default
    return float(v)


@dataclass
class ResolornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    eps: float = 0.0
    residual_mult: float = 1.0
    layers: tuple = ()
    eos_token_id: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ResolornConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        p = []
        name = raw.get("architecture") or (raw.get("architectures") or [""])[0]
        vocab = _int(p, "config", raw, "vocab")
        width = _int(p, "config", raw, "width")
        max_positions = _int(p, "config", raw, "max_positions")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            p.append("config: missing 'norm' (an object with 'eps')")
            norm = {}
        eps = _float(p, "norm", norm, "eps", required=isinstance(raw.get("norm"), dict))
        mult = _float(p, "config", raw, "residual_mult", required=False, default=1.0)
        entries = raw.get("layers")
        layers = []
        if not isinstance(entries, list) or not entries:
            p.append("config: 'layers' must be a list with at least one layer")
            entries = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                p.append(f"{where}: must be an object")
                continue
            kind = entry.get("type")
            if kind not in MIXERS:
                p.append(f"{where}: unknown mixer type {kind!r} (known: {', '.join(MIXERS)})")
                continue
            m = entry.get("mixer")
            if not isinstance(m, dict):
                p.append(f"{where}: missing 'mixer'")
                continue
            mask = m.get("mask")
            window = _int(p, f"{where}.mixer.mask", mask, "size") if isinstance(mask, dict) else 0
            kv_from = m.get("kv_from")
            if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
                p.append(f"{where}.mixer: 'kv_from' must be a layer's index, got {kv_from!r}")
                kv_from = None
            mixer = LatentAttentionConfig(
                heads=_int(p, f"{where}.mixer", m, "heads"), dim=_int(p, f"{where}.mixer", m, "dim"),
                vdim=_int(p, f"{where}.mixer", m, "vdim"), q_rank=_int(p, f"{where}.mixer", m, "q_rank"),
                kv_rank=_int(p, f"{where}.mixer", m, "kv_rank"), scale=_float(p, f"{where}.mixer", m, "scale"),
                window=window, kv_from=kv_from)
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
                    p.append(f"{where}.mlp: 'kind' must be 'dense' or 'moe'")
                elif f["kind"] == "dense":
                    mlp = FeedForwardConfig("dense", _int(p, f"{where}.mlp", f, "ff"))
                else:
                    router = f.get("router") if isinstance(f.get("router"), dict) else {}
                    shared = f.get("shared")
                    mlp = FeedForwardConfig(
                        "moe", _int(p, f"{where}.mlp.expert", f.get("expert"), "ff"),
                        experts=_int(p, f"{where}.mlp.router", router, "experts"), top=_int(p, f"{where}.mlp.router", router, "top"),
                        shared_ff=_int(p, f"{where}.mlp.shared", shared, "ff") if isinstance(shared, dict) else 0)
            layers.append(ResolornLayer(kind, mixer, mlp))
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else (tuple(eos) if isinstance(eos, (list, tuple)) else (eos,))
        cfg = cls(model_type="resolorn", architectures=(name or "Resolorn",), vocab=vocab, width=width, max_positions=max_positions,
                  eps=eps, residual_mult=mult, layers=tuple(layers), eos_token_id=eos)
        cfg._raw = dict(raw)
        p = cfg.validate()
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        return cfg

    def validate(self) -> list:
        p = []
        if not self.eps > 0:
            p.append("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if not m.scale > 0:
                p.append(f"layers[{i}].mixer: scale must be positive")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    p.append(f"layers[{i}].mixer: kv_from {m.kv_from} must name an earlier layer")
                else:
                    src = self.layers[m.kv_from].mixer
                    if src.kv_from is not None:
                        p.append(f"layers[{i}].mixer: kv_from names layer {m.kv_from}, which keeps no latents of its own")
                    elif src.kv_rank != m.kv_rank:
                        p.append(f"layers[{i}].mixer: kv_rank {m.kv_rank} differs from layer {m.kv_from}'s {src.kv_rank}")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                if f.top > f.experts:
                    p.append(f"layers[{i}].mlp: top {f.top} of {f.experts} experts")
                if f.top > 32:
                    p.append(f"layers[{i}].mlp: at most 32 experts a token")
        return p

    @property
    def max_position_embeddings(self) -> int:
        """The longest sequence the model takes (what the engine limits requests to)."""
        return self.max_positions

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def cache_windows(self) -> dict:
        """layer that keeps latents -> how long they must be kept: the widest window among the layers that read them
        (0: for ever, if any of them has no window)."""
        readers = {}
        for i, layer in enumerate(self.layers):
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            readers.setdefault(owner, []).append(layer.mixer.window)
        return {owner: (0 if 0 in ws else max(ws)) for owner, ws in readers.items()}

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0] if self.architectures else "Resolorn",
               "layers": [layer.to_dict() for layer in self.layers], "max_positions": self.max_positions,
               "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
