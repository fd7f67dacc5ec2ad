"""Configuration of the Gugalorn decoder.

config.json of this family is nested:

    architecture      "Gugalorn"
    vocab, width
    norm.eps          the eps of every RMS norm
    embedding.scale   what a token's embedding is multiplied with (the output head reads the table unscaled)
    canon.taps        taps of the causal convolution that every mixer's input passes first
    layers[]          one entry a layer, in order:
        type          which mixer: "mamba2" or "parallel"
        mixer         mamba2:   heads, vdim, state, groups, conv (taps of the inner convolution), norm_groups
                      parallel: left (softmax attention: heads, kv_heads, dim, vdim, scale, rot.dims, rot.base),
                                right (gated linear attention: heads, dim, vdim), left_scale, right_scale
        mlp           null, or kind "dense" with ff

Every size and constant is read from here; every problem of a file is reported in one ``ConfigError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import ConfigError, ModelConfig
from .resolorn import _float, _int

MIXERS = ("mamba2", "parallel")


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0
    rot_base: float = 10000.0

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SinkAttentionConfig
    right: GatedLinearConfig
    left_scale: float = 1.0
    right_scale: float = 1.0

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class GugalornLayer:
    type: str
    mixer: object
    ff: int = 0                 # 0: the layer has no feed-forward

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": {"ff": self.ff, "kind": "dense"} if self.ff else None, "type": self.type}


def _mamba2(p, where, m) -> Mamba2Config:
    return Mamba2Config(heads=_int(p, where, m, "heads"), vdim=_int(p, where, m, "vdim"), state=_int(p, where, m, "state"),
                        groups=_int(p, where, m, "groups"), conv=_int(p, where, m, "conv"),
                        norm_groups=_int(p, where, m, "norm_groups", required=False, default=1))


def _parallel(p, where, m) -> Optional[ParallelMixerConfig]:
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, dict) or not isinstance(right, dict):
        p.append(f"{where}: a parallel mixer needs 'left' and 'right'")
        return None
    rot = left.get("rot") if isinstance(left.get("rot"), dict) else {}
    lc = SinkAttentionConfig(
        heads=_int(p, f"{where}.left", left, "heads"), kv_heads=_int(p, f"{where}.left", left, "kv_heads"),
        dim=_int(p, f"{where}.left", left, "dim"), vdim=_int(p, f"{where}.left", left, "vdim"),
        scale=_float(p, f"{where}.left", left, "scale"),
        rot_dims=_int(p, f"{where}.left.rot", rot, "dims", minimum=0, required=False, default=0),
        rot_base=_float(p, f"{where}.left.rot", rot, "base", required=False, default=10000.0))
    rc = GatedLinearConfig(heads=_int(p, f"{where}.right", right, "heads"), dim=_int(p, f"{where}.right", right, "dim"),
                           vdim=_int(p, f"{where}.right", right, "vdim"))
    return ParallelMixerConfig(lc, rc, left_scale=_float(p, where, m, "left_scale", required=False, default=1.0),
                               right_scale=_float(p, where, m, "right_scale", required=False, default=1.0))


@dataclass
class GugalornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 0.0
    embedding_scale: float = 1.0
    canon_taps: int = 0
    layers: tuple = ()
    eos_token_id: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "GugalornConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        p = []
        name = raw.get("architecture") or (raw.get("architectures") or [""])[0]
        vocab = _int(p, "config", raw, "vocab")
        width = _int(p, "config", raw, "width")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            p.append("config: missing 'norm' (an object with 'eps')")
            norm = {}
        eps = _float(p, "norm", norm, "eps", required=isinstance(raw.get("norm"), dict))
        emb = raw.get("embedding") if isinstance(raw.get("embedding"), dict) else {}
        scale = _float(p, "embedding", emb, "scale", required=False, default=1.0)
        canon = raw.get("canon") if isinstance(raw.get("canon"), dict) else {}
        taps = _int(p, "canon", canon, "taps", required=False, default=0)   # absent: no input convolution
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
            mixer = _mamba2(p, f"{where}.mixer", m) if kind == "mamba2" else _parallel(p, f"{where}.mixer", m)
            f = entry.get("mlp")
            ff = 0
            if f is not None:
                if not isinstance(f, dict) or f.get("kind", "dense") != "dense":
                    p.append(f"{where}.mlp: 'kind' must be 'dense'")
                else:
                    ff = _int(p, f"{where}.mlp", f, "ff")
            if mixer is not None:
                layers.append(GugalornLayer(kind, mixer, ff))
        if p:
            raise ConfigError("invalid configuration: " + "; ".join(p))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else (tuple(eos) if isinstance(eos, (list, tuple)) else (eos,))
        cfg = cls(model_type="gugalorn", architectures=(name or "Gugalorn",), vocab=vocab, width=width, eps=eps,
                  embedding_scale=scale, canon_taps=taps, layers=tuple(layers), eos_token_id=eos)
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
            m, where = layer.mixer, f"layers[{i}].mixer"
            if layer.type == "mamba2":
                if m.heads % m.groups:
                    p.append(f"{where}: {m.heads} heads do not divide into {m.groups} groups")
                if (m.heads * m.vdim) % m.norm_groups:
                    p.append(f"{where}: {m.heads * m.vdim} inner numbers do not divide into {m.norm_groups} norm groups")
                if m.state > 256:
                    p.append(f"{where}: a state of {m.state} rows a head is beyond what the recurrence kernel takes (256)")
            else:
                a, g = m.left, m.right
                if a.heads % a.kv_heads:
                    p.append(f"{where}.left: {a.heads} heads over {a.kv_heads} kv heads")
                if a.rot_dims % 2 or a.rot_dims > a.dim:
                    p.append(f"{where}.left.rot: dims {a.rot_dims} must be even and at most dim {a.dim}")
                if g.dim > 256:
                    p.append(f"{where}.right: dim {g.dim} is beyond what the recurrence kernel takes (256)")
        return p

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0] if self.architectures else "Gugalorn",
               **({"canon": {"taps": self.canon_taps}} if self.canon_taps else {}), "embedding": {"scale": self.embedding_scale}, "layers": [layer.to_dict() for layer in self.layers],
               "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
