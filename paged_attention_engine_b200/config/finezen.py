"""Typed configuration of the Finezen decoder, read from its own config.json keys.

    {"architecture": "Finezen", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "residual_mult": m, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": ..., "mixer": {...}, "mlp": {...} | null}, ...]}

`loop` (absent: every layer runs once): layers a .. b - 1 run n times in a row with the same
weights and a cache of their own per pass. A layer's mixer is one of two kinds:

  attention         heads, kv_heads, dim (query/key head size), vdim, scale, mask {size} (absent:
                    every earlier key), rot {base, dims, scaling {factor, original, fast, slow}}
                    (`scaling` absent: plain frequencies; `rot` absent: no rotation).
  latent_attention  heads, dim, vdim, kv_rank (the key/value latent), q_rank (the query latent),
                    scale, mask {size} (absent: every earlier key). No positions.

Its feed-forward (`mlp`) is null, or a mixture of gated experts:

  {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}, "shared": {"ff": F'}}

with `shared` (an expert that every token uses, behind a gate of its own) absent when there is none.

Every size and constant that can differ between two models of the design is read here; nothing
has a default except where a key's absence means that the mechanism is absent.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .zugarax import Rotation, WindowAttention, _get, _positive

LAYER_TYPES = ("attention", "latent_attention")
YARN_KEYS = ("factor", "original", "fast", "slow")


def _window(raw, where: str) -> int:
    if raw.get("mask") is None:
        return 0
    return _positive(_get(raw["mask"], "size", int, where + "mask."), where + "mask.size")


@dataclass(frozen=True)
class WindowLatentAttention:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int             # 0: every earlier key

    def to_dict(self) -> dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
               "scale": self.scale}
        if self.window:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class GatedExperts:
    ff: int                 # an expert's hidden size
    experts: int
    top: int
    shared_ff: int          # 0: no shared expert

    def to_dict(self) -> dict[str, Any]:
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class FinezenLayer:
    type: str
    mixer: Any
    mlp: GatedExperts | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _read_mixer(kind: str, raw, m: str):
    size = lambda key: _positive(_get(raw, key, int, m), m + key)
    if kind == "attention":
        heads, kv_heads = size("heads"), size("kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {m}heads {heads} is not a multiple of kv_heads {kv_heads}")
        dim = size("dim")
        rot = Rotation.read(raw["rot"], m + "rot.", YARN_KEYS) if raw.get("rot") is not None else None
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"config.json: {m}rot.dims {rot.dims} exceeds dim {dim}")
        return WindowAttention(heads, kv_heads, dim, size("vdim"), _get(raw, "scale", float, m), _window(raw, m), rot)
    return WindowLatentAttention(size("heads"), size("dim"), size("vdim"), size("kv_rank"), size("q_rank"),
                                 _get(raw, "scale", float, m), _window(raw, m))


def _read_mlp(raw, w: str) -> GatedExperts:
    kind = _get(raw, "kind", str, w)
    if kind != "moe":
        raise ConfigError(f"config.json: {w}kind '{kind}' is not moe")
    r = raw.get("router")
    if not isinstance(r, Mapping):
        raise ConfigError(f"config.json: key '{w}router' is missing")
    experts = _positive(_get(r, "experts", int, w + "router."), w + "router.experts")
    top = _positive(_get(r, "top", int, w + "router."), w + "router.top")
    if top > experts:
        raise ConfigError(f"config.json: {w}router.top {top} exceeds the {experts} experts")
    shared = 0
    if raw.get("shared") is not None:
        shared = _positive(_get(raw["shared"], "ff", int, w + "shared."), w + "shared.ff")
    return GatedExperts(_positive(_get(raw.get("expert"), "ff", int, w + "expert."), w + "expert.ff"), experts, top, shared)


@dataclass(frozen=True)
class FinezenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    loop: Loop | None
    layers: tuple[FinezenLayer, ...]
    architecture: str = "Finezen"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FinezenConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' is missing or empty")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of {', '.join(LAYER_TYPES)}")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: key '{where}mixer' is missing")
            mlp = _read_mlp(entry["mlp"], where + "mlp.") if entry.get("mlp") is not None else None
            layers.append(FinezenLayer(kind, _read_mixer(kind, entry["mixer"], where + "mixer."), mlp))
        loop = None
        if raw.get("loop") is not None:
            l = raw["loop"]
            loop = Loop(_get(l, "start", int, "loop."), _get(l, "stop", int, "loop."), _positive(_get(l, "times", int, "loop."), "loop.times"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not lie within the {len(layers)} layers")
        return cls(
            vocab=_positive(_get(raw, "vocab", int, ""), "vocab"),
            width=_positive(_get(raw, "width", int, ""), "width"),
            embedding_scale=_get(raw.get("embedding"), "scale", float, "embedding."),
            norm_eps=_positive(_get(raw.get("norm"), "eps", float, "norm."), "norm.eps"),
            residual_mult=_get(raw, "residual_mult", float, ""),
            loop=loop,
            layers=tuple(layers),
            architecture=str(raw.get("architecture", "Finezen")),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "FinezenConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        return out

    def runs(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding's output is added before it) in running order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        out = [(i, False) for i in range(self.loop.start)]
        for p in range(self.loop.times):
            out += [(i, p > 0 and i == self.loop.start) for i in range(self.loop.start, self.loop.stop)]
        return out + [(i, False) for i in range(self.loop.stop, n)]
