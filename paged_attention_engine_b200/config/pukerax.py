"""Typed configuration of the Pukerax decoder, read from its own config.json keys.

    {"architecture": "Pukerax", "vocab": V, "width": W, "streams": S, "norm": {"eps": e},
     "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

`streams` absent: one residual stream with plain sums; S >= 1: S streams joined by
hyper-connections. A layer's mixer is a latent attention:

  heads, dim (unrotated query/key channels per head), rot_dim (rotated ones), vdim, kv_rank
  (the key/value latent), q_rank (the query latent; absent: queries are projected directly),
  scale, rot {base, dims} (dims <= rot_dim: the leading channels of the rotated part turn).

Its feed-forward (`mlp`) is null, or

  {"kind": "dense", "ff": F}
  {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k, "scale": s,
   "identity": I, "groups": {"count": g, "keep": m}}, "shared": {"ff": F'}}

with `identity` (experts that return their input), `groups` (only experts of the best groups
can be chosen) and `shared` (an expert that every token uses) each absent when the mechanism is.

Every size and constant that can differ between two models of the design is read here; nothing
has a default except where a key's absence means that the mechanism is absent.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .zugarax import _get, _positive


@dataclass(frozen=True)
class QueryLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int             # 0: queries are projected directly
    scale: float
    rot_base: float
    rot_dims: int

    def to_dict(self) -> dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
               "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.q_rank:
            out["q_rank"] = self.q_rank
        return out


@dataclass(frozen=True)
class Router:
    experts: int            # routed experts with weights
    top: int
    scale: float
    identity: int           # further experts that return their input
    group_count: int        # 0: every expert can be chosen
    group_keep: int

    @property
    def total(self) -> int:
        return self.experts + self.identity

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.identity:
            out["identity"] = self.identity
        if self.group_count:
            out["groups"] = {"count": self.group_count, "keep": self.group_keep}
        return out


@dataclass(frozen=True)
class FeedForward:
    kind: str               # "dense" or "moe"
    ff: int                 # dense: the hidden size; moe: an expert's
    router: Router | None
    shared_ff: int          # 0: no shared expert

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": self.router.to_dict()}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class PukeraxLayer:
    type: str
    mixer: QueryLatentAttention
    mlp: FeedForward | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


def _read_mixer(raw, m: str) -> QueryLatentAttention:
    size = lambda key: _positive(_get(raw, key, int, m), m + key)
    rot = raw.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: key '{m}rot' is missing")
    rot_dim = size("rot_dim")
    dims = _positive(_get(rot, "dims", int, m + "rot."), m + "rot.dims")
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {m}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
    q_rank = 0
    if raw.get("q_rank") is not None:
        q_rank = size("q_rank")
    return QueryLatentAttention(size("heads"), size("dim"), rot_dim, size("vdim"), size("kv_rank"), q_rank,
                                _get(raw, "scale", float, m), _positive(_get(rot, "base", float, m + "rot."), m + "rot.base"), dims)


def _read_mlp(raw, w: str) -> FeedForward:
    kind = _get(raw, "kind", str, w)
    if kind == "dense":
        return FeedForward("dense", _positive(_get(raw, "ff", int, w), w + "ff"), None, 0)
    if kind != "moe":
        raise ConfigError(f"config.json: {w}kind '{kind}' is not one of dense, moe")
    r = raw.get("router")
    if not isinstance(r, Mapping):
        raise ConfigError(f"config.json: key '{w}router' is missing")
    experts = _positive(_get(r, "experts", int, w + "router."), w + "router.experts")
    identity = int(r.get("identity") or 0)
    if identity < 0:
        raise ConfigError(f"config.json: {w}router.identity {identity} is negative")
    top = _positive(_get(r, "top", int, w + "router."), w + "router.top")
    count = keep = 0
    if r.get("groups") is not None:
        count = _positive(_get(r["groups"], "count", int, w + "router.groups."), w + "router.groups.count")
        keep = _positive(_get(r["groups"], "keep", int, w + "router.groups."), w + "router.groups.keep")
        if (experts + identity) % count or keep > count:
            raise ConfigError(f"config.json: {w}router.groups: {experts + identity} experts do not form {count} equal groups of which {keep} are kept")
    reachable = (experts + identity) // count * keep if count else experts + identity
    if top > reachable:
        raise ConfigError(f"config.json: {w}router.top {top} exceeds the {reachable} experts that can be chosen")
    shared = 0
    if raw.get("shared") is not None:
        shared = _positive(_get(raw["shared"], "ff", int, w + "shared."), w + "shared.ff")
    return FeedForward("moe", _positive(_get(raw.get("expert"), "ff", int, w + "expert."), w + "expert.ff"),
                       Router(experts, top, _get(r, "scale", float, w + "router."), identity, count, keep), shared)


@dataclass(frozen=True)
class PukeraxConfig:
    vocab: int
    width: int
    streams: int            # 0: a single stream with plain residual sums
    norm_eps: float
    layers: tuple[PukeraxLayer, ...]
    architecture: str = "Pukerax"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PukeraxConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' is missing or empty")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}type '{kind}' is not latent_attention")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: key '{where}mixer' is missing")
            mlp = _read_mlp(entry["mlp"], where + "mlp.") if entry.get("mlp") is not None else None
            layers.append(PukeraxLayer(kind, _read_mixer(entry["mixer"], where + "mixer."), mlp))
        streams = 0
        if raw.get("streams") is not None:
            streams = _positive(_get(raw, "streams", int, ""), "streams")
        return cls(
            vocab=_positive(_get(raw, "vocab", int, ""), "vocab"),
            width=_positive(_get(raw, "width", int, ""), "width"),
            streams=streams,
            norm_eps=_positive(_get(raw.get("norm"), "eps", float, "norm."), "norm.eps"),
            layers=tuple(layers),
            architecture=str(raw.get("architecture", "Pukerax")),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "PukeraxConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.streams:
            out["streams"] = self.streams
        return out
