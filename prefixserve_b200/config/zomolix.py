"""Typed Zomolix configuration, read from the keys of a model folder's config.json.

Zomolix is a decoder whose layers are listed one by one: each entry of ``layers`` names its mixer (``attention``:
grouped-query attention with biases, a partial split-half rotation and a sliding window that keeps a sequence's first
keys; ``latent_attention``: attention through a shared low-rank latent with a sink in the softmax and a gate on its
output), the mixer's sizes, and its feed-forward (routed experts with a shared one, or none).  An attention layer may
read another attention layer's keys and values instead of projecting its own.  Keys:

    architecture: "Zomolix"
    vocab, width, norm.eps, embedding.scale
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp = {...} | null
      attention:        heads, kv_heads, dim, vdim, scale, rot.{base, dims, scaling}, mask.{size, keep_first} (absent:
                        every earlier key is seen), kv_from (absent: projections of its own)
      latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot.{base, dims, scaling}
      rot.scaling:      {factor, original, fast, slow} (absent: plain frequencies)
      mlp:              kind "moe", expert.{ff, limit}, router.{experts, top, groups.{count, keep}},
                        shared.{ff, limit} (absent: no shared expert)

Every size and constant the engine uses for such a model comes from here; what the design fixes (the constants of the
experts' activation) is in ``architectures/zomolix``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .llama import UnsupportedModelError
from .nerenex import _need, _positive

ARCHITECTURE = "Zomolix"


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int                      # how many leading elements of a head (or of the rotated part) turn
    factor: float | None = None    # frequency scaling by wavelength with a ramp between two pair indices; None: none
    original: int = 0
    fast: float = 1.0
    slow: float = 1.0

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "RotationConfig":
        cfg = RotationConfig(base=float(_need(m, "base", where)), dims=_positive(_need(m, "dims", where), f"{where}.dims"))
        if cfg.dims % 2:
            raise UnsupportedModelError(f"config.json: {where}.dims {cfg.dims} must be even")
        if not cfg.base > 1:
            raise UnsupportedModelError(f"config.json: {where}.base must exceed 1, is {cfg.base}")
        sc = m.get("scaling")
        if sc is not None:
            w = f"{where}.scaling"
            cfg = RotationConfig(cfg.base, cfg.dims, factor=float(_need(sc, "factor", w)),
                                 original=_positive(_need(sc, "original", w), f"{w}.original"),
                                 fast=float(_need(sc, "fast", w)), slow=float(_need(sc, "slow", w)))
            if not (cfg.factor > 0 and cfg.fast > 0 and cfg.slow > 0):
                raise UnsupportedModelError(f"config.json: {w}: factor, fast and slow must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return out


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int        # query/key size per head
    vdim: int       # value size per head
    scale: float
    rot: RotationConfig | None = None
    window: int | None = None   # mask.size: position i sees j when i - j < window ...
    keep_first: int = 0         # ... or j < keep_first
    kv_from: int | None = None  # the layer whose keys and values this one reads; None: its own

    kind = "attention"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "AttentionConfig":
        rot, mask = m.get("rot"), m.get("mask")
        dim = _positive(_need(m, "dim", where), f"{where}.dim")
        cfg = AttentionConfig(
            heads=_positive(_need(m, "heads", where), f"{where}.heads"),
            kv_heads=_positive(_need(m, "kv_heads", where), f"{where}.kv_heads"),
            dim=dim,
            vdim=_positive(m.get("vdim", dim), f"{where}.vdim"),
            scale=float(_need(m, "scale", where)),
            rot=None if rot is None else RotationConfig.from_dict(rot, f"{where}.rot"),
            window=None if mask is None or mask.get("size") is None else _positive(mask["size"], f"{where}.mask.size"),
            keep_first=0 if mask is None else int(mask.get("keep_first") or 0),
            kv_from=None if m.get("kv_from") is None else int(m["kv_from"]),
        )
        if cfg.heads % cfg.kv_heads:
            raise UnsupportedModelError(f"config.json: {where}: {cfg.heads} heads cannot share {cfg.kv_heads} key/value heads")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise UnsupportedModelError(f"config.json: {where}.rot.dims {cfg.rot.dims} exceeds the head size {cfg.dim}")
        if cfg.keep_first < 0:
            raise UnsupportedModelError(f"config.json: {where}.mask.keep_first must not be negative")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.window is not None:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int        # unrotated query/key size per head
    rot_dim: int    # rotated query/key size per head (the key's is shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig | None = None

    kind = "latent_attention"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        rot = m.get("rot")
        cfg = LatentAttentionConfig(
            heads=_positive(_need(m, "heads", where), f"{where}.heads"),
            dim=_positive(_need(m, "dim", where), f"{where}.dim"),
            rot_dim=_positive(_need(m, "rot_dim", where), f"{where}.rot_dim"),
            vdim=_positive(_need(m, "vdim", where), f"{where}.vdim"),
            kv_rank=_positive(_need(m, "kv_rank", where), f"{where}.kv_rank"),
            scale=float(_need(m, "scale", where)),
            rot=None if rot is None else RotationConfig.from_dict(rot, f"{where}.rot"),
        )
        if cfg.rot is not None and cfg.rot.dims > cfg.rot_dim:
            raise UnsupportedModelError(f"config.json: {where}.rot.dims {cfg.rot.dims} exceeds the rotated part of {cfg.rot_dim}")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "kv_rank": self.kv_rank, "scale": self.scale}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    ff: int
    limit: float
    groups: int = 1
    keep: int = 1
    shared_ff: int | None = None
    shared_limit: float | None = None

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "RoutedFF":
        if m.get("kind") != "moe":
            raise UnsupportedModelError(f"config.json: {where}.kind {m.get('kind')!r} is not built (moe)")
        expert, router, shared = _need(m, "expert", where), _need(m, "router", where), m.get("shared")
        groups = router.get("groups") or {}
        count = _positive(groups.get("count", 1), f"{where}.router.groups.count")
        cfg = RoutedFF(
            experts=_positive(_need(router, "experts", f"{where}.router"), f"{where}.router.experts"),
            top=_positive(_need(router, "top", f"{where}.router"), f"{where}.router.top"),
            ff=_positive(_need(expert, "ff", f"{where}.expert"), f"{where}.expert.ff"),
            limit=float(_need(expert, "limit", f"{where}.expert")),
            groups=count,
            keep=_positive(groups.get("keep", count), f"{where}.router.groups.keep"),
            shared_ff=None if shared is None else _positive(_need(shared, "ff", f"{where}.shared"), f"{where}.shared.ff"),
            shared_limit=None if shared is None else float(_need(shared, "limit", f"{where}.shared")),
        )
        if cfg.experts % cfg.groups or cfg.keep > cfg.groups:
            raise UnsupportedModelError(f"config.json: {where}.router: {cfg.experts} experts cannot form {cfg.groups} equal groups of which {cfg.keep} are kept")
        if cfg.top > cfg.keep * (cfg.experts // cfg.groups):
            raise UnsupportedModelError(f"config.json: {where}.router: {cfg.keep} groups of {cfg.experts // cfg.groups} experts cannot give {cfg.top} choices")
        if not cfg.limit > 0 or (cfg.shared_limit is not None and not cfg.shared_limit > 0):
            raise UnsupportedModelError(f"config.json: {where}: the limits must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                               "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


_MIXERS = {"attention": AttentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class ZomolixLayer:
    mixer: AttentionConfig | LatentAttentionConfig
    mlp: RoutedFF | None


@dataclass(frozen=True)
class ZomolixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[ZomolixLayer, ...]
    stop_token_ids: frozenset[int] = frozenset()

    architecture = ARCHITECTURE

    @staticmethod
    def from_dicts(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "ZomolixConfig":
        if raw.get("architecture") != ARCHITECTURE and ARCHITECTURE not in (raw.get("architectures") or []):
            raise UnsupportedModelError(f"config.json does not describe a {ARCHITECTURE} model")
        layers: list[ZomolixLayer] = []
        for i, entry in enumerate(_need(raw, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mixer = _MIXERS[kind].from_dict(_need(entry, "mixer", where), f"{where}.mixer")
            mlp = entry.get("mlp")
            layers.append(ZomolixLayer(mixer, None if mlp is None else RoutedFF.from_dict(mlp, f"{where}.mlp")))
        if not layers:
            raise UnsupportedModelError("config.json: a model needs at least one layer")
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, AttentionConfig) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if 0 <= m.kv_from < i else None
                if not isinstance(src, AttentionConfig) or src.kv_from is not None:
                    raise UnsupportedModelError(f"config.json: layers[{i}].mixer.kv_from must name an earlier attention layer with projections of its own")
                if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise UnsupportedModelError(f"config.json: layers[{i}] reads the keys and values of layer {m.kv_from}, whose sizes differ")
        stops: set[int] = set()
        eos = (generation or {}).get("eos_token_id")
        if eos is not None:
            stops.update(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return ZomolixConfig(
            vocab=_positive(_need(raw, "vocab", "the top level"), "vocab"),
            width=_positive(_need(raw, "width", "the top level"), "width"),
            norm_eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            layers=tuple(layers),
            stop_token_ids=frozenset(stops),
        )

    def to_config_json(self) -> dict[str, Any]:
        return {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab,
            "width": self.width,
            "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": layer.mixer.kind, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
        }
