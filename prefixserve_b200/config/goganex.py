"""Typed Goganex configuration, read from the keys of a model folder's config.json.

Goganex is a decoder whose layers are listed one by one: each entry of ``layers`` names its mixer (``attention``:
rotated, unit-normed queries and keys with a factor per head and a sink in the softmax; ``parallel``: an attention
whose keys are its values beside a minGRU recurrence), the mixer's sizes, and its feed-forward (or none).  A run of
the layers may be repeated with the same weights (``loop``).  Keys:

    architecture: "Goganex"
    vocab, width, norm.eps, embedding.scale
    loop.{start, stop, times}                     (absent: every layer once)
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp = {kind: "dense", ff, limit} | null
      attention: heads, kv_heads, dim, vdim, scale, rot.{base, dims, scaling.{factor, low, high, original}}
                 (rot absent: no rotation; scaling absent: plain frequencies)
      parallel:  left.{heads, kv_heads, dim, vdim, scale}, right.{width}

Every size and constant the engine uses for such a model comes from here; what the design fixes (the constants of the
feed-forward's activation, the sink's score, the weight of a parallel mixer's branches) is in ``architectures/goganex``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .llama import UnsupportedModelError
from .nerenex import _need, _positive

ARCHITECTURE = "Goganex"


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int                      # how many leading elements of a head turn (pairs 2i, 2i+1)
    factor: float | None = None    # frequency scaling by wavelength; None: none
    low: float = 1.0
    high: float = 1.0
    original: int = 0

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "RotationConfig":
        sc = m.get("scaling")
        cfg = RotationConfig(base=float(_need(m, "base", where)), dims=_positive(_need(m, "dims", where), f"{where}.dims"))
        if cfg.dims % 2:
            raise UnsupportedModelError(f"config.json: {where}.dims {cfg.dims} must be even")
        if sc is not None:
            w = f"{where}.scaling"
            cfg = RotationConfig(cfg.base, cfg.dims, factor=float(_need(sc, "factor", w)), low=float(_need(sc, "low", w)),
                                 high=float(_need(sc, "high", w)), original=_positive(_need(sc, "original", w), f"{w}.original"))
            if cfg.high == cfg.low:
                raise UnsupportedModelError(f"config.json: {w}: low and high must differ")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            out["scaling"] = {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}
        return out


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int        # query/key size per head
    vdim: int       # value size per head
    scale: float
    rot: RotationConfig | None = None

    kind = "attention"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "AttentionConfig":
        rot = m.get("rot")
        dim = _positive(_need(m, "dim", where), f"{where}.dim")
        cfg = AttentionConfig(
            heads=_positive(_need(m, "heads", where), f"{where}.heads"),
            kv_heads=_positive(_need(m, "kv_heads", where), f"{where}.kv_heads"),
            dim=dim,
            vdim=_positive(m.get("vdim", dim), f"{where}.vdim"),
            scale=float(_need(m, "scale", where)),
            rot=None if rot is None else RotationConfig.from_dict(rot, f"{where}.rot"),
        )
        if cfg.heads % cfg.kv_heads:
            raise UnsupportedModelError(f"config.json: {where}: {cfg.heads} heads cannot share {cfg.kv_heads} key/value heads")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise UnsupportedModelError(f"config.json: {where}.rot.dims {cfg.rot.dims} exceeds the head size {cfg.dim}")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class ParallelConfig:
    left: AttentionConfig   # its projected keys are its values (vdim == dim), no rotation
    right_width: int        # channels of the recurrence

    kind = "parallel"

    @staticmethod
    def from_dict(m: Mapping[str, Any], where: str) -> "ParallelConfig":
        left = AttentionConfig.from_dict(_need(m, "left", where), f"{where}.left")
        if left.vdim != left.dim:
            raise UnsupportedModelError(f"config.json: {where}.left: the keys are the values, so vdim {left.vdim} must equal dim {left.dim}")
        right = _need(m, "right", where)
        return ParallelConfig(left=left, right_width=_positive(_need(right, "width", f"{where}.right"), f"{where}.right.width"))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": {"width": self.right_width}}


@dataclass(frozen=True)
class ClippedFF:
    ff: int
    limit: float

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


_MIXERS = {"attention": AttentionConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class GoganexLayer:
    mixer: AttentionConfig | ParallelConfig
    mlp: ClippedFF | None


@dataclass(frozen=True)
class GoganexConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[GoganexLayer, ...]
    loop_start: int = 0     # layers loop_start .. loop_stop - 1 run loop_times times in a row
    loop_stop: int = 0
    loop_times: int = 1
    stop_token_ids: frozenset[int] = frozenset()

    architecture = ARCHITECTURE

    def run_order(self) -> tuple[int, ...]:
        """The layers in the order they run, a repeated run written out."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return tuple(range(n))
        inside = tuple(range(self.loop_start, self.loop_stop))
        return tuple(range(self.loop_start)) + inside * self.loop_times + tuple(range(self.loop_stop, n))

    @staticmethod
    def from_dicts(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "GoganexConfig":
        if raw.get("architecture") != ARCHITECTURE and ARCHITECTURE not in (raw.get("architectures") or []):
            raise UnsupportedModelError(f"config.json does not describe a {ARCHITECTURE} model")
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mixer = _MIXERS[kind].from_dict(_need(entry, "mixer", where), f"{where}.mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise UnsupportedModelError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not built (dense)")
                ff = ClippedFF(ff=_positive(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff"), limit=float(_need(mlp, "limit", f"{where}.mlp")))
                if not ff.limit > 0:
                    raise UnsupportedModelError(f"config.json: {where}.mlp.limit must be positive, is {ff.limit}")
            layers.append(GoganexLayer(mixer, ff))
        if not layers:
            raise UnsupportedModelError("config.json: a model needs at least one layer")
        loop = raw.get("loop")
        start = stop = 0
        times = 1
        if loop is not None:
            start, stop, times = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop"))
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise UnsupportedModelError(f"config.json: loop {start}..{stop} x {times} does not fit {len(layers)} layers")
        stops: set[int] = set()
        eos = (generation or {}).get("eos_token_id")
        if eos is not None:
            stops.update(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return GoganexConfig(
            vocab=_positive(_need(raw, "vocab", "the top level"), "vocab"),
            width=_positive(_need(raw, "width", "the top level"), "width"),
            norm_eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            layers=tuple(layers),
            loop_start=start, loop_stop=stop, loop_times=times,
            stop_token_ids=frozenset(stops),
        )

    def to_config_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab,
            "width": self.width,
            "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": layer.mixer.kind, "mixer": layer.mixer.to_dict(),
                        "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers],
        }
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
