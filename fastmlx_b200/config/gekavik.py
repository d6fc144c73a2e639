"""Typed configuration of the Gekavik design, read from config.json.

A Gekavik model is a list of layers, each with a norm in front of and behind its mixer and its
feed-forward (dynamic tanh) and a multiplier on what enters the residual stream.  A layer's mixer is
`attention` (grouped queries with biased projections, q and k normalised per head before an
interleaved rotation of the head's first dimensions, a sliding window that keeps a request's first
tokens, an element-wise output gate) or `latent_attention` (keys and values read out of one cached
latent per token, queries through a latent of their own, no positions, a plain sliding window, a gate
value per head); its feed-forward is a mixture of small experts with a grouped router and a shared
expert, or none.  A run of layers may loop: layers start .. stop-1 run `times` times in a row with the
same weights and a cache of their own per pass, and in front of every pass the stream is mixed with
the token embeddings again.  Every size and constant stands in config.json.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ModelConfig


def _int(d: Mapping, key: str, where: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"gekavik: {where}.{key} must be an integer >= {low}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"gekavik: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                   # 0: every earlier token is seen
    keep_first: int               # a request's first tokens that stay visible behind the window
    rot_dims: int                 # 0: no rotation
    rot_base: float

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "WindowedAttentionConfig":
        rot = d.get("rot") or {}
        mask = d.get("mask") or {}
        rot_dims = _int(rot, "dims", where + ".rot", 0) if rot else 0
        c = WindowedAttentionConfig(
            _int(d, "heads", where), _int(d, "kv_heads", where), _int(d, "dim", where), _int(d, "vdim", where),
            _float(d, "scale", where), _int(mask, "size", where + ".mask") if mask else 0,
            _int(mask, "keep_first", where + ".mask", 0) if mask.get("keep_first") is not None else 0,
            rot_dims, _float(rot, "base", where + ".rot") if rot_dims else 1.0)
        if c.heads % c.kv_heads:
            raise ConfigError(f"gekavik: {where}: {c.heads} heads are no multiple of {c.kv_heads} kv_heads")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"gekavik: {where}.rot.dims must be even and at most dim, got {c.rot_dims}")
        if c.rot_dims and c.rot_base <= 0:
            raise ConfigError(f"gekavik: {where}.rot.base must be positive, got {c.rot_base}")
        if c.dim > 256 or c.vdim > 256:
            raise ConfigError(f"gekavik: {where}: head sizes up to 256")
        return c


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int                   # 0: every earlier token is seen

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        mask = d.get("mask") or {}
        c = LatentAttentionConfig(_int(d, "heads", where), _int(d, "dim", where), _int(d, "vdim", where),
                                  _int(d, "q_rank", where), _int(d, "kv_rank", where), _float(d, "scale", where),
                                  _int(mask, "size", where + ".mask") if mask else 0)
        if c.kv_rank > 512:
            raise ConfigError(f"gekavik: {where}.kv_rank up to 512, got {c.kv_rank}")
        return c


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0            # 0: no shared expert
    shared_limit: float = 0.0
    kind: str = "moe"

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "ExpertsConfig":
        if d.get("kind", "moe") != "moe":
            raise ConfigError(f"gekavik: {where}.kind must be 'moe', got {d.get('kind')!r}")
        router, expert = d.get("router"), d.get("expert")
        if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
            raise ConfigError(f"gekavik: {where} needs `router` and `expert`")
        groups = router.get("groups") or {}
        shared = d.get("shared") or {}
        c = ExpertsConfig(_int(router, "experts", where + ".router"), _int(router, "top", where + ".router"),
                          _int(expert, "ff", where + ".expert"), _float(expert, "limit", where + ".expert"),
                          _int(groups, "count", where + ".router.groups") if groups else 1,
                          _int(groups, "keep", where + ".router.groups") if groups else 1,
                          _int(shared, "ff", where + ".shared") if shared else 0,
                          _float(shared, "limit", where + ".shared") if shared else 0.0)
        if c.top > c.experts or c.experts % c.groups or c.keep > c.groups:
            raise ConfigError(f"gekavik: {where}.router: top {c.top} of {c.experts} experts in {c.groups} groups, {c.keep} kept")
        if c.top > (c.experts // c.groups) * c.keep:
            raise ConfigError(f"gekavik: {where}.router: {c.keep} groups of {c.experts // c.groups} hold fewer than top={c.top}")
        return c


@dataclass(frozen=True)
class LayerConfig:
    type: str                     # "attention" | "latent_attention"
    mixer: WindowedAttentionConfig | LatentAttentionConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class GekavikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    layers: tuple[LayerConfig, ...] = ()
    loop: LoopConfig | None = None
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    raw: tuple = ()               # the config.json items as read, for to_dict

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> int:
        return -1

    def layer_passes(self) -> list[tuple[int, int | None]]:
        """(layer, pass number or None) in the order the layers run; a pass number stands at the first layer
        of each pass of the loop."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        order = [(i, None) for i in range(lp.start)]
        for p in range(lp.times):
            order += [(i, p if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, n)]

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "GekavikConfig":
        layers = c.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("gekavik: `layers` must be a list with at least one layer")
        out = []
        for i, spec in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(spec, Mapping) or not isinstance(spec.get("mixer"), Mapping):
                raise ConfigError(f"gekavik: {where} must be an object with a `mixer`")
            kind = spec.get("type")
            if kind == "attention":
                mixer = WindowedAttentionConfig.from_dict(spec["mixer"], where + ".mixer")
            elif kind == "latent_attention":
                mixer = LatentAttentionConfig.from_dict(spec["mixer"], where + ".mixer")
            else:
                raise ConfigError(f"gekavik: {where}.type must be 'attention' or 'latent_attention', got {kind!r}")
            mlp = spec.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"gekavik: {where}.mlp must be an object or null")
                mlp = ExpertsConfig.from_dict(mlp, where + ".mlp")
            out.append(LayerConfig(kind, mixer, mlp))
        loop = c.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("gekavik: `loop` must be an object")
            loop = LoopConfig(_int(loop, "start", "loop", 0), _int(loop, "stop", "loop", 0), _int(loop, "times", "loop", 1))
            if not 0 <= loop.start < loop.stop <= len(out):
                raise ConfigError(f"gekavik: loop {loop.start}..{loop.stop} lies outside the {len(out)} layers")
        norm = c.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("gekavik: `norm` must be an object with `eps`")
        eps = _float(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"gekavik: norm.eps must not be negative, got {eps}")
        mult = _float(c, "residual_mult", "config") if c.get("residual_mult") is not None else 1.0
        return GekavikConfig(vocab=_int(c, "vocab", "config"), width=_int(c, "width", "config"), layers=tuple(out),
                             loop=loop, norm_eps=eps, residual_mult=mult,
                             raw=tuple(sorted(c.items(), key=lambda kv: kv[0])))

    def to_dict(self) -> dict:
        return dict(self.raw)
