"""Typed configuration of the Medirax design, read from config.json.

A Medirax model is a list of parallel layers (one norm; a mixer and an optional dense
feed-forward read its output), each with a mixer of its own kind and sizes: `delta` (the
gated delta rule with short convolutions) or `attention` (grouped queries, partial rotary
positions, q and k normalised after the rotation, capped scores, a sliding window).  A
run of layers may loop: layers start .. stop-1 run `times` times in a row with the same
weights and a cache of their own for every pass.  Every size and constant stands in
config.json; nothing is defaulted from another layer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ModelConfig


def _int(d: Mapping, key: str, where: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"medirax: {where}.{key} must be an integer >= {low}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"medirax: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                     # taps of the short convolutions

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "DeltaMixerConfig":
        c = DeltaMixerConfig(_int(d, "heads", where), _int(d, "kv_heads", where), _int(d, "dim", where),
                             _int(d, "vdim", where), _int(d, "conv", where))
        if c.heads % c.kv_heads:
            raise ConfigError(f"medirax: {where}: {c.heads} heads are no multiple of {c.kv_heads} kv_heads")
        if c.conv > 16 or c.dim > 256:
            raise ConfigError(f"medirax: {where}: at most 16 taps and a dim of 256, got conv={c.conv}, dim={c.dim}")
        return c


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                # 0: scores are not capped
    window: int                   # 0: every earlier token is seen
    rot_dims: int                 # 0: no rotation
    rot_base: float

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "AttentionMixerConfig":
        rot = d.get("rot") or {}
        mask = d.get("mask") or {}
        rot_dims = _int(rot, "dims", where + ".rot", 0) if rot else 0
        c = AttentionMixerConfig(
            _int(d, "heads", where), _int(d, "kv_heads", where), _int(d, "dim", where), _int(d, "vdim", where),
            _float(d, "scale", where), _float(d, "softcap", where) if d.get("softcap") is not None else 0.0,
            _int(mask, "size", where + ".mask") if mask else 0, rot_dims,
            _float(rot, "base", where + ".rot") if rot_dims else 1.0)
        if c.heads % c.kv_heads:
            raise ConfigError(f"medirax: {where}: {c.heads} heads are no multiple of {c.kv_heads} kv_heads")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"medirax: {where}.rot.dims must be even and at most dim, got {c.rot_dims}")
        if c.rot_dims and c.rot_base <= 0:
            raise ConfigError(f"medirax: {where}.rot.base must be positive, got {c.rot_base}")
        if c.softcap < 0 or c.dim > 256 or c.vdim > 256:
            raise ConfigError(f"medirax: {where}: softcap >= 0 and head sizes up to 256")
        return c


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class LayerConfig:
    type: str                     # "delta" | "attention"
    mixer: DeltaMixerConfig | AttentionMixerConfig
    mlp: DenseMlpConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MediraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    layers: tuple[LayerConfig, ...] = ()
    loop: LoopConfig | None = None
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    raw: tuple = ()               # the config.json items as read, for to_dict

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> int:
        return -1

    def layer_order(self) -> list[int]:
        """Indices of the layers in the order they run, a looped run repeated."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        lp = self.loop
        return list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "MediraxConfig":
        layers = c.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("medirax: `layers` must be a list with at least one layer")
        out = []
        for i, spec in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(spec, Mapping) or not isinstance(spec.get("mixer"), Mapping):
                raise ConfigError(f"medirax: {where} must be an object with a `mixer`")
            kind = spec.get("type")
            if kind == "delta":
                mixer = DeltaMixerConfig.from_dict(spec["mixer"], where + ".mixer")
            elif kind == "attention":
                mixer = AttentionMixerConfig.from_dict(spec["mixer"], where + ".mixer")
            else:
                raise ConfigError(f"medirax: {where}.type must be 'delta' or 'attention', got {kind!r}")
            mlp = spec.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"medirax: {where}.mlp.kind must be 'dense', got {mlp!r}")
                mlp = DenseMlpConfig(_int(mlp, "ff", where + ".mlp"))
            out.append(LayerConfig(kind, mixer, mlp))
        loop = c.get("loop")
        if loop is not None:
            loop = LoopConfig(_int(loop, "start", "loop", 0), _int(loop, "stop", "loop", 0), _int(loop, "times", "loop", 1))
            if not 0 <= loop.start <= loop.stop <= len(out):
                raise ConfigError(f"medirax: loop {loop.start}..{loop.stop} lies outside the {len(out)} layers")
        norm = c.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("medirax: `norm` must be an object with `eps`")
        eps = _float(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"medirax: norm.eps must not be negative, got {eps}")
        scale = _float(c, "logit_scale", "config") if c.get("logit_scale") is not None else 1.0
        return MediraxConfig(vocab=_int(c, "vocab", "config"), width=_int(c, "width", "config"), layers=tuple(out),
                             loop=loop, norm_eps=eps, logit_scale=scale, raw=tuple(sorted(c.items(), key=lambda kv: kv[0])))

    def to_dict(self) -> dict:
        return dict(self.raw)
