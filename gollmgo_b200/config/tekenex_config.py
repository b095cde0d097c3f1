"""Typed configuration of the Tekenex decoder, read from its config.json.

The file names the design in ``architecture`` and lists the layers one by one: each entry has
``type`` (its mixer), the mixer's sizes and constants in ``mixer``, and its feed-forward in
``mlp`` (``kind`` "dense" or "moe", or null for a layer without one).  ``norm.eps`` is the one
epsilon of every norm; ``vocab`` and ``width`` are the table's sizes.  Every size and constant
is taken from the file; a key this engine does not know inside a layer is reported on standard
error and ignored.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError


def _int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _only(d: dict, known, where: str) -> None:
    extra = sorted(set(d) - set(known))
    if extra:
        print(f"[gollmgo_b200] config.json: {where} has keys this engine does not know and ignores: {extra}",
              file=sys.stderr, flush=True)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int               # of a head's query and key
    vdim: int              # of a head's value
    kv_rank: int           # of the latent that keys and values are expanded from
    scale: float           # of the scores


@dataclass(frozen=True)
class GatedExpertConfig:
    ff: int


@dataclass(frozen=True)
class TekenexMlpConfig:
    kind: str                                  # "dense" | "moe"
    ff: int = 0                                # dense: width of the hidden layer
    experts: int = 0
    top: int = 0
    expert: Optional[GatedExpertConfig] = None
    shared: Optional[GatedExpertConfig] = None


@dataclass(frozen=True)
class TekenexLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[TekenexMlpConfig]


@dataclass(frozen=True)
class TekenexConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[TekenexLayerConfig, ...]
    max_position_embeddings: int
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None

    @staticmethod
    def from_dict(d: dict) -> "TekenexConfig":
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' (with 'eps') is missing")
        eps = _num(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            _only(e, ("type", "mixer", "mlp"), where)
            kind = e.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known (known: latent_attention)")
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            _only(m, ("heads", "dim", "vdim", "kv_rank", "scale"), where + ".mixer")
            mixer = LatentMixerConfig(_int(m, "heads", where + ".mixer"), _int(m, "dim", where + ".mixer"),
                                      _int(m, "vdim", where + ".mixer"), _int(m, "kv_rank", where + ".mixer"),
                                      _num(m, "scale", where + ".mixer"))
            layers.append(TekenexLayerConfig(kind, mixer, _mlp(e.get("mlp"), where + ".mlp")))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return TekenexConfig(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), eps=eps,
                             layers=tuple(layers),
                             max_position_embeddings=int(d.get("max_position_embeddings", 1 << 17)),
                             eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))


def _mlp(f, where: str) -> Optional[TekenexMlpConfig]:
    if f is None:
        return None
    if not isinstance(f, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    kind = f.get("kind")
    if kind == "dense":
        _only(f, ("kind", "ff"), where)
        return TekenexMlpConfig("dense", ff=_int(f, "ff", where))
    if kind == "moe":
        _only(f, ("kind", "router", "expert", "shared"), where)
        r, ex, sh = f.get("router"), f.get("expert"), f.get("shared")
        if not isinstance(r, dict) or not isinstance(ex, dict):
            raise ConfigError(f"config.json: {where} needs 'router' and 'expert'")
        _only(r, ("experts", "top"), where + ".router")
        _only(ex, ("ff",), where + ".expert")
        experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router picks {top} of {experts} experts")
        shared = None
        if sh is not None:
            if not isinstance(sh, dict):
                raise ConfigError(f"config.json: {where}.shared must be an object or null")
            _only(sh, ("ff",), where + ".shared")
            shared = GatedExpertConfig(_int(sh, "ff", where + ".shared"))
        return TekenexMlpConfig("moe", experts=experts, top=top,
                                expert=GatedExpertConfig(_int(ex, "ff", where + ".expert")), shared=shared)
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not known (known: dense, moe)")
