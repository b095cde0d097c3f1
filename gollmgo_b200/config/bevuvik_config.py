"""Typed configuration of the Bevuvik decoder, read from its config.json.

The file names the design in ``architecture`` and lists the layers one by one: each entry has
``type`` (its mixer: "attention" = differential attention, "parallel" = a softmax attention and
a gated delta rule side by side), the mixer's sizes and constants in ``mixer`` and its
feed-forward in ``mlp`` (or null).  ``loop`` (optional) says which layers run several times in a
row; ``residual_mult`` scales what a layer adds to the stream; ``norm.eps`` is the one epsilon.
Every size and constant is taken from the file; a key that is absent switches its feature off
(no ``rot``: no rotation; no ``mask``: every earlier key is seen; no ``softcap``: scores are
not capped; no ``loop``: every layer runs once).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError
from .tekenex_config import _int, _num, _only


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    # stretching for long contexts, or None: (factor, original, fast, slow)
    scaling: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: Optional[int]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class SoftmaxBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    rot: Optional[RotaryConfig]


@dataclass(frozen=True)
class DeltaBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SoftmaxBranchConfig
    right: DeltaBranchConfig


@dataclass(frozen=True)
class BevuvikMlpConfig:
    kind: str
    ff: int
    limit: float


@dataclass(frozen=True)
class BevuvikLayerConfig:
    type: str
    mixer: object                                # DiffAttentionConfig | ParallelMixerConfig
    mlp: Optional[BevuvikMlpConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BevuvikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[BevuvikLayerConfig, ...]
    loop: Optional[LoopConfig]
    max_position_embeddings: int
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None

    @staticmethod
    def from_dict(d: dict) -> "BevuvikConfig":
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
            kind, m = e.get("type"), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            if kind == "attention":
                mixer = _diff_attention(m, where + ".mixer")
            elif kind == "parallel":
                _only(m, ("left", "right"), where + ".mixer")
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                mixer = ParallelMixerConfig(_softmax_branch(m["left"], where + ".mixer.left"),
                                            _delta_branch(m["right"], where + ".mixer.right"))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known (known: attention, parallel)")
            layers.append(BevuvikLayerConfig(kind, mixer, _mlp(e.get("mlp"), where + ".mlp")))
        loop = None
        lp = d.get("loop")
        if lp is not None:
            if not isinstance(lp, dict):
                raise ConfigError("config.json: 'loop' must be an object or null")
            _only(lp, ("start", "stop", "times"), "loop")
            start = lp.get("start")
            if isinstance(start, bool) or not isinstance(start, int) or start < 0:
                raise ConfigError(f"config.json: loop.start must be an integer >= 0, got {start!r}")
            loop = LoopConfig(start, _int(lp, "stop", "loop"), _int(lp, "times", "loop"))
            if not (loop.start < loop.stop <= len(layers)):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not lie inside the {len(layers)} layers")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        mult = d.get("residual_mult", 1.0)
        if isinstance(mult, bool) or not isinstance(mult, (int, float)):
            raise ConfigError(f"config.json: residual_mult must be a number, got {mult!r}")
        return BevuvikConfig(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), eps=eps,
                             residual_mult=float(mult), layers=tuple(layers), loop=loop,
                             max_position_embeddings=int(d.get("max_position_embeddings", 1 << 17)),
                             eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))


def _heads(m: dict, where: str):
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    return heads, kv, _int(m, "dim", where), _int(m, "vdim", where)


def _rot(r, where: str) -> Optional[RotaryConfig]:
    if r is None:
        return None
    if not isinstance(r, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    _only(r, ("dims", "base", "scaling"), where)
    dims = _int(r, "dims", where)
    if dims % 2:
        raise ConfigError(f"config.json: {where}.dims must be even, got {dims}")
    scaling = None
    sc = r.get("scaling")
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}.scaling must be an object or null")
        _only(sc, ("factor", "original", "fast", "slow"), where + ".scaling")
        scaling = tuple(_num(sc, k, where + ".scaling") for k in ("factor", "original", "fast", "slow"))
    return RotaryConfig(dims, _num(r, "base", where), scaling)


def _window(m: dict, where: str) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object or null")
    _only(mask, ("size",), where + ".mask")
    return _int(mask, "size", where + ".mask")


def _diff_attention(m: dict, where: str) -> DiffAttentionConfig:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask", "rot"), where)
    heads, kv, dim, vdim = _heads(m, where)
    rot = _rot(m.get("rot"), where + ".rot")
    if rot is not None and rot.dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {rot.dims} is more than dim {dim}")
    return DiffAttentionConfig(heads, kv, dim, vdim, _num(m, "scale", where), _num(m, "diff", where),
                               _window(m, where), rot)


def _softmax_branch(m: dict, where: str) -> SoftmaxBranchConfig:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask", "rot"), where)
    heads, kv, dim, vdim = _heads(m, where)
    rot = _rot(m.get("rot"), where + ".rot")
    if rot is not None and rot.dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {rot.dims} is more than dim {dim}")
    cap = m.get("softcap")
    return SoftmaxBranchConfig(heads, kv, dim, vdim, _num(m, "scale", where),
                               None if cap is None else _num(m, "softcap", where), _window(m, where), rot)


def _delta_branch(m: dict, where: str) -> DeltaBranchConfig:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
    heads, kv, dim, vdim = _heads(m, where)
    return DeltaBranchConfig(heads, kv, dim, vdim, _int(m, "conv", where))


def _mlp(f, where: str) -> Optional[BevuvikMlpConfig]:
    if f is None:
        return None
    if not isinstance(f, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    if f.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}.kind {f.get('kind')!r} is not known (known: dense)")
    _only(f, ("kind", "ff", "limit"), where)
    return BevuvikMlpConfig("dense", _int(f, "ff", where), _num(f, "limit", where))
