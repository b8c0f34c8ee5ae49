"""Typed reader of a Bogetar ``config.json``.

A Bogetar model is a list of layers, each with a mixer of type ``delta`` (gated delta rule with one decay per
head) or ``parallel`` (windowed attention with logistic, unnormalised key weights beside gated linear attention,
their outputs added with two weights) and a feed-forward (``moe`` with grouped expert selection, or none).  A
norm in groups stands before and after each part, a short convolution over time before each part's input, and a
layer scale behind each output norm.  Every size and every constant that can differ between models is read here
and nowhere else; the rank of the linear attention's decay projection is given by a tensor's shape alone
(``decay_rank`` in the mixer's sizes serves models made without a checkpoint).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("delta", "parallel")
MLP_KINDS = ("moe",)


def _need(d: Mapping[str, Any], key: str, what: str, kind=(int, float)):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"Bogetar config: {what} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"Bogetar config: {what} '{key}' = {v!r} has the wrong type")
    return v


def _positive_int(d: Mapping[str, Any], key: str, what: str) -> int:
    v = _need(d, key, what, int)
    if v < 1:
        raise ConfigError(f"Bogetar config: {what} '{key}' = {v} must be positive")
    return v


def _positive(d: Mapping[str, Any], key: str, what: str) -> float:
    v = float(_need(d, key, what))
    if not v > 0:
        raise ConfigError(f"Bogetar config: {what} '{key}' = {v} must be positive")
    return v


def _object(d: Mapping[str, Any], key: str, what: str) -> Mapping[str, Any]:
    v = d.get(key) if isinstance(d, Mapping) else None
    if not isinstance(v, Mapping):
        raise ConfigError(f"Bogetar config: {what} lacks the object '{key}'")
    return v


@dataclass(frozen=True)
class BogetarLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]        # None: a layer without a feed-forward


@dataclass(frozen=True)
class BogetarConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    norm_groups: int
    taps: int                               # of the convolutions before each part's input
    layers: Tuple[BogetarLayer, ...]

    @classmethod
    def from_json_dict(cls, j: Mapping[str, Any]) -> "BogetarConfig":
        vocab = _positive_int(j, "vocab", "the model")
        width = _positive_int(j, "width", "the model")
        norm = _object(j, "norm", "the model")
        eps = _positive(norm, "eps", "norm")
        groups = _positive_int(norm, "groups", "norm") if "groups" in norm else 1
        if width % groups:
            raise ConfigError(f"Bogetar config: a width of {width} does not split into {groups} norm groups")
        taps = _positive_int(_object(j, "canon", "the model"), "taps", "canon")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("Bogetar config: 'layers' must be a non-empty list")
        layers: List[BogetarLayer] = []
        for i, l in enumerate(raw):
            what = f"layer {i}"
            if not isinstance(l, Mapping) or l.get("type") not in MIXER_TYPES:
                raise ConfigError(f"Bogetar config: {what} needs a 'type' among {MIXER_TYPES}")
            m = _object(l, "mixer", what)
            (_check_delta if l["type"] == "delta" else _check_parallel)(m, what)
            mlp = l.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, what + " mlp")
            layers.append(BogetarLayer(l["type"], m, mlp))
        return cls(str(j.get("architecture", "Bogetar")), vocab, width, eps, groups, taps, tuple(layers))


def _check_heads(m: Mapping[str, Any], what: str) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m, k, what)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"Bogetar config: {what}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")


def _check_delta(m: Mapping[str, Any], what: str) -> None:
    _check_heads(m, what)
    _positive_int(m, "conv", what)


def _check_parallel(m: Mapping[str, Any], what: str) -> None:
    left, right = _object(m, "left", what), _object(m, "right", what)
    _check_heads(left, what + " left")
    _positive_int(_object(left, "mask", what + " left"), "size", what + " left mask")
    _need(left, "scale", what + " left")
    rot = left.get("rot")
    if rot is not None:
        dims = _positive_int(rot, "dims", what + " left rot")
        if dims % 2 or dims > left["dim"]:
            raise ConfigError(f"Bogetar config: {what} left rotates {dims} of {left['dim']} dimensions")
        _positive(rot, "base", what + " left rot")
    for k in ("heads", "dim", "vdim"):
        _positive_int(right, k, what + " right")
    _positive(right, "tau", what + " right")
    _need(m, "left_scale", what)
    _need(m, "right_scale", what)


def _check_mlp(mlp: Any, what: str) -> None:
    if not isinstance(mlp, Mapping) or mlp.get("kind", "moe") not in MLP_KINDS:
        raise ConfigError(f"Bogetar config: {what} must be of a kind among {MLP_KINDS}")
    expert = _object(mlp, "expert", what)
    _positive_int(expert, "ff", what + " expert")
    _positive(expert, "limit", what + " expert")
    router = _object(mlp, "router", what)
    E, top = _positive_int(router, "experts", what + " router"), _positive_int(router, "top", what + " router")
    count = keep = 1
    if router.get("groups") is not None:
        g = _object(router, "groups", what + " router")
        count, keep = _positive_int(g, "count", what + " groups"), _positive_int(g, "keep", what + " groups")
    if E % count or keep > count:
        raise ConfigError(f"Bogetar config: {what}: {E} experts in {count} groups of which {keep} are kept")
    if top > keep * (E // count):
        raise ConfigError(f"Bogetar config: {what}: top {top} exceeds the {keep * (E // count)} experts of {keep} groups")


def expert_groups(router: Mapping[str, Any]) -> Tuple[int, int]:
    g = router.get("groups")
    return (int(g["count"]), int(g["keep"])) if g is not None else (1, 1)
