"""Typed reader of a Tofinex ``config.json``.

A Tofinex model is a list of layers, each an ``attention`` mixer (grouped-query attention with normalised,
neighbour-rotated heads, capped scores, a softmax that counts one key more, values that may be blended with
the first blending layer's) and a feed-forward (``dense``, ``moe`` with an optional shared expert, or none),
whose OUTPUTS are normalised and added to the residual times ``residual_mult``.  Every size and every constant
that can differ between models is read here and nowhere else.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _need(d: Mapping[str, Any], key: str, what: str, kind=(int, float)):
    if key not in d:
        raise ConfigError(f"Tofinex config: {what} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"Tofinex config: {what} '{key}' = {v!r} has the wrong type")
    return v


def _positive_int(d: Mapping[str, Any], key: str, what: str) -> int:
    v = _need(d, key, what, int)
    if v < 1:
        raise ConfigError(f"Tofinex config: {what} '{key}' = {v} must be positive")
    return v


def _positive(d: Mapping[str, Any], key: str, what: str) -> float:
    v = float(_need(d, key, what))
    if not v > 0:
        raise ConfigError(f"Tofinex config: {what} '{key}' = {v} must be positive")
    return v


def _cap(d: Mapping[str, Any], key: str, what: str) -> float:
    """A cap ``c`` of ``c tanh(z / c)``: positive, or absent / null / 0 for none."""
    if d.get(key) is None:
        return 0.0
    v = float(_need(d, key, what))
    if v < 0:
        raise ConfigError(f"Tofinex config: {what} '{key}' = {v} must not be negative")
    return v


@dataclass(frozen=True)
class TofinexLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]        # None: a layer without a feed-forward

    @property
    def blends_values(self) -> bool:
        return bool(self.mixer.get("v_mix", False))


@dataclass(frozen=True)
class TofinexConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: float
    layers: Tuple[TofinexLayer, ...]

    @property
    def first_blending_layer(self) -> Optional[int]:
        for i, l in enumerate(self.layers):
            if l.blends_values:
                return i
        return None

    @classmethod
    def from_json_dict(cls, j: Mapping[str, Any]) -> "TofinexConfig":
        vocab = _positive_int(j, "vocab", "the model")
        width = _positive_int(j, "width", "the model")
        norm = j.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("Tofinex config: 'norm' must be an object with 'eps'")
        eps = float(_need(norm, "eps", "norm"))
        if eps < 0:
            raise ConfigError(f"Tofinex config: norm 'eps' = {eps} must not be negative")
        mult = float(_need(j, "residual_mult", "the model")) if "residual_mult" in j else 1.0
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("Tofinex config: 'layers' must be a non-empty list")
        layers: List[TofinexLayer] = []
        for i, l in enumerate(raw):
            what = f"layer {i}"
            if not isinstance(l, Mapping) or l.get("type") not in MIXER_TYPES:
                raise ConfigError(f"Tofinex config: {what} needs a 'type' among {MIXER_TYPES}")
            m = l.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"Tofinex config: {what} lacks its 'mixer' sizes")
            _check_mixer(m, what)
            mlp = l.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, what)
            layers.append(TofinexLayer(l["type"], dict(m), None if mlp is None else dict(mlp)))
        # the layers that blend values share the first one's: they must be of one size
        first = next((l for l in layers if l.blends_values), None)
        for i, l in enumerate(layers):
            if l.blends_values and (l.mixer["kv_heads"] * l.mixer["vdim"]
                                    != first.mixer["kv_heads"] * first.mixer["vdim"]):
                raise ConfigError(f"Tofinex config: layer {i} blends values of {l.mixer['kv_heads']} x "
                                  f"{l.mixer['vdim']} with the first blending layer's "
                                  f"{first.mixer['kv_heads']} x {first.mixer['vdim']}")
        return cls(str(j.get("architecture", "Tofinex")), vocab, width, eps, mult,
                   _cap(j, "logit_softcap", "the model"), tuple(layers))


def _check_mixer(m: Mapping[str, Any], what: str) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m, k, what)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"Tofinex config: {what}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
    _positive(m, "scale", what)
    _cap(m, "softcap", what)
    if "v_mix" in m and not isinstance(m["v_mix"], bool):
        raise ConfigError(f"Tofinex config: {what} 'v_mix' = {m['v_mix']!r} must be true or false")
    rot = m.get("rot")
    if rot is not None:
        if not isinstance(rot, Mapping):
            raise ConfigError(f"Tofinex config: {what} 'rot' must be an object")
        dims = _need(rot, "dims", what + " rot", int)
        if dims < 0 or dims % 2 or dims > m["dim"]:
            raise ConfigError(f"Tofinex config: {what} rotates {dims} of {m['dim']} dimensions")
        if dims:
            _positive(rot, "base", what + " rot")


def _check_mlp(mlp: Any, what: str) -> None:
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"Tofinex config: {what} has an 'mlp' whose 'kind' is not among {MLP_KINDS}")
    if mlp["kind"] == "dense":
        _positive_int(mlp, "ff", what + " mlp")
        return
    ex, ro = mlp.get("expert"), mlp.get("router")
    if not isinstance(ex, Mapping) or not isinstance(ro, Mapping):
        raise ConfigError(f"Tofinex config: {what} mlp of kind 'moe' needs 'expert' and 'router'")
    _positive_int(ex, "ff", what + " expert")
    n, k = _positive_int(ro, "experts", what + " router"), _positive_int(ro, "top", what + " router")
    if k > n:
        raise ConfigError(f"Tofinex config: {what} router picks {k} of {n} experts")
    sh = mlp.get("shared")
    if sh is not None:
        if not isinstance(sh, Mapping):
            raise ConfigError(f"Tofinex config: {what} 'shared' must be an object with 'ff'")
        _positive_int(sh, "ff", what + " shared expert")
