"""Typed reader of a Nipapel ``config.json``.

A Nipapel model is a list of layers, each with one of two mixers (``attention``: grouped-query attention with
normalised heads behind a window that keeps the first tokens; ``latent_attention``: attention through a
latent, optionally reading the latents another layer caches) and a feed-forward (``dense``, ``moe`` or
none).  Every size and every constant that can differ between models is read here and nowhere else.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _need(d: Mapping[str, Any], key: str, what: str, kind=(int, float)):
    if key not in d:
        raise ConfigError(f"Nipapel config: {what} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"Nipapel config: {what} '{key}' = {v!r} has the wrong type")
    return v


def _positive_int(d: Mapping[str, Any], key: str, what: str) -> int:
    v = _need(d, key, what, int)
    if v < 1:
        raise ConfigError(f"Nipapel config: {what} '{key}' = {v} must be positive")
    return v


def _positive(d: Mapping[str, Any], key: str, what: str) -> float:
    v = float(_need(d, key, what))
    if not v > 0:
        raise ConfigError(f"Nipapel config: {what} '{key}' = {v} must be positive")
    return v


@dataclass(frozen=True)
class NipapelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]        # None: a layer without a feed-forward


@dataclass(frozen=True)
class NipapelConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[NipapelLayer, ...]

    @classmethod
    def from_json_dict(cls, j: Mapping[str, Any]) -> "NipapelConfig":
        vocab = _positive_int(j, "vocab", "the model")
        width = _positive_int(j, "width", "the model")
        norm = j.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("Nipapel config: 'norm' must be an object with 'eps'")
        eps = float(_need(norm, "eps", "norm"))
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("Nipapel config: 'layers' must be a non-empty list")
        layers: List[NipapelLayer] = []
        for i, l in enumerate(raw):
            what = f"layer {i}"
            if not isinstance(l, Mapping) or l.get("type") not in MIXER_TYPES:
                raise ConfigError(f"Nipapel config: {what} needs a 'type' among {MIXER_TYPES}")
            m = l.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"Nipapel config: {what} lacks its 'mixer' sizes")
            _check_mixer(l["type"], m, what)
            mlp = l.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, what)
            layers.append(NipapelLayer(l["type"], dict(m), None if mlp is None else dict(mlp)))
        # a layer that borrows latents names an earlier latent layer that caches its own, of the same geometry
        for i, l in enumerate(layers):
            src = l.mixer.get("kv_from")
            if src is None:
                continue
            what = f"layer {i}"
            if l.type != "latent_attention" or isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"Nipapel config: {what} 'kv_from' = {src!r} must name an earlier layer")
            o = layers[src]
            if o.type != "latent_attention" or o.mixer.get("kv_from") is not None:
                raise ConfigError(f"Nipapel config: {what} borrows from layer {src}, which caches no latents of its own")
            same = all(o.mixer[k] == l.mixer[k] for k in ("kv_rank", "rot_dim")) and \
                all(o.mixer["rot"][k] == l.mixer["rot"][k] for k in ("base", "dims"))
            if not same:
                raise ConfigError(f"Nipapel config: {what} and layer {src} differ in latent size or rotation")
        return cls(str(j.get("architecture", "Nipapel")), vocab, width, eps, tuple(layers))


def _check_mask(m: Mapping[str, Any], what: str, may_keep: bool) -> None:
    mask = m.get("mask")
    if not isinstance(mask, Mapping):
        raise ConfigError(f"Nipapel config: {what} lacks 'mask'")
    _positive_int(mask, "size", what + " mask")
    if "keep_first" in mask:
        if not may_keep:
            raise ConfigError(f"Nipapel config: {what} mask: 'keep_first' belongs to the 'attention' mixer")
        if _need(mask, "keep_first", what + " mask", int) < 0:
            raise ConfigError(f"Nipapel config: {what} mask 'keep_first' must not be negative")


def _check_rot(m: Mapping[str, Any], what: str, within: int, required: bool) -> None:
    rot = m.get("rot")
    if rot is None:
        if required:
            raise ConfigError(f"Nipapel config: {what} lacks 'rot'")
        return
    if not isinstance(rot, Mapping):
        raise ConfigError(f"Nipapel config: {what} 'rot' must be an object")
    dims = _positive_int(rot, "dims", what + " rot")
    if dims % 2 or dims > within:
        raise ConfigError(f"Nipapel config: {what} rotates {dims} of {within} dimensions")
    _positive(rot, "base", what + " rot")


def _check_mixer(kind: str, m: Mapping[str, Any], what: str) -> None:
    _positive(m, "scale", what)
    if kind == "attention":
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(m, k, what)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"Nipapel config: {what}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
        _check_mask(m, what, True)
        _check_rot(m, what, m["dim"], False)
    else:
        for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
            _positive_int(m, k, what)
        _check_mask(m, what, False)
        _check_rot(m, what, m["rot_dim"], True)
        if m["rot"]["dims"] != m["rot_dim"]:
            raise ConfigError(f"Nipapel config: {what}: the rotation covers {m['rot']['dims']} dimensions, "
                              f"the rotated part has {m['rot_dim']}")


def _check_mlp(mlp: Any, what: str) -> None:
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"Nipapel config: {what} has an 'mlp' whose 'kind' is not among {MLP_KINDS}")
    if mlp["kind"] == "dense":
        _positive_int(mlp, "ff", what + " mlp")
        _positive(mlp, "limit", what + " mlp")
        return
    ex, ro = mlp.get("expert"), mlp.get("router")
    if not isinstance(ex, Mapping) or not isinstance(ro, Mapping):
        raise ConfigError(f"Nipapel config: {what} mlp of kind 'moe' needs 'expert' and 'router'")
    _positive_int(ex, "ff", what + " expert")
    _positive(ex, "limit", what + " expert")
    n, k = _positive_int(ro, "experts", what + " router"), _positive_int(ro, "top", what + " router")
    if k > n:
        raise ConfigError(f"Nipapel config: {what} router picks {k} of {n} experts")
