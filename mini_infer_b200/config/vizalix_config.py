"""Typed reader of a Vizalix ``config.json``.

A Vizalix model is a list of layers, each with one of three mixers (``channel_delta``, ``attention``,
``mamba2``), its sizes, and a dense gated feed-forward or none; a stretch of the layers may run several times
in a row (``loop``).  Every size and every constant that can differ between models is read here and nowhere
else; sizes that only a tensor's shape gives (the ranks of the low-rank decay and gate projections of
``channel_delta``) are taken from the checkpoint's header when the model is built from a folder, or from the
optional keys ``decay_rank`` / ``gate_rank``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("channel_delta", "attention", "mamba2")


def _need(d: Mapping[str, Any], key: str, what: str, kind=(int, float)):
    if key not in d:
        raise ConfigError(f"Vizalix config: {what} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"Vizalix config: {what} '{key}' = {v!r} has the wrong type")
    return v


def _positive_int(d: Mapping[str, Any], key: str, what: str) -> int:
    v = _need(d, key, what, int)
    if v < 1:
        raise ConfigError(f"Vizalix config: {what} '{key}' = {v} must be positive")
    return v


@dataclass(frozen=True)
class VizalixLayer:
    type: str
    mixer: Mapping[str, Any]
    ff: Optional[int]               # width of the feed-forward, None for a layer without one


@dataclass(frozen=True)
class VizalixLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class VizalixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[VizalixLayer, ...]
    loop: Optional[VizalixLoop]

    @classmethod
    def from_json_dict(cls, j: Mapping[str, Any]) -> "VizalixConfig":
        vocab = _positive_int(j, "vocab", "the model")
        width = _positive_int(j, "width", "the model")
        norm = j.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("Vizalix config: 'norm' must be an object with 'eps'")
        eps = float(_need(norm, "eps", "norm"))
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("Vizalix config: 'layers' must be a non-empty list")
        layers: List[VizalixLayer] = []
        for i, l in enumerate(raw):
            what = f"layer {i}"
            if not isinstance(l, Mapping) or l.get("type") not in MIXER_TYPES:
                raise ConfigError(f"Vizalix config: {what} needs a 'type' among {MIXER_TYPES}")
            m = l.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"Vizalix config: {what} lacks its 'mixer' sizes")
            _check_mixer(l["type"], m, what)
            mlp = l.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"Vizalix config: {what} has an 'mlp' that is not of kind 'dense'")
                ff = _positive_int(mlp, "ff", what + " mlp")
            layers.append(VizalixLayer(l["type"], dict(m), ff))
        loop = None
        lj = j.get("loop")
        if lj is not None:
            if not isinstance(lj, Mapping):
                raise ConfigError("Vizalix config: 'loop' must be an object")
            start, stop = _need(lj, "start", "loop", int), _need(lj, "stop", "loop", int)
            times = _positive_int(lj, "times", "loop")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"Vizalix config: loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = VizalixLoop(start, stop, times)
        return cls(str(j.get("architecture", "Vizalix")), vocab, width, eps, tuple(layers), loop)

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """The order of layer runs: ``(layer, pass)`` where ``pass`` is the number of the loop pass that
        this run opens (the run is the first of its pass), else None."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        out += [(i, None) for i in range(lp.stop, n)]
        return out


def _check_mixer(kind: str, m: Mapping[str, Any], what: str) -> None:
    if kind == "channel_delta":
        for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
            _positive_int(m, k, what)
    elif kind == "attention":
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(m, k, what)
        mask = m.get("mask")
        if not isinstance(mask, Mapping):
            raise ConfigError(f"Vizalix config: {what} lacks 'mask'")
        _positive_int(mask, "size", what + " mask")
        _need(m, "scale", what)
        rot = m.get("rot")
        if rot is not None:
            if not isinstance(rot, Mapping):
                raise ConfigError(f"Vizalix config: {what} 'rot' must be an object")
            dims = _positive_int(rot, "dims", what + " rot")
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"Vizalix config: {what} rotates {dims} of {m['dim']} dimensions")
            _need(rot, "base", what + " rot")
            sc = rot.get("scaling")
            if sc is not None:
                for k in ("factor", "low", "high", "original"):
                    _need(sc, k, what + " rot scaling")
    else:
        for k in ("heads", "vdim", "state", "conv"):
            _positive_int(m, k, what)
    if kind != "mamba2" and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"Vizalix config: {what}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
