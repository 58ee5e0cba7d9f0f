"""Typed configuration of the Rogisun decoder, read from its config.json.

The file gives ``width``, ``vocab``, ``norm.eps``, ``canon.taps`` (the taps of the convolution in front of every
sub-layer) and ``layers``: a list whose entries name the layer's mixer (``type``: "lightning", "mamba2" or
"parallel"), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: an object of kind "moe", or
null for a layer without one). Every size and constant is taken from there; nothing is assumed equal between
layers. Two optional keys serve the random-weights mode only: ``max_position`` (the longest sequence the engine
plans for) and, in a delta-rule mixer, ``rank`` (the width of its two-step projections, which a weight file gives
by its shapes).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from .base import ConfigError, ModelConfig

_MIXER_KEYS = {
    "lightning": ("heads", "dim", "vdim", "decay"),
    "mamba2": ("heads", "vdim", "state", "groups", "norm_groups", "conv"),
    "parallel": ("left", "right", "left_scale", "right_scale"),
}
_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "mask")
_RIGHT_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")


def _need(d: Dict[str, Any], keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d or d[k] is None]
    if missing:
        raise ConfigError(f"{where} lacks the keys: {', '.join(missing)}")


def _positive(d: Dict[str, Any], keys, where: str) -> None:
    for k in keys:
        if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] <= 0:
            raise ConfigError(f"{where}.{k} must be a positive integer, got {d[k]!r}")


@dataclass(frozen=True)
class RogisunConfig(ModelConfig):
    width: int
    vocab: int
    eps: float
    canon_taps: int
    layers: Tuple[Dict[str, Any], ...]
    max_position: int = 1 << 17

    architecture = "Rogisun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RogisunConfig":
        _need(d, ("width", "vocab", "norm", "canon", "layers"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        _need(d["canon"], ("taps",), "canon")
        _positive(d, ("width", "vocab"), "config.json")
        _positive(d["canon"], ("taps",), "canon")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind = layer["type"]
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"{where}.type {kind!r} is not known ({', '.join(sorted(_MIXER_KEYS))})")
            m = layer["mixer"]
            _need(m, _MIXER_KEYS[kind], where + ".mixer")
            if kind == "lightning":
                _positive(m, ("heads", "dim", "vdim"), where + ".mixer")
                if not isinstance(m["decay"], list) or len(m["decay"]) != m["heads"]:
                    raise ConfigError(f"{where}.mixer.decay must list one decay per head")
            elif kind == "mamba2":
                _positive(m, ("heads", "vdim", "state", "groups", "norm_groups", "conv"), where + ".mixer")
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"{where}.mixer: heads must split into groups and heads * vdim into norm_groups")
            else:
                _need(m["left"], _LEFT_KEYS, where + ".mixer.left")
                _need(m["right"], _RIGHT_KEYS, where + ".mixer.right")
                _need(m["left"]["mask"], ("size",), where + ".mixer.left.mask")
                _positive(m["left"], ("heads", "kv_heads", "dim", "vdim"), where + ".mixer.left")
                _positive(m["left"]["mask"], ("size",), where + ".mixer.left.mask")
                _positive(m["right"], ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".mixer.right")
                for side in ("left", "right"):
                    if m[side]["heads"] % m[side]["kv_heads"]:
                        raise ConfigError(f"{where}.mixer.{side}: heads must be a multiple of kv_heads")
            f = layer.get("mlp")
            if f is not None:
                _need(f, ("kind", "expert", "router"), where + ".mlp")
                if f["kind"] != "moe":
                    raise ConfigError(f"{where}.mlp.kind {f['kind']!r} is not known (moe)")
                _need(f["expert"], ("ff", "limit"), where + ".mlp.expert")
                _need(f["router"], ("experts", "top"), where + ".mlp.router")
                _positive(f["expert"], ("ff",), where + ".mlp.expert")
                _positive(f["router"], ("experts", "top"), where + ".mlp.router")
                if f["router"]["top"] > f["router"]["experts"]:
                    raise ConfigError(f"{where}.mlp.router: top exceeds experts")
            layers.append(copy.deepcopy({"type": kind, "mixer": m, "mlp": f}))
        eps = float(d["norm"]["eps"])
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        return cls(width=int(d["width"]), vocab=int(d["vocab"]), eps=eps, canon_taps=int(d["canon"]["taps"]), layers=tuple(layers),
                   max_position=int(d.get("max_position") or (1 << 17)))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                "canon": {"taps": self.canon_taps}, "layers": copy.deepcopy(list(self.layers)), "max_position": self.max_position}
