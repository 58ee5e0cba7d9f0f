"""Typed configuration of the Bapavik decoder, read from its config.json.

The file gives ``width``, ``vocab``, ``norm.eps``, ``embedding.scale``, ``layers`` and optionally ``loop``. A layer
names its mixer (``type``: "attention" or "latent_attention"), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``: an object of kind "dense" or "moe", or null for a layer without one). ``loop`` = {start, stop,
times}: layers start .. stop-1 run ``times`` times in a row with the same weights (each pass has a cache of its own),
then the rest follow. Every size and constant is taken from the file; nothing is assumed equal between layers.
``max_position`` (the longest sequence the engine plans for) is optional.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig

_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
}


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d or d[k] is None]
    if missing:
        raise ConfigError(f"{where} lacks the keys: {', '.join(missing)}")


def _positive(d, keys, where: str) -> None:
    for k in keys:
        if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] <= 0:
            raise ConfigError(f"{where}.{k} must be a positive integer, got {d[k]!r}")


@dataclass(frozen=True)
class BapavikConfig(ModelConfig):
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    max_position: int = 1 << 17

    architecture = "Bapavik"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "BapavikConfig":
        _need(d, ("width", "vocab", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        _positive(d, ("width", "vocab"), "config.json")
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
            if kind == "attention":
                _positive(m, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads must be a multiple of kv_heads")
                if m.get("q_temp") is not None:
                    _need(m["q_temp"], ("coef", "every"), where + ".mixer.q_temp")
                    _positive(m["q_temp"], ("every",), where + ".mixer.q_temp")
                if m.get("softcap") is not None and not float(m["softcap"]) > 0:
                    raise ConfigError(f"{where}.mixer.softcap must be positive")
            else:
                _positive(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where + ".mixer")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                _positive(m["rot"], ("dims",), where + ".mixer.rot")
                if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most rot_dim")
            f = layer.get("mlp")
            if f is not None:
                _need(f, ("kind",), where + ".mlp")
                if f["kind"] == "dense":
                    _need(f, ("ff", "limit"), where + ".mlp")
                    _positive(f, ("ff",), where + ".mlp")
                elif f["kind"] == "moe":
                    _need(f, ("expert", "router"), where + ".mlp")
                    _need(f["expert"], ("ff",), where + ".mlp.expert")
                    _need(f["router"], ("experts", "top"), where + ".mlp.router")
                    _positive(f["expert"], ("ff",), where + ".mlp.expert")
                    _positive(f["router"], ("experts", "top"), where + ".mlp.router")
                    if f["router"]["top"] > f["router"]["experts"]:
                        raise ConfigError(f"{where}.mlp.router: top exceeds experts")
                else:
                    raise ConfigError(f"{where}.mlp.kind {f['kind']!r} is not known (dense, moe)")
            layers.append(copy.deepcopy({"type": kind, "mixer": m, "mlp": f}))
        eps = float(d["norm"]["eps"])
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            _need(lp, ("start", "stop", "times"), "loop")
            start, stop, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop {lp!r} does not fit {len(layers)} layers (0 <= start <= stop <= layers, times >= 1)")
            loop = (start, stop, times)
        scale = 1.0
        if d.get("embedding") is not None:
            _need(d["embedding"], ("scale",), "embedding")
            scale = float(d["embedding"]["scale"])
        return cls(width=int(d["width"]), vocab=int(d["vocab"]), eps=eps, embedding_scale=scale, layers=tuple(layers), loop=loop,
                   max_position=int(d.get("max_position") or (1 << 17)))

    def layer_order(self) -> Tuple[int, ...]:
        """Indices of the layers in running order."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(list(self.layers)),
               "max_position": self.max_position}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out
