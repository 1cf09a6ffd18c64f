"""Nipolorn's configuration, read from its own config.json.

The file is nested: `vocab`, `width`, `norm.eps`, and `layers`, a list with one entry per layer:
`type` (which mixer the layer has), `mixer` (that mixer's sizes and constants) and `mlp` (the
feed-forward's, or null for a layer without one).  The architecture is named by a top-level
`architecture` string.  Every size and constant is taken from there; the kinds of mixer and
feed-forward that the design knows are checked here, key by key, so that an error names the key.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("parallel",)
MLPS = ("dense", "moe")


def _get(d: dict, path: str, kind, where: str, positive: bool = True):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, dict) or key not in cur or cur[key] is None:
            raise ConfigError(f"NipolornConfig: {where}{path} is missing")
        cur = cur[key]
    if isinstance(cur, bool) or not isinstance(cur, (int, float)) or (kind is int and int(cur) != cur):
        raise ConfigError(f"NipolornConfig: {where}{path} = {cur!r}, expected {'a whole number' if kind is int else 'a number'}")
    cur = kind(cur)
    if positive and not cur > 0:
        raise ConfigError(f"NipolornConfig: {where}{path} = {cur} must be positive")
    return cur


@dataclasses.dataclass(frozen=True)
class NipolornConfig(ModelConfig):
    architecture: ClassVar[str] = "Nipolorn"

    vocab: int
    width: int
    norm_eps: float
    layers: tuple          # the entries of config.json's `layers`, checked, as plain dicts

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "NipolornConfig":
        vocab = _get(d, "vocab", int, "")
        width = _get(d, "width", int, "")
        eps = _get(d, "norm.eps", float, "")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("NipolornConfig: layers is missing or empty")
        cfg = cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            at = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"NipolornConfig: layers[{i}] is not an object")
            if layer.get("type") not in MIXERS:
                raise ConfigError(f"NipolornConfig: {at}type = {layer.get('type')!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"NipolornConfig: {at}mixer is missing")
            for key in ("left.dim", "left.heads", "left.kv_heads", "left.vdim", "left.mask.size", "right.conv", "right.groups",
                        "right.heads", "right.norm_groups", "right.state", "right.vdim"):
                _get(m, key, int, at + "mixer.")
            if m["left"]["mask"].get("keep_first") is None:      # a window that keeps no first tokens
                m["left"]["mask"]["keep_first"] = 0
            _get(m, "left.mask.keep_first", int, at + "mixer.", positive=False)
            if m["left"]["mask"]["keep_first"] < 0:
                raise ConfigError(f"NipolornConfig: {at}mixer.left.mask.keep_first is negative")
            _get(m, "left.scale", float, at + "mixer.")
            _get(m, "left_scale", float, at + "mixer.", positive=False)
            _get(m, "right_scale", float, at + "mixer.", positive=False)
            if m["left"]["heads"] % m["left"]["kv_heads"]:
                raise ConfigError(f"NipolornConfig: {at}mixer.left.heads is not a multiple of kv_heads")
            if m["right"]["heads"] % m["right"]["groups"]:
                raise ConfigError(f"NipolornConfig: {at}mixer.right.heads is not a multiple of groups")
            if (m["right"]["heads"] * m["right"]["vdim"]) % m["right"]["norm_groups"]:
                raise ConfigError(f"NipolornConfig: {at}mixer.right: heads * vdim is not a multiple of norm_groups")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLPS:
                raise ConfigError(f"NipolornConfig: {at}mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                  f"is not one of {MLPS}")
            if mlp["kind"] == "dense":
                _get(mlp, "ff", int, at + "mlp.")
                _get(mlp, "limit", float, at + "mlp.")
            else:
                _get(mlp, "expert.ff", int, at + "mlp.")
                experts = _get(mlp, "router.experts", int, at + "mlp.")
                top = _get(mlp, "router.top", int, at + "mlp.")
                if top > experts:
                    raise ConfigError(f"NipolornConfig: {at}mlp.router.top = {top} exceeds experts = {experts}")
                if mlp.get("shared") is not None:
                    _get(mlp, "shared.ff", int, at + "mlp.")

    def check_dtype(self, dtype: str) -> None:
        """Nothing is refused: every part of this design has a kernel for every size in both compute types (rows
        that are no multiples of 16 bytes take the slower ones)."""

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
