"""Muzozen's configuration, read from its own config.json.

The file is nested: `vocab`, `width`, `norm.eps`, `embedding` (`scale`, and `bigram` with `buckets`,
`mul_prev`, `mul_cur` for the table of token pairs, or no `bigram` for a model without one), and
`layers`, a list with one entry per layer: `type` (which mixer the layer has: `delta` or
`latent_attention`), `mixer` (that mixer's sizes and constants) and `mlp` (the feed-forward's, or
null for a layer without one).  The architecture is named by a top-level `architecture` string.
Every size and constant is taken from there and checked here, key by key, so that an error names
the key.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("delta", "latent_attention")
MLPS = ("dense",)


def _get(d: dict, path: str, kind, where: str, positive: bool = True):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, dict) or key not in cur or cur[key] is None:
            raise ConfigError(f"MuzozenConfig: {where}{path} is missing")
        cur = cur[key]
    if isinstance(cur, bool) or not isinstance(cur, (int, float)) or (kind is int and int(cur) != cur):
        raise ConfigError(f"MuzozenConfig: {where}{path} = {cur!r}, expected {'a whole number' if kind is int else 'a number'}")
    cur = kind(cur)
    if positive and not cur > 0:
        raise ConfigError(f"MuzozenConfig: {where}{path} = {cur} must be positive")
    return cur


@dataclasses.dataclass(frozen=True)
class MuzozenConfig(ModelConfig):
    architecture: ClassVar[str] = "Muzozen"

    vocab: int
    width: int
    norm_eps: float
    embedding: dict        # {"scale": s, "bigram": {"buckets", "mul_prev", "mul_cur"} or None}
    layers: tuple          # the entries of config.json's `layers`, checked, as plain dicts

    def __hash__(self):
        return hash((self.vocab, self.width, self.norm_eps, len(self.layers)))

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "MuzozenConfig":
        vocab = _get(d, "vocab", int, "")
        width = _get(d, "width", int, "")
        eps = _get(d, "norm.eps", float, "")
        emb = d.get("embedding")
        if not isinstance(emb, dict):
            raise ConfigError("MuzozenConfig: embedding is missing")
        embedding = {"scale": _get(emb, "scale", float, "embedding.", positive=False), "bigram": None}
        if emb.get("bigram") is not None:
            b = emb["bigram"]
            embedding["bigram"] = {"buckets": _get(b, "buckets", int, "embedding.bigram."),
                                   "mul_prev": _get(b, "mul_prev", int, "embedding.bigram.", positive=False),
                                   "mul_cur": _get(b, "mul_cur", int, "embedding.bigram.", positive=False)}
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("MuzozenConfig: layers is missing or empty")
        cfg = cls(vocab=vocab, width=width, norm_eps=eps, embedding=embedding, layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            at = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"MuzozenConfig: layers[{i}] is not an object")
            if layer.get("type") not in MIXERS:
                raise ConfigError(f"MuzozenConfig: {at}type = {layer.get('type')!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"MuzozenConfig: {at}mixer is missing")
            if layer["type"] == "delta":
                for key in ("conv", "dim", "heads", "kv_heads", "vdim"):
                    _get(m, key, int, at + "mixer.")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"MuzozenConfig: {at}mixer.heads is not a multiple of kv_heads")
            else:
                self._check_latent(i, m, at + "mixer.")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLPS:
                raise ConfigError(f"MuzozenConfig: {at}mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                  f"is not one of {MLPS}")
            _get(mlp, "ff", int, at + "mlp.")

    def _check_latent(self, i: int, m: dict, at: str) -> None:
        for key in ("dim", "heads", "kv_rank", "q_rank", "rot_dim", "vdim", "rot.dims"):
            _get(m, key, int, at)
        _get(m, "scale", float, at)
        _get(m, "rot.base", float, at)
        if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
            raise ConfigError(f"MuzozenConfig: {at}rot.dims = {m['rot']['dims']} must be even and at most rot_dim")
        if m["rot"].get("scaling") is not None:
            for key in ("factor", "fast", "slow"):
                _get(m, "rot.scaling." + key, float, at)
            _get(m, "rot.scaling.original", float, at)
        src = m.get("kv_from")
        if src is None:
            return
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
            raise ConfigError(f"MuzozenConfig: {at}kv_from = {src!r} must name an earlier layer")
        other = self.layers[src]
        if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
            raise ConfigError(f"MuzozenConfig: {at}kv_from = {src} names a layer without cached rows of its own")
        for key in ("kv_rank", "rot_dim", "rot"):
            if other["mixer"].get(key) != m.get(key):
                raise ConfigError(f"MuzozenConfig: {at}kv_from = {src}: the two layers differ in {key}")

    def check_dtype(self, dtype: str) -> None:
        """Nothing is refused: every part of this design has a kernel for every size in both compute types (rows
        that are no multiples of 16 bytes take the slower ones)."""

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": copy.deepcopy(self.embedding),
                "layers": copy.deepcopy(list(self.layers))}
