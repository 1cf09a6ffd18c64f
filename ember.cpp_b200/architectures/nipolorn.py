"""Nipolorn as a ModelSpec.

Token embedding without positions (no layer uses them in its scores); per layer the `sandwich`
arrangement (an RMS norm with a gain stored around zero before and after each sublayer); the
mixer two members side by side on the same input, a windowed attention that also keeps the
sequence's first tokens and a Mamba-2 recurrence, added with the configuration's two factors; the
feed-forward a clamped gated layer (`g = min(g, limit)`, `u` within +-limit,
`g * sigmoid(1.702 g) * (u + 1)`), or experts picked by a table over token ids with an optional
shared expert, or none; a last norm and an untied head.  The constants 1.702 and 1 of the clamped
layer are the design's, everything else comes from the configuration.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.nipolorn import NipolornConfig
from ..parts.spec import Application, LayerSpec, ModelSpec, PartSpec

GATE_ALPHA = 1.702
UP_SHIFT = 1.0


def build_spec(cfg: NipolornConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", name, {"width": d, "eps": eps, "weight": "", "offset": 1.0})  # noqa: E731
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        a, r = m["left"], m["right"]
        left = PartSpec("causal_attention", p + "mix.left.", {
            "width": d, "n_heads": a["heads"], "kv_heads": a["kv_heads"], "head_dim": a["dim"], "value_dim": a["vdim"],
            "scale": a["scale"], "window": a["mask"]["size"], "keep_first": a["mask"]["keep_first"],
            "qkv": ("q", "k", "v"), "out": "o", "stored": "out_in", "bias": False, "suffix": ""})
        right = PartSpec("mamba2", p + "mix.right.", {
            "width": d, "heads": r["heads"], "vdim": r["vdim"], "groups": r["groups"], "state": r["state"],
            "conv": r["conv"], "norm_groups": r["norm_groups"], "eps": eps})
        mixer = PartSpec("parallel", p + "mix.", {"width": d, "members": (
            ("left", left, m["left_scale"]), ("right", right, m["right_scale"]))})
        mlp = layer.get("mlp")
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = PartSpec("gated", p + "mlp.", {"width": d, "inner": mlp["ff"], "activation": "clamped_sigmoid",
                                                 "limit": mlp["limit"], "alpha": GATE_ALPHA, "shift": UP_SHIFT, "suffix": ""})
        else:
            shared = mlp.get("shared")
            ffn = PartSpec("table_experts", p + "mlp.", {
                "width": d, "vocab": cfg.vocab, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "inner": mlp["expert"]["ff"], "shared_inner": shared["ff"] if shared else 0, "suffix": ""})
        more = (("after_mixer", norm(p + "norm1b")),) + ((("after_ffn", norm(p + "norm2b")),) if ffn is not None else ())
        layers.append(LayerSpec("sandwich", norm(p + "norm1"), mixer, norm(p + "norm2") if ffn is not None else None, ffn, more))
    return ModelSpec(width=d, vocab_size=cfg.vocab, token_table="embed", position=PartSpec("none", ""),
                     layers=tuple(layers), schedule=tuple(Application(i) for i in range(len(layers))),
                     final_norm=norm("final.norm"), head="head")


register_architecture(NipolornConfig.architecture, NipolornConfig, build_spec)
