"""Muzozen as a ModelSpec.

The token's row times a factor, plus a row of a table of token pairs (`pair_table`), normed; no
position table (the attention layers rotate their queries and keys).  Per layer the `shared_norm`
arrangement: one RMS norm whose output the mixer and the feed-forward both read, their outputs
added to the stream.  The mixer is a gated delta rule or an attention over cached low-rank rows,
which may read the rows that an earlier layer cached; the feed-forward is dense with the tanh
GELU and no biases, or absent; a last norm and an untied head.  Every number comes from the
configuration.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.muzozen import MuzozenConfig
from ..parts.spec import Application, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: MuzozenConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", name, {"width": d, "eps": eps, "weight": ""})  # noqa: E731
    layers, schedule, entry_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        cache_of = None
        if layer["type"] == "delta":
            mixer = PartSpec("gated_delta_rule", p + "mix.", {
                "width": d, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                "conv": m["conv"], "eps": eps})
        else:
            src = m.get("kv_from")
            cache_of = None if src is None else entry_of[src]
            rot = m["rot"]
            mixer = PartSpec("latent_attention", p + "mix.", {
                "width": d, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
                "rotary": {"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling")},
                "shares_cache": src is not None})
        mlp = layer.get("mlp")
        ffn = None if mlp is None else PartSpec("dense", p + "mlp.", {
            "width": d, "inner": mlp["ff"], "activation": "gelu_tanh", "up": "up", "down": "down", "stored": "out_in",
            "bias": False, "suffix": "", "any_size": True})
        entry_of[i] = len(schedule)
        schedule.append(Application(i, cache_of))
        layers.append(LayerSpec("shared_norm", norm(p + "norm1"), mixer, None, ffn))
    pair = cfg.embedding["bigram"]
    extras = () if pair is None else (PartSpec("pair_table", "", {
        "width": d, "buckets": pair["buckets"], "mul_prev": pair["mul_prev"], "mul_cur": pair["mul_cur"], "table": "bigram"}),)
    return ModelSpec(width=d, vocab_size=cfg.vocab, token_table="embed", position=PartSpec("none", ""),
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"), head="head",
                     embedding_scale=float(cfg.embedding["scale"]), embed_parts=extras, embed_norm=norm("embed.norm"))


register_architecture(MuzozenConfig.architecture, MuzozenConfig, build_spec)
