"""Small Nipolorn configurations and helpers shared by the CPU and GPU tests.

The first two configurations differ from one another in every size and option (a third has sizes that are no
multiples of 8 anywhere): attention with values
wider than keys and grouped heads / plain heads with equal sizes; a window shorter than a page
with kept first tokens / a window longer than a page with none; Mamba-2 with groups, four taps and
split norm / one group, two taps, one norm part and sizes that are no powers of two; a clamped
gated layer, experts with and without a shared one, top 2 and top 1, and a layer without a
feed-forward.
"""
import copy
import json
import os

import numpy as np


def _layer(left, right, mlp, ls, rs):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


LEFT_A = {"dim": 16, "vdim": 32, "heads": 4, "kv_heads": 2, "scale": 0.31, "mask": {"size": 20, "keep_first": 3}}
RIGHT_A = {"heads": 4, "vdim": 16, "groups": 2, "state": 8, "conv": 4, "norm_groups": 2}
LEFT_B = {"dim": 32, "vdim": 32, "heads": 3, "kv_heads": 3, "scale": 0.15, "mask": {"size": 70, "keep_first": 0}}
RIGHT_B = {"heads": 2, "vdim": 40, "groups": 1, "state": 20, "conv": 2, "norm_groups": 1}

CONFIGS = {
    "nip_a": {"architecture": "Nipolorn", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        _layer(LEFT_A, RIGHT_A, {"kind": "dense", "ff": 104, "limit": 0.8}, 0.7, 1.1),
        _layer(LEFT_A, RIGHT_A, {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 40}}, 0.5, 0.8),
        _layer(LEFT_A, RIGHT_A, None, 1.0, 0.4),
        _layer(LEFT_A, RIGHT_A, {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 3, "top": 1}, "shared": None}, 0.9, 0.9),
    ]},
    "nip_b": {"architecture": "Nipolorn", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "layers": [
        _layer(LEFT_B, RIGHT_B, {"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 4, "top": 3}, "shared": {"ff": 16}}, 1.2, 0.6),
        _layer(LEFT_B, RIGHT_B, {"kind": "dense", "ff": 160, "limit": 2.5}, 0.8, 1.0),
    ]},
}
# sizes that are no multiples of 8 anywhere: rows that are no whole 16-byte pieces in bfloat16
LEFT_C = {"dim": 12, "vdim": 10, "heads": 3, "kv_heads": 1, "scale": 0.25, "mask": {"size": 9, "keep_first": 2}}
RIGHT_C = {"heads": 3, "vdim": 6, "groups": 1, "state": 7, "conv": 3, "norm_groups": 3}
CONFIGS["nip_c"] = {"architecture": "Nipolorn", "vocab": 101, "width": 60, "norm": {"eps": 1e-5}, "layers": [
    _layer(LEFT_C, RIGHT_C, {"kind": "dense", "ff": 50, "limit": 1.5}, 0.9, 0.7),
    _layer(LEFT_C, RIGHT_C, {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 10}}, 0.6, 1.2),
]}
SEEDS = {"nip_a": 3, "nip_b": 4, "nip_c": 5}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write_model(folder: str, cfg: dict, seed: int, scale_up: float = 8.0) -> str:
    """A model folder with random weights through the library's own random-weights mode, the matrices
    scaled up so that attention and the recurrence matter in the logits."""
    import torch

    import ember_cpp_b200 as E
    from ember_cpp_b200.weights import read_folder, write_file
    E.write_random_model(folder, E.config.config_from_dict(cfg), seed)
    tensors = {name: t.clone() for name, t in read_folder(folder).items()}     # (the file is mapped: copies, then rewrite)
    for name, t in tensors.items():
        if t.dtype.is_floating_point and t.dim() == 2 and not name.endswith(".conv"):
            tensors[name] = (t.float() * (2.0 if name in ("embed", "head") else scale_up)).to(torch.bfloat16)
    write_file(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder


def ids(seed: int, vocab: int, n: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def row_error(got, ref) -> float:
    """Worst row of rms(delta - mean(delta)) / rms(ref - mean(ref))."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got[None], ref[None]
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))).max())


# of a row's spread (see row_error).  bfloat16: these models' weights are scaled up so that every mechanism shows in
# the logits, which also lets the roundings of activations through: the engine is within this of the exact rows
TOL = {"float32": 2e-5, "bfloat16": 8e-2}
