"""Small Muzozen configurations and helpers shared by the CPU and GPU tests.

The configurations differ from one another in every size and option: the pair table's constants
(one model has no pair table), an embedding factor of 2 / 1 / 0.5; attention over cached rows with
and without YaRN scaling, with all or only some of the shared key part's dimensions rotated, with
layers that read an earlier layer's rows (directly after it, and with layers in between); the
delta rule with grouped and ungrouped heads, one head, convolutions of 4, 2, 3 and 1 taps; layers
without a feed-forward; a delta layer first or an attention first; and one model whose sizes are
no multiples of 8 anywhere.
"""
import copy
import json
import os

import numpy as np


def _rot(dims, base, scaling=None):
    return {"dims": dims, "base": base, "scaling": scaling}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, kv_from=None, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


YARN_A = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
YARN_B = {"factor": 2.5, "original": 40, "fast": 6.0, "slow": 0.5}
ROT_A, ROT_B, ROT_C = _rot(16, 10000.0, YARN_A), _rot(8, 500.0, None), _rot(6, 2000.0, YARN_B)

CONFIGS = {
    "muz_a": {"architecture": "Muzozen", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
              "embedding": {"scale": 2.0, "bigram": {"buckets": 211, "mul_prev": 31, "mul_cur": 7}}, "layers": [
        _latent(4, 16, 16, 24, 24, 32, 0.2, ROT_A, ff=96),
        _delta(4, 2, 16, 8, 4, ff=96),
        _latent(4, 16, 16, 24, 24, 32, 0.2, ROT_A, kv_from=0),
        _delta(2, 2, 32, 16, 2, ff=40),
        _latent(2, 8, 16, 8, 8, 16, 0.3, ROT_B, ff=72),          # eight of the key part's sixteen dimensions are rotated
        _latent(3, 32, 16, 16, 40, 16, 0.15, ROT_B, kv_from=4, ff=72),
        _latent(4, 8, 16, 40, 16, 32, 0.25, ROT_A, kv_from=0, ff=24),
    ]},
    "muz_b": {"architecture": "Muzozen", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
              "embedding": {"scale": 1.0, "bigram": {"buckets": 64, "mul_prev": 5, "mul_cur": 1}}, "layers": [
        _delta(1, 1, 48, 40, 1, ff=160),
        _latent(1, 48, 32, 48, 16, 64, 0.1, _rot(32, 1e6, YARN_A), ff=160),
        _delta(6, 3, 24, 16, 3),
        _latent(5, 16, 32, 24, 48, 64, 0.12, _rot(32, 1e6, YARN_A), kv_from=1, ff=64),
    ]},
    # sizes that are no multiples of 8 anywhere: rows that are no whole 16-byte pieces in bfloat16; no pair table
    "muz_c": {"architecture": "Muzozen", "vocab": 101, "width": 60, "norm": {"eps": 1e-5},
              "embedding": {"scale": 0.5}, "layers": [
        _latent(3, 12, 6, 10, 14, 20, 0.25, ROT_C, ff=50),
        _delta(3, 1, 12, 6, 3, ff=50),
        _latent(2, 10, 6, 14, 6, 20, 0.3, ROT_C, kv_from=0),
    ]},
}
# odd sizes everywhere, only delta-rule layers in front of one attention layer that nothing shares, a key part of two values
CONFIGS["muz_d"] = {"architecture": "Muzozen", "vocab": 77, "width": 36, "norm": {"eps": 1e-6},
                    "embedding": {"scale": 3.0, "bigram": {"buckets": 13, "mul_prev": 100003, "mul_cur": 99991}}, "layers": [
    _delta(5, 5, 7, 3, 5, ff=27),
    _delta(2, 1, 130, 9, 2),
    _latent(5, 3, 2, 7, 5, 9, 0.4, _rot(2, 37.0, {"factor": 1.5, "original": 16, "fast": 4.0, "slow": 1.0}), ff=11),
]}
# only attention layers (no state besides the pair table's), every later one reading the first one's rows
CONFIGS["muz_e"] = {"architecture": "Muzozen", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
                    "embedding": {"scale": 1.0, "bigram": {"buckets": 5, "mul_prev": 1, "mul_cur": 1}}, "layers": [
    _latent(2, 16, 16, 16, 16, 32, 0.2, ROT_A, ff=48),
    _latent(4, 8, 16, 8, 8, 32, 0.2, ROT_A, kv_from=0),
    _latent(1, 32, 16, 32, 24, 32, 0.1, ROT_A, kv_from=0, ff=16),
]}
SEEDS = {"muz_a": 11, "muz_b": 12, "muz_c": 13, "muz_d": 14, "muz_e": 15}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write_model(folder: str, cfg: dict, seed: int, scale_up: float = 6.0) -> str:
    """A model folder with random weights through the library's own random-weights mode, the matrices
    scaled up so that attention and the recurrence matter in the logits."""
    import torch

    import ember_cpp_b200 as E
    from ember_cpp_b200.weights import read_folder, write_file
    E.write_random_model(folder, E.config.config_from_dict(cfg), seed)
    tensors = {name: t.clone() for name, t in read_folder(folder).items()}     # (the file is mapped: copies, then rewrite)
    for name, t in tensors.items():
        if t.dtype.is_floating_point and t.dim() == 2 and not name.endswith(".conv"):
            tensors[name] = (t.float() * (2.0 if name in ("embed", "head", "bigram") else scale_up)).to(torch.bfloat16)
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
TOL = {"float32": 3e-5, "bfloat16": 8e-2}
