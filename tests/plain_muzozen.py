"""Plain Muzozen: whole sequences, no cache, no state carried between calls, one function for each
mechanism.

Muzozen is a decoder whose embedding adds a row chosen by the (previous token, token) pair to the
token's row and norms the sum; whose layers read one RMS norm and add a mixer and a feed-forward
that both take its output; and whose mixers are a gated delta-rule recurrence or an attention
whose keys and values are expanded from a cached low-rank row, with a rotated key part shared by
the heads, a YaRN-scaled rotation, and layers that read another layer's cached rows.

Nothing here is shared with the engine: own safetensors reader, own arithmetic (numpy, float64),
loops over tokens where the definition is a recurrence.  It is the exact value that the engine's
float32 and bfloat16 paths approximate.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------------- model folder
def read_safetensors(path: str) -> dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        kind = meta["dtype"].upper()
        if kind == "BF16":
            a = (np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif kind == "F32":
            a = np.frombuffer(data[b:e], dtype="<f4").astype(np.float64)
        elif kind == "I32":
            a = np.frombuffer(data[b:e], dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"plain reader: dtype {kind} of {name}")
        out[name] = a.reshape(meta["shape"])
    return out


class PlainMuzozen:
    def __init__(self, folder: str | None = None, cfg: dict | None = None, weights: dict | None = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                cfg = json.load(f)
            weights = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.w = cfg, {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}


# --------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


# --------------------------------------------------------------------------- embedding
def pair_rows(tokens, buckets: int, mul_prev: int, mul_cur: int) -> list:
    """The row of the pair table for every token: the extra last row for a sequence's first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (int(tokens[i - 1]) * mul_prev + int(t) * mul_cur) % buckets)
    return rows


def embed(m: PlainMuzozen, tokens) -> np.ndarray:
    e = m.cfg["embedding"]
    x = m.w["embed"][np.asarray(tokens)] * e["scale"]
    b = e.get("bigram")
    if b:
        x = x + m.w["bigram"][pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])]
    return rms_norm(x, m.w["embed.norm"], m.cfg["norm"]["eps"])


# --------------------------------------------------------------------------- rotation
def rotation_tables(rot: dict, n_positions: int):
    """cos and sin [positions, dims / 2] of the rotation, with YaRN's blend of stretched and original
    frequencies and its factor on both tables where the configuration asks for scaling."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    mag = 1.0
    s = rot.get("scaling")
    if s:
        def at(turns):
            return dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(at(s["fast"])), 0)
        hi = min(math.ceil(at(s["slow"])), dims - 1)
        ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / s["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(s["factor"]) + 1.0
    a = np.arange(n_positions)[:, None] * f[None, :]
    return np.cos(a) * mag, np.sin(a) * mag


def rotate(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dims: int) -> np.ndarray:
    """x [T, ..., n]: the first `dims` of the last axis are rotated, dimension i paired with i + dims / 2."""
    half = dims // 2
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = cos[:x.shape[0]].reshape(shape), sin[:x.shape[0]].reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., dims:]], axis=-1)


# --------------------------------------------------------------------------- attention over a low-rank row
def latent_rows(m: PlainMuzozen, p: str, mx: dict, h: np.ndarray):
    """What a layer with a down projection of its own caches: the normed low-rank row and the rotated key part."""
    eps = m.cfg["norm"]["eps"]
    down = h @ m.w[p + "dkv"].T
    c = rms_norm(down[:, :mx["kv_rank"]], m.w[p + "dkv.norm"], eps)
    cos, sin = rotation_tables(mx["rot"], h.shape[0])
    return c, rotate(down[:, mx["kv_rank"]:], cos, sin, mx["rot"]["dims"])


def latent_attention(m: PlainMuzozen, p: str, mx: dict, h: np.ndarray, c: np.ndarray, k_rot: np.ndarray) -> np.ndarray:
    T, H, d, r, vd = h.shape[0], mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    eps = m.cfg["norm"]["eps"]
    q = (rms_norm(h @ m.w[p + "dq"].T, m.w[p + "dq.norm"], eps) @ m.w[p + "uq"].T).reshape(T, H, d + r)
    cos, sin = rotation_tables(mx["rot"], T)
    q_rot = rotate(q[..., d:], cos, sin, mx["rot"]["dims"])
    k = (c @ m.w[p + "uk"].T).reshape(T, H, d)
    v = (c @ m.w[p + "uv"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    for i in range(T):
        for hd in range(H):
            s = (k[:i + 1, hd] @ q[i, hd, :d] + k_rot[:i + 1] @ q_rot[i, hd]) * mx["scale"]
            w = np.exp(s - s.max())
            out[i, hd] = (w / w.sum()) @ v[:i + 1, hd]
    return out.reshape(T, H * vd) @ m.w[p + "o"].T


# --------------------------------------------------------------------------- gated delta rule
def causal_conv_silu(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """x [T, channels], w [channels, taps] with the last tap on the current token; zeros before the start."""
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x])
    y = sum(padded[j:j + x.shape[0]] * w[:, j] for j in range(taps))
    return silu(y)


def unit(x: np.ndarray) -> np.ndarray:
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


def delta_recurrence(q, k, v, beta, decay):
    """q, k [T, dim], v [T, vdim], beta and decay [T] of one head; the state starts at zero."""
    S = np.zeros((q.shape[1], v.shape[1]))
    out = np.zeros_like(v)
    for t in range(q.shape[0]):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(m: PlainMuzozen, p: str, mx: dict, h: np.ndarray) -> np.ndarray:
    T, H, KV, d, vd = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    w = m.w
    q = unit(causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, KV, d)) * d ** -0.5
    k = unit(causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, KV, d))
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(T, H, vd)
    beta = sigmoid(h @ w[p + "b"].T)
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    for hd in range(H):
        j = hd // (H // KV)
        o = delta_recurrence(q[:, j], k[:, j], v[:, hd], beta[:, hd], decay[:, hd])
        out[:, hd] = o / np.sqrt((o * o).mean(-1, keepdims=True) + m.cfg["norm"]["eps"]) * w[p + "norm"] * gate[:, hd]
    return out.reshape(T, H * vd) @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forward, layers, model
def dense_ffn(m: PlainMuzozen, p: str, h: np.ndarray) -> np.ndarray:
    return gelu_tanh(h @ m.w[p + "up"].T) @ m.w[p + "down"].T


def forward(m: PlainMuzozen, tokens, return_layers: bool = False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer)."""
    eps = m.cfg["norm"]["eps"]
    x = embed(m, tokens)
    cached, streams = {}, []
    for i, layer in enumerate(m.cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = rms_norm(x, m.w[p + "norm1"], eps)
        if layer["type"] == "delta":
            y = delta_mixer(m, p + "mix.", mx, h)
        elif layer["type"] == "latent_attention":
            src = mx.get("kv_from")
            if src is None:
                cached[i] = latent_rows(m, p + "mix.", mx, h)
                src = i
            y = latent_attention(m, p + "mix.", mx, h, *cached[src])
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + dense_ffn(m, p + "mlp.", h)
        x = x + y
        streams.append(x)
    logits = rms_norm(x, m.w["final.norm"], eps) @ m.w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits


def generate(m: PlainMuzozen, prompt, steps: int) -> list:
    """Greedy: the first largest logit, the whole sequence run again for every token."""
    seq = list(prompt)
    for _ in range(steps):
        seq.append(int(np.argmax(forward(m, seq)[-1])))
    return seq[len(prompt):]
