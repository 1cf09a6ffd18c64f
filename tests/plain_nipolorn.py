"""Plain Nipolorn: whole sequences, no cache, no state carried between calls, one function for
each mechanism.

Nipolorn is a decoder whose layers wrap every sublayer in two RMS norms (one before, one after) and
whose mixer runs a sliding-window attention with kept first tokens beside a Mamba-2 recurrence, both
on the same input, their outputs added with two fixed factors.  Its feed-forwards are a clamped
gated layer or a set of small experts picked by a table indexed with the token id.

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
        elif kind == "I64":
            a = np.frombuffer(data[b:e], dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"plain reader: dtype {kind} of {name}")
        out[name] = a.reshape(meta["shape"])
    return out


class PlainNipolorn:
    def __init__(self, folder: str | None = None, cfg: dict | None = None, weights: dict | None = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                cfg = json.load(f)
            weights = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.w = cfg, weights


# --------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """Rows divided by sqrt(mean of squares + eps)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def offset_rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The model's norm: the gain is stored as its distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


# --------------------------------------------------------------------------- attention with window and kept first tokens
def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (i - j < window or j < keep_first)


def windowed_attention(h, wq, wk, wv, wo, heads, kv_heads, dim, vdim, scale, window, keep_first):
    """h [T, width] -> [T, width].  No rotation; one softmax over the visible keys of each query."""
    T = h.shape[0]
    q = (h @ wq.T).reshape(T, heads, dim)
    k = (h @ wk.T).reshape(T, kv_heads, dim)
    v = (h @ wv.T).reshape(T, kv_heads, vdim)
    per = heads // kv_heads
    out = np.zeros((T, heads, vdim))
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        for a in range(heads):
            g = a // per
            s = np.array([q[i, a] @ k[j, g] for j in js]) * scale
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, a] = sum(pj * v[j, g] for pj, j in zip(p, js))
    return out.reshape(T, heads * vdim) @ wo.T


# --------------------------------------------------------------------------- Mamba-2
def causal_conv_silu(u, taps_w, bias):
    """u [T, C]; taps_w [C, taps], the last column multiplies the current token; zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        acc = bias.copy()
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                acc = acc + taps_w[:, j] * u[src]
        out[t] = silu(acc)
    return out


def ssd_recurrence(x, B, C, dt, A_log, D, heads, vdim, groups, state):
    """x [T, heads*vdim], B, C [T, groups*state], dt [T, heads] (already positive).  Token by token:
    S <- exp(-exp(A_log) dt) S + dt B x^T (S: state x vdim), y = S^T C + D x."""
    T = x.shape[0]
    per = heads // groups
    y = np.zeros((T, heads, vdim))
    for a in range(heads):
        g = a // per
        S = np.zeros((state, vdim))
        for t in range(T):
            xt = x[t, a * vdim:(a + 1) * vdim]
            Bt, Ct = B[t, g * state:(g + 1) * state], C[t, g * state:(g + 1) * state]
            S = math.exp(-math.exp(A_log[a]) * dt[t, a]) * S + dt[t, a] * np.outer(Bt, xt)
            y[t, a] = S.T @ Ct + D[a] * xt
    return y.reshape(T, heads * vdim)


def gated_group_norm(y, z, w, parts, eps):
    """The gate first, then each of `parts` equal pieces of a row by its own root mean square."""
    g = y * silu(z)
    T, n = g.shape
    g = rms_unit(g.reshape(T, parts, n // parts), eps).reshape(T, n)
    return g * w


def mamba2(h, w_in, conv_w, conv_b, dt_bias, A_log, D, norm_w, w_o, heads, vdim, groups, state, norm_groups, eps):
    inner, gn = heads * vdim, groups * state
    proj = h @ w_in.T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * gn], proj[:, 2 * inner + 2 * gn:]
    xbc = causal_conv_silu(xbc, conv_w, conv_b)
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:]
    dt = softplus(dt + dt_bias)
    y = ssd_recurrence(x, B, C, dt, A_log, D, heads, vdim, groups, state)
    return gated_group_norm(y, z, norm_w, norm_groups, eps) @ w_o.T


# --------------------------------------------------------------------------- feed-forwards
def clamped_gated(h, w_gate, w_up, w_down, limit):
    g = np.minimum(h @ w_gate.T, limit)
    u = np.clip(h @ w_up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def silu_gated(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def table_experts(h, ids, table, experts, shared):
    """experts: list of (gate, up, down); table [vocab, top]; each chosen expert weighs 1/top."""
    top = table.shape[1]
    out = np.zeros((h.shape[0], experts[0][2].shape[0]))
    for t, tok in enumerate(ids):
        for e in table[tok]:
            out[t] += silu_gated(h[t:t + 1], *experts[int(e)])[0] / top
    if shared is not None:
        out += silu_gated(h, *shared)
    return out


# --------------------------------------------------------------------------- the model
def mixer(m: PlainNipolorn, i: int, h):
    c, w, p = m.cfg["layers"][i]["mixer"], m.w, f"l{i}.mix."
    eps = m.cfg["norm"]["eps"]
    a, r = c["left"], c["right"]
    left = windowed_attention(h, w[p + "left.q"], w[p + "left.k"], w[p + "left.v"], w[p + "left.o"], a["heads"],
                              a["kv_heads"], a["dim"], a["vdim"], a["scale"], a["mask"]["size"], a["mask"]["keep_first"])
    right = mamba2(h, w[p + "right.in"], w[p + "right.conv"], w[p + "right.conv.b"], w[p + "right.dt_bias"],
                   w[p + "right.A_log"], w[p + "right.D"], w[p + "right.norm"], w[p + "right.o"], r["heads"], r["vdim"],
                   r["groups"], r["state"], r["norm_groups"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def feed_forward(m: PlainNipolorn, i: int, h, ids):
    c, w, p = m.cfg["layers"][i]["mlp"], m.w, f"l{i}.mlp."
    if c["kind"] == "dense":
        return clamped_gated(h, w[p + "gate"], w[p + "up"], w[p + "down"], c["limit"])
    experts = [(w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"]) for e in range(c["router"]["experts"])]
    shared = (w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"]) if c.get("shared") else None
    return table_experts(h, ids, w[p + "table"], experts, shared)


def layer(m: PlainNipolorn, i: int, x, ids):
    w, eps, p = m.w, m.cfg["norm"]["eps"], f"l{i}."
    x = x + offset_rms_norm(mixer(m, i, offset_rms_norm(x, w[p + "norm1"], eps)), w[p + "norm1b"], eps)
    if m.cfg["layers"][i].get("mlp"):
        x = x + offset_rms_norm(feed_forward(m, i, offset_rms_norm(x, w[p + "norm2"], eps), ids), w[p + "norm2b"], eps)
    return x


def forward(m: PlainNipolorn, ids, streams: list | None = None) -> np.ndarray:
    """Logits [T, vocab] of a whole sequence; `streams` collects the residual stream after each layer."""
    x = m.w["embed"][np.asarray(ids)]
    for i in range(len(m.cfg["layers"])):
        x = layer(m, i, x, ids)
        if streams is not None:
            streams.append(x.copy())
    return offset_rms_norm(x, m.w["final.norm"], m.cfg["norm"]["eps"]) @ m.w["head"].T


def generate(m: PlainNipolorn, prompt, n_new: int) -> list[int]:
    """Greedy: the first largest logit of the last position, the whole sequence run anew each time."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(m, ids)[-1])))
    return ids[len(prompt):]
