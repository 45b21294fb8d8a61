"""A plain, slow implementation of the Kofutar design: numpy, one function a mechanism, whole
sequences at once (no cache, no batch), in the precision of the arrays it is given (tests pass
float64). It shares nothing with the package: the tests compare the engine with it.

A model is (config, tensors): config.json's dict and {name: array}. Notation: T tokens, W the
model's width, H heads, G key/value heads, d the query/key size of a head, e its value size.
"""
from __future__ import annotations

import math

import numpy as np


# ---------------------------------------------------------------------------------------- small pieces
def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean squared deviation."""
    c = x - x.mean(axis=-1, keepdims=True)
    return c / np.sqrt(np.mean(c * c, axis=-1, keepdims=True) + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, positions, rot):
    """x [T, n, d]: the first rot["dims"] components of every vector are turned pairwise, component
    i with i + dims/2, by the angle position * base^(-2i/dims) / factor; the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    freq = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(half)]) / factor
    a = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]          # [T, half]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = np.array(x, copy=True)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_softmax(scores, sink=None):
    """scores [T, T] -> weights; row i sees columns 0..i. With `sink`, e^sink joins the denominator
    (a column without a value)."""
    T = scores.shape[0]
    out = np.zeros_like(scores)
    for i in range(T):
        row = scores[i, : i + 1]
        top = row.max() if sink is None else max(row.max(), sink)
        p = np.exp(row - top)
        total = p.sum() + (0.0 if sink is None else math.exp(sink - top))
        out[i, : i + 1] = p / total
    return out


# ---------------------------------------------------------------------------------------- mixers
def attention_mixer(h, t, prefix, m, eps):
    """Grouped queries; every head's query and key is RMS-normed with a weight shared by the heads,
    then rotated; softmax over the keys up to the row's own."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = np.arange(T)
    q = (h @ t[f"{prefix}.q"].T).reshape(T, H, d)
    k = (h @ t[f"{prefix}.k"].T).reshape(T, G, d)
    v = (h @ t[f"{prefix}.v"].T).reshape(T, G, e)
    q = rms_unit(q, eps) * t[f"{prefix}.q.norm"]
    k = rms_unit(k, eps) * t[f"{prefix}.k.norm"]
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    out = np.zeros((T, H, e), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        w = causal_softmax((q[:, a] @ k[:, g].T) * m["scale"])
        out[:, a] = w @ v[:, g]
    return out.reshape(T, H * e) @ t[f"{prefix}.o"].T


def latent_attention_mixer(h, t, prefix, m, eps):
    """Queries and keys/values through low-rank latents; one rotated key part for all heads; a sink in
    the softmax's denominator; a sigmoid gate on the heads' outputs."""
    H, d, r, e, kv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = np.arange(T)
    rot = dict(m["rot"])
    rot["dims"] = r
    cq = rms_unit(h @ t[f"{prefix}.dq"].T, eps) * t[f"{prefix}.dq.norm"]
    q = (cq @ t[f"{prefix}.uq"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, rot)
    down = h @ t[f"{prefix}.dkv"].T
    c = rms_unit(down[:, :kv], eps) * t[f"{prefix}.dkv.norm"]
    k_rot = rotate(down[:, None, kv:], pos, rot)[:, 0]                              # [T, r]
    k_plain = (c @ t[f"{prefix}.uk"].T).reshape(T, H, d)
    v = (c @ t[f"{prefix}.uv"].T).reshape(T, H, e)
    out = np.zeros((T, H, e), dtype=h.dtype)
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = causal_softmax(s, float(t[f"{prefix}.sink"][a])) @ v[:, a]
    gate = sigmoid(h @ t[f"{prefix}.g"].T)
    return (out.reshape(T, H * e) * gate) @ t[f"{prefix}.o"].T


def short_conv(x, w):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c] with zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        y[j:] += x[: T - j] * w[:, taps - 1 - j]
    return y


def delta_recurrence(q, k, v, g, beta):
    """One head. q, k [T, d], v [T, e], g, beta [T]: per row S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q, so the read-out sees the row's own write. Returns o [T, e]."""
    T, d = k.shape
    S = np.zeros((d, v.shape[1]), dtype=v.dtype)
    out = np.zeros_like(v)
    for i in range(T):
        S = g[i] * S
        u = beta[i] * (v[i] - S.T @ k[i])
        S = S + np.outer(k[i], u)
        out[i] = S.T @ q[i]
    return out


def unit(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + eps)


def delta_inputs(x, conv, a_log, dt_bias, H, G, d, e):
    """From the stacked projections x [T, 2 G d + H e + 2 H] (q | k | v | b | a) and the filters
    conv [2 G d + H e, taps]: unit q (times d^-1/2) and k [T, G, d], v [T, H, e], decay and step size [T, H]."""
    T = x.shape[0]
    n = G * d
    y = silu(short_conv(x[:, : 2 * n + H * e], conv))
    q = unit(y[:, :n].reshape(T, G, d)) * d ** -0.5
    k = unit(y[:, n : 2 * n].reshape(T, G, d))
    v = y[:, 2 * n :].reshape(T, H, e)
    beta = sigmoid(x[:, 2 * n + H * e : 2 * n + H * e + H])
    g = np.exp(-np.exp(a_log) * softplus(x[:, 2 * n + H * e + H :] + dt_bias))
    return q, k, v, g, beta


def delta_mixer(h, t, prefix, m, eps):
    """The gated delta rule behind short convolutions; each head's read-out is divided by its root mean
    square, times a weight shared by the heads, times silu of a gate."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    x = np.concatenate([h @ t[f"{prefix}.{r}"].T for r in ("q", "k", "v", "b", "a")], axis=1)
    conv = np.concatenate([t[f"{prefix}.{r}.conv"] for r in ("q", "k", "v")], axis=0)
    q, k, v, g, beta = delta_inputs(x, conv, t[f"{prefix}.A_log"], t[f"{prefix}.dt_bias"], H, G, d, e)
    out = np.stack([delta_recurrence(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], g[:, a], beta[:, a]) for a in range(H)], axis=1)
    out = rms_unit(out, eps) * t[f"{prefix}.norm"]
    gate = silu(h @ t[f"{prefix}.g"].T).reshape(T, H, e)
    return (out * gate).reshape(T, H * e) @ t[f"{prefix}.o"].T


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer, "delta": delta_mixer}


def dense_ffn(h, t, prefix):
    return (gelu_tanh(h @ t[f"{prefix}.gate"].T) * (h @ t[f"{prefix}.up"].T)) @ t[f"{prefix}.down"].T


# ---------------------------------------------------------------------------------------- the model
def layer_runs(config):
    """The layers in the order they run: [(layer, first of a pass?)]. The layers start..stop-1 of
    `loop` run `times` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for _ in range(times):
        runs += [(i, i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(config, t, tokens, residuals=None):
    """Logits [T, vocab] of a whole sequence; `residuals`, a list, receives the stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x = t["embed"][np.asarray(tokens)]
    x0 = x
    for i, opens in layer_runs(config):
        if opens:
            x = np.concatenate([x, x0], axis=-1) @ t["loop.in"].T
        rec, p = config["layers"][i], f"l{i}"
        a = MIXERS[rec["type"]](layer_norm(x, t[f"{p}.norm1"], eps), t, f"{p}.mix", rec["mixer"], eps)
        x = x + layer_norm(a, t[f"{p}.norm1b"], eps)
        if rec.get("mlp") is not None:
            f = dense_ffn(layer_norm(x, t[f"{p}.norm2"], eps), t, f"{p}.mlp")
            x = x + layer_norm(f, t[f"{p}.norm2b"], eps)
        if residuals is not None:
            residuals.append(x)
    return layer_norm(x, t["final.norm"], eps) @ t["head"].T
