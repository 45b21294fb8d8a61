"""A plain, slow implementation of the Fusitar design: numpy, one function a mechanism, whole
sequences at once (no cache, no batch), in the precision of the arrays it is given (tests pass
float64). It shares nothing with the package: the tests compare the engine with it.

A model is (config, tensors): config.json's dict and {name: array}. Notation: T tokens, W the
model's width, H heads, G key/value heads, d the query/key size of a head, e its value size.
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def embed(table, tokens, scale):
    return table[np.asarray(tokens)] * scale


# ---------------------------------------------------------------------------------------- attention
def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def attention_scores(q, k, scale, size, keep_first):
    """Softmax weights [T, T] of one head: q [T, d], k [T, d]."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    for i in range(T):
        for j in range(T):
            if not visible(i, j, size, keep_first):
                s[i, j] = -np.inf
    s = s - s.max(axis=1, keepdims=True)
    p = np.exp(s)
    return p / p.sum(axis=1, keepdims=True)


def attention_mixer(h, t, prefix, m, eps):
    """h [T, W] -> [T, W]; `m` is the layer's mixer record, `t` the tensors, `prefix` "l<i>.mix"."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ t[f"{prefix}.q"].T
    k = h @ t[f"{prefix}.k"].T
    v = h @ t[f"{prefix}.v"].T
    q = rms_norm(q, t[f"{prefix}.q.norm"], eps)            # over all heads' rows at once
    k = rms_norm(k, t[f"{prefix}.k.norm"], eps)
    q = q.reshape(T, H, d)
    k = k.reshape(T, G, d)
    v = v.reshape(T, G, e)
    out = np.zeros((T, H, e), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        p = attention_scores(q[:, head], k[:, g], m["scale"], m["mask"]["size"], m["mask"]["keep_first"])
        out[:, head] = p @ v[:, g]
    y = out.reshape(T, H * e) * sigmoid(h @ t[f"{prefix}.g"].T)
    return y @ t[f"{prefix}.o"].T


# -------------------------------------------------------------------------------------------- mLSTM
def mlstm_gates(h, t, prefix, cap):
    """(log input gate, log forget gate), each [T, H]."""
    zi = h @ t[f"{prefix}.i"].T + t[f"{prefix}.i.b"]
    zf = h @ t[f"{prefix}.f"].T + t[f"{prefix}.f.b"]
    return cap * np.tanh(zi / cap), log_sigmoid(cap * np.tanh(zf / cap))


def mlstm_recurrence(q, k, v, gi, gf):
    """One head, token by token: q, k [T, d], v [T, e], gi, gf [T] -> o [T, e]. The matrix
    memory S [d, e], the normaliser n [d] and the running maximum m all start at zero."""
    T, d = q.shape
    e = v.shape[1]
    S = np.zeros((d, e), dtype=q.dtype)
    n = np.zeros((d,), dtype=q.dtype)
    m = 0.0
    o = np.zeros((T, e), dtype=q.dtype)
    for s in range(T):
        m_new = max(gf[s] + m, gi[s])
        a = math.exp(gf[s] + m - m_new)
        b = math.exp(gi[s] - m_new)
        S = a * S + b * np.outer(k[s], v[s])
        n = a * n + b * k[s]
        m = m_new
        o[s] = (S.T @ q[s]) / (max(abs(float(n @ q[s])), math.exp(-m)) + 1e-6)
    return o


def mlstm_mixer(h, t, prefix, m, eps):
    H, d, e = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t[f"{prefix}.q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ t[f"{prefix}.k"].T).reshape(T, H, d)
    v = (h @ t[f"{prefix}.v"].T).reshape(T, H, e)
    gi, gf = mlstm_gates(h, t, prefix, m["gate_cap"])
    o = np.zeros((T, H, e), dtype=h.dtype)
    for head in range(H):
        o[:, head] = rms_unit(mlstm_recurrence(q[:, head], k[:, head], v[:, head], gi[:, head], gf[:, head]), eps)
    y = o.reshape(T, H * e) * t[f"{prefix}.norm"] * sigmoid(h @ t[f"{prefix}.g"].T)
    return y @ t[f"{prefix}.o"].T


# -------------------------------------------------------------------------------- mixture of experts
def route(z, correction, top, groups, keep):
    """Router logits z [E] of one token -> (chosen experts, their weights)."""
    s = sigmoid(z)
    choice = s + correction
    E = z.shape[0]
    per = E // groups
    group_score = []
    for g in range(groups):
        part = np.sort(choice[g * per : (g + 1) * per])[::-1]
        group_score.append(part[:2].sum())
    order = sorted(range(groups), key=lambda g: (-group_score[g], g))
    allowed = set(order[:keep])
    masked = np.array([choice[x] if (x // per) in allowed else -np.inf for x in range(E)])
    chosen = sorted(range(E), key=lambda x: (-masked[x], x))[:top]
    return chosen, [s[x] for x in chosen]


def moe(h, t, prefix, mlp):
    r = mlp["router"]
    z = h @ t[f"{prefix}.router"].T
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        chosen, weights = route(z[i], t[f"{prefix}.correction"], r["top"], r["groups"]["count"], r["groups"]["keep"])
        for x, w in zip(chosen, weights):
            a = np.maximum(t[f"{prefix}.e{x}.up"] @ h[i], 0.0) ** 2
            out[i] += w * (t[f"{prefix}.e{x}.down"] @ a)
    return out


# --------------------------------------------------------------------------------------------- model
MIXERS = {"attention": attention_mixer, "mlstm": mlstm_mixer}


def forward(config, t, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence; with `return_layers` also the residual after every layer."""
    eps = config["norm"]["eps"]
    x = embed(t["embed"], tokens, config["embedding"]["scale"])
    after = []
    for i, layer in enumerate(config["layers"]):
        a = MIXERS[layer["type"]](x, t, f"l{i}.mix", layer["mixer"], eps)
        x = x + rms_norm(a, t[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            f = moe(x, t, f"l{i}.mlp", layer["mlp"])
            x = x + rms_norm(f, t[f"l{i}.norm2"], eps)
        after.append(x.copy())
    logits = rms_norm(x, t["final.norm"], eps) @ t["embed"].T
    return (logits, np.stack(after)) if return_layers else logits
