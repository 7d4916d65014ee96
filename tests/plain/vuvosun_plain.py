"""A plain, slow implementation of the Vuvosun design in numpy float64: one function per mechanism, one token after the
other wherever the design has a recurrence.  It shares no code with the package and is what the tests compare it with.

A model is (config dict, {tensor name: float64 array}).  ``forward`` runs one sequence from its first token and returns the
logits of every position and the residual stream (the sum of the streams) after every layer.
"""
from __future__ import annotations

import math

import numpy as np


def rms_div(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -np.logaddexp(0.0, -z)


def rotate_adjacent(x, positions, dims, base):
    """x [T, heads, dim]: dimension 2i turns with 2i + 1 by positions * base^(-2i/dims), for the first ``dims`` dimensions."""
    out = x.copy()
    for i in range(dims // 2):
        ang = positions * (base ** (-2.0 * i / dims))
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def sees(i, j, size, keep_first):
    """Does position i see position j: the causal window of ``size`` keys (None: all) and the first ``keep_first`` tokens."""
    return j <= i and (size is None or i - j < size or j < keep_first)


def windowed_sink_attention(h, w, m, eps):
    """The softmax mixer: grouped queries, rotation, value norm, window with kept first tokens, sink, output gate."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, dk)
    k = (h @ w["k"].T).reshape(T, G, dk)
    v = (h @ w["v"].T).reshape(T, G, dv)
    pos = np.arange(T, dtype=np.float64)
    mask = m.get("mask") or {}
    q = rotate_adjacent(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_adjacent(k, pos, m["rot"]["dims"], m["rot"]["base"])
    v = rms_div(v, eps)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if sees(i, j, mask.get("size"), mask.get("keep_first", 0))]
            s = np.array([q[i, hh] @ k[j, g] for j in js]) * m["scale"]
            top = max(s.max(), w["sink"][hh])
            e = np.exp(s - top)
            out[i, hh] = (e[:, None] * v[js, g]).sum(0) / (e.sum() + math.exp(w["sink"][hh] - top))
    gate = sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * dv) * gate) @ w["o"].T


def short_conv(x, taps):
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, j] x_(t - n + 1 + j), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, x.shape[1])), x], axis=0)
    return sum(padded[j:j + T] * taps[:, j] for j in range(n))


def gated_delta(h, w, m, eps):
    """The delta-rule mixer: short convolutions, unit keys and queries, a decay and a write strength per head."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)
    decay = np.exp(-np.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    o = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    o = rms_div(o, eps) * w["norm"]
    gate = silu(h @ w["g"].T).reshape(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ w["o"].T


def mlstm(h, w, m, eps):
    """The matrix memory with exponential gates and a running maximum that starts at zero."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = logsigmoid(cap * np.tanh((h @ w["f"].T + w["f.b"]) / cap))
    o = np.zeros((T, H, dv))
    for hh in range(H):
        S, n, mx = np.zeros((dk, dv)), np.zeros(dk), 0.0
        for t in range(T):
            new = max(gf[t, hh] + mx, gi[t, hh])
            keep, add = math.exp(gf[t, hh] + mx - new), math.exp(gi[t, hh] - new)
            S = keep * S + add * np.outer(k[t, hh], v[t, hh])
            n = keep * n + add * k[t, hh]
            mx = new
            o[t, hh] = S.T @ q[t, hh] / (max(abs(n @ q[t, hh]), math.exp(-mx)) + 1e-6)
    o = rms_div(o, eps).reshape(T, H * dv) * w["norm"]
    return (o * sigmoid(h @ w["g"].T)) @ w["o"].T


def polynorm_ff(h, w, eps):
    z = h @ w["up"].T
    a, b, c, e = w["act"]
    return (a * rms_div(z, eps) + b * rms_div(z ** 2, eps) + c * rms_div(z ** 3, eps) + e) @ w["down"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def mixer(kind, h, w, m, eps):
    if kind == "mlstm":
        return mlstm(h, w, m, eps)
    if kind == "parallel":
        left = windowed_sink_attention(h, sub(w, "left."), m["left"], eps)
        right = gated_delta(h, sub(w, "right."), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    raise ValueError(kind)


def hyper_step(streams, hc, run, norm_w, eps):
    """One sublayer over the streams [s, T, W]: read a blend, run, mix the streams and write the result into each."""
    u = np.einsum("s,stw->tw", hc["in"], streams)
    y = run(rms_div(u, eps) * norm_w)
    return np.einsum("sr,stw->rtw", hc["mix"], streams) + hc["out"][:, None, None] * y[None]


def forward(config, tensors, tokens):
    eps = config["norm"]["eps"]
    x = tensors["embed"][np.asarray(tokens)]
    x = rms_div(x, eps) * tensors["embed.norm"]
    streams = np.stack([x] * config["streams"])
    after = []
    for i, layer in enumerate(config["layers"]):
        w = sub(tensors, f"l{i}.")
        streams = hyper_step(streams, sub(w, "hc1."), lambda hh: mixer(layer["type"], hh, sub(w, "mix."), layer["mixer"], eps), w["norm1"], eps)
        if layer.get("mlp") is not None:
            streams = hyper_step(streams, sub(w, "hc2."), lambda hh: polynorm_ff(hh, sub(w, "mlp."), eps), w["norm2"], eps)
        after.append(streams.sum(0))
    x = rms_div(streams.sum(0), eps) * tensors["final.norm"]
    return x @ tensors["embed"].T, np.stack(after)
