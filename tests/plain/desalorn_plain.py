"""A plain, slow implementation of the Desalorn design in float64 numpy: one function per mechanism, whole sequences at
once, nothing shared with the package.  The tests compare the engine with it.

``cfg`` is the model's description as the configuration file gives it (a dict), ``P`` maps tensor names to arrays.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x over the root of (mean square + eps), along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, w, groups, eps):
    """Rows [T, W] cut into ``groups`` equal runs; every run has its own mean square; one weight over the whole row."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    return unit_rms(parts, eps).reshape(T, W) * w


def rotate(x, positions, dims, base, adjacent):
    """x [T, heads, d]: the first ``dims`` of every head turn by position * base^(-2i/dims); pairs are (i, i + dims/2),
    or (2i, 2i + 1) with ``adjacent``.  The rest of a head passes."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if adjacent:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def distance_bucket(n, rows, far):
    """Row of the distance table for a distance n >= 0: one row a distance below rows/2, then logarithmic steps that reach
    the last row at ``far``."""
    half = rows // 2
    if rows < 2:
        return 0
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_attention(h, P, pre, m, eps):
    """Grouped queries with biases, one norm over all of q and one over all of k, capped scores, a bias by distance, the
    heads' scores blended by a matrix, causal softmax, one sigmoid gate a head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ P[pre + "q"].T + P[pre + "q.b"]
    k = h @ P[pre + "k"].T + P[pre + "k.b"]
    v = h @ P[pre + "v"].T + P[pre + "v.b"]
    q = unit_rms(q, eps) * P[pre + "q.norm"]
    k = unit_rms(k, eps) * P[pre + "k.norm"]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    rel, talk = P[pre + "rel"], P[pre + "talk"]
    rows, cap = rel.shape[0], m.get("softcap")
    s = np.empty((H, T, T))
    for hd in range(H):
        s[hd] = (q[:, hd] @ k[:, hd // (H // G)].T) * m["scale"]
    if cap is not None:
        s = cap * np.tanh(s / cap)
    for i in range(T):
        for j in range(i + 1):
            s[:, i, j] += rel[distance_bucket(i - j, rows, m["bias_max"])]
    s = np.einsum("hg,gij->hij", talk, s)
    out = np.zeros((T, H, dv))
    for i in range(T):
        w = s[:, i, : i + 1]
        w = np.exp(w - w.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        for hd in range(H):
            out[i, hd] = w[hd] @ v[: i + 1, hd // (H // G)]
    gate = sigmoid(h @ P[pre + "g"].T)                     # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ P[pre + "o"].T + P[pre + "o.b"]


def retention(h, P, pre, m, eps, state=None, start=0):
    """Linear attention with one fixed decay a head: S <- decay S + k v^T, o = S^T q, token after token.  ``state``
    [H, d, dv] (None: zeros) is what earlier tokens left; returns (rows, state)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(start, start + T)
    q = rotate((h @ P[pre + "q"].T).reshape(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], False)
    k = rotate((h @ P[pre + "k"].T).reshape(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], False) * d ** -0.5
    v = (h @ P[pre + "v"].T).reshape(T, H, dv)
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    decay = np.asarray(m["decay"], dtype=np.float64)
    o = np.empty((T, H, dv))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T, S


def latent_attention(h, P, pre, m, eps):
    """Queries through a normed latent; keys and values from one normed latent a token plus one rotated key part that the
    heads share; a window of the last ``mask.size`` positions."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = unit_rms(h @ P[pre + "dq"].T, eps) * P[pre + "dq.norm"]
    q = (cq @ P[pre + "uq"].T).reshape(T, H, d + dr)
    q_plain = q[..., :d]
    q_rot = rotate(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"], True)
    down = h @ P[pre + "dkv"].T
    c = unit_rms(down[:, :r], eps) * P[pre + "dkv.norm"]
    k_rot = rotate(down[:, None, r:], pos, m["rot"]["dims"], m["rot"]["base"], True)[:, 0]
    k_plain = (c @ P[pre + "uk"].T).reshape(T, H, d)
    v = (c @ P[pre + "uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    span = m["mask"]["size"]
    for i in range(T):
        lo = max(0, i - span + 1)
        for hd in range(H):
            s = (k_plain[lo: i + 1, hd] @ q_plain[i, hd] + k_rot[lo: i + 1] @ q_rot[i, hd]) * m["scale"]
            w = np.exp(s - s.max())
            out[i, hd] = (w / w.sum()) @ v[lo: i + 1, hd]
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def route(z, correction, top, groups, keep):
    """Router outputs z [T, E] -> (experts [T, top], weights [T, top]).  Scores are sigmoids; the choice goes by score +
    correction among the experts of the ``keep`` groups whose two best such numbers add up highest; the weights are the
    chosen experts' scores as they are."""
    T, E = z.shape
    s = sigmoid(z)
    pick = s + correction
    per = E // groups
    ids = np.zeros((T, top), dtype=np.int64)
    wts = np.zeros((T, top))
    for t in range(T):
        by_group = pick[t].reshape(groups, per)
        rank = np.sort(by_group, axis=1)[:, ::-1]
        total = rank[:, :2].sum(axis=1)
        open_groups = np.argsort(-total, kind="stable")[:keep]
        masked = np.full(E, -np.inf)
        for g in open_groups:
            masked[g * per: (g + 1) * per] = pick[t, g * per: (g + 1) * per]
        chosen = np.argsort(-masked, kind="stable")[:top]
        ids[t], wts[t] = chosen, s[t, chosen]
    return ids, wts


def gated_expert(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def mixture(h, P, pre, f, router_input=None):
    """``router_input``: the rows the router reads where they differ from ``h`` (a rounded copy)."""
    r = f["router"]
    z = (h if router_input is None else router_input) @ P[pre + "router"].T
    ids, wts = route(z, P[pre + "correction"], r["top"], r["groups"]["count"], r["groups"]["keep"])
    out = np.zeros((h.shape[0], P[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            out[t] += w * gated_expert(h[t: t + 1], P, f"{pre}e{e}.")[0]
    if f.get("shared") is not None:
        out += gated_expert(h, P, pre + "shared.")
    return out


MIXERS = {"attention": lambda h, P, pre, m, eps: softmax_attention(h, P, pre, m, eps),
          "retention": lambda h, P, pre, m, eps: retention(h, P, pre, m, eps)[0],
          "latent_attention": lambda h, P, pre, m, eps: latent_attention(h, P, pre, m, eps)}


def forward(cfg, P, tokens, after_layer=None):
    """Logits [T, vocab] of one sequence from its first token."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = P["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        h = group_norm(x, P[f"l{i}.norm1"], groups, eps)
        y = MIXERS[layer["type"]](h, P, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + mixture(h, P, f"l{i}.mlp.", layer["mlp"])
        x = x + cfg["residual_mult"] * y
        if after_layer is not None:
            after_layer(i, x)
    return group_norm(x, P["final.norm"], groups, eps) @ P["head"].T


def tensor_shapes(cfg, rel_rows=None):
    """name -> shape of every tensor of a model; ``rel_rows``: rows of the attention layers' distance tables."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        out[f"l{i}.norm1"] = (W,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            out.update({p + "q": (H * d, W), p + "q.b": (H * d,), p + "k": (G * d, W), p + "k.b": (G * d,), p + "v": (G * dv, W),
                        p + "v.b": (G * dv,), p + "q.norm": (H * d,), p + "k.norm": (G * d,), p + "rel": (rel_rows, H),
                        p + "talk": (H, H), p + "g": (H, W), p + "o": (W, H * dv), p + "o.b": (W,)})
        elif layer["type"] == "retention":
            out.update({p + "q": (H * d, W), p + "k": (H * d, W), p + "v": (H * dv, W), p + "g": (H * dv, W), p + "o": (W, H * dv)})
        else:
            r, dr, qr = m["kv_rank"], m["rot_dim"], m["q_rank"]
            out.update({p + "dq": (qr, W), p + "dq.norm": (qr,), p + "uq": (H * (d + dr), qr), p + "dkv": (r + dr, W),
                        p + "dkv.norm": (r,), p + "uk": (H * d, r), p + "uv": (H * dv, r), p + "o": (W, H * dv)})
        f = layer.get("mlp")
        if f is not None:
            q = f"l{i}.mlp."
            E, F = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                out.update({f"{q}e{e}.gate": (F, W), f"{q}e{e}.up": (F, W), f"{q}e{e}.down": (W, F)})
            out.update({q + "router": (E, W), q + "correction": (E,)})
            if f.get("shared") is not None:
                S = f["shared"]["ff"]
                out.update({q + "shared.gate": (S, W), q + "shared.up": (S, W), q + "shared.down": (W, S)})
    return out
