"""Plain, slow Revepel in numpy: the oracle the engine is compared with.

Whole sequences, no cache, no batching, float64, one function per mechanism, token by token and key by key; it
shares no code with the package (only the file readers of the other oracle).

    layer:    n = rms(x) w;  m = n + (n_prev - n) shift;  x <- x + sig(R1 n + b1) mixer(m) + sig(R2 n + b2) ff(n)
    mixers:   a selective state space, a delta rule with a decay per key channel, a windowed attention whose
              weights are sigmoids; see the functions
    ff:       a few of many small two-matrix feed-forwards, chosen by sigmoid scores that scale their inputs,
              and one that every token takes
    output:   logits = head rms(x) w_final * logit_scale; the embedding is E[id] * scale
"""
from __future__ import annotations

import math
import os

import numpy as np

from plain_gemma2 import read_config, read_safetensors  # noqa: F401  (file formats only)


def load_folder(folder):
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    return read_config(folder), {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_rows(x, eps):
    """Every row divided by its root mean square, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def shifted(n, shift):
    """Row t moves towards row t - 1 (zeros before the first) by the fraction `shift`, channel by channel."""
    prev = np.vstack([np.zeros((1, n.shape[1])), n[:-1]])
    return n + (prev - n) * shift


def short_conv(x, taps_w, bias=None):
    """Causal convolution over time per channel: x [T, C], taps_w [C, K] whose last column meets the current token."""
    T, C = x.shape
    K = taps_w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        for j in range(K):
            s = t - (K - 1 - j)
            if s >= 0:
                out[t] += taps_w[:, j] * x[s]
    return out if bias is None else out + bias


# ---- the selective state space ----

def state_space_head(x, B, C, dt, a, d_skip):
    """One head: S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T (S [N, P], zero at the start); y_t = S_t^T C_t + d_skip x_t."""
    T, P = x.shape
    S = np.zeros((B.shape[1], P))
    y = np.zeros((T, P))
    for t in range(T):
        S = math.exp(-a * dt[t]) * S + dt[t] * np.outer(B[t], x[t])
        y[t] = S.T @ C[t] + d_skip * x[t]
    return y


def state_space(w, p, m, h, eps):
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    r = h @ w[p + "in"].T
    z, xbc, dt = r[:, :inner], r[:, inner:2 * inner + 2 * G * N], r[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
    dt = softplus(dt + w[p + "dt_bias"])
    y = np.zeros((h.shape[0], inner))
    for a in range(H):
        g = a // (H // G)
        y[:, a * P:(a + 1) * P] = state_space_head(x[:, a * P:(a + 1) * P], B[:, g * N:(g + 1) * N], C[:, g * N:(g + 1) * N],
                                                   dt[:, a], math.exp(w[p + "A_log"][a]), w[p + "D"][a])
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_rows(y.reshape(h.shape[0], parts, inner // parts), eps).reshape(h.shape[0], inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---- the delta rule with a decay per key channel ----

def delta_head(q, k, v, beta, g):
    """One head: S <- g_t (.) S row by row; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t."""
    T, e = v.shape
    S = np.zeros((k.shape[1], e))
    o = np.zeros((T, e))
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def unit(v):
    return v / np.sqrt(np.sum(v * v, axis=-1, keepdims=True) + 1e-6)


def channel_delta(w, p, m, h, eps):
    H, J, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"]))
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"]))
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"]))
    beta = sigmoid(h @ w[p + "b"].T)
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"])                  # [T, H * d]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)                                       # [T, H * e]
    out = np.zeros((T, H * e))
    for a in range(H):
        j = a // (H // J)
        qa = unit(q[:, j * d:(j + 1) * d]) * d ** -0.5
        ka = unit(k[:, j * d:(j + 1) * d])
        g = np.exp(-math.exp(w[p + "A_log"][a]) * step[:, a * d:(a + 1) * d])
        o = delta_head(qa, ka, v[:, a * e:(a + 1) * e], beta[:, a], g)
        out[:, a * e:(a + 1) * e] = rms_rows(o, eps) * w[p + "norm"]
    return (out * gate) @ w[p + "o"].T


# ---- attention with sigmoid weights ----

def rotary_angles(rot):
    """Frequencies of the rotated pairs and the factor on cos and sin."""
    n, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / n) for i in range(n // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda turns: n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), n - 1)
    ramp = np.clip((np.arange(n // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def turn(vec, pos, rot):
    out = np.array(vec, dtype=np.float64)
    if not rot:
        return out
    f, mag = rotary_angles(rot)
    n = rot["dims"]
    for i in range(n // 2):
        c, s = math.cos(pos * f[i]) * mag, math.sin(pos * f[i]) * mag
        u, v = vec[i], vec[i + n // 2]
        out[i], out[i + n // 2] = u * c - v * s, v * c + u * s
    return out


def keys_values(w, p, m, h):
    """Rotated keys [T, J, d] and values [T, J, e] of a layer that has projections of its own."""
    T, J, d, e = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T).reshape(T, J, d)
    v = (h @ w[p + "v"].T).reshape(T, J, e)
    k = np.stack([np.stack([turn(k[t, j], t, m.get("rot")) for j in range(J)]) for t in range(T)])
    return k, v


def sigmoid_attention(w, p, m, h, k, v):
    T, H, J, d, e = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    out = np.zeros((T, H, e))
    for t in range(T):
        for a in range(H):
            j = a // (H // J)
            qa = turn(q[t, a], t, m.get("rot"))
            first = 0 if not m.get("mask") else max(0, t - m["mask"]["size"] + 1)
            for s in range(first, t + 1):
                out[t, a] += sigmoid(float(qa @ k[s, j]) * m["scale"] + w[p + "pb"][a]) * v[s, j]
    return out.reshape(T, H * e) @ w[p + "o"].T


# ---- the feed-forward ----

def relu2(z):
    return np.maximum(z, 0.0) ** 2


def two_matrix(w, p, h):
    return relu2(h @ w[p + "up"].T) @ w[p + "down"].T


def routed(w, p, f, h, margins=None):
    """margins: a list that receives, per token, the gap between the last chosen score and the best one left out
    (infinite where every expert is chosen): a choice with a small gap may flip between number formats."""
    E, top = f["router"]["experts"], f["router"]["top"]
    out = np.zeros_like(h)
    gaps = np.full(h.shape[0], np.inf)
    for t in range(h.shape[0]):
        s = sigmoid(w[p + "router"] @ h[t])
        order = np.argsort(-s, kind="stable")
        if top < E:
            gaps[t] = s[order[top - 1]] - s[order[top]]
        for e in order[:top]:
            out[t] += two_matrix(w, f"{p}e{e}.", (s[e] * h[t])[None])[0]
    if margins is not None:
        margins.append(gaps)
    if f.get("shared"):
        out += two_matrix(w, p + "shared.", h)
    return out


# ---- the model ----

def forward(cfg, w, ids, layers_out=None, margins=None):
    """float64 logits [T, vocab]; layers_out: a list that receives the stream after every layer; margins: a list that
    receives every routed layer's gaps (see `routed`)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(ids)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        n = rms_rows(x, eps) * w[p + "norm1"]
        mixed = shifted(n, w[p + "shift"])
        if layer["type"] == "mamba2":
            a = state_space(w, p + "mix.", m, mixed, eps)
        elif layer["type"] == "channel_delta":
            a = channel_delta(w, p + "mix.", m, mixed, eps)
        else:
            if m.get("kv_from") is None:
                kept[i] = keys_values(w, p + "mix.", m, mixed)
            k, v = kept[i if m.get("kv_from") is None else m["kv_from"]]
            a = sigmoid_attention(w, p + "mix.", m, mixed, k, v)
        branch = sigmoid(n @ w[p + "rg1"].T + w[p + "rg1.b"]) * a
        if layer.get("mlp") is not None:
            branch = branch + sigmoid(n @ w[p + "rg2"].T + w[p + "rg2.b"]) * routed(w, p + "mlp.", layer["mlp"], n, margins)
        x = x + branch
        if layers_out is not None:
            layers_out.append(x.copy())
    n = rms_rows(x, eps) * w["final.norm"]
    return (n @ w["head"].T) * cfg["logit_scale"]


def generate_greedy(cfg, w, ids, n_new):
    ids = list(ids)
    out = []
    for _ in range(n_new):
        tok = int(np.argmax(forward(cfg, w, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out
