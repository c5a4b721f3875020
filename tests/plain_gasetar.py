"""Plain, slow Gasetar in numpy: the oracle the engine is compared with.

Whole sequences, no cache, no batching, float64, one function per mechanism, query by query and key by key, written
from the design's equations; it shares no code with the package (only the file readers of the other oracle).

    layer:   n = norm(x; norm1);  x <- x + m * (mixer(n) + ff(n))          (ff may be absent; m = residual_mult)
    norm:    v / sqrt(mean(v^2) + eps) * w
    mixers:  attention with a norm over the whole query and key projections, or latent attention with sinks (below)
    ff:      W_down (silu(W_gate n) * (W_up n)), alone or as routed experts plus a shared one (below)
    input:   x = E[token] * embedding.scale
    output:  z = E norm(x; final.norm) * logit_scale;  logits = cap * tanh(z / cap) with cap = logit_softcap
"""
from __future__ import annotations

import math
import os

import numpy as np

from plain_gemma2 import read_config, read_safetensors  # noqa: F401  (file formats only)


def load_folder(folder):
    w = read_safetensors(os.path.join(folder, "model.safetensors"))
    return read_config(folder), {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def rotary_frequencies(rot):
    """f_i = base^(-2i/n) for the n/2 pairs.  With scaling (factor F, low, high, original L) and the wavelength
    l_i = 2 pi / f_i:  l_i < L / high keeps f_i;  l_i > L / low gives f_i / F;  in between, with
    s = (L / l_i - low) / (high - low), f_i <- (1 - s) f_i / F + s f_i."""
    n, base = rot["dims"], rot["base"]
    out = []
    sc = rot.get("scaling")
    for i in range(n // 2):
        f = base ** (-2.0 * i / n)
        if sc:
            l = 2.0 * math.pi / f
            if l > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif l >= sc["original"] / sc["high"]:
                s = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate(v, pos, rot):
    """One vector at position pos: value i of its first rot['dims'] values is paired with value i + dims/2; the pair
    turns by pos * f_i; the rest pass."""
    out = np.array(v, dtype=np.float64)
    if not rot:
        return out
    half = rot["dims"] // 2
    for i, f in enumerate(rotary_frequencies(rot)):
        c, s = math.cos(pos * f), math.sin(pos * f)
        a, b = v[i], v[i + half]
        out[i], out[i + half] = a * c - b * s, b * c + a * s
    return out


def softmax_with_sink(scores, sink=None):
    """Weights of the keys; with a sink the denominator also holds exp(sink), which has no key and no value."""
    top = max(float(np.max(scores)), sink if sink is not None else -math.inf)
    e = np.exp(np.asarray(scores) - top)
    return e / (e.sum() + (math.exp(sink - top) if sink is not None else 0.0))


def attention(h, w, prefix, m, eps):
    T = h.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    vd = m.get("vdim", d)
    q = rms_norm(h @ w[prefix + "q"].T, w[prefix + "q.norm"], eps).reshape(T, H, d)       # one norm over all heads' values
    k = rms_norm(h @ w[prefix + "k"].T, w[prefix + "k.norm"], eps).reshape(T, G, d)
    v = (h @ w[prefix + "v"].T).reshape(T, G, vd)
    rot = m.get("rot")
    q = np.stack([[rotate(q[t, a], t, rot) for a in range(H)] for t in range(T)])
    k = np.stack([[rotate(k[t, g], t, rot) for g in range(G)] for t in range(T)])
    window = m["mask"]["size"] if m.get("mask") else None
    cap = m.get("softcap")
    out = np.zeros((T, H, vd))
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            g = a // (H // G)
            s = np.array([q[i, a] @ k[j, g] * m["scale"] for j in range(first, i + 1)])
            if cap:
                s = cap * np.tanh(s / cap)
            p = softmax_with_sink(s)
            out[i, a] = (p[:, None] * v[first:i + 1, g]).sum(axis=0)
    return out.reshape(T, H * vd) @ w[prefix + "o"].T


def latent_attention(h, w, prefix, m, eps):
    T = h.shape[0]
    H, d, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, d + rd)
    dk = h @ w[prefix + "dkv"].T
    c = rms_norm(dk[:, :r], w[prefix + "dkv.norm"], eps)
    kr = np.stack([rotate(dk[t, r:], t, m["rot"]) for t in range(T)])
    k_un = (c @ w[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, vd)
    gate = 1.0 / (1.0 + np.exp(-(h @ w[prefix + "g"].T)))          # a gate for every value of every head
    out = np.zeros((T, H, vd))
    for i in range(T):
        for a in range(H):
            q_rot = rotate(q[i, a, d:], i, m["rot"])
            s = [(q[i, a, :d] @ k_un[j, a] + q_rot @ kr[j]) * m["scale"] for j in range(i + 1)]
            p = softmax_with_sink(s, float(w[prefix + "sink"][a]))
            out[i, a] = (p[:, None] * v[:i + 1, a]).sum(axis=0)
    return (out.reshape(T, H * vd) * gate) @ w[prefix + "o"].T


def gated(x, w, prefix):
    return (silu(x @ w[prefix + "gate"].T) * (x @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def router(h, w, prefix, f):
    """Chosen experts [T, top] by the largest logits W_r h + b, their weights (softmax over the chosen logits alone) and
    each token's margin: the gap between the last chosen and the first not chosen logit (inf when all are chosen)."""
    z = h @ w[prefix + "router"].T + w[prefix + "router.b"]
    top = f["router"]["top"]
    order = np.argsort(-z, axis=-1, kind="stable")
    chosen = order[:, :top]
    zc = np.take_along_axis(z, chosen, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    srt = np.take_along_axis(z, order, axis=-1)
    margin = srt[:, top - 1] - srt[:, top] if top < z.shape[1] else np.full(h.shape[0], np.inf)
    return chosen, e / e.sum(axis=-1, keepdims=True), margin


def feed_forward(h, w, prefix, f, margins=None):
    if f["kind"] == "dense":
        return gated(h, w, prefix)
    chosen, weight, margin = router(h, w, prefix, f)
    if margins is not None:
        margins.append(margin)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k, e in enumerate(chosen[t]):
            out[t] += weight[t, k] * gated(h[t], w, prefix + f"e{int(e)}.")
    if f.get("shared"):
        out += gated(h, w, prefix + "shared.")
    return out


def forward(cfg, w, ids, margins=None, streams=None):
    """float64 logits [T, vocab]; margins: list that receives every routed layer's per-token margin;
    streams: list that receives the residual stream after every layer."""
    x = w["embed"][np.asarray(ids)] * cfg.get("embedding", {}).get("scale", 1.0)
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = rms_norm(x, w[p + "norm1"], eps)
        mix = attention if layer["type"] == "attention" else latent_attention
        branch = mix(n, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            branch = branch + feed_forward(n, w, p + "mlp.", layer["mlp"], margins)
        x = x + m * branch
        if streams is not None:
            streams.append(x.copy())
    z = (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z


def min_margin(cfg, w, ids):
    margins = []
    forward(cfg, w, ids, margins)
    return min((float(m.min()) for m in margins), default=math.inf)
