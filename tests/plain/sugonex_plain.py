"""Plain, slow implementation of the Sugonex decoder in numpy: whole sequences, no cache, one
function per mechanism.  It shares no code with the engine: it reads config.json keys itself and
walks tokens and keys with ordinary loops where the engine has kernels.

A Sugonex layer reads the stream once and adds two branches to it side by side,

    x <- x + mixer(N1(x)) + ff(N2(x)),      N(x) = x / rms(x) * (1 + w)

where the mixer is attention over a cached latent (with a rotated key part shared by the heads and an
output gate, or without positions and with a sliding window) or a gated delta rule, and ff is a gated
feed-forward (absent in some layers).  A span of layers may run several times with the same weights;
each pass starts by adding its own learned vector to the stream.  The logits come from the embedding
matrix, scaled and soft-capped.

All arithmetic is float64; tensors come as a dict of arrays.
"""

from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1 / (1 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0)


def gelu_tanh(z):
    return 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z**3)))


def rotate_half_pairs(x, positions, dims, base):
    """x [T, ..., d]: dimension i < dims/2 pairs with i + dims/2; the pair (u, v) at position p turns by
    the angle p * base^(-2i/dims).  Dimensions from ``dims`` on pass unchanged."""
    out = x.copy()
    half = dims // 2
    shape = (len(positions),) + (1,) * (x.ndim - 2)
    for i in range(half):
        a = positions * base ** (-2.0 * i / dims)
        c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def softmax(s):
    e = np.exp(s - s.max())
    return e / e.sum()


def latent_attention(h, w, px, mix, eps, gated):
    """Attention whose keys and values are both made from one small vector per token.

    W_dkv h gives kv_rank numbers, RMS-normed with a plain weight: the latent c.  If the mixer has a rotated part
    (``rot_dim``), W_dkv h has rot_dim more rows: one key part, turned by the token's position, that every head
    shares; q then holds per head ``dim`` plain numbers followed by ``rot_dim`` that are turned the same way.
    Per head the plain key is its rows of W_uk c and the value its rows of W_uv c.  Token i sees j <= i, and with
    ``mask.size`` only the last that many (itself included).  ``gated``: the heads' outputs are multiplied by
    sigmoid(W_g h) before W_o."""
    T = h.shape[0]
    H, d, dv, r = mix["heads"], mix["dim"], mix["vdim"], mix["kv_rank"]
    dr = int(mix.get("rot_dim", 0) or 0)
    pos = np.arange(T, dtype=np.float64)
    q = (h @ w[px + "q"].T).reshape(T, H, d + dr)
    down = h @ w[px + "dkv"].T
    c = rms_unit(down[:, :r], eps) * w[px + "dkv.norm"]
    k_plain = (c @ w[px + "uk"].T).reshape(T, H, d)
    v = (c @ w[px + "uv"].T).reshape(T, H, dv)
    q_plain = q[:, :, :d]
    if dr:
        rot = mix["rot"]
        q_turn = rotate_half_pairs(q[:, :, d:], pos, rot["dims"], rot["base"])
        k_turn = rotate_half_pairs(down[:, r:], pos, rot["dims"], rot["base"])
    span = (mix.get("mask") or {}).get("size")
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - span + 1) if span else 0
        for a in range(H):
            s = k_plain[lo : i + 1, a] @ q_plain[i, a]
            if dr:
                s = s + k_turn[lo : i + 1] @ q_turn[i, a]
            out[i, a] = softmax(s * mix["scale"]) @ v[lo : i + 1, a]
    out = out.reshape(T, H * dv)
    if gated:
        out = out * sigmoid(h @ w[px + "g"].T)
    return out @ w[px + "o"].T


def causal_conv(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    out = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += taps_w[:, j] * x[src]
    return out


def unit_vector(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def delta_rule(h, w, px, mix, eps):
    """The gated delta rule: a matrix S per head (key size x value size) that forgets, corrects what it holds under
    the current key toward the current value, and is read with the query, token by token."""
    T = h.shape[0]
    H, G, d, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    q = silu(causal_conv(h @ w[px + "q"].T, w[px + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[px + "k"].T, w[px + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[px + "v"].T, w[px + "v.conv"])).reshape(T, H, dv)
    q = unit_vector(q) * d**-0.5
    k = unit_vector(k)
    beta = sigmoid(h @ w[px + "b"].T)
    keep = np.exp(-np.exp(w[px + "A_log"]) * softplus(h @ w[px + "a"].T + w[px + "dt_bias"]))
    S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] *= keep[t, a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, g])
            S[a] += np.outer(k[t, g], u)
            o[t, a] = S[a].T @ q[t, g]
    o = rms_unit(o, eps) * w[px + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[px + "g"].T)
    return o @ w[px + "o"].T


def gated_feed_forward(h, w, px):
    return (gelu_tanh(h @ w[px + "gate"].T) * (h @ w[px + "up"].T)) @ w[px + "down"].T


def gated_latent_attention(h, w, px, mix, eps):
    """The kind with a rotated key part: its output is gated."""
    return latent_attention(h, w, px, mix, eps, gated=True)


def windowed_latent_attention(h, w, px, mix, eps):
    """The kind without positions: no gate."""
    return latent_attention(h, w, px, mix, eps, gated=False)


MIXERS = {"latent_attention": gated_latent_attention, "latent_attention_2": windowed_latent_attention, "delta": delta_rule}


def layer_runs(cfg):
    """[(layer, pass or None)]: pass t at the layer that is entered through the t-th loop vector."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def layer(x, w, cfg, i):
    spec = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    px = f"l{i}."
    add = MIXERS[spec["type"]](offset_norm(x, w[px + "norm1"], eps), w, px + "mix.", spec["mixer"], eps)
    if spec.get("mlp"):
        add = add + gated_feed_forward(offset_norm(x, w[px + "norm2"], eps), w, px + "mlp.")
    return x + add


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one whole sequence.  ``trace``: a list that receives the stream after every layer run."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    x = w["embed"][np.asarray(tokens)]
    for i, t in layer_runs(cfg):
        if t is not None:
            x = x + w["loop.step"][t]
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x.copy())
    y = offset_norm(x, w["final.norm"], cfg["norm"]["eps"])
    logits = (y @ w["embed"].T) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits


def greedy(cfg, w, prompt, new_tokens):
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]
