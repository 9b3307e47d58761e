"""Plain, slow implementation of the Pazenex decoder in numpy: whole sequences, no cache, one
function per mechanism.  It shares no code with the engine: it reads config.json keys itself
and walks tokens and keys with ordinary loops where the engine has kernels.

A Pazenex model is a list of layers, each a token mixer (softmax attention with a sink, or a
Mamba-2 state-space mixer) and an optional feed-forward, every sublayer between two layer norms:

    x <- x + LN_b(mixer(LN_a(x)));   x <- x + LN_d(ff(LN_c(x)))

A span of the layers may run several times in a row with the same weights; before each run of
the span a learned vector of that run is added to the stream, and before every run but the
first the embedding output is added again.

All arithmetic is float64 unless another dtype is asked for; tensors are given as a dict of arrays.
"""

from __future__ import annotations

import math

import numpy as np


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, var the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z**3)))


def relu_squared(z):
    return np.maximum(z, 0) ** 2


def sigmoid(z):
    return 1 / (1 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0)


def rotate_half_pairs(x, positions, dims, base, factor):
    """x [T, heads, d]: dimension i < dims/2 is paired with i + dims/2; the pair (u, v) at position p
    becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims) / factor.  Dimensions from
    ``dims`` on pass unchanged."""
    out = x.copy()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims) / factor
        a = positions * f
        c, s = np.cos(a)[:, None], np.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def sink_softmax(scores):
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): a sink with score 0 and no value takes part of the mass."""
    m = max(0.0, float(scores.max()))
    e = np.exp(scores - m)
    return e / (math.exp(-m) + e.sum())


def sink_attention(h, w, px, mix, eps):
    """The attention mixer on a whole sequence h [T, width].

    q = Wq h, k = Wk h; the values are k as projected (no norm, no rotation, no value matrix);
    q and k are each divided by the RMS of their whole projection (all heads together) and
    multiplied by a weight of that size; rotary on the first ``rot.dims`` dimensions of each
    head; scores (q . k) * scale over keys j <= i (the last ``window`` of them, if the mixer
    has that key) with the sink softmax; the heads' outputs times sigmoid(Wg h), then Wo."""
    T = h.shape[0]
    H, G, d, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    pos = np.arange(T, dtype=np.float64)
    q = h @ w[px + "q"].T
    k = h @ w[px + "k"].T
    v = k.reshape(T, G, d)
    q = (rms_unit(q, eps) * w[px + "q.norm"]).reshape(T, H, d)
    kn = (rms_unit(k, eps) * w[px + "k.norm"]).reshape(T, G, d)
    rot = mix["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_half_pairs(q, pos, rot["dims"], rot["base"], factor)
    kn = rotate_half_pairs(kn, pos, rot["dims"], rot["base"], factor)
    out = np.zeros((T, H, dv), dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - mix["window"] + 1) if mix.get("window") else 0
        for a in range(H):
            g = a // (H // G)
            s = (kn[lo : i + 1, g] @ q[i, a]) * mix["scale"]
            p = sink_softmax(s)
            out[i, a] = p @ v[lo : i + 1, g]
    gate = sigmoid(h @ w[px + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[px + "o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    out = np.zeros_like(x)
    for t in range(T):
        acc = bias.copy()
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                acc = acc + taps_w[:, j] * x[src]
        out[t] = acc
    return out


def ssm_scan(x, dt, A, B, C, D, heads_per_group):
    """x [T, heads, P], dt [T, heads] (after softplus), A [heads] (> 0), B, C [T, groups, N], D [heads].
    S_t = exp(-A dt_t) S_{t-1} + dt_t B_t x_t^T  (N x P per head);  y_t = S_t^T C_t + D x_t."""
    T, Hh, P = x.shape
    N = B.shape[2]
    y = np.zeros_like(x)
    for a in range(Hh):
        g = a // heads_per_group
        S = np.zeros((N, P), dtype=x.dtype)
        for t in range(T):
            S = math.exp(-A[a] * dt[t, a]) * S + dt[t, a] * np.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + D[a] * x[t, a]
    return y


def gated_group_norm(y, z, w, parts, eps):
    """(y * silu(z)), cut into ``parts`` equal runs of the last axis, each divided by its own RMS; times w."""
    T, n = y.shape
    g = (y * silu(z)).reshape(T, parts, n // parts)
    return rms_unit(g, eps).reshape(T, n) * w


def mamba2(h, w, px, mix, eps):
    """The Mamba-2 mixer on a whole sequence.  W_in h = [z | x | B | C | dt]; x, B, C pass the causal
    convolution and silu; dt <- softplus(dt + dt_bias); the scan; y * silu(z) normed in parts; Wo."""
    T = h.shape[0]
    Hh, P, N, G = mix["heads"], mix["vdim"], mix["state"], mix["groups"]
    inner = Hh * P
    u = h @ w[px + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner : 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_conv(xbc, w[px + "conv"], w[px + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner : inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N :].reshape(T, G, N)
    dt = softplus(dt + w[px + "dt_bias"])
    y = ssm_scan(x, dt, np.exp(w[px + "A_log"]), B, C, w[px + "D"], Hh // G)
    y = gated_group_norm(y.reshape(T, inner), z, w[px + "norm"], mix["norm_groups"], eps)
    return y @ w[px + "o"].T


def feed_forward(h, w, px, mlp):
    if mlp["kind"] != "dense":
        raise ValueError(f"feed-forward kind {mlp['kind']!r}")
    return relu_squared(h @ w[px + "up"].T) @ w[px + "down"].T


def run_layer(x, w, i, spec, eps):
    px = f"l{i}."
    h = layer_norm(x, w[px + "norm1"], eps)
    if spec["type"] == "attention":
        m = sink_attention(h, w, px + "mix.", spec["mixer"], eps)
    elif spec["type"] == "mamba2":
        m = mamba2(h, w, px + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(f"layer type {spec['type']!r}")
    x = x + layer_norm(m, w[px + "norm1b"], eps)
    if spec.get("mlp"):
        f = feed_forward(layer_norm(x, w[px + "norm2"], eps), w, px + "mlp.", spec["mlp"])
        x = x + layer_norm(f, w[px + "norm2b"], eps)
    return x


def layer_runs(cfg):
    """[(layer, pass number or None)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] < 1 or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, dtype=np.float64, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and, if asked, the stream after every layer run)."""
    w = {k: np.asarray(v).astype(dtype) if np.asarray(v).dtype.kind == "f" else np.asarray(v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    embedded = x.copy()
    loop = cfg.get("loop")
    streams = []
    for i, t in layer_runs(cfg):
        if t is not None and i == loop["start"]:
            if t > 0:
                x = x + embedded
            x = x + w["loop.step"][t]
        x = run_layer(x, w, i, cfg["layers"][i], eps)
        streams.append(x.copy())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
