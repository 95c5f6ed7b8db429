"""The Luvapel decoder, plain: numpy, 64-bit, whole sequences, no cache, one function per
mechanism. It shares no code with the package and is what the tests compare the engine with.

    x = embed[token] * embedding.scale
    per layer:   x <- x + norm1(gate1(x) * mixer(x));   x <- x + norm2(gate2(x) * ff(x))
                 (the sublayers read x itself; gate(x) = sigmoid(W_rg x + b_rg); a layer may name
                 another layer whose tensors it runs with)
    logits = head(norm_final(x))

``weights``: name -> array. ``config``: the config.json dictionary.
"""
import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rotate_interleaved(v, positions, base, dims):
    """v [T, heads, dim]: the first ``dims`` channels of each head rotated, channel 2i with 2i+1,
    by the angle position * base^(-2i/dims); the other channels are left alone."""
    out = v.copy()
    i = np.arange(dims // 2)
    f = base ** (-2.0 * i / dims)
    a = positions[:, None].astype(np.float64) * f[None, :]          # [T, dims/2]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def windowed_attention(W, p, h, m, eps):
    """Grouped-query attention whose values are the keys as projected; queries and keys normed per
    head, rotated; a temperature per head; a sliding window; gated output."""
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dim)
    k = (h @ W[p + "k"].T).reshape(T, G, dim)
    v = k.copy()
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    pos = np.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_interleaved(q, pos, rot["base"], rot["dims"])
        k = rotate_interleaved(k, pos, rot["base"], rot["dims"])
    window = m["mask"]["size"] if m.get("mask") is not None else None
    out = np.zeros((T, H, dim))
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"] * W[p + "temp"][n]
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        seen = j <= i
        if window is not None:
            seen &= (i - j) < window
        s = np.where(seen, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        e = np.exp(s)
        out[:, n] = (e / e.sum(axis=1, keepdims=True)) @ v[:, g]
    out = out.reshape(T, H * dim) * sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def causal_conv(x, w):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c], zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for j in range(min(taps, T)):
        y[j:] += x[:T - j] * w[:, taps - 1 - j]
    return y


def gated_delta(W, p, h, m, eps):
    """The gated delta rule with one decay per head."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dim)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dim)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)                                             # [T, H]
    g = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))   # [T, H]
    gate = silu(h @ W[p + "g"].T).reshape(T, H, vdim)
    o = np.zeros((T, H, vdim))
    for n in range(H):
        kv = n // (H // G)
        S = np.zeros((dim, vdim))
        for t in range(T):
            S = g[t, n] * S
            u = beta[t, n] * (v[t, n] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            o[t, n] = S.T @ q[t, kv]
    o = rms(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * vdim) @ W[p + "o"].T


def parallel_mixer(W, p, h, m, eps):
    left = windowed_attention(W, p + "left.", h, m["left"], eps)
    right = gated_delta(W, p + "right.", h, m["right"], eps)
    return 0.5 * (rms(left, eps) * W[p + "left.out"] + rms(right, eps) * W[p + "right.out"])


def general_delta(W, p, h, m, eps):
    """The generalized delta rule: a decay and a removal rate per head and key channel."""
    T = h.shape[0]
    H, dim = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).reshape(T, H, dim)
    k = (h @ W[p + "k"].T).reshape(T, H, dim)
    v = (h @ W[p + "v"].T).reshape(T, H, dim)
    w = np.exp(-np.exp(-0.5) * sigmoid(np.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, dim)
    a = sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).reshape(T, H, dim)
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    o = np.zeros((T, H, dim))
    for n in range(H):
        S = np.zeros((dim, dim))
        for t in range(T):
            S = w[t, n][:, None] * S - np.outer(a[t, n] * u[t, n], u[t, n] @ S) + np.outer(k[t, n], v[t, n])
            o[t, n] = S.T @ r[t, n]
    o = rms(o, eps).reshape(T, H * dim) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def feed_forward(W, p, h):
    z = np.maximum(h @ W[p + "up"].T, 0.0)
    return (z * z) @ W[p + "down"].T


MIXERS = {"parallel": parallel_mixer, "general_delta": general_delta}


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence. ``layers_out``: a list that receives the residual after
    every layer."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        src = i
        while config["layers"][src].get("weights_of") is not None:       # the layer that has the tensors
            src = config["layers"][src]["weights_of"]
        p = f"l{src}."
        y = MIXERS[layer["type"]](W, p + "mix.", x, layer["mixer"], eps)
        y = y * sigmoid(x @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + rms(y, eps) * W[p + "norm1"]
        if layer.get("mlp") is not None:
            y = feed_forward(W, p + "mlp.", x)
            y = y * sigmoid(x @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + rms(y, eps) * W[p + "norm2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T
