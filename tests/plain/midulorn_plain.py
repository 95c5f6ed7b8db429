"""The Midulorn design, plain: numpy, 64-bit, whole sequences, no cache, one function per mechanism.

The oracle of the tests. Written from the design's equations, in the notation below; it shares no
code with ``garuda_b200``.

  rms(v, w)      = v / sqrt(mean(v^2) + eps) * w
  layer          : x <- rms(alpha x + mixer(x), w1);  x <- rms(alpha x + ff(x), w2)
  logits         = E rms(x, w_final) * logit_scale,  x_0 = E[token] * embedding_scale
"""
import numpy as np


def rms(v, w, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def xielu(z, p, q):
    """softplus(p) z^2 + z/2 above zero; (1/2 + softplus(q)) (e^z - 1 - z) + z/2 at and below."""
    below = np.minimum(z, 0.0)
    return np.where(z > 0, softplus(p) * z * z + 0.5 * z, (0.5 + softplus(q)) * (np.expm1(below) - below) + 0.5 * z)


def dense_ff(W, p, h):
    a = W[p + "act"]
    return xielu(h @ W[p + "up"].T, a[0], a[1]) @ W[p + "down"].T


def softmax_sink(s, sink):
    """Rows of ``s`` (masked entries -inf) through a softmax whose denominator also holds exp(sink)."""
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def routed_ff(W, p, experts, top, h):
    """Every token's ``top`` experts by their share of the softmax over all experts; shares not renormalized."""
    z = h @ W[p + "router"].T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            q = f"{p}e{e}."
            out[t] += s[t, e] * ((silu(W[q + "gate"] @ h[t]) * (W[q + "up"] @ h[t])) @ W[q + "down"].T)
    return out


def rotate_half(v, positions, base, dims):
    """The first ``dims`` channels of ``v [T, n]``: channel i with channel i + dims/2, by positions * base^(-2i/dims)."""
    half = dims // 2
    angle = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * np.arange(half) / dims)[None, :]
    c, s = np.cos(angle), np.sin(angle)
    out = v.copy()
    out[:, :half] = v[:, :half] * c - v[:, half:dims] * s
    out[:, half:dims] = v[:, half:dims] * c + v[:, :half] * s
    return out


def latent_attention(W, p, m, eps, h):
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = np.arange(T)
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rd)
    down = h @ W[p + "dkv"].T
    c = rms(down[:, :rank], W[p + "dkv.norm"], eps)
    key_rot = rotate_half(down[:, rank:], pos, base, dims)
    k = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vd)
    gate = sigmoid(h @ W[p + "g"].T)
    causal = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, vd))
    for n in range(H):
        s = (q[:, n, :dim] @ k[:, n].T + rotate_half(q[:, n, dim:], pos, base, dims) @ key_rot.T) * m["scale"]
        out[:, n] = softmax_sink(np.where(causal, s, -np.inf), W[p + "sink"][n]) @ v[:, n] * gate[:, n:n + 1]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def min_gru(W, p, h):
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    states = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        states[t] = S
    return (states * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def causal_conv(u, taps):
    """``y_t = sum_j taps[:, j] u_(t - n + 1 + j)`` with ``n`` taps, zeros before the first token."""
    T, n = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, u.shape[1])), u], axis=0)
    return sum(padded[j:j + T] * taps[:, j][None, :] for j in range(n))


def chunked_attention(W, p, m, eps, h, shared):
    """``shared``: what the first layer with mixed values leaves for the later ones."""
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ W[p + n].T + W[p + n + ".b"] for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (causal_conv(u, W[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms(q.reshape(T, H, dim), W[p + "q.norm"], eps)
    k = rms(k.reshape(T, G, dim), W[p + "k.norm"], eps)
    v = v.reshape(T, G, vd)
    if m.get("v_mix"):
        if "values" in shared:
            lam = float(W[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["values"].reshape(v.shape)      # channel by channel of the flat row
        else:
            shared["values"] = v
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = j <= i
    if m.get("mask"):
        seen &= (i // m["mask"]["size"]) == (j // m["mask"]["size"])
    dist = np.maximum(i - j, 0).astype(np.float64)
    out = np.zeros((T, H, vd))
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"] - W[p + "r1"][n] * np.log1p(W[p + "r2"][n] * dist)
        out[:, n] = softmax_sink(np.where(seen, s, -np.inf), W[p + "sink"][n]) @ v[:, g]
    return out.reshape(T, H * vd) @ W[p + "o"].T + W[p + "o.b"]


def forward(cfg, W, tokens, layers_out=None):
    """Logits ``[T, vocab]`` (64-bit) at every position. ``W``: name -> array. ``layers_out``: a list that
    receives the residual after every layer."""
    W = {n: np.asarray(a, dtype=np.float64) for n, a in W.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            y = chunked_attention(W, p + "mix.", m, eps, x, shared)
        elif layer["type"] == "latent_attention":
            y = latent_attention(W, p + "mix.", m, eps, x)
        elif layer["type"] == "mingru":
            y = min_gru(W, p + "mix.", x)
        else:
            raise ValueError(layer["type"])
        x = rms(alpha * x + y, W[p + "norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            y = dense_ff(W, p + "mlp.", x) if f["kind"] == "dense" else routed_ff(W, p + "mlp.", f["router"]["experts"], f["router"]["top"], x)
            x = rms(alpha * x + y, W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms(x, W["final.norm"], eps) @ W["embed"].T * cfg["logit_scale"]
