"""A recurrent mixer: the gated delta rule with a decay per key channel.

With ``h`` the mixer's input, ``H`` heads that each keep a state ``S [dim,
vdim]`` per request (32-bit, zero at the start), ``G`` query/key heads (head
``n`` uses query/key head ``n // (H / G)``):

    q, k = W_q h, W_k h  (G x dim),   v = W_v h  (H x vdim)
    each passes a causal convolution over time per channel (``taps`` taps, the last one on the
    current token, zeros before the sequence) and SiLU
    q <- q / sqrt(sum q^2 + 1e-6) * dim^-1/2,   k <- k / sqrt(sum k^2 + 1e-6)     per head
    beta = sigmoid(W_b h)                                                        per head
    g = exp(-exp(A_n) * softplus(W_a2 (W_a1 h) + dt_bias))                       per head and key channel
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q         per token, in this order
    out = W_o concat_n [ o_n / sqrt(mean(o_n^2) + eps) * w_norm * sigmoid(W_g2 (W_g1 h))_n ]

Decays, gates, unit vectors, the state and everything between them are 32-bit;
the matrix products and the convolution's inputs are in the compute dtype with
32-bit results. The state of a request is one row of a fixed-size state array:
``S`` of all heads, then the convolution's last ``taps - 1`` inputs.

Three products feed the recurrence: ``[W_q; W_k; W_v; W_b]`` (32-bit result),
``[W_a1; W_g1]`` (the low-rank pair's first halves, result in the compute
dtype) and ``diag(W_a2, W_g2)`` on that (32-bit result; the zero blocks add
exact zeros). The ranks of the two low-rank pairs are read from the tensors.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import FixedState, Mixer, TensorSpec, register_mixer


@register_mixer("channel_delta_rule")
class ChannelDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: Optional[int] = None, gate_rank: Optional[int] = None, init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} query/key heads")
        if taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {taps}")
        self.width, self.heads, self.kv_heads = int(width), int(heads), int(kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.gate_rank = int(gate_rank) if gate_rank else None
        self.init_std = float(init_std)
        self.qk_dim, self.v_dim = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk_dim + self.v_dim

    def tensors(self):
        init, d = ("normal", self.init_std), self.width
        H, taps = self.heads, self.taps
        conv = ("normal", 0.4)
        return {
            "q": TensorSpec((self.qk_dim, d), init=init), "q.conv": TensorSpec((self.qk_dim, taps), role="vector", init=conv),
            "k": TensorSpec((self.qk_dim, d), init=init), "k.conv": TensorSpec((self.qk_dim, taps), role="vector", init=conv),
            "v": TensorSpec((self.v_dim, d), init=init), "v.conv": TensorSpec((self.v_dim, taps), role="vector", init=conv),
            "b": TensorSpec((H, d), init=init),
            "A_log": TensorSpec((H,), role="vector", init=("normal", 0.5)),
            "norm": TensorSpec((self.vdim,), role="vector", init=("normal_about_one", 0.1)),
            "a1": TensorSpec((self.decay_rank, d), init=init),
            "a2": TensorSpec((H * self.dim, self.decay_rank), init=init),
            "dt_bias": TensorSpec((H * self.dim,), role="vector", init=("normal", 0.5)),
            "g1": TensorSpec((self.gate_rank, d), init=init),
            "g2": TensorSpec((self.v_dim, self.gate_rank), init=init),
            "o": TensorSpec((d, self.v_dim), init=init),
        }

    def cache_need(self):
        return FixedState((self.heads * self.dim * self.vdim + (self.taps - 1) * self.channels,), torch.float32)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        t = tensors
        ra, rg = t["a1"].shape[0], t["g1"].shape[0]
        if t["a2"].shape[1] != ra or t["g2"].shape[1] != rg:
            raise ValueError(f"the low-rank pairs do not fit: a1 {tuple(t['a1'].shape)} a2 {tuple(t['a2'].shape)}, "
                             f"g1 {tuple(t['g1'].shape)} g2 {tuple(t['g2'].shape)}")
        self.w_in = torch.cat([t["q"], t["k"], t["v"], t["b"]], dim=0).contiguous()
        # the low-rank pairs: first halves stacked (padded to a multiple of 8 columns for the
        # tensor-core products), second halves as one block-diagonal matrix
        r = ra + rg
        rp = (r + 7) // 8 * 8
        low = torch.zeros(rp, self.width, dtype=t["a1"].dtype, device=t["a1"].device)
        low[:ra], low[ra:r] = t["a1"], t["g1"]
        second = torch.zeros(self.heads * self.dim + self.v_dim, rp, dtype=t["a2"].dtype, device=t["a2"].device)
        second[:self.heads * self.dim, :ra] = t["a2"]
        second[self.heads * self.dim:, ra:r] = t["g2"]
        self.w_low, self.w_second, self.low_rank = low.contiguous(), second.contiguous(), rp
        vec = torch.float32
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).to(vec).contiguous()
        self.a_log = t["A_log"].to(vec).contiguous()
        self.dt_bias = t["dt_bias"].to(vec).contiguous()
        self.norm_w = t["norm"].to(vec).contiguous()
        self.w_o = t["o"].contiguous()

    def forward(self, ctx, h, cache, residual=None):
        ops, ws = self.ops, ctx.ws
        T = h.shape[0]
        proj = ws.get("delta_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, proj)
        low = ws.get("delta_low", (T, self.low_rank), self.dtype)
        ops.linear(h, self.w_low, low)
        second = ws.get("delta_second", (T, self.w_second.shape[0]), torch.float32)
        ops.linear(low, self.w_second, second)
        out = ws.get("delta_out", (T, self.v_dim), self.dtype)
        ops.delta_rule(ctx, proj, second, self.conv_w, self.a_log, self.dt_bias, self.norm_w, self.eps, cache.state,
                       self.heads, self.kv_heads, self.dim, self.vdim, self.taps, out)
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y


@register_mixer("head_delta_rule")
class HeadDeltaRule(Mixer):
    """The gated delta rule with one decay per head. As ``ChannelDeltaRule`` but

        g = exp(-exp(A_n) * softplus(W_a h + dt_bias))        one number per head and token
        out = W_o concat_n [ o_n / sqrt(mean(o_n^2) + eps) * w_norm * silu(W_g h)_n ]

    with ``W_a [H, d]`` and ``W_g [H vdim, d]`` full projections (no low-rank pairs) and
    ``gate`` = ``silu`` or ``sigmoid``. One product makes ``[q | k | v | beta | decay | gate]`` in
    32-bit; the recurrence kernels are those of the channel-decay rule, with the head's decay for
    every key channel. The state of a request is one row of a fixed-size state array: ``S`` of
    all heads, then the convolution's last ``taps - 1`` inputs."""
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 gate: str = "silu", init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} query/key heads")
        if taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {taps}")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"the output gate is 'silu' or 'sigmoid', got {gate!r}")
        self.width, self.heads, self.kv_heads = int(width), int(heads), int(kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(taps), float(eps)
        self.gate, self.init_std = gate, float(init_std)
        self.qk_dim, self.v_dim = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk_dim + self.v_dim

    def tensors(self):
        init, d = ("normal", self.init_std), self.width
        H, taps = self.heads, self.taps
        conv = ("normal", 0.4)
        return {
            "q": TensorSpec((self.qk_dim, d), init=init), "q.conv": TensorSpec((self.qk_dim, taps), role="vector", init=conv),
            "k": TensorSpec((self.qk_dim, d), init=init), "k.conv": TensorSpec((self.qk_dim, taps), role="vector", init=conv),
            "v": TensorSpec((self.v_dim, d), init=init), "v.conv": TensorSpec((self.v_dim, taps), role="vector", init=conv),
            "b": TensorSpec((H, d), init=init),
            "A_log": TensorSpec((H,), role="vector", init=("normal", 0.5)),
            "norm": TensorSpec((self.vdim,), role="vector", init=("normal_about_one", 0.1)),
            "a": TensorSpec((H, d), init=init),
            "dt_bias": TensorSpec((H,), role="vector", init=("normal", 0.5)),
            "g": TensorSpec((self.v_dim, d), init=init),
            "o": TensorSpec((d, self.v_dim), init=init),
        }

    def cache_need(self):
        return FixedState((self.heads * self.dim * self.vdim + (self.taps - 1) * self.channels,), torch.float32)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        t = tensors
        rows = [t["q"], t["k"], t["v"], t["b"], t["a"], t["g"]]
        n = sum(r.shape[0] for r in rows)
        pad = (-n) % 8            # whole groups of eight rows for the tensor-core products
        if pad:
            rows.append(torch.zeros(pad, self.width, dtype=t["q"].dtype, device=t["q"].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        vec = torch.float32
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).to(vec).contiguous()
        self.a_log = t["A_log"].to(vec).contiguous()
        self.dt_bias = t["dt_bias"].to(vec).contiguous()
        self.norm_w = t["norm"].to(vec).contiguous()
        self.w_o = t["o"].contiguous()

    def forward(self, ctx, h, cache, residual=None, out_name: str = "delta_y"):
        ops, ws = self.ops, ctx.ws
        T, H = h.shape[0], self.heads
        proj = ws.get("hdelta_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, proj)
        first = self.channels + H
        out = ws.get("delta_out", (T, self.v_dim), self.dtype)
        ops.delta_rule(ctx, proj[:, :first], proj[:, first:first + H + self.v_dim], self.conv_w, self.a_log, self.dt_bias,
                       self.norm_w, self.eps, cache.state, H, self.kv_heads, self.dim, self.vdim, self.taps, out,
                       decay_per_head=True, gate=self.gate)
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True)
            return None
        y = ws.get(out_name, (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y


@register_mixer("general_delta_rule")
class GeneralDeltaRule(Mixer):
    """The generalized delta rule: ``H`` heads that each keep a state ``S [dim, dim]`` per request
    (32-bit, zero at the start), a decay and a removal rate per head and key channel:

        r, k, v = W_r h, W_k h, W_v h                      (H x dim each)
        w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 h) + w0))
        a = sigmoid(W_a h + a0)
        u = k / sqrt(sum k^2 + 1e-6)                        per head
        S <- diag(w) S - (a * u)(u^T S) + k v^T             both terms read the old S
        o = S^T r
        out = W_o ( concat_n [o_n / sqrt(mean(o_n^2) + eps)] * w_norm * sigmoid(W_g h) )

    Decays, rates, unit keys, the state and everything between them are 32-bit. One product
    makes ``[r | k | v | a | g | W_w1 h]`` in 32-bit, a second the decay's pre-activation from
    ``tanh(W_w1 h)``; the rank of that pair is read from the tensors."""
    graph_safe = True

    def __init__(self, width: int, heads: int, dim: int, eps: float, decay_scale: float = math.exp(-0.5),
                 decay_rank: Optional[int] = None, init_std: float = 0.02):
        self.width, self.heads, self.dim, self.eps = int(width), int(heads), int(dim), float(eps)
        self.decay_scale = float(decay_scale)
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.init_std = float(init_std)
        self.inner = self.heads * self.dim

    def tensors(self):
        init, d, n = ("normal", self.init_std), self.width, self.inner
        t = {name: TensorSpec((n, d), init=init) for name in ("r", "k", "v", "a", "g")}
        t.update({
            "a.b": TensorSpec((n,), role="vector", init=("normal", 0.5)),
            "w1": TensorSpec((self.decay_rank, d), init=init),
            "w2": TensorSpec((n, self.decay_rank), init=("normal", 0.5)),
            "w0": TensorSpec((n,), role="vector", init=("normal", 1.0)),
            "norm": TensorSpec((n,), role="vector", init=("normal_about_one", 0.1)),
            "o": TensorSpec((d, n), init=init),
        })
        return t

    def cache_need(self):
        return FixedState((self.heads * self.dim * self.dim,), torch.float32)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        t, n = tensors, self.inner
        rank = t["w1"].shape[0]
        if t["w2"].shape[1] != rank:
            raise ValueError(f"the decay's low-rank pair does not fit: w1 {tuple(t['w1'].shape)} w2 {tuple(t['w2'].shape)}")
        rp = (rank + 7) // 8 * 8           # padded to whole groups of eight for the tensor-core products
        low = torch.zeros(rp, self.width, dtype=t["w1"].dtype, device=t["w1"].device)
        low[:rank] = t["w1"]
        self.w_in = torch.cat([t["r"], t["k"], t["v"], t["a"], t["g"], low], dim=0).contiguous()
        self.cols = (0, n, 2 * n, 3 * n, 4 * n)
        self.col_low, self.rank = 5 * n, rp
        second = torch.zeros(n, rp, dtype=t["w2"].dtype, device=t["w2"].device)
        second[:, :rank] = t["w2"]
        self.w_second = second.contiguous()
        self.w0 = t["w0"].float().contiguous()
        self.a0 = t["a.b"].float().contiguous()
        self.norm_w = t["norm"].float().contiguous()
        self.w_o = t["o"].contiguous()

    def forward(self, ctx, h, cache, residual=None, out_name: str = "gdelta_y"):
        ops, ws = self.ops, ctx.ws
        T = h.shape[0]
        proj = ws.get("gdelta_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, proj)
        low = ws.get("gdelta_low", (T, self.rank), self.dtype)
        ops.activation(proj[:, self.col_low:self.col_low + self.rank], low, "tanh")
        zdec = ws.get("gdelta_zdec", (T, self.inner), torch.float32)
        ops.linear(low, self.w_second, zdec)
        out = ws.get("gdelta_out", (T, self.inner), self.dtype)
        ops.general_delta(ctx, proj, self.cols, zdec, self.w0, self.a0, self.decay_scale, self.norm_w, self.eps,
                          cache.state, self.heads, self.dim, self.dim, out)
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True)
            return None
        y = ws.get(out_name, (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y
