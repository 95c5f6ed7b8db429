"""Dense SwiGLU feed-forward: ``down(silu(gate h) * (up h))``, no bias.

garuda/src/llama/mod.rs:1002-1020 (``expert_batch``; the dense model is the one
expert that every token goes through, :914-921) and garuda/src/simd/mod.rs:161-163
(``silu(x) = x / (1 + exp(-x))``). Gate and up are one matrix product against
their rows stacked; the activation is computed in 32-bit from the 32-bit
accumulators and rounded once.
"""
from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, width: int, inner: int, init_std: float = 0.02):
        self.width, self.inner = int(width), int(inner)
        self.init_std = float(init_std)

    def tensors(self):
        init = ("normal", self.init_std)
        return {"gate_proj.weight": TensorSpec((self.inner, self.width), init=init),
                "up_proj.weight": TensorSpec((self.inner, self.width), init=init),
                "down_proj.weight": TensorSpec((self.width, self.inner), init=init)}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.w_gate_up = ops.pack_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.w_down = tensors["down_proj.weight"].contiguous()

    # ``h`` may be a norm that is half done (``CudaOps.linear_swiglu`` takes it), and the last product
    # may fold in the first half of the norm that follows (``emit_norm``)
    takes_pending_norm = True
    emits_norm = True

    def forward(self, ctx, h, residual=None, emit_norm=None):
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.inner), self.dtype)
        self.ops.linear_swiglu(ctx, h, self.w_gate_up, act)
        if residual is not None:
            if emit_norm is None:
                self.ops.linear(act, self.w_down, residual, accumulate=True)
            else:
                ctx.pending_norm = self.ops.linear(act, self.w_down, residual, accumulate=True, ctx=ctx,
                                                   emit_norm=emit_norm)
            return None
        y = ctx.ws.get("ffn_out", (T, self.width), torch.float32)
        self.ops.linear(act, self.w_down, y)
        return y


@register_feed_forward("gated")
class GatedFeedForward(FeedForward):
    """``down(act(gate h, up h))`` with the activation and the tensors' names as parameters:
    ``activation`` is ``"silu"`` (``silu(g) u``), ``"gelu_tanh"`` (``gelu_tanh(g) u``) or
    ``"clamped_swish"`` (``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(g, limit)`` and
    ``u' = clamp(u, -limit, limit)``). The activation is 32-bit on the 32-bit accumulators.
    The last product adds ``alpha * output`` into the residual."""
    graph_safe = True
    scales_residual = True

    def __init__(self, width: int, inner: int, activation: str = "silu", limit: float = 0.0,
                 names=("gate", "up", "down"), init_std: float = 0.02):
        if activation not in ("silu", "gelu_tanh", "clamped_swish"):
            raise ValueError(f"unknown gated activation {activation!r}")
        self.width, self.inner = int(width), int(inner)
        self.activation, self.limit = activation, float(limit)
        self.names = tuple(names)
        self.init_std = float(init_std)

    def tensors(self):
        init = ("normal", self.init_std)
        g, u, d = self.names
        return {g: TensorSpec((self.inner, self.width), init=init), u: TensorSpec((self.inner, self.width), init=init),
                d: TensorSpec((self.width, self.inner), init=init)}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        g, u, d = self.names
        self.w_gate_up = ops.pack_gate_up(tensors[g], tensors[u])
        self.w_down = tensors[d].contiguous()

    def forward(self, ctx, h, residual=None, alpha: float = 1.0):
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.inner), self.dtype)
        self.ops.linear_gated(ctx, h, self.w_gate_up, act, self.activation, self.limit)
        if residual is not None:
            self.ops.linear(act, self.w_down, residual, accumulate=True, alpha=alpha)
            return None
        y = ctx.ws.get("ffn_out", (T, self.width), torch.float32)
        self.ops.linear(act, self.w_down, y)
        return y


@register_feed_forward("plain")
class PlainFeedForward(FeedForward):
    """``down(act(up h))`` without a gate: ``activation`` is ``"relu2"`` (the square of relu),
    ``"silu"``, ``"tanh"``, ``"sigmoid"`` or ``"xielu"``, computed in 32-bit on the product's 32-bit
    result and rounded once. ``names``: the tensors' local names.

    ``xielu`` has two learned numbers ``p, q`` (tensor ``act_name``, ``[2]``): ``softplus(p) z^2 + z / 2``
    for ``z > 0`` and ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` for ``z <= 0``; both factors are
    formed once, in 64-bit, when the weights are loaded. The last product adds ``alpha * output`` into
    the residual."""
    graph_safe = True
    scales_residual = True

    def __init__(self, width: int, inner: int, activation: str = "relu2", names=("up", "down"), init_std: float = 0.02,
                 act_name: str = "act"):
        if activation not in ("relu2", "silu", "tanh", "sigmoid", "xielu"):
            raise ValueError(f"unknown activation {activation!r}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.names = tuple(names)
        self.act_name = act_name
        self.init_std = float(init_std)

    def tensors(self):
        init = ("normal", self.init_std)
        u, d = self.names
        t = {u: TensorSpec((self.inner, self.width), init=init), d: TensorSpec((self.width, self.inner), init=init)}
        if self.activation == "xielu":
            t[self.act_name] = TensorSpec((2,), role="vector", init=("normal", 0.5))
        return t

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        u, d = self.names
        self.w_up = tensors[u].contiguous()
        self.w_down = tensors[d].contiguous()
        if self.activation == "xielu":
            import math
            p, q = (float(v) for v in tensors[self.act_name].double().cpu())
            softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))
            self.a_pos, self.a_neg = softplus(p), 0.5 + softplus(q)

    def forward(self, ctx, h, residual=None, alpha: float = 1.0):
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.inner), self.dtype)
        if self.activation == "xielu":
            self.ops.linear_xielu(ctx, h, self.w_up, act, self.a_pos, self.a_neg)
        else:
            self.ops.linear_act(ctx, h, self.w_up, act, self.activation)
        if residual is not None:
            self.ops.linear(act, self.w_down, residual, accumulate=True, alpha=alpha)
            return None
        y = ctx.ws.get("ffn_out", (T, self.width), torch.float32)
        self.ops.linear(act, self.w_down, y)
        return y
