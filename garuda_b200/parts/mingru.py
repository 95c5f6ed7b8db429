"""minGRU: a recurrence per channel whose gate and candidate are functions of the current token alone.

With ``x`` the mixer's input and one state ``S`` of ``inner`` channels per request:

    z = sigmoid(W_z x + b_z)              the gate
    u = W_x x + b_x;  n = u + 1/2 where u >= 0, sigmoid(u) where u < 0      the candidate
    S_t = (1 - z) S_(t-1) + z n           channel by channel, from S = 0 at a request's start
    out = W_o (S_t * silu(W_g x))

One product makes ``[W_z x | W_x x | W_g x]`` as a 32-bit row; the gate, the candidate, the
recurrence and the output gate are 32-bit arithmetic in one kernel (two for long prompt portions,
which are cut into stretches that run side by side); only ``S_t * silu(.)`` is rounded to the compute
dtype, as the operand of the output product. ``S`` is a ``FixedState`` row, zeroed by the step that
runs a request's first token and carried from step to step.

``names``: the tensors' local names; the biases are the weights' names with ``.b`` added
(``bias=False``: none).
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FixedState, Mixer, TensorSpec, register_mixer


@register_mixer("mingru")
class MinGRU(Mixer):
    graph_safe = True
    scales_residual = True

    def __init__(self, width: int, inner: int, bias: bool = True, names: Optional[dict] = None, init_std: float = 0.02):
        self.width, self.inner, self.bias = int(width), int(inner), bool(bias)
        if min(self.width, self.inner) < 1:
            raise ValueError("a recurrence needs positive sizes")
        self.names = dict({"z": "z", "x": "x", "g": "g", "o": "o"}, **(names or {}))
        self.init_std = float(init_std)

    def tensors(self):
        init, n = ("normal", self.init_std), self.names
        t = {n[k]: TensorSpec((self.inner, self.width), init=init) for k in ("z", "x", "g")}
        t[n["o"]] = TensorSpec((self.width, self.inner), init=init)
        if self.bias:
            t[n["z"] + ".b"] = TensorSpec((self.inner,), role="vector", init=("normal", 0.5))
            t[n["x"] + ".b"] = TensorSpec((self.inner,), role="vector", init=("normal", 0.5))
        return t

    def cache_need(self):
        return FixedState((self.inner,))

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        n = self.names
        self.w_in = torch.cat([tensors[n["z"]], tensors[n["x"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.b_z = tensors[n["z"] + ".b"].float().contiguous() if self.bias else None
        self.b_x = tensors[n["x"] + ".b"].float().contiguous() if self.bias else None

    def forward(self, ctx, h, cache, residual=None, alpha: float = 1.0):
        ops, ws = self.ops, ctx.ws
        T, W = h.shape[0], self.inner
        proj = ws.get("mingru_proj", (T, 3 * W), torch.float32)
        ops.linear(h, self.w_in, proj)
        gated = ws.get("mingru_out", (T, W), self.dtype)
        ops.mingru(ctx, proj, (0, W, 2 * W), self.b_z, self.b_x, cache.state, gated)
        if residual is not None:
            ops.linear(gated, self.w_o, residual, accumulate=True, alpha=alpha)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(gated, self.w_o, y)
        return y
