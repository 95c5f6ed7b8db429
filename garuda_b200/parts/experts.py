"""A feed-forward of routed experts: a router picks ``top`` of ``experts`` small
gated feed-forwards per token, their outputs are summed with the router's
weights, and an optional shared expert runs for every token.

    z      = W_r h + b_r                      (32-bit)
    chosen = the ``top`` largest z, weights = softmax over the chosen z only
    expert(h) = W_down act(W_gate h, W_up h)  (``act`` as in ``GatedFeedForward``)
    out    = sum_chosen weight_e * expert_e(h) + shared(h)

Variants, by constructor parameter: ``router_score="sigmoid"`` weighs a chosen expert by
``sigmoid(z_e)`` (the choice is still of the largest; nothing is renormalized);
``router_score="softmax_all"`` weighs it by its share of the softmax over all experts' logits
(not renormalized over the chosen either);
``scale_input=True`` puts the weight on what goes into the expert, ``out = sum_chosen
expert_e(weight_e * h)``; ``router_bias=False`` drops ``b_r``; ``activation="silu"`` is the plain
SiLU gate.

Tensor names: ``router``, ``router.b``, ``e<i>.gate|up|down``, ``shared.gate|up|down``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True
    scales_residual = True

    def __init__(self, width: int, experts: int, top: int, inner: int, activation: str = "clamped_swish",
                 limit: float = 0.0, shared_inner: Optional[int] = None, shared_limit: float = 0.0,
                 router_bias: bool = True, init_std: float = 0.02, router_score: str = "softmax_chosen",
                 scale_input: bool = False):
        if router_score not in ("softmax_chosen", "sigmoid", "softmax_all"):
            raise ValueError(f"unknown router score {router_score!r}")
        self.router_score, self.scale_input = router_score, bool(scale_input)
        if not 1 <= top <= experts:
            raise ValueError(f"a token uses 1 to {experts} experts, got {top}")
        self.width, self.experts, self.top, self.inner = int(width), int(experts), int(top), int(inner)
        self.activation, self.limit = activation, float(limit)
        self.shared_inner = int(shared_inner) if shared_inner else None
        self.shared_limit = float(shared_limit)
        self.router_bias = bool(router_bias)
        self.init_std = float(init_std)

    def tensors(self):
        init = ("normal", self.init_std)
        t = {"router": TensorSpec((self.experts, self.width), init=init)}
        if self.router_bias:
            t["router.b"] = TensorSpec((self.experts,), role="vector", init=("normal", 0.02))
        for e in range(self.experts):
            t[f"e{e}.gate"] = TensorSpec((self.inner, self.width), init=init)
            t[f"e{e}.up"] = TensorSpec((self.inner, self.width), init=init)
            t[f"e{e}.down"] = TensorSpec((self.width, self.inner), init=init)
        if self.shared_inner:
            t["shared.gate"] = TensorSpec((self.shared_inner, self.width), init=init)
            t["shared.up"] = TensorSpec((self.shared_inner, self.width), init=init)
            t["shared.down"] = TensorSpec((self.width, self.shared_inner), init=init)
        return t

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.w_router = tensors["router"].contiguous()
        self.b_router = tensors["router.b"].float().contiguous() if self.router_bias else None
        E = self.experts
        # the experts' gate and up rows stacked in the kernels' layout; [E, width, inner]
        self.w_gate_up = ops.pack_expert_gate_up([tensors[f"e{e}.gate"] for e in range(E)],
                                                 [tensors[f"e{e}.up"] for e in range(E)])
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared_inner:
            self.w_shared_gate_up = ops.pack_gate_up(tensors["shared.gate"], tensors["shared.up"])
            self.w_shared_down = tensors["shared.down"].contiguous()

    def forward(self, ctx, h, residual=None, alpha: float = 1.0):
        ops, ws = self.ops, ctx.ws
        T = h.shape[0]
        target = residual
        if target is None:
            target = ws.get("ffn_out", (T, self.width), torch.float32)
            target.zero_()
            alpha = 1.0
        ids = ws.get("expert_ids", (T, self.top), torch.int32)
        weights = ws.get("expert_weights", (T, self.top), torch.float32)
        if self.router_score == "softmax_chosen" and not self.scale_input:
            ops.route_topk(h, self.w_router, self.b_router, self.top, ids, weights)
            ops.routed_feed_forward(ctx, h, self.w_gate_up, self.w_down, ids, weights, target, self.activation,
                                    self.limit, alpha)
        else:
            ops.route_topk(h, self.w_router, self.b_router, self.top, ids, weights, score=self.router_score)
            ops.routed_feed_forward(ctx, h, self.w_gate_up, self.w_down, ids, weights, target, self.activation,
                                    self.limit, alpha, scale_input=self.scale_input)
        if self.shared_inner:
            act = ws.get("shared_act", (T, self.shared_inner), self.dtype)
            ops.linear_gated(ctx, h, self.w_shared_gate_up, act, self.activation, self.shared_limit)
            ops.linear(act, self.w_shared_down, target, accumulate=True, alpha=alpha)
        return None if residual is not None else target
