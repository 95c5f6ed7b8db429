"""How a mixer, a feed-forward and their norms are arranged in one layer.

``pre_norm`` is the reference's block (garuda/src/llama/mod.rs:851-893):
``x += mixer(norm1(x)); x += ffn(norm2(x))``, the residual stream ``x`` in
32-bit throughout. A part may add into the residual itself (fused into its
last matrix product); if it returns a tensor instead, the block adds it.

Two things a model may add to that: a residual multiplier ``m`` (``x += m *
mixer(...)``, likewise the feed-forward), and branches that run after the
feed-forward and add to ``x`` from ``x`` itself (``parts.ResidualBranch``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .base import PartSpec, SublayerGate, TensorSpec, build_part, register_block, register_gate


@dataclass(frozen=True)
class BlockSpec:
    """One layer as data: which parts, with which parameters and tensor prefixes."""
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: PartSpec
    feed_forward_norm: Optional[PartSpec]
    arrangement: str = "pre_norm"
    residual_mult: float = 1.0                 # x += residual_mult * part(norm(x))
    branches: Tuple[PartSpec, ...] = ()        # after the feed-forward, in order
    # for an arrangement over a residual of several streams: how each sublayer is joined to them
    mixer_connection: Optional[PartSpec] = None
    feed_forward_connection: Optional[PartSpec] = None
    # for the arrangement that norms a sublayer's output: a gate on that output, per sublayer
    mixer_gate: Optional[PartSpec] = None
    feed_forward_gate: Optional[PartSpec] = None
    # for the arrangement that norms after the sum: x <- norm(post_alpha * x + part(x))
    post_alpha: float = 1.0


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward else None
        self.feed_forward_norm = (build_part("norm", spec.feed_forward_norm)
                                  if spec.feed_forward_norm else None)
        self.branches = [build_part("branch", b) for b in spec.branches]
        self.mult = float(spec.residual_mult)

    def parts(self):
        """(part, tensor-name prefix) pairs, for the loader."""
        s = self.spec
        out = [(self.mixer_norm, s.mixer_norm.prefix), (self.mixer, s.mixer.prefix)]
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, s.feed_forward_norm.prefix),
                    (self.feed_forward, s.feed_forward.prefix)]
        out += [(b, bs.prefix) for b, bs in zip(self.branches, s.branches)]
        return out

    def takes_pending_norm(self, ops):
        """The norm part that the layer in front may fold into its last product (see
        ``forward``'s ``pending``), or None."""
        if self.mult == 1.0 and getattr(ops, "folds_norms", False) and getattr(self.mixer, "takes_pending_norm", False) \
                and hasattr(self.mixer_norm, "fold"):
            return self.mixer_norm
        return None

    @property
    def graph_safe(self):
        return all(part.graph_safe for part, _ in self.parts())

    @staticmethod
    def _take_pending(ctx, x, added_in_place):
        """The one place where a folded norm changes hands: what the part that just ran left in
        ``ctx.pending_norm`` is taken out (the field is empty afterwards) and checked to be the
        norm of this block's residual stream. A part that returned its output instead of adding
        it in cannot have folded a norm of the sum; whatever it left is dropped."""
        p, ctx.pending_norm = ctx.pending_norm, None
        if p is None or not added_in_place:
            return None
        if p.x.data_ptr() != x.data_ptr() or tuple(p.x.shape) != tuple(x.shape):
            raise RuntimeError("a folded norm was left behind that is not of this block's residual stream")
        return p

    def forward(self, ctx, x, cache, pending=None, next_norm=None):
        """``pending``: this layer's first norm of ``x``, already half done by the layer in
        front (a ``PendingNorm``). ``next_norm``: the norm part that the next layer starts with,
        if that layer takes such a result. Returns the pending norm for the next layer, or None.
        Parts that know nothing of this are run with the plain norms."""
        ops = ctx.ops
        if self.mult != 1.0 or self.branches:
            return self._forward_scaled(ctx, x, cache)
        folds = getattr(ops, "folds_norms", False)
        h = pending if pending is not None else self.mixer_norm.forward(ctx, x)
        ff = self.feed_forward
        kw = {}
        if (folds and ff is not None and getattr(self.mixer, "emits_norm", False)
                and getattr(ff, "takes_pending_norm", False) and hasattr(self.feed_forward_norm, "fold")):
            kw["emit_norm"] = self.feed_forward_norm
        elif folds and ff is None and next_norm is not None and getattr(self.mixer, "emits_norm", False):
            kw["emit_norm"] = next_norm
        ctx.pending_norm = None
        y = self.mixer.forward(ctx, h, cache, residual=x, **kw)
        if y is not None:
            ops.residual_add(x, y)
        out = self._take_pending(ctx, x, y is None and "emit_norm" in kw)
        if ff is None:
            return out
        h2 = out if out is not None else self.feed_forward_norm.forward(ctx, x)
        kw = {}
        if folds and next_norm is not None and getattr(ff, "emits_norm", False):
            kw["emit_norm"] = next_norm
        y2 = ff.forward(ctx, h2, residual=x, **kw)
        if y2 is not None:
            ops.residual_add(x, y2)
        return self._take_pending(ctx, x, y2 is None and "emit_norm" in kw)

    def _run(self, ctx, part, x, h, *cache):
        """``x += mult * part(h)``: by the part itself if it takes the multiplier, else here."""
        if part.scales_residual:
            y = part.forward(ctx, h, *cache, residual=x, alpha=self.mult)
            if y is not None:
                ctx.ops.residual_axpy(x, y, self.mult)
        else:
            y = part.forward(ctx, h, *cache)
            if y is None:
                raise RuntimeError(f"{type(part).__name__} returned nothing although it was given no residual to add to")
            ctx.ops.residual_axpy(x, y, self.mult)

    def _forward_scaled(self, ctx, x, cache):
        """The block of a model with a residual multiplier or with branches: plain norms (nothing
        is folded across parts), every part's output scaled as it is added."""
        ctx.pending_norm = None
        self._run(ctx, self.mixer, x, self.mixer_norm.forward(ctx, x), cache)
        if self.feed_forward is not None:
            self._run(ctx, self.feed_forward, x, self.feed_forward_norm.forward(ctx, x))
        for branch in self.branches:
            branch.forward(ctx, x, self.mult)
        ctx.pending_norm = None
        return None


@register_gate("linear_sigmoid")
class LinearSigmoidGate(SublayerGate):
    """``sigmoid(W h + b)``, one gate per channel of the model's width. ``weight_name``: the local
    name of ``W [d, d]``; the bias is that name with ``.b`` added (``bias=False``: none)."""
    graph_safe = True

    def __init__(self, width: int, weight_name: str = "gate", bias: bool = True, init_std: float = 0.02):
        self.width, self.weight_name, self.has_bias, self.init_std = int(width), weight_name, bool(bias), float(init_std)

    def tensors(self):
        t = {self.weight_name: TensorSpec((self.width, self.width), init=("normal", self.init_std))}
        if self.has_bias:
            t[self.weight_name + ".b"] = TensorSpec((self.width,), role="vector", init=("normal", 0.5))
        return t

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.weight_name + ".b"].float().contiguous() if self.has_bias else None

    def logits(self, ctx, h, name="gate_logits"):
        out = ctx.ws.get(name, (h.shape[0], self.width), torch.float32)
        self.ops.linear(h, self.weight, out)
        return out


class BranchOutputs:
    """What a mixer made of several mixers hands to a block that norms sublayer outputs: the
    members' 32-bit outputs ``ys`` with a weight each; the mixer's output is the mean over the
    members of ``rms(y_b) * w_b``, which the block's one pass over the row computes."""

    def __init__(self, ys, weights, eps):
        self.ys, self.weights, self.eps = list(ys), list(weights), float(eps)

    def materialize(self, ctx, name="branches_out"):
        T, d = self.ys[0].shape
        out = ctx.ws.get(name, (T, d), torch.float32)
        ctx.ops.sublayer_merge(self.ys, self.weights, self.eps, out=out)
        return out


@register_block("sublayer_norm")
class SublayerNormBlock:
    """A layer whose sublayers read the residual itself and whose outputs are normed:
    ``x += norm1(gate1 * mixer(x)); x += norm2(gate2 * ffn(x))``, with ``gate = sigmoid(W x + b)``
    per channel from the sublayer's own input (``BlockSpec.mixer_gate`` / ``feed_forward_gate``;
    None: no gate). The residual is 32-bit; a sublayer's input is the residual rounded to the
    compute dtype (the residual itself in 32-bit runs); its output stays 32-bit through the gate,
    the norm and the sum, which are one pass over the row."""

    def __init__(self, spec: BlockSpec):
        if spec.residual_mult != 1.0 or spec.branches or spec.mixer_connection is not None:
            raise ValueError("a layer that norms its sublayers' outputs takes no multiplier, branches or streams")
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.mixer_gate = build_part("gate", spec.mixer_gate) if spec.mixer_gate else None
        self.feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward else None
        self.feed_forward_norm = build_part("norm", spec.feed_forward_norm) if spec.feed_forward else None
        self.feed_forward_gate = (build_part("gate", spec.feed_forward_gate)
                                  if spec.feed_forward and spec.feed_forward_gate else None)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "fold"):
                raise ValueError("a layer that norms its sublayers' outputs takes RMS norms")

    def parts(self):
        s = self.spec
        out = [(self.mixer_norm, s.mixer_norm.prefix), (self.mixer, s.mixer.prefix)]
        if self.mixer_gate is not None:
            out.append((self.mixer_gate, s.mixer_gate.prefix))
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, s.feed_forward_norm.prefix), (self.feed_forward, s.feed_forward.prefix)]
            if self.feed_forward_gate is not None:
                out.append((self.feed_forward_gate, s.feed_forward_gate.prefix))
        return out

    @property
    def graph_safe(self):
        return all(part.graph_safe for part, _ in self.parts())

    def takes_pending_norm(self, ops):
        """What the layer in front may leave for this one: nothing to fold, but a layer of the same
        arrangement writes this layer's rounded input in its last pass over the row."""
        return _ROUNDED_INPUT

    def _input(self, ctx, x, turn=0):
        if ctx.dtype == torch.float32:
            return x
        h = ctx.ws.get(f"sublayer_in_{turn}", tuple(x.shape), ctx.dtype)
        ctx.ops.cast(x, h)
        return h

    def _join(self, ctx, x, h, y, gate, norm, turn=None):
        """``x += norm(gate(h) * y)``. ``turn``: also write the new ``x`` rounded to the compute dtype
        into that buffer and return it (the next sublayer's input)."""
        weight, eps = norm.fold()
        logits = gate.logits(ctx, h) if gate is not None else None
        bias = gate.bias if gate is not None else None
        rounded = None
        if turn is not None and ctx.dtype == torch.bfloat16:
            rounded = ctx.ws.get(f"sublayer_in_{turn}", tuple(x.shape), ctx.dtype)
        if isinstance(y, BranchOutputs):
            ctx.ops.sublayer_merge(y.ys, y.weights, eps, x=x, gate=logits, gate_bias=bias, weight=weight, branch_eps=y.eps,
                                   rounded=rounded)
        else:
            ctx.ops.sublayer_merge([y], None, eps, x=x, gate=logits, gate_bias=bias, weight=weight, rounded=rounded)
        return rounded

    def forward(self, ctx, x, cache, pending=None, next_norm=None):
        """``pending``: this layer's input already rounded, by the layer in front. ``next_norm``: what
        the next layer said it takes; if that is a rounded input, the last pass writes it and it is
        returned."""
        ctx.pending_norm = None
        last = 1 if next_norm is _ROUNDED_INPUT else None
        h = pending if pending is not None else self._input(ctx, x, 1)
        ff = self.feed_forward
        # two buffers in turn: a sublayer's input is read by its gate while the pass writes the next one
        h2 = self._join(ctx, x, h, self.mixer.forward(ctx, h, cache), self.mixer_gate, self.mixer_norm,
                        turn=0 if ff is not None else last)
        if ff is None:
            return h2
        if h2 is None:
            h2 = self._input(ctx, x, 0)
        return self._join(ctx, x, h2, ff.forward(ctx, h2), self.feed_forward_gate, self.feed_forward_norm, turn=last)


class _RoundedInput:
    """Marker: the next layer takes its input (the residual rounded to the compute dtype) from
    the pass that last wrote the residual."""

    def __repr__(self):
        return "rounded input"


_ROUNDED_INPUT = _RoundedInput()


@register_block("post_norm")
class PostNormBlock:
    """A layer whose norms come after the sums and whose sublayers read the residual itself:
    ``x <- norm1(alpha * x + mixer(x)); x <- norm2(alpha * x + ffn(x))`` with ``alpha =
    BlockSpec.post_alpha``. The residual is 32-bit; a sublayer's input is the residual rounded to the
    compute dtype (the residual itself in 32-bit runs).

    An RMS norm does not see a factor on its input but for ``eps``: ``rms_eps(alpha v) =
    rms_(eps / alpha^2)(v)``. So a sublayer adds ``output / alpha`` into ``x`` (in its last product's
    epilogue, like every other block's sublayers), and one pass over the row then norms ``x`` in
    place with ``eps / alpha^2``, adds a deferred output bias on the way and writes the rounded
    input of the sublayer that reads ``x`` next. A part that cannot add into the residual returns its
    output, and the pass computes ``alpha * x + output`` as written."""

    def __init__(self, spec: BlockSpec):
        if spec.residual_mult != 1.0 or spec.branches or spec.mixer_connection is not None or spec.mixer_gate is not None:
            raise ValueError("a layer that norms after the sum takes no multiplier, branches, streams or gates")
        if not spec.post_alpha > 0:
            raise ValueError(f"post_alpha must be positive, got {spec.post_alpha}")
        self.spec = spec
        self.alpha = float(spec.post_alpha)
        self.mixer = build_part("mixer", spec.mixer)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward else None
        self.feed_forward_norm = build_part("norm", spec.feed_forward_norm) if spec.feed_forward else None
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "fold"):
                raise ValueError("a layer that norms after the sum takes RMS norms")

    def parts(self):
        s = self.spec
        out = [(self.mixer_norm, s.mixer_norm.prefix), (self.mixer, s.mixer.prefix)]
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, s.feed_forward_norm.prefix), (self.feed_forward, s.feed_forward.prefix)]
        return out

    @property
    def graph_safe(self):
        return all(part.graph_safe for part, _ in self.parts())

    def takes_pending_norm(self, ops):
        """A layer in front that makes a pass over the row anyway writes this layer's rounded input."""
        return _ROUNDED_INPUT

    def _input(self, ctx, x, turn):
        """The residual in the compute dtype. A 32-bit run gets a copy too: a part that adds into
        the residual in its last product may read its input again after that (a shared expert behind
        the routed ones)."""
        h = ctx.ws.get(f"sublayer_in_{turn}", tuple(x.shape), ctx.dtype)
        ctx.ops.cast(x, h)
        return h

    def _sublayer(self, ctx, x, h, part, norm, cache, turn):
        """``x <- norm(alpha * x + part(h))``; ``turn``: also write the new ``x`` rounded into that
        buffer and return it."""
        weight, eps = norm.fold()
        a = self.alpha
        kw = {"defer_bias": True} if part.defers_bias else {}
        args = (ctx, h) if cache is _NO_CACHE else (ctx, h, cache)
        rounded = None
        if turn is not None and ctx.dtype == torch.bfloat16:
            rounded = ctx.ws.get(f"sublayer_in_{turn}", tuple(x.shape), ctx.dtype)
        bias = part.output_bias if part.defers_bias else None
        if part.scales_residual:
            y = part.forward(*args, residual=x, alpha=1.0 / a, **kw)
            if y is None:
                if bias is not None:
                    bias = self._scaled(part, bias, 1.0 / a)
                ctx.ops.post_norm(x, None, 1.0, weight, eps / (a * a), row=bias, rounded=rounded)
                return rounded
        else:
            y = part.forward(*args, **kw)
            if y is None:
                raise RuntimeError(f"{type(part).__name__} returned nothing although it was given no residual to add to")
        ctx.ops.post_norm(x, y, a, weight, eps, row=bias, rounded=rounded)
        return rounded

    def _scaled(self, part, bias, factor):
        cache = self.__dict__.setdefault("_bias_rows", {})
        key = (id(part), factor)
        if key not in cache:
            cache[key] = (bias * factor).contiguous()
        return cache[key]

    def forward(self, ctx, x, cache, pending=None, next_norm=None):
        """``pending``: this layer's input already rounded, by the layer in front. ``next_norm``: what
        the next layer said it takes; if that is a rounded input, the last pass writes it and it is
        returned."""
        ctx.pending_norm = None
        last = 1 if next_norm is _ROUNDED_INPUT else None
        h = pending if pending is not None else self._input(ctx, x, 1)
        ff = self.feed_forward
        h2 = self._sublayer(ctx, x, h, self.mixer, self.mixer_norm, cache, 0 if ff is not None else last)
        if ff is None:
            return h2
        if h2 is None:
            h2 = self._input(ctx, x, 0)
        return self._sublayer(ctx, x, h2, ff, self.feed_forward_norm, _NO_CACHE, last)


_NO_CACHE = object()
