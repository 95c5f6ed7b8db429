"""Several mixers side by side: all read the same input, each output is RMS-normed over the
model's width with a weight of its own, and the mixer's output is their mean:

    y = (1 / n) * sum_b  y_b / sqrt(mean(y_b^2) + eps) * w_b

Each member keeps its own cache or state (pages for an attention, a fixed-size state for a
recurrent one), so the mixer's cache need is the tuple of its members' needs. A block that
norms sublayer outputs takes the members' outputs as they are and does the norms, the mean, its
own gate and norm and the residual sum in one pass over the row; any other block gets the mean
as a tensor.
"""
from __future__ import annotations

import torch

from .base import Mixer, PartSpec, TensorSpec, build_part, register_mixer
from .block import BranchOutputs


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """``members``: a list of ``{"name": registered mixer, "params": {...}, "prefix": local
    prefix of its tensors, "out": local name of its output norm's weight}``."""

    def __init__(self, width: int, eps: float, members):
        if not 1 <= len(members) <= 4:
            raise ValueError(f"one to four mixers run side by side, got {len(members)}")
        self.width, self.eps = int(width), float(eps)
        self.specs = [dict(m) for m in members]
        self.members = [build_part("mixer", PartSpec(m["name"], dict(m.get("params", {})))) for m in self.specs]

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.members)

    def tensors(self):
        t = {}
        for spec, member in zip(self.specs, self.members):
            for local, ts in member.tensors().items():
                t[spec["prefix"] + local] = ts
            t[spec["out"]] = TensorSpec((self.width,), role="vector", init=("normal_about_one", 0.1))
        return t

    def cache_need(self):
        return tuple(m.cache_need() for m in self.members)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.out_weights = []
        for spec, member in zip(self.specs, self.members):
            member.load({local: tensors[spec["prefix"] + local] for local in member.tensors()}, ops, dtype)
            self.out_weights.append(tensors[spec["out"]].float().contiguous())

    def forward(self, ctx, h, cache, residual=None):
        ys = [member.forward(ctx, h, cache.parts[i], out_name=f"member_y{i}")
              for i, member in enumerate(self.members)]
        out = BranchOutputs(ys, self.out_weights, self.eps)
        if residual is not None:
            self.ops.residual_add(residual, out.materialize(ctx))
            return None
        return out
