"""The Midulorn decoder as a ``ModelSpec``.

An embedding times a constant; layers whose norms come after the sums, ``x <- norm(alpha x +
sublayer(x))``, the sublayers reading the residual itself. A layer's mixer is one of three:
attention behind short causal convolutions, with normed queries and keys, no position encoding
but a term that grows with the logarithm of the distance, a mask of fixed stretches of
positions, a learned sink per head, biases on its four projections, and values that are mixed
with those of the first such layer; attention over a cached latent with one rotated key part
for all heads (pairs ``(i, i + dims / 2)``), a learned sink per head and a gate per head; or a
recurrence per channel whose gate and candidate are functions of the current token alone. The feed-forward is
``down(xielu(up h))`` or routed experts weighed by their share of a softmax over all experts,
or absent. A final norm; the head is the embedding table, the logits times a constant.
Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.midulorn_config import MidulornConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.block import BlockSpec
from .decoder import ModelSpec, LayerCall


def _norm(cfg, prefix, name):
    return PartSpec("rms", dict(width=cfg.width, eps=cfg.eps, weight_name=name), prefix=prefix)


def _mixer(cfg, layer, p, first_mixed):
    m = layer.mixer
    if layer.type == "mingru":
        return PartSpec("mingru", dict(width=cfg.width, inner=m.width, bias=True), prefix=p)
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", dict(
            width=cfg.width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
            eps=cfg.eps, rot_base=m.rot_base, rot_dims=m.rot_dims, rot_layout="half", sink=True, head_gate=True), prefix=p)
    mix = None
    if m.v_mix:
        mix = "source" if first_mixed else "mix"
    return PartSpec("convolved_attention", dict(
        width=cfg.width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, taps=m.taps,
        qk_norm=True, eps=cfg.eps, bias=True, distance=True, chunk=m.chunk, sink=True, value_mix=mix), prefix=p)


def _feed_forward(cfg, f, p):
    if f is None:
        return None
    if f.kind == "dense":
        return PartSpec("plain", dict(width=cfg.width, inner=f.ff, activation="xielu"), prefix=p)
    return PartSpec("routed_experts", dict(width=cfg.width, experts=f.experts, top=f.top, inner=f.ff, activation="silu",
                                           router_bias=False, router_score="softmax_all"), prefix=p)


def midulorn_spec(cfg: MidulornConfig) -> ModelSpec:
    layers, ignored, seen_mixed = [], [], False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        first_mixed = layer.type == "attention" and layer.mixer.v_mix and not seen_mixed
        seen_mixed = seen_mixed or first_mixed
        ff = _feed_forward(cfg, layer.mlp, p + "mlp.")
        if ff is None:
            ignored.append(p + "norm2")
        if layer.type == "attention" and not layer.mixer.v_mix:
            ignored.append(p + "mix.vmix")           # (a folder may carry the mixing weight of a layer that mixes nothing)
        layers.append(BlockSpec(mixer=_mixer(cfg, layer, p + "mix.", first_mixed), feed_forward=ff,
                                mixer_norm=_norm(cfg, p, "norm1"),
                                feed_forward_norm=_norm(cfg, p, "norm2") if ff is not None else None,
                                arrangement="post_norm", post_alpha=cfg.post_alpha))
    return ModelSpec(
        architecture=cfg.architecture, width=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding="embed", layers=layers, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=_norm(cfg, "", "final.norm"), head=None, embedding_scale=cfg.embedding_scale,
        logit_scale=cfg.logit_scale, eos_token_ids=cfg.eos_token_ids, ignored_tensors=tuple(ignored))


register_architecture("Midulorn", MidulornConfig.from_dict, midulorn_spec)
