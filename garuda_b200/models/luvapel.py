"""The Luvapel decoder as a ``ModelSpec``.

An embedding times a constant; layers whose sublayers read the residual itself and whose
outputs are gated per channel (``sigmoid(W x + b)`` of the sublayer's input), RMS-normed and then
added. A layer's mixer is either two mixers side by side (sliding-window attention with normed,
partly rotated queries and keys, the keys as projected for values, a temperature per head and a
gated output; and a gated delta rule with one decay per head behind short convolutions), their
outputs normed and averaged, or a generalized delta rule with a decay and a removal rate per key
channel. The feed-forward is ``down(relu(up h)^2)``, or absent. A layer may run with the tensors
of an earlier layer, keeping a cache and a state of its own. A final norm and an output head.
Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm2``,
``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.up|down``.
"""
from __future__ import annotations

from ..config.luvapel_config import LuvapelConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.block import BlockSpec
from .decoder import ModelSpec, LayerCall


def _norm(cfg, prefix, name):
    return PartSpec("rms", dict(width=cfg.width, eps=cfg.eps, weight_name=name), prefix=prefix)


def _mixer(cfg, layer, p):
    m = layer.mixer
    if layer.type == "general_delta":
        return PartSpec("general_delta_rule", dict(width=cfg.width, heads=m.heads, dim=m.dim, eps=cfg.eps,
                                                   decay_rank=m.decay_rank), prefix=p + "mix.")
    a, r = m.left, m.right
    left = dict(name="normed_key_attention", prefix="left.", out="left.out", params=dict(
        width=cfg.width, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, scale=a.scale, window=a.window,
        rot_base=a.rot_base, rot_dims=a.rot_dims, rot_layout="interleaved", qk_norm=True, eps=cfg.eps, temperature=True,
        values="keys", gate=True))
    right = dict(name="head_delta_rule", prefix="right.", out="right.out", params=dict(
        width=cfg.width, heads=r.heads, kv_heads=r.kv_heads, dim=r.dim, vdim=r.vdim, taps=r.taps, eps=cfg.eps, gate="silu"))
    return PartSpec("parallel_mixers", dict(width=cfg.width, eps=cfg.eps, members=[left, right]), prefix=p + "mix.")


def luvapel_spec(cfg: LuvapelConfig) -> ModelSpec:
    layers, ignored, at = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        ff = None
        if layer.mlp is not None:
            ff = PartSpec("plain", dict(width=cfg.width, inner=layer.mlp.ff, activation="relu2"), prefix=p + "mlp.")
        else:
            ignored += [p + "norm2", p + "rg2", p + "rg2.b"]
        gate = lambda name: PartSpec("linear_sigmoid", dict(width=cfg.width, weight_name=name), prefix=p)
        at[i] = len(layers)
        layers.append(BlockSpec(mixer=_mixer(cfg, layer, p), feed_forward=ff, mixer_norm=_norm(cfg, p, "norm1"),
                                feed_forward_norm=_norm(cfg, p, "norm2") if ff is not None else None,
                                arrangement="sublayer_norm", mixer_gate=gate("rg1"),
                                feed_forward_gate=gate("rg2") if ff is not None else None))
    # a layer that names another runs that layer's block again, with a cache and a state of its own
    order = [LayerCall(at[i if layer.weights_of is None else layer.weights_of]) for i, layer in enumerate(cfg.layers)]
    return ModelSpec(
        architecture=cfg.architecture, width=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding="embed", layers=layers, order=order, final_norm=_norm(cfg, "", "final.norm"), head="head",
        embedding_scale=cfg.embedding_scale, eos_token_ids=cfg.eos_token_ids, ignored_tensors=tuple(ignored))


register_architecture("Luvapel", LuvapelConfig.from_dict, luvapel_spec)
