"""Typed configuration of the Luvapel design, read from its config.json.

Keys: ``architecture`` ("Luvapel"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``, ``layers`` (a list; each entry has ``type`` = ``parallel`` |
``general_delta``, the mixer's sizes under ``mixer``, its feed-forward under
``mlp`` or null, and optionally ``weights_of``: the index of another layer
whose tensors this layer runs with, keeping a cache and a state of its own),
``max_positions`` (optional: the longest sequence; the design itself has no
limit).

``parallel``: ``left`` (windowed attention: ``heads``, ``kv_heads``, ``dim``,
``vdim``, ``scale``, ``mask.size`` (optional: no mask, every earlier position
is read), ``rot.base`` and ``rot.dims`` (optional: no rotation)) and ``right``
(gated delta rule: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps).
``general_delta``: ``heads``, ``dim``; the rank of its decay's low-rank pair
comes from the tensors (``decay_rank`` may name it for random weights).
``mlp``: ``kind`` = ``dense``, ``ff``. Every size and constant of a model comes
from here; a key that is missing where the design needs it is an error that
names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .kavenex_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("parallel", "general_delta")
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]            # mask.size: positions a query looks back over, itself included
    rot_base: Optional[float]        # None: no rotation
    rot_dims: int


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: GatedDeltaConfig


@dataclass(frozen=True)
class GeneralDeltaConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class LuvapelLayer:
    type: str
    mixer: object
    mlp: Optional[DenseMlpConfig]
    weights_of: Optional[int] = None


def _heads(m, where):
    heads, kv_heads = _get(m, "heads", where, int, 1), _get(m, "kv_heads", where, int, 1)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{where}heads' = {heads} is not a multiple of '{where}kv_heads' = {kv_heads}")
    return heads, kv_heads


def _read_mixer(kind, m, wm):
    if kind == "general_delta":
        rank = m.get("decay_rank")
        return GeneralDeltaConfig(_get(m, "heads", wm, int, 1), _get(m, "dim", wm, int, 1), int(rank) if rank else None)
    left, wl = _get(m, "left", wm), wm + "left."
    heads, kv_heads = _heads(left, wl)
    dim, vdim = _get(left, "dim", wl, int, 1), _get(left, "vdim", wl, int, 1)
    if vdim != dim:
        raise ConfigError(f"config.json: '{wl}vdim' = {vdim} differs from '{wl}dim' = {dim}, but this mixer's values "
                          f"are its keys as projected")
    window = None
    if left.get("mask") is not None:
        window = _get(left["mask"], "size", wl + "mask.", int, 1)
    base, dims = None, 0
    if left.get("rot") is not None:
        base = _get(left["rot"], "base", wl + "rot.", float, 0.0)
        dims = _get(left["rot"], "dims", wl + "rot.", int, 2)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: '{wl}rot.dims' = {dims} must be even and at most '{wl}dim' = {dim}")
    attention = WindowAttentionConfig(heads, kv_heads, dim, vdim, _get(left, "scale", wl, float, 0.0), window, base, dims)
    right, wr = _get(m, "right", wm), wm + "right."
    heads, kv_heads = _heads(right, wr)
    delta = GatedDeltaConfig(heads, kv_heads, _get(right, "dim", wr, int, 1), _get(right, "vdim", wr, int, 1),
                             _get(right, "conv", wr, int, 1))
    return ParallelMixerConfig(attention, delta)


@dataclass(frozen=True)
class LuvapelConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[LuvapelLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "LuvapelConfig":
        vocab = _get(d, "vocab", "", int, 1)
        width = _get(d, "width", "", int, 1)
        scale = _get(d.get("embedding"), "scale", "embedding.", float)
        eps = _get(d.get("norm"), "eps", "norm.", float, 0.0)
        entries = _get(d, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            kind = _get(e, "type", w)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{w}type' = {kind!r} is not a mixer of this design {MIXER_TYPES}")
            mixer = _read_mixer(kind, _get(e, "mixer", w), w + "mixer.")
            mlp = None
            if e.get("mlp") is not None:
                f = e["mlp"]
                mk = _get(f, "kind", w + "mlp.")
                if mk != "dense":
                    raise ConfigError(f"config.json: '{w}mlp.kind' = {mk!r}: this design's feed-forward is 'dense'")
                mlp = DenseMlpConfig(_get(f, "ff", w + "mlp.", int, 1))
            src = e.get("weights_of")
            if src is not None:
                src = _get(e, "weights_of", w, int, 0)
                if src >= len(entries) or src == i:
                    raise ConfigError(f"config.json: '{w}weights_of' = {src} must name another layer")
            layers.append(LuvapelLayer(kind, mixer, mlp, src))
        for i, layer in enumerate(layers):
            # a layer may name one that names another: follow to the layer that has the tensors
            src, seen = layer.weights_of, {i}
            while src is not None and layers[src].weights_of is not None:
                if src in seen:
                    raise ConfigError(f"config.json: 'layers[{i}].weights_of' leads back to itself")
                seen.add(src)
                src = layers[src].weights_of
            if src is not None:
                if (layers[src].type, layers[src].mixer, layers[src].mlp) != (layer.type, layer.mixer, layer.mlp):
                    raise ConfigError(f"config.json: layer {i} runs with the tensors of layer {src} but its sizes differ")
                layers[i] = LuvapelLayer(layer.type, layer.mixer, layer.mlp, src)
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        return cls(architecture=d.get("architecture", "Luvapel"), vocab=vocab, width=width, embedding_scale=scale,
                   eps=eps, layers=tuple(layers), max_positions=int(d.get("max_positions") or DEFAULT_MAX_POSITIONS),
                   eos_token_ids=eos, raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)
