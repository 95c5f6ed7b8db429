"""Typed configuration of the Midulorn design, read from its config.json.

Keys: ``architecture`` ("Midulorn"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``, ``postln_alpha``, ``logit_scale``, ``layers`` (a list; each entry
has ``type`` = ``attention`` | ``latent_attention`` | ``mingru``, the mixer's
sizes under ``mixer``, its feed-forward under ``mlp`` or null),
``max_positions`` (optional: the longest sequence; the design itself has no
limit).

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv``
(taps; optional: no convolution), ``mask.size`` (optional: every earlier
position is read), ``v_mix`` (optional).
``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``,
``scale``, ``rot.base``, ``rot.dims``.
``mingru``: ``width``.
``mlp``: ``kind`` = ``dense`` (``ff``) | ``moe`` (``expert.ff``,
``router.experts``, ``router.top``).
Every size and constant of a model comes from here; a key that is missing
where the design needs it is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .kavenex_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("attention", "latent_attention", "mingru")
DEFAULT_MAX_POSITIONS = 32768


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    taps: Optional[int]          # None: no convolution
    chunk: Optional[int]         # mask.size: a query reads the positions of its own stretch of this many
    v_mix: bool


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class MinGruConfig:
    width: int


@dataclass(frozen=True)
class MlpConfig:
    kind: str                    # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class MidulornLayer:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


def _read_mixer(kind, m, wm):
    if kind == "mingru":
        return MinGruConfig(_get(m, "width", wm, int, 1))
    heads = _get(m, "heads", wm, int, 1)
    dim, vdim = _get(m, "dim", wm, int, 1), _get(m, "vdim", wm, int, 1)
    scale = _get(m, "scale", wm, float, 0.0)
    if kind == "latent_attention":
        rot_dim = _get(m, "rot_dim", wm, int, 0)
        rot = _get(m, "rot", wm)
        base, dims = _get(rot, "base", wm + "rot.", float, 0.0), _get(rot, "dims", wm + "rot.", int, 0)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: '{wm}rot.dims' = {dims} must be even and at most '{wm}rot_dim' = {rot_dim}")
        return LatentConfig(heads, dim, rot_dim, vdim, _get(m, "kv_rank", wm, int, 1), scale, base, dims)
    kv_heads = _get(m, "kv_heads", wm, int, 1)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{wm}heads' = {heads} is not a multiple of '{wm}kv_heads' = {kv_heads}")
    taps = _get(m, "conv", wm, int, 1) if m.get("conv") is not None else None
    if taps is not None and taps > 16:
        raise ConfigError(f"config.json: '{wm}conv' = {taps}: at most 16 taps")
    chunk = _get(m["mask"], "size", wm + "mask.", int, 1) if m.get("mask") is not None else None
    return ChunkedAttentionConfig(heads, kv_heads, dim, vdim, scale, taps, chunk, bool(m.get("v_mix", False)))


def _read_mlp(f, w):
    kind = _get(f, "kind", w)
    if kind == "dense":
        return MlpConfig("dense", _get(f, "ff", w, int, 1))
    if kind == "moe":
        router = _get(f, "router", w)
        experts, top = _get(router, "experts", w + "router.", int, 1), _get(router, "top", w + "router.", int, 1)
        if top > experts:
            raise ConfigError(f"config.json: '{w}router.top' = {top} is more than '{w}router.experts' = {experts}")
        return MlpConfig("moe", _get(_get(f, "expert", w), "ff", w + "expert.", int, 1), experts, top)
    raise ConfigError(f"config.json: '{w}kind' = {kind!r}: this design's feed-forwards are 'dense' and 'moe'")


@dataclass(frozen=True)
class MidulornConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    post_alpha: float
    logit_scale: float
    layers: Tuple[MidulornLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "MidulornConfig":
        vocab = _get(d, "vocab", "", int, 1)
        width = _get(d, "width", "", int, 1)
        scale = _get(d.get("embedding"), "scale", "embedding.", float)
        eps = _get(d.get("norm"), "eps", "norm.", float, 0.0)
        alpha = _get(d, "postln_alpha", "", float, 0.0)
        logit_scale = _get(d, "logit_scale", "", float)
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
            mlp = _read_mlp(e["mlp"], w + "mlp.") if e.get("mlp") is not None else None
            layers.append(MidulornLayer(kind, mixer, mlp))
        mixed = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if any(m.kv_heads * m.vdim != mixed[0].kv_heads * mixed[0].vdim for m in mixed):
            raise ConfigError("config.json: layers with 'v_mix' must have values of one width (kv_heads * vdim)")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        return cls(architecture=d.get("architecture", "Midulorn"), vocab=vocab, width=width, embedding_scale=scale,
                   eps=eps, post_alpha=alpha, logit_scale=logit_scale, layers=tuple(layers),
                   max_positions=int(d.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos, raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)
