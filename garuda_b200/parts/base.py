"""Interfaces of the parts a decoder is put together from, and their registries.

A part is a mixer (attention here), a feed-forward, a norm or a position
encoding. Each takes its sizes and constants as constructor parameters, names
the tensors it needs, and knows nothing about the model it sits in: the same
class serves any layer of any architecture, and a model may name different
parts in different layers. The reference keeps these as methods of one struct
(garuda/src/llama/mod.rs:733-1020); here each is a class chosen by name.

A new part is added by subclassing the matching base class and registering it
with ``register_mixer`` / ``register_feed_forward`` / ``register_norm`` /
``register_position_encoding``; a model's layer list then refers to it by that
name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Optional, Tuple

import torch


# --------------------------------------------------------------------------
# what a part asks of the loader and of the cache
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs. ``role`` is ``"matrix"`` (an operand of a
    contraction or an embedding table: held in the compute dtype), ``"vector"``
    (a norm weight or the like: a tensor stored in 32-bit stays 32-bit) or
    ``"table"`` (integers: held as int32). ``init`` describes the random-weights
    mode: ``("normal", std)``, ``("ones",)``, ``("normal_about_one", std)``, ``("uniform", low, high)`` or ``("normal_about_identity", std)``. A size that
    the configuration does not give (the rank of a low-rank pair of matrices) is written ``None``
    in ``shape``: the loader takes what the file has there and checks the other sizes;
    random weights use ``free`` for it."""
    shape: Tuple[Optional[int], ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    free: int = 16

    def fits(self, shape) -> bool:
        return len(shape) == len(self.shape) and all(w is None or int(w) == int(s) for w, s in zip(self.shape, shape))

    def concrete(self) -> Tuple[int, ...]:
        return tuple(self.free if s is None else int(s) for s in self.shape)


@dataclass(frozen=True)
class PagedKV:
    """A mixer that keeps one key and one value vector per position.
    ``window``: positions a query may look back over, itself included
    (garuda/src/cache/mod.rs:333-338); ``None`` keeps everything. ``value_dim``: the width of
    a value vector where it differs from the key's (``None``: ``head_dim``). ``keep_first``: with a
    window, the first positions of a request that every later query still reads; their pages stay
    with the request while the pages between them and the window go back to the pool. ``chunk``
    n (instead of a window): a query reads only the positions of its own stretch of n,
    ``floor(j / n) = floor(i / n)``; the pages of the stretches in front go back to the pool."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None
    keep_first: int = 0
    chunk: Optional[int] = None


@dataclass(frozen=True)
class PagedLatent:
    """A mixer that keeps one vector per position, shared by all its heads (a compressed
    latent from which keys and values are computed, with whatever rides along: a rotated key
    part). The pool is ``[num_pages, 1, page_size, width]`` and comes as ``LayerCache.k``;
    there is no second pool. ``window`` as for ``PagedKV``."""
    width: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A mixer that keeps a state of fixed size per request
    (garuda/src/cache/mod.rs:630-648 is the reference's example)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one layer call sees of the cache during a step.

    For ``PagedKV``: ``k`` and ``v`` are this call's slices of its group's page
    pool, ``[num_pages, kv_heads, page_size, head_dim]``; ``block_table`` is the
    group's table for the requests of the batch, ``[R, max_pages]`` int32 (-1
    where a page has been given back). ``writes`` is False for a call that reads
    another call's cache. For ``FixedState``: ``state`` is ``[max_slots, *shape]``
    and the batch's ``slots`` index it. For a mixer made of several mixers (its ``cache_need()``
    is a tuple): ``parts`` holds one ``LayerCache`` (or None) per entry of the tuple.
    """
    need: object
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None
    writes: bool = True
    parts: Optional[tuple] = None


# --------------------------------------------------------------------------
# base classes
# --------------------------------------------------------------------------

class Part:
    """Common behaviour: tensors by local name, bound once after loading."""

    #: Whether a decode step through this part may be captured in a CUDA graph and replayed: every
    #: launch must read the batch from the device arrays of ``ctx.batch`` only (a replayed step has
    #: no host copies, ``ctx.batch.host`` is empty), launch the same kernels whatever the batch
    #: holds, and allocate nothing. The built-in parts say True; a part that says nothing is run
    #: kernel by kernel.
    graph_safe = False
    #: A mixer or feed-forward that says True takes ``alpha`` in ``forward`` and adds ``alpha *
    #: output`` into the residual itself (a model's residual multiplier); for one that does not,
    #: the block scales and adds what it returns.
    scales_residual = False
    #: A part whose output ends with a constant row (an output projection's bias) may say True and
    #: keep that row, 32-bit ``[width]``, as ``output_bias``: a block that makes a pass over the residual
    #: anyway then calls ``forward(..., defer_bias=True)``, gets the output without the row and adds
    #: the row (scaled as the output is) in its own pass. Without ``defer_bias`` the part adds it itself.
    defers_bias = False
    output_bias = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], ops, dtype: torch.dtype) -> None:
        """Receive the device tensors named by ``tensors()`` (already in the dtype
        their role asks for). ``ops`` is the kernel set, ``dtype`` the compute dtype."""
        self.ops = ops
        self.dtype = dtype


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` is the 32-bit residual stream ``[T, d]``; returns ``[T, d]`` (or
        ``[len(rows), d]``) in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into a change of the query and key vectors."""
    #: a rotary encoding that the fused rotate-and-store kernel can apply
    rotary = None
    #: False for an encoding that leaves queries and keys alone
    changes_vectors = True

    def apply(self, ctx, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """In place on ``q [T, Hq, hd]`` and ``k [T, Hkv, hd]`` (32-bit)."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        """``PagedKV``, ``PagedLatent``, ``FixedState`` or ``None``; a mixer that is made of several
        mixers gives a tuple with one of these per member, and gets a ``LayerCache`` whose ``parts``
        are the members' caches in that order."""
        return None

    def forward(self, ctx, h: torch.Tensor, cache: Optional[LayerCache],
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """``h``: normed input ``[T, d]`` in the compute dtype. Either returns
        the output ``[T, d]`` or, when ``residual`` (32-bit ``[T, d]``) is given
        and the part can add into it itself, adds there and returns ``None``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Connection(Part):
    """How a sublayer is joined to a residual that is kept as several streams ``x [T, S, d]``
    (32-bit): ``read`` gives the sublayer's normed input, ``write`` takes its output ``y [T, d]``
    (32-bit) and updates every stream."""

    def read(self, ctx, x: torch.Tensor, norm) -> torch.Tensor:
        raise NotImplementedError

    def write(self, ctx, x: torch.Tensor, y: torch.Tensor) -> None:
        raise NotImplementedError


class SublayerGate(Part):
    """A gate on a sublayer's output, computed from the sublayer's input: ``logits(ctx, h)`` gives
    32-bit ``[T, d]`` logits (without the bias, which ``bias`` holds, 32-bit ``[d]`` or None); the
    block multiplies the sublayer's output by their sigmoid."""
    bias = None

    def logits(self, ctx, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class ResidualBranch(Part):
    """Something a layer adds to the residual stream after its mixer and feed-forward, computed
    from the stream itself and the step's tokens (a per-layer token embedding, gated): it reads
    no norm of the block and keeps no cache."""

    def forward(self, ctx, x: torch.Tensor, alpha: float = 1.0) -> None:
        """Adds ``alpha * branch(x)`` into ``x`` (32-bit ``[T, d]``)."""
        raise NotImplementedError


# --------------------------------------------------------------------------
# registries: name -> class
# --------------------------------------------------------------------------

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {}, "branch": {},
    "connection": {}, "gate": {},
}


def _register(kind: str, name: str, cls=None):
    def deco(c):
        _REGISTRIES[kind][name] = c
        return c
    return deco(cls) if cls is not None else deco


def register_mixer(name, cls=None): return _register("mixer", name, cls)
def register_feed_forward(name, cls=None): return _register("feed_forward", name, cls)
def register_norm(name, cls=None): return _register("norm", name, cls)
def register_position_encoding(name, cls=None): return _register("position_encoding", name, cls)
def register_block(name, cls=None): return _register("block", name, cls)
def register_branch(name, cls=None): return _register("branch", name, cls)
def register_connection(name, cls=None): return _register("connection", name, cls)
def register_gate(name, cls=None): return _register("gate", name, cls)


@dataclass(frozen=True)
class PartSpec:
    """A part named as data: registry ``kind``, registered ``name``, constructor
    parameters, and the prefix its tensor names get in the checkpoint. A local tensor name that
    starts with ``@`` is a name of the model's own, shared by parts of several layers: it takes no
    prefix (``@side.embed`` is the checkpoint's ``side.embed``)."""
    name: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


def tensor_name(prefix: str, local: str) -> str:
    """The checkpoint's name of a part's tensor."""
    return local[1:] if local.startswith("@") else prefix + local


def build_part(kind: str, spec: PartSpec):
    try:
        cls = _REGISTRIES[kind][spec.name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[kind])) or "none"
        raise KeyError(f"no {kind} named '{spec.name}' is registered (registered: {known})") from None
    return cls(**spec.params)
