"""Tiny Luvapel configurations of the tests, their model folders and plain logits.

The configurations differ from one another in every size and option: windows shorter and longer
than a page and no mask at all; rotations of the whole head, of its first channels only, none;
groups of one, two and four query heads per key head; delta-rule heads that share query/key
heads or not; one to five taps; key and value widths that are unequal and no multiple of 8;
layers without a feed-forward; layers that run with an earlier layer's tensors (of both kinds);
widths and ranks that no tensor-core kernel takes, and sizes that they do take.
"""
from __future__ import annotations

import tempfile

import numpy as np
import torch


def _par(left, right, mlp, **kw):
    return dict({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}, **kw)


def _left(heads, kv_heads, dim, scale, size=None, base=None, dims=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if base is not None:
        m["rot"] = {"base": base, "dims": dims}
    return m


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _gd(heads, dim, mlp, rank=6, **kw):
    return dict({"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}, **kw)


def _ff(n):
    return {"kind": "dense", "ff": n}


# a window shorter than a page of 8, a rotation of half the head, delta heads that share key heads,
# a layer without a feed-forward, a layer of each kind that runs with an earlier layer's tensors
LA = {"architecture": "Luvapel", "vocab": 131, "width": 48, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
      "layers": [_par(_left(4, 2, 16, 0.45, size=6, base=10000.0, dims=8), _right(4, 2, 12, 20, 3), _ff(40)),
                 _gd(3, 16, None),
                 _par(_left(4, 2, 16, 0.45, size=6, base=10000.0, dims=8), _right(4, 2, 12, 20, 3), _ff(40), weights_of=0),
                 _gd(2, 24, _ff(56), rank=5),
                 _gd(3, 16, None, weights_of=1)]}

# no mask and no rotation, as many key heads as heads, one tap, one delta head, the general rule first
LB = {"architecture": "Luvapel", "vocab": 97, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
      "layers": [_gd(1, 40, _ff(24), rank=3),
                 _par(_left(3, 3, 8, 0.6), _right(1, 1, 8, 12, 1), None)]}

# sizes the tensor-core kernels take: head width 64, groups of four, a window of more than two pages
# of 32, the whole head rotated; a wider general rule
LC = {"architecture": "Luvapel", "vocab": 320, "width": 128, "embedding": {"scale": 6.0}, "norm": {"eps": 1e-5},
      "layers": [_par(_left(8, 2, 64, 0.2, size=70, base=1000000.0, dims=64), _right(4, 2, 32, 64, 2), _ff(192)),
                 _gd(2, 64, _ff(256), rank=16),
                 _gd(2, 64, _ff(256), rank=16, weights_of=1),
                 _par(_left(2, 1, 128, 0.12, size=33, base=500.0, dims=32), _right(2, 2, 64, 32, 5), _ff(128))]}

# one layer of mixers side by side and nothing else: what the attention reads is exactly its window
LD = {"architecture": "Luvapel", "vocab": 64, "width": 32, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
      "layers": [_par(_left(2, 1, 16, 0.7, size=9, base=100.0, dims=16), _right(1, 1, 8, 8, 2), None)]}

CASES = {"LA": (LA, 31), "LB": (LB, 32), "LC": (LC, 33), "LD": (LD, 34)}

# Random N(0, 0.02) weights leave every gate at one half and every decay alike; these factors spread
# the gates' and decays' logits, the delta rules' writes and the logits (the attention's scores are
# spread by the configurations' scale, since queries and keys are normed).
SHARPEN = {"mix.left.g": 6.0, "mix.left.o": 5.0, "mix.right.q": 5.0, "mix.right.k": 5.0, "mix.right.v": 6.0,
           "mix.right.b": 8.0, "mix.right.a": 8.0, "mix.right.g": 6.0, "mix.right.o": 5.0, "mix.r": 5.0, "mix.k": 5.0,
           "mix.v": 5.0, "mix.a": 8.0, "mix.g": 6.0, "mix.w1": 8.0, "mix.o": 5.0, ".rg1": 8.0, ".rg2": 8.0, ".up": 6.0,
           ".down": 4.0, "head": 6.0, "embed": 25.0}

_DIRS, _PLAIN = {}, {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed = CASES[name]
        d = tempfile.mkdtemp(prefix=f"garuda_luvapel_{name}_")
        write_random_model(d, cfg, seed, store_dtype=store_dtype, scale=SHARPEN)
        _DIRS[key] = d
    return _DIRS[key]


def weights(name: str, store_dtype=torch.float32) -> dict:
    from tests.helpers import folder_weights
    return folder_weights(model_dir(name, store_dtype))


def plain_logits(name: str, store_dtype, tokens) -> np.ndarray:
    from tests.plain import luvapel_plain
    key = (name, store_dtype, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = luvapel_plain.forward(CASES[name][0], weights(name, store_dtype), tokens).astype(np.float32)
    return _PLAIN[key]


def random_tokens(name: str, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, CASES[name][0]["vocab"], n).tolist()
