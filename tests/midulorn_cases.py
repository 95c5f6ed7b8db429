"""Tiny Midulorn configurations for the tests, their model folders and the plain model's logits.

The configurations differ from one another in every size and option: chunks of 5, 12, 24 and 70
positions and no mask; 1 to 5 taps and no convolution; one, two and three query heads per key
head; key and value widths that are unequal and no multiple of 8; a rotation of the whole rotated
part and of its first channels only; latent widths that the tensor-core kernel takes and ones
it does not; layers without a feed-forward; one to three layers with mixed values; residual
factors of 1, 1.7, 2 and 3.5; one expert chosen of several, all of them chosen, and more.
"""
import tempfile

import numpy as np
import torch


def _att(heads, kv_heads, dim, vdim, scale, conv=None, size=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if size:
        m["mask"] = {"size": size}
    if v_mix:
        m["v_mix"] = True
    return m


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# all three mixers, both feed-forwards; sizes no tensor-core kernel takes (widths 40 and 44, heads of 12, 20, 10)
MA = {"architecture": "Midulorn", "vocab": 96, "width": 40, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
      "postln_alpha": 1.7, "logit_scale": 0.5,
      "layers": [_layer("attention", _att(4, 2, 12, 20, 0.4, conv=3, size=12, v_mix=True), _dense(56)),
                 _layer("latent_attention", _lat(3, 10, 6, 14, 20, 0.35, 100.0), _moe(5, 2, 24)),
                 _layer("mingru", {"width": 44}, None),
                 _layer("attention", _att(2, 1, 12, 40, 0.3, conv=2, size=5, v_mix=True), _moe(4, 4, 16)),
                 _layer("mingru", {"width": 24}, _dense(48))]}

# sizes the tensor-core kernels take (heads of 64 and 32, a latent of 64 + 16, widths that are multiples of 8);
# no convolution in one layer, no mask in another, one layer with mixed values only
MB = {"architecture": "Midulorn", "vocab": 160, "width": 128, "embedding": {"scale": 11.0}, "norm": {"eps": 1e-6},
      "postln_alpha": 2.0, "logit_scale": 0.3,
      "layers": [_layer("latent_attention", _lat(4, 32, 16, 32, 64, 0.15, 500000.0), _dense(256)),
                 _layer("attention", _att(4, 2, 64, 64, 0.11, conv=4, size=70), _moe(8, 3, 64)),
                 _layer("mingru", {"width": 256}, _moe(6, 1, 128)),
                 _layer("attention", _att(6, 2, 32, 64, 0.2, size=24, v_mix=True), _dense(192)),
                 _layer("attention", _att(2, 2, 64, 32, 0.12, conv=5), None),
                 _layer("latent_attention", _lat(2, 16, 32, 48, 128, 0.2, 10000.0, dims=16), _moe(3, 2, 96))]}

# one layer of attention and nothing else: what a query reads is exactly its own stretch of positions
MC = {"architecture": "Midulorn", "vocab": 64, "width": 32, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
      "postln_alpha": 1.0, "logit_scale": 1.0,
      "layers": [_layer("attention", _att(2, 1, 16, 16, 0.6, conv=1, size=9), None)]}

# three layers with mixed values between recurrences, a residual factor far from one
MD = {"architecture": "Midulorn", "vocab": 200, "width": 72, "embedding": {"scale": 8.5}, "norm": {"eps": 1e-5},
      "postln_alpha": 3.5, "logit_scale": 0.2,
      "layers": [_layer("attention", _att(3, 1, 24, 48, 0.25, conv=2, size=33, v_mix=True), _moe(7, 3, 40)),
                 _layer("mingru", {"width": 100}, _dense(144)),
                 _layer("attention", _att(2, 1, 40, 48, 0.2, conv=3, size=33, v_mix=True), _dense(80)),
                 _layer("latent_attention", _lat(5, 8, 8, 24, 48, 0.3, 2000.0), _dense(96)),
                 _layer("attention", _att(3, 3, 16, 16, 0.3, conv=3, v_mix=True), _moe(2, 1, 72))]}

CASES = {"MA": (MA, 41), "MB": (MB, 42), "MC": (MC, 43), "MD": (MD, 44)}

# Random N(0, 0.02) weights leave every gate at one half, every expert alike and the logits flat; these
# factors spread the gates' and the router's logits, the recurrences' candidates and the logits. (The
# chunked attention's scores are spread by the configurations' scale, since queries and keys are normed;
# a factor matches every tensor whose name holds the key, so "mix.v" also scales that projection's bias and taps.)
SHARPEN = {"mix.uk": 8.0, "mix.v": 3.0, "mix.o": 3.0, "mix.g": 5.0, "mix.dkv": 3.0, "mix.uv": 3.0,
           "mix.z": 5.0, "mix.x": 5.0, ".router": 12.0, ".gate": 3.0, ".up": 3.0, ".down": 3.0, "embed": 25.0}

_DIRS, _PLAIN = {}, {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed = CASES[name]
        d = tempfile.mkdtemp(prefix=f"garuda_midulorn_{name}_")
        write_random_model(d, cfg, seed, store_dtype=store_dtype, scale=SHARPEN)
        _DIRS[key] = d
    return _DIRS[key]


def weights(name: str, store_dtype=torch.float32) -> dict:
    from tests.helpers import folder_weights
    return folder_weights(model_dir(name, store_dtype))


def plain_logits(name: str, store_dtype, tokens) -> np.ndarray:
    from tests.plain import midulorn_plain
    key = (name, store_dtype, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = midulorn_plain.forward(CASES[name][0], weights(name, store_dtype), tokens).astype(np.float32)
    return _PLAIN[key]


def random_tokens(name: str, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, CASES[name][0]["vocab"], n).tolist()
