"""Causal grouped-query attention over the paged cache.

garuda/src/llama/mod.rs:743-757 (Q, K, V projections, no bias), :766-821
(``attend_one``: rotate q and k at the token's position, store the rotated key
and the raw value, then for every query head ``h`` read kv head ``h // g``:
``s_j = dot(q, K_j) / sqrt(head_dim)`` over ``j`` in ``[start, pos]``, softmax,
``sum_j p_j V_j``), :879-880 (output projection). A step's tokens are first all
stored and then all read, each query over keys up to its own position, which
is the same thing as the reference's token-by-token order.

The three projections are one matrix product against the rows of
``q_proj, k_proj, v_proj`` stacked (the reference runs three, :753-755); its
result stays 32-bit until after the rotation.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import (FixedState, Mixer, PagedKV, TensorSpec, PartSpec, build_part, register_mixer)


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int,
                 position: Optional[dict] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, reads_shared_cache: bool = False,
                 init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.heads, self.kv_heads, self.head_dim = int(width), int(heads), int(kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.reads_shared_cache = bool(reads_shared_cache)
        self.init_std = float(init_std)
        pos = position or {"name": "none", "params": {}}
        self.position = build_part("position_encoding", PartSpec(pos["name"], dict(pos.get("params", {}))))
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim

    # ---- declarations ------------------------------------------------------
    def tensors(self):
        init = ("normal", self.init_std)
        t = {"q_proj.weight": TensorSpec((self.q_dim, self.width), init=init),
             "o_proj.weight": TensorSpec((self.width, self.q_dim), init=init)}
        if not self.reads_shared_cache:
            t["k_proj.weight"] = TensorSpec((self.kv_dim, self.width), init=init)
            t["v_proj.weight"] = TensorSpec((self.kv_dim, self.width), init=init)
        # a position encoding with tensors of its own (a learned table) keeps them under "position."
        for local, ts in self.position.tensors().items():
            t["position." + local] = ts
        return t

    @property
    def graph_safe(self):
        return self.position.graph_safe

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.position.load({local: tensors["position." + local] for local in self.position.tensors()}, ops, dtype)
        if self.reads_shared_cache:
            self.w_qkv = tensors["q_proj.weight"].contiguous()
        else:
            self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                    tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()

    # ---- one step ------------------------------------------------------------
    # ``h`` may be a norm that is half done (``CudaOps.qkv_rope_append`` takes it), and the output
    # product may fold in the first half of the norm that follows (``emit_norm``)
    takes_pending_norm = True
    emits_norm = True

    def forward(self, ctx, h, cache, residual=None, emit_norm=None):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T = h.shape[0]
        writes = cache.writes and not self.reads_shared_cache
        cols = self.q_dim + (2 * self.kv_dim if writes else 0)
        # a call that reads another call's cache projects queries only (the first rows)
        w_qkv = self.w_qkv if self.w_qkv.shape[0] == cols else self.w_qkv[:cols]
        q = ws.get("q_heads", (T, self.heads, self.head_dim), self.dtype)
        rotary = self.position.rotary
        kv_heads = self.kv_heads if writes else 0
        if rotary is not None or not self.position.changes_vectors:
            # the product, the rotation and the write into the pages, fused where the kernels allow
            ops.qkv_rope_append(ctx, h, w_qkv, q, cache.k if writes else None, cache.v if writes else None,
                                b.positions, b.token_req, cache.block_table, self.heads, kv_heads,
                                self.head_dim, rotary, cache.page_size)
        else:
            # an encoding the fused kernel does not know: let the part change q and k in place
            qkv = ws.get("qkv", (T, cols), torch.float32)
            if hasattr(ops, "normed"):
                h = ops.normed(ctx, h)
            ops.linear(h, w_qkv, qkv)
            qv = qkv[:, :self.q_dim].unflatten(1, (self.heads, self.head_dim))
            kv = (qkv[:, self.q_dim:self.q_dim + self.kv_dim].unflatten(1, (self.kv_heads, self.head_dim))
                  if writes else None)
            self.position.apply(ctx, qv, kv, b.positions)
            ops.rope_kv_append(qkv, q, cache.k if writes else None, cache.v if writes else None,
                               b.positions, b.token_req, cache.block_table, self.heads, kv_heads,
                               self.head_dim, None, cache.page_size)
        out = ws.get("attn_ctx", (T, self.q_dim), self.dtype)
        ops.paged_attention(q, cache.k, cache.v, cache.block_table, b.cu_q, b.kv_lens, b.token_req, out,
                            self.scale, self.window or 0, cache.page_size,
                            b.num_requests, b.max_q_len, b.max_kv_len, ws=ws, min_q_len=b.min_q_len)
        if residual is not None:
            if emit_norm is None:
                ops.linear(out, self.w_o, residual, accumulate=True)
            else:
                ctx.pending_norm = ops.linear(out, self.w_o, residual, accumulate=True, ctx=ctx, emit_norm=emit_norm)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y


@register_mixer("capped_sink_attention")
class CappedSinkAttention(Mixer):
    """Grouped-query attention over the paged cache with keys and values of widths of their own,
    optional biases on the three projections, and no position encoding: positions enter only
    through the mask. With ``q, k, v`` the projected rows (``dim`` wide for queries and keys,
    ``vdim`` for values), query head ``h`` reading key/value head ``h // (heads / kv_heads)``:

        s_ij = (q_i . k_j) * scale;          softcap c:  s_ij <- c tanh(s_ij / c)
        i reads j  iff  j <= i and (i - j < window  or  j < keep_first)
        sink:  p_ij = exp(s_ij) / (1 + sum_j' exp(s_ij'))    (else the ordinary softmax)
        out_i = W_o concat_h sum_j p_ij v_j

    ``names``: the tensors' local names (``q, k, v, o``; a bias is the weight's name with ``.b``
    added). Kept positions keep their true places: nothing is renumbered."""
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: Optional[int] = None,
                 scale: Optional[float] = None, softcap: Optional[float] = None, window: Optional[int] = None,
                 keep_first: int = 0, sink: bool = False, bias: bool = False, names: Optional[dict] = None,
                 init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.heads, self.kv_heads, self.dim = int(width), int(heads), int(kv_heads), int(dim)
        self.vdim = int(vdim) if vdim else self.dim
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dim)
        self.softcap = float(softcap) if softcap else 0.0
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.sink, self.bias = bool(sink), bool(bias)
        self.names = dict({"q": "q", "k": "k", "v": "v", "o": "o"}, **(names or {}))
        self.init_std = float(init_std)
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim

    def tensors(self):
        init, n = ("normal", self.init_std), self.names
        t = {n["q"]: TensorSpec((self.q_dim, self.width), init=init), n["k"]: TensorSpec((self.k_dim, self.width), init=init),
             n["v"]: TensorSpec((self.v_dim, self.width), init=init),
             n["o"]: TensorSpec((self.width, self.heads * self.vdim), init=init)}
        if self.bias:
            for key, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)):
                t[n[key] + ".b"] = TensorSpec((rows,), role="vector", init=("normal", 0.02))
        return t

    def cache_need(self):
        return PagedKV(self.kv_heads, self.dim, self.window, value_dim=self.vdim, keep_first=self.keep_first)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        n = self.names
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.b_qkv = (torch.cat([tensors[n[k] + ".b"].float() for k in ("q", "k", "v")]).contiguous()
                      if self.bias else None)
        self.w_o = tensors[n["o"]].contiguous()

    def forward(self, ctx, h, cache, residual=None):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T = h.shape[0]
        qkv = ws.get("qkv", (T, self.w_qkv.shape[0]), torch.float32)
        ops.linear(h, self.w_qkv, qkv)
        q = ws.get("q_heads", (T, self.heads, self.dim), self.dtype)
        ops.qkv_bias_append(qkv, self.b_qkv, q, cache.k, cache.v, b.positions, b.token_req, cache.block_table,
                            self.heads, self.kv_heads, self.dim, self.vdim, cache.page_size)
        out = ws.get("attn_ctx", (T, self.heads * self.vdim), self.dtype)
        ops.paged_attention(q, cache.k, cache.v, cache.block_table, b.cu_q, b.kv_lens, b.token_req, out,
                            self.scale, self.window or 0, cache.page_size, b.num_requests, b.max_q_len, b.max_kv_len,
                            ws=ws, min_q_len=b.min_q_len, softcap=self.softcap, keep_first=self.keep_first, sink=self.sink)
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y


@register_mixer("normed_key_attention")
class NormedKeyAttention(Mixer):
    """Grouped-query attention over the paged cache whose queries and keys are RMS-normed per head
    before they are rotated, whose values may be the keys as projected, with a temperature per
    head and a gate on the concatenated heads. With ``h`` the mixer's input, query head ``n``
    reading key/value head ``n // (heads / kv_heads)``:

        q, k = W_q h, W_k h;   v = k (as projected; ``values="keys"``) or W_v h (``"projected"``)
        q <- rms(q) * w_q, k <- rms(k) * w_k     per head, over ``dim`` (``qk_norm``)
        q, k rotated at their positions: channel 2i with 2i+1, the first ``rot_dims`` channels, angle
             position * rot_base^(-2i / rot_dims)    (``rot_base`` None: not rotated)
        s_ij = (q_i . k_j) * scale * temp_n;   i reads j  iff  0 <= i - j < window  (None: j <= i)
        out = W_o (concat_n softmax(s) v * sigmoid(W_g h))       (``gate``)

    The temperature multiplies the query's norm weight when the weights are loaded (the rotation
    is linear), so the attention kernel sees one scale. One product makes ``[q | k | (v) | gate]``
    in 32-bit; one kernel norms, rotates and stores. ``names``: the tensors' local names."""
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, scale: Optional[float] = None,
                 window: Optional[int] = None, rot_base: Optional[float] = None, rot_dims: int = 0,
                 rot_layout: str = "interleaved", qk_norm: bool = True, eps: float = 1e-6, temperature: bool = True,
                 values: str = "keys", vdim: Optional[int] = None, gate: bool = True, names: Optional[dict] = None,
                 init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if values not in ("keys", "projected"):
            raise ValueError(f"values are 'keys' or 'projected', got {values!r}")
        if temperature and not qk_norm:
            raise ValueError("a temperature per head goes with normed queries (it is folded into their norm's weight)")
        self.width, self.heads, self.kv_heads, self.dim = int(width), int(heads), int(kv_heads), int(dim)
        self.vdim = self.dim if values == "keys" or not vdim else int(vdim)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dim)
        self.window = int(window) if window else None
        self.qk_norm, self.eps, self.temperature = bool(qk_norm), float(eps), bool(temperature)
        self.values, self.gate = values, bool(gate)
        self.names = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                           "temp": "temp"}, **(names or {}))
        self.init_std = float(init_std)
        self.rotary = None
        if rot_base is not None and rot_dims:
            from .rotary import Rotary
            # frequencies in 64-bit, rounded once; channels beyond the rotated width get frequency zero
            freqs = [float(rot_base) ** (-2.0 * i / int(rot_dims)) for i in range(int(rot_dims) // 2)]
            self.rotary = Rotary(float(rot_base), self.dim, layout=rot_layout, inv_freq=freqs, rotary_dim=int(rot_dims)).rotary
            if self.rotary is None:
                raise ValueError("a rotation narrower than the head takes the interleaved pairing here")
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.ctx_dim = self.heads * self.vdim

    def tensors(self):
        init, n = ("normal", self.init_std), self.names
        t = {n["q"]: TensorSpec((self.q_dim, self.width), init=init), n["k"]: TensorSpec((self.k_dim, self.width), init=init),
             n["o"]: TensorSpec((self.width, self.ctx_dim), init=init)}
        if self.values == "projected":
            t[n["v"]] = TensorSpec((self.v_dim, self.width), init=init)
        if self.gate:
            t[n["g"]] = TensorSpec((self.ctx_dim, self.width), init=init)
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((self.dim,), role="vector", init=("normal_about_one", 0.1))
            t[n["k_norm"]] = TensorSpec((self.dim,), role="vector", init=("normal_about_one", 0.1))
        if self.temperature:
            t[n["temp"]] = TensorSpec((self.heads,), role="vector", init=("normal_about_one", 0.2))
        return t

    def cache_need(self):
        return PagedKV(self.kv_heads, self.dim, self.window, value_dim=self.vdim)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]]]
        self.col_q, self.col_k = 0, self.q_dim
        self.col_v = self.col_k
        at = self.q_dim + self.k_dim
        if self.values == "projected":
            rows.append(tensors[n["v"]])
            self.col_v, at = at, at + self.v_dim
        self.col_g = at
        if self.gate:
            rows.append(tensors[n["g"]])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.k_weight = tensors[n["k_norm"]].float().contiguous() if self.qk_norm else None
        self.q_weight = None
        if self.qk_norm:
            per_head = tensors[n["q_norm"]].float()[None, :].expand(self.heads, self.dim)
            if self.temperature:
                per_head = per_head * tensors[n["temp"]].float()[:, None]
            self.q_weight = per_head.contiguous()

    def forward(self, ctx, h, cache, residual=None, out_name: str = "attn_y"):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T = h.shape[0]
        proj = ws.get("attn_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, proj)
        q = ws.get("q_heads", (T, self.heads, self.dim), self.dtype)
        ops.qk_norm_rope_append(proj, (self.col_q, self.col_k, self.col_v), q, cache.k, cache.v, b.positions, b.token_req,
                                cache.block_table, self.heads, self.kv_heads, self.dim, self.vdim, self.q_weight,
                                self.k_weight, self.eps, self.rotary, cache.page_size)
        out = ws.get("attn_ctx", (T, self.ctx_dim), self.dtype)
        ops.paged_attention(q, cache.k, cache.v, cache.block_table, b.cu_q, b.kv_lens, b.token_req, out,
                            self.scale, self.window or 0, cache.page_size, b.num_requests, b.max_q_len, b.max_kv_len,
                            ws=ws, min_q_len=b.min_q_len)
        if self.gate:
            ops.gate_mul(out, proj[:, self.col_g:self.col_g + self.ctx_dim], "sigmoid")
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True)
            return None
        y = ws.get(out_name, (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y


@register_mixer("convolved_attention")
class ConvolvedAttention(Mixer):
    """Grouped-query attention over the paged cache behind a short causal convolution on every
    projected channel, without a position encoding: positions enter through the mask and through a
    term that grows with the distance. With ``x`` the mixer's input, query head ``n`` reading key/value
    head ``n // (heads / kv_heads)``, each option off at its neutral value:

        q, k, v = W_q x + b_q, W_k x + b_k, W_v x + b_v                       (``bias``)
        y_t = sum_j w[c, j] u_(t - taps + 1 + j) per channel c of q, k, v    (``taps``; zeros before the start)
        q, k <- rms(q) * w_q, rms(k) * w_k per head, the weights shared by the heads   (``qk_norm``)
        v <- (1 - lambda) v + lambda v_first                                  (``value_mix="mix"``)
        s_ij = (q_i . k_j) * scale - r1_n ln(1 + r2_n (i - j))                (``distance``)
        i reads j  iff  j <= i and floor(i / chunk) = floor(j / chunk)        (``chunk``; None: every j <= i)
        p_ij = exp(s_ij) / (exp(sink_n) + sum_j' exp(s_ij'))                  (``sink``)
        out = W_o concat_n sum_j p_ij v_j + b_o

    ``value_mix``: ``"source"`` marks the layer whose values (after the convolution) the later
    layers mix into theirs; ``"mix"`` such a later layer, with ``lambda`` its tensor ``vmix``. Both name
    the same ``value_mix_key``; the values travel in the step's context, for the step's tokens only.
    The mixed values are what the cache holds. The convolution's state, the last ``taps - 1`` projected
    rows of a request (biases included), is a ``FixedState`` beside the pages.
    ``names``: the tensors' local names (a bias is the weight's name with ``.b`` added, a convolution's
    taps ``.conv``, ``[channels, taps]`` with the last column on the current token)."""
    graph_safe = True
    scales_residual = True
    defers_bias = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: Optional[int] = None,
                 scale: Optional[float] = None, taps: int = 0, qk_norm: bool = True, eps: float = 1e-6, bias: bool = True,
                 distance: bool = False, chunk: Optional[int] = None, sink: bool = False, value_mix: Optional[str] = None,
                 value_mix_key: str = "v_first", names: Optional[dict] = None, init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix is None, 'source' or 'mix', got {value_mix!r}")
        self.width, self.heads, self.kv_heads, self.dim = int(width), int(heads), int(kv_heads), int(dim)
        self.vdim = int(vdim) if vdim else self.dim
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dim)
        self.has_conv = bool(taps)               # (one tap is a convolution too: a factor per channel)
        self.taps = max(int(taps or 0), 1)
        self.qk_norm, self.eps, self.bias = bool(qk_norm), float(eps), bool(bias)
        self.distance, self.sink = bool(distance), bool(sink)
        self.chunk = int(chunk) if chunk else None
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.names = dict({"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1",
                           "r2": "r2", "sink": "sink", "vmix": "vmix"}, **(names or {}))
        self.init_std = float(init_std)
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.channels = self.q_dim + self.k_dim + self.v_dim

    def tensors(self):
        init, n = ("normal", self.init_std), self.names
        t = {n["q"]: TensorSpec((self.q_dim, self.width), init=init), n["k"]: TensorSpec((self.k_dim, self.width), init=init),
             n["v"]: TensorSpec((self.v_dim, self.width), init=init),
             n["o"]: TensorSpec((self.width, self.heads * self.vdim), init=init)}
        if self.bias:
            for key, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim), ("o", self.width)):
                t[n[key] + ".b"] = TensorSpec((rows,), role="vector", init=("normal", 0.02))
        if self.has_conv:
            for key, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)):
                t[n[key] + ".conv"] = TensorSpec((rows, self.taps), role="vector", init=("normal", 0.5))
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((self.dim,), role="vector", init=("normal_about_one", 0.1))
            t[n["k_norm"]] = TensorSpec((self.dim,), role="vector", init=("normal_about_one", 0.1))
        if self.distance:
            t[n["r1"]] = TensorSpec((self.heads,), role="vector", init=("uniform", 0.1, 1.0))
            t[n["r2"]] = TensorSpec((self.heads,), role="vector", init=("uniform", 0.05, 2.0))
        if self.sink:
            t[n["sink"]] = TensorSpec((self.heads,), role="vector", init=("normal", 1.0))
        if self.value_mix is not None:
            t[n["vmix"]] = TensorSpec((), role="vector", init=("uniform", 0.2, 0.8))
        return t

    def cache_need(self):
        paged = PagedKV(self.kv_heads, self.dim, None, value_dim=self.vdim, chunk=self.chunk)
        if self.taps > 1:
            return (paged, FixedState(((self.taps - 1) * self.channels,)))
        return paged

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        n = self.names
        keys = ("q", "k", "v")
        self.w_qkv = torch.cat([tensors[n[k]] for k in keys], dim=0).contiguous()
        self.b_qkv = torch.cat([tensors[n[k] + ".b"].float() for k in keys]).contiguous() if self.bias else None
        self.conv_w = None
        if self.has_conv:
            self.conv_w = torch.cat([tensors[n[k] + ".conv"].float() for k in keys], dim=0).contiguous()
        else:
            self.conv_w = torch.ones((self.channels, 1), dtype=torch.float32, device=self.w_qkv.device)
        self.q_weight = tensors[n["q_norm"]].float().contiguous() if self.qk_norm else None
        self.k_weight = tensors[n["k_norm"]].float().contiguous() if self.qk_norm else None
        self.far = (tensors[n["r1"]].float().contiguous(), tensors[n["r2"]].float().contiguous()) if self.distance else None
        self.sinks = tensors[n["sink"]].float().contiguous() if self.sink else None
        self.mix = float(tensors[n["vmix"]].float().reshape(-1)[0]) if self.value_mix == "mix" else 0.0
        self.w_o = tensors[n["o"]].contiguous()
        self.output_bias = tensors[n["o"] + ".b"].float().contiguous() if self.bias else None
        self._scaled_bias = {}

    def _bias_times(self, alpha: float):
        if alpha == 1.0:
            return self.output_bias
        if alpha not in self._scaled_bias:
            self._scaled_bias[alpha] = (self.output_bias * alpha).contiguous()
        return self._scaled_bias[alpha]

    def forward(self, ctx, h, cache, residual=None, alpha: float = 1.0, defer_bias: bool = False):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T = h.shape[0]
        paged, state = (cache.parts[0], cache.parts[1].state) if cache.parts is not None else (cache, None)
        if not cache.writes:
            raise ValueError("a convolved attention keeps a cache of its own")
        proj = ws.get("qkv", (T, self.channels), torch.float32)
        ops.linear(h, self.w_qkv, proj)
        q = ws.get("q_heads", (T, self.heads, self.dim), self.dtype)
        v_in = v_out = None
        key = ("shared_values", self.value_mix_key)
        if self.value_mix == "source":
            v_out = ws.get(f"shared_values_{self.value_mix_key}", (T, self.v_dim), torch.float32)
            ctx.step_cache[key] = v_out
        elif self.value_mix == "mix":
            v_in = ctx.step_cache.get(key)
            if v_in is None or tuple(v_in.shape) != (T, self.v_dim):
                raise ValueError(f"no layer in front has left values '{self.value_mix_key}' of {self.v_dim} channels to mix in")
        ops.conv_qkv_append(ctx, proj, self.b_qkv, self.conv_w, self.taps, state, q, paged.k, paged.v, paged.block_table,
                            self.heads, self.kv_heads, self.dim, self.vdim, self.q_weight, self.k_weight, self.eps,
                            paged.page_size, v_first_in=v_in, v_first_out=v_out, mix=self.mix)
        out = ws.get("attn_ctx", (T, self.heads * self.vdim), self.dtype)
        ops.paged_attention(q, paged.k, paged.v, paged.block_table, b.cu_q, b.kv_lens, b.token_req, out, self.scale, 0,
                            paged.page_size, b.num_requests, b.max_q_len, b.max_kv_len, ws=ws, min_q_len=b.min_q_len,
                            sink_values=self.sinks, distance=self.far, chunk=self.chunk or 0)
        add_bias = self.output_bias is not None and not defer_bias
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True, alpha=alpha)
            if add_bias:
                ops.residual_axpy(residual, None, 1.0, self._bias_times(alpha))
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        if add_bias:
            ops.residual_axpy(y, None, 1.0, self.output_bias)
        return y
