"""Causal attention whose keys and values are linear maps of one cached latent
vector per position.

Per position ``j`` the mixer caches ``[c_j | r_j]``: ``c_j`` the first ``rank``
outputs of the down projection, RMS-normed with a weight; ``r_j`` its last
``rot_dim`` outputs, rotated at position ``j`` (one rotated key part for all
heads). Head ``h`` has an unrotated query part ``q^n`` (``dim`` wide) and a
rotated one ``q^r``; its key at ``j`` is ``[W_uk,h c_j | r_j]`` and its value
``W_uv,h c_j``:

    s_ij = (q^n_i . W_uk,h c_j + q^r_i . r_j) * scale
         = ((W_uk,h^T q^n_i) . c_j + q^r_i . r_j) * scale
    o_i  = W_uv,h sum_j softmax_j(s_ij) c_j

so the query is mapped through ``W_uk^T`` once, attention runs over the cached
rows with all heads reading the same row (as paged attention with one key/value
head whose values are the first ``rank`` channels of its keys), and ``W_uv``
is applied to the result: per token the work on the cache is one pass over
``rank + rot_dim`` numbers per position, whatever the number of heads.

The rotation turns pairs ``(2i, 2i + 1)`` of the first ``rot_dims`` channels of
the rotated parts by ``pos * base^(-2i / rot_dims)``; angles are 32-bit. With
``rot_layout="half"`` the pairs are ``(i, i + rot_dims / 2)`` instead: a score is a
dot product, which does not change when queries and keys are permuted alike, so
the rows of the query and down projections that make the rotated channels are
reordered once, when the weights are loaded (channel ``i`` to ``2i``, channel ``i +
rot_dims / 2`` to ``2i + 1``), and the kernels turn neighbouring pairs as before.

Two options, each off by default. ``sink``: every head has a learned number
``sink_h`` (tensor ``sink``, ``[heads]``) and the softmax's denominator also holds
``exp(sink_h)``, an entry without a key or a value that is not scaled.
``head_gate``: head ``h``'s output is multiplied by ``sigmoid(W_g x)_h`` (tensor
``g``, ``[heads, width]``), ``x`` the mixer's input; the gate is a number per head,
so it is applied to the head's mixed latent, in front of ``W_uv``.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .base import Mixer, PagedLatent, TensorSpec, register_mixer
from .rotary import RotaryParams


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    scales_residual = True

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 eps: float, rot_base: float = 10000.0, rot_dims: Optional[int] = None,
                 window: Optional[int] = None, init_std: float = 0.02,
                 names=("q", "dkv", "dkv.norm", "uk", "uv", "o"), rot_layout: str = "interleaved", sink: bool = False,
                 head_gate: bool = False, sink_name: str = "sink", gate_name: str = "g"):
        self.width, self.heads, self.dim, self.rot_dim = int(width), int(heads), int(dim), int(rot_dim)
        self.vdim, self.rank = int(vdim), int(kv_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        dims = self.rot_dim if rot_dims is None else int(rot_dims)
        if rot_layout not in ("interleaved", "half"):
            raise ValueError(f"the rotation pairs channels 'interleaved' or by 'half', got {rot_layout!r}")
        self.rot_layout, self.sink, self.head_gate = rot_layout, bool(sink), bool(head_gate)
        self.sink_name, self.gate_name = sink_name, gate_name
        if dims % 2 or not 0 <= dims <= self.rot_dim:
            raise ValueError(f"the rotation turns an even number of at most {self.rot_dim} channels, got {dims}")
        if min(self.heads, self.dim, self.vdim, self.rank) < 1 or self.rot_dim < 0:
            raise ValueError("latent attention needs positive sizes")
        self.rot_dims = dims
        self.init_std = float(init_std)
        self.names = tuple(names)
        self.rotary = None
        if dims:
            # one frequency per pair, base^(-2i/dims), taken in 64-bit and rounded once
            i = np.arange(dims // 2, dtype=np.float64)
            freqs = np.power(float(rot_base), -2.0 * i / dims).astype(np.float32)
            self.rotary = RotaryParams(float(rot_base), dims, True, tuple(float(f) for f in freqs))
        self.q_width = self.heads * (self.dim + self.rot_dim)
        self.row = self.rank + self.rot_dim

    def tensors(self):
        init = ("normal", self.init_std)
        q, dkv, norm, uk, uv, o = self.names
        t = {q: TensorSpec((self.q_width, self.width), init=init),
             dkv: TensorSpec((self.row, self.width), init=init),
             norm: TensorSpec((self.rank,), role="vector", init=("ones",)),
             uk: TensorSpec((self.heads * self.dim, self.rank), init=init),
             uv: TensorSpec((self.heads * self.vdim, self.rank), init=init),
             o: TensorSpec((self.width, self.heads * self.vdim), init=init)}
        if self.sink:
            t[self.sink_name] = TensorSpec((self.heads,), role="vector", init=("normal", 1.0))
        if self.head_gate:
            t[self.gate_name] = TensorSpec((self.heads, self.width), init=init)
        return t

    def cache_need(self):
        return PagedLatent(self.row, self.window)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        q, dkv, norm, uk, uv, o = self.names
        w_q, w_dkv = tensors[q], tensors[dkv]
        if self.rot_layout == "half" and self.rot_dims:
            # pairs (i, i + dims/2) become neighbours: the same permutation of the rotated channels of
            # every head's query and of the shared key part leaves every score as it is
            half = self.rot_dims // 2
            perm = torch.arange(self.rot_dim)
            perm[:self.rot_dims] = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
            per_head = torch.cat([torch.arange(self.dim), self.dim + perm])
            q_rows = (torch.arange(self.heads)[:, None] * (self.dim + self.rot_dim) + per_head[None, :]).reshape(-1)
            d_rows = torch.cat([torch.arange(self.rank), self.rank + perm])
            w_q, w_dkv = w_q[q_rows.to(w_q.device)], w_dkv[d_rows.to(w_dkv.device)]
        # the query, the down projection and the heads' gates are one product against their rows stacked
        rows = [w_q, w_dkv] + ([tensors[self.gate_name]] if self.head_gate else [])
        self.w_qd = torch.cat(rows, dim=0).contiguous()
        self.sinks = tensors[self.sink_name].float().contiguous() if self.sink else None
        self.norm_w = tensors[norm]
        # W_uk per head, transposed once: [H * rank, dim], so that the query's map into the latent's
        # coordinates is a product against rows like every other
        self.w_uk_t = (tensors[uk].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
                       .view(self.heads * self.rank, self.dim))
        self.w_uv = tensors[uv].contiguous()
        self.w_o = tensors[o].contiguous()

    def forward(self, ctx, h, cache, residual=None, alpha: float = 1.0):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T, H = h.shape[0], self.heads
        cols = self.q_width + self.row
        qd = ws.get("latent_qd", (T, self.w_qd.shape[0]), torch.float32)
        ops.linear(h, self.w_qd, qd)
        gate = None
        if self.head_gate:
            qd, gate = qd[:, :cols], qd[:, cols:]
        # the query in the latent's coordinates: [W_uk^T q^n | q^r]
        q_lat = ws.get("latent_q", (T, H, self.row), self.dtype)
        q_nope = ws.get("latent_q_nope", (T, H, self.dim), self.dtype)
        if cache.writes:
            # one kernel: the queries prepared, the step's cache rows normed, rotated and written
            ops.latent_rows(qd, H, self.dim, self.rot_dim, self.rank, self.rotary, b.positions, q_nope, q_lat,
                            self.norm_w, self.eps, b.token_req, cache.block_table, cache.k, cache.page_size)
        else:
            ops.latent_query_prepare(qd[:, :self.q_width], H, self.dim, self.rot_dim, self.rotary, b.positions,
                                     q_nope, q_lat)
        ops.head_linear(q_nope, self.w_uk_t, q_lat, n=self.rank, k=self.dim, transposed=False)
        mixed = ws.get("latent_ctx", (T, H * self.rank), self.dtype)
        if self.sinks is None:
            ops.paged_attention(q_lat, cache.k, cache.k, cache.block_table, b.cu_q, b.kv_lens, b.token_req, mixed,
                                self.scale, self.window or 0, cache.page_size, b.num_requests, b.max_q_len,
                                b.max_kv_len, ws=ws, min_q_len=b.min_q_len, value_dim=self.rank)
        else:
            ops.paged_attention(q_lat, cache.k, cache.k, cache.block_table, b.cu_q, b.kv_lens, b.token_req, mixed,
                                self.scale, self.window or 0, cache.page_size, b.num_requests, b.max_q_len,
                                b.max_kv_len, ws=ws, min_q_len=b.min_q_len, value_dim=self.rank, sink_values=self.sinks)
        if gate is not None:
            ops.group_gate_mul(mixed, gate, self.rank)
        out = ws.get("attn_ctx", (T, H * self.vdim), self.dtype)
        ops.head_linear(mixed.unflatten(1, (H, self.rank)), self.w_uv, out.unflatten(1, (H, self.vdim)),
                        n=self.vdim, k=self.rank, transposed=False)
        if residual is not None:
            ops.linear(out, self.w_o, residual, accumulate=True, alpha=alpha)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y
