"""Plain references of the engine's kernels, one function per kernel, on the CPU.

Two uses. The ``-m gpu`` tests compare each CUDA kernel with the function of the
same name here. And because the functions take the same arguments as the
product's kernel set, an instance of ``CpuOps`` can stand in for it, so that
the step function, the cache and the batching logic can be exercised on a
machine without a GPU. It is never used outside the tests: the product path has
no CPU fallback.

Written from the reference's formulas (cited per function); shares no code with
``garuda_b200``.
"""
from __future__ import annotations


import numpy as np
import torch


class CpuOps:
    name = "cpu-reference"

    device = "cpu"

    def __init__(self):
        self.tc = None

    # garuda/src/llama/mod.rs:198-200, :1078-1085
    def embedding(self, table, ids, out, scale=1.0):
        rows = table[ids.long()].float() * scale
        out[: ids.shape[0]] = rows[:, None, :] if out.dim() == 3 else rows

    def scale_softcap(self, x, scale=1.0, cap=0.0):
        """x * scale, then cap * tanh(x / cap)"""
        x *= scale
        if cap > 0:
            x.copy_(cap * torch.tanh(x / cap))

    # garuda/src/simd/mod.rs:166-173; garuda/src/llama/mod.rs:733-738
    def rmsnorm(self, x, weight, eps, out, rows=None):
        xs = x if rows is None else x[rows.long()]
        ms = (xs * xs).sum(-1, keepdim=True) / xs.shape[-1]
        out.copy_(((xs * (1.0 / torch.sqrt(ms + eps))) * weight.float()).to(out.dtype))

    # garuda/src/simd/mod.rs:96-129
    def linear(self, a, w, out, accumulate=False, alpha=1.0):
        y = a.float() @ w.float().t()
        if accumulate:
            out += alpha * y
        else:
            out.copy_(y.to(out.dtype))

    def pack_gate_up(self, gate, up):
        return torch.cat([gate, up], 0).contiguous()

    # garuda/src/llama/mod.rs:1002-1020; garuda/src/simd/mod.rs:161-163
    def linear_swiglu(self, ctx, h, w_gate_up, act):
        y = h.float() @ w_gate_up.float().t()
        self.silu_mul(y, act)

    def silu_mul(self, gate_up, out):
        F = out.shape[1]
        g, u = gate_up[:, :F].float(), gate_up[:, F:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    # garuda/src/simd/mod.rs:176-179
    def residual_add(self, x, y):
        x += y.float()

    # garuda/src/simd/mod.rs:196-206
    def _rotate(self, v, positions, rotary):
        """``rotary``: anything with ``theta``, ``interleaved`` and ``inv_freq`` (one frequency per
        pair in place of the formula, or None)."""
        hd = v.shape[-1]
        interleaved = rotary.interleaved
        if getattr(rotary, "inv_freq", None) is not None:
            inv = torch.tensor(list(rotary.inv_freq), dtype=torch.float32)
        else:
            i = np.arange(hd // 2, dtype=np.float32)
            inv = torch.from_numpy(np.float32(1.0) / np.power(np.float32(rotary.theta),
                                                              np.float32(2.0) * i / np.float32(hd), dtype=np.float32))
        ang = positions.float()[:, None] * inv[None, :]
        s, c = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
        out = torch.empty_like(v)
        if interleaved:
            a, b = v[..., 0::2], v[..., 1::2]
            out[..., 0::2] = a * c - b * s
            out[..., 1::2] = a * s + b * c
        else:
            a, b = v[..., : hd // 2], v[..., hd // 2:]
            out[..., : hd // 2] = a * c - b * s
            out[..., hd // 2:] = a * s + b * c
        return out

    def rope_inplace(self, x, positions, rotary):
        x.copy_(self._rotate(x.clone(), positions, rotary))

    # garuda/src/llama/mod.rs:743-757 (the projections), then rotate and store
    def qkv_rope_append(self, ctx, h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                        heads, kv_heads, head_dim, rotary, page_size):
        qkv = h.float() @ w_qkv.float().t()
        self.rope_kv_append(qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            head_dim, rotary, page_size)

    # garuda/src/llama/mod.rs:784-791 (rotate, then store the rotated key and the raw value)
    def rope_kv_append(self, qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                       heads, kv_heads, head_dim, rotary, page_size):
        T = qkv.shape[0]
        x = qkv.float()
        q = x[:, : heads * head_dim].reshape(T, heads, head_dim)
        if rotary is not None:
            q = self._rotate(q, positions, rotary)
        q_out.copy_(q.to(q_out.dtype))
        if not kv_heads:
            return
        k = x[:, heads * head_dim: (heads + kv_heads) * head_dim].reshape(T, kv_heads, head_dim)
        v = x[:, (heads + kv_heads) * head_dim:].reshape(T, kv_heads, head_dim)
        if rotary is not None:
            k = self._rotate(k, positions, rotary)
        for t in range(T):
            pos = int(positions[t])
            page = int(block_table[int(token_req[t]), pos // page_size])
            assert page >= 0, "a position without a page"
            k_pool[page, :, pos % page_size, :] = k[t].to(k_pool.dtype)
            v_pool[page, :, pos % page_size, :] = v[t].to(v_pool.dtype)

    # garuda/src/llama/mod.rs:793-818; garuda/src/cache/mod.rs:333-338
    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out,
                        scale, window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1,
                        value_dim=None, softcap=0.0, keep_first=0, sink=False, sink_values=None, distance=None, chunk=0):
        """softcap c: s <- c tanh(s / c); keep_first n: a windowed query also reads positions below n;
        sink: p_j = exp(s_j) / (1 + sum exp(s_k)); sink_values: exp(sink_values[h]) in place of the 1;
        distance (r1, r2): s_j -= r1[h] ln(1 + r2[h] (pos - j)); chunk n: keys from floor(pos / n) n on"""
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        g = Hq // Hkv
        vd = v_pool.shape[3] if value_dim is None else value_dim
        res = torch.zeros(T, Hq, vd)
        for t in range(T):
            r = int(token_req[t])
            q_len = int(cu_q[r + 1] - cu_q[r])
            pos = int(kv_lens[r]) - q_len + (t - int(cu_q[r]))
            start = max(0, pos + 1 - window) if window else 0
            if chunk:
                start = pos // chunk * chunk
            js = torch.arange(start, pos + 1)
            if window and keep_first and start > 0:
                js = torch.cat([torch.arange(0, min(keep_first, start)), js])
            pages = block_table[r, (js // page_size)].long()
            assert (pages >= 0).all(), "attention reads a position whose page was given back"
            K = k_pool[pages, :, (js % page_size), :].float()    # [n, Hkv, hd]
            V = v_pool[pages, :, (js % page_size), :vd].float()
            for h in range(Hq):
                s = (K[:, h // g, :] @ q[t, h].float()) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if distance is not None:
                    s = s - float(distance[0][h]) * torch.log1p(float(distance[1][h]) * (pos - js).float())
                if sink_values is not None:
                    p = torch.softmax(torch.cat([s, sink_values[h].float().reshape(1)]), 0)[:-1]
                elif sink:
                    p = torch.softmax(torch.cat([s, torch.zeros(1)]), 0)[:-1]
                else:
                    p = torch.softmax(s, 0)
                res[t, h] = p @ V[:, h // g, :]
        out.copy_(res.reshape(T, Hq * vd).to(out.dtype))

    # ---- parts the reference has no counterpart of: each is the formula in its docstring ----
    def layernorm(self, x, weight, bias, eps, out, rows=None):
        """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations"""
        xs = x if rows is None else x[rows.long()]
        mu = xs.mean(-1, keepdim=True)
        var = ((xs - mu) ** 2).mean(-1, keepdim=True)
        y = (xs - mu) / torch.sqrt(var + eps) * weight.float()
        if bias is not None:
            y = y + bias.float()
        out.copy_(y.to(out.dtype))

    def residual_axpy(self, x, y=None, alpha=1.0, row=None):
        if y is not None:
            x += alpha * y.float()
        if row is not None:
            x += row.float()[None, :]

    def rms_add(self, x, y, weight, eps, alpha=1.0):
        """x += alpha * y / sqrt(mean(y^2) + eps) * w"""
        x += alpha * (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)) * weight.float()

    @staticmethod
    def _gelu_tanh(z):
        return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))

    def gelu_gather_mul(self, z, table, ids, col0, out):
        e = table[ids.long(), col0:col0 + out.shape[1]].float()
        out.copy_((self._gelu_tanh(z.float()) * e).to(out.dtype))

    def cast(self, x, out):
        out.copy_(x.to(out.dtype))

    def gated_act(self, gate_up, out, kind="silu", limit=0.0, group=0):
        F = out.shape[1]
        g, u = gate_up[:, :F].float(), gate_up[:, F:].float()
        if kind == "silu":
            y = g / (1.0 + torch.exp(-g)) * u
        elif kind == "gelu_tanh":
            y = self._gelu_tanh(g) * u
        else:
            g = torch.clamp(g, max=limit)
            u = torch.clamp(u, -limit, limit)
            y = g / (1.0 + torch.exp(-1.702 * g)) * (u + 1.0)
        out.copy_(y.to(out.dtype))

    def linear_gated(self, ctx, h, w_gate_up, act, kind="silu", limit=0.0):
        self.gated_act(h.float() @ w_gate_up.float().t(), act, kind, limit)

    def route_topk(self, h, w_router, bias, top, ids, weights, score="softmax_chosen"):
        z = h.float() @ w_router.float().t()
        if bias is not None:
            z = z + bias.float()
        order = torch.sort(-z, dim=-1, stable=True).indices[:, :top]
        ids.copy_(order.to(torch.int32))
        chosen = torch.gather(z, 1, order)
        if score == "softmax_all":
            weights.copy_(torch.gather(torch.softmax(z, -1), 1, order))
        else:
            weights.copy_(torch.sigmoid(chosen) if score == "sigmoid" else torch.softmax(chosen, -1))

    def moe_gate_up(self, h, w_gate_up, ids, act, kind, limit, in_scale=None):
        T, top = ids.shape
        F = act.shape[2]
        for t in range(T):
            for j in range(top):
                x = h[t].float() * (float(in_scale[t, j]) if in_scale is not None else 1.0)
                gu = (w_gate_up[int(ids[t, j])].float() @ x)[None, :]
                self.gated_act(gu, act[t, j][None, :], kind, limit)

    def moe_down(self, act, w_down, ids, weights, x, alpha=1.0):
        T, top, F = act.shape
        for t in range(T):
            total = torch.zeros(x.shape[1])
            for j in range(top):
                wt = weights[t, j] if weights is not None else 1.0
                total += wt * (w_down[int(ids[t, j])].float() @ act[t, j].float())
            x[t] += alpha * total

    def pack_expert_gate_up(self, gates, ups):
        return torch.stack([torch.cat([g, u], 0) for g, u in zip(gates, ups)]).contiguous()

    def routed_feed_forward(self, ctx, h, w_gate_up, w_down, ids, weights, x, kind, limit, alpha=1.0, scale_input=False):
        T, top = ids.shape
        act = torch.zeros(T, top, w_down.shape[2], dtype=h.dtype)
        self.moe_gate_up(h, w_gate_up, ids, act, kind, limit, weights if scale_input else None)
        self.moe_down(act, w_down, ids, None if scale_input else weights, x, alpha)

    # ---- a norm after the sum, gates per head, xIELU, a gated recurrence per channel, convolved projections ----
    def post_norm(self, x, y, alpha, weight, eps, row=None, rounded=None):
        v = alpha * x
        if y is not None:
            v = v + y
        if row is not None:
            v = v + row
        x.copy_(v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight.float())
        if rounded is not None:
            rounded.copy_(x.to(rounded.dtype))

    def group_gate_mul(self, x, gate, group):
        x.copy_((x.float() * torch.sigmoid(gate.float()).repeat_interleave(group, dim=1)).to(x.dtype))

    def xielu(self, z, out, a_pos, a_neg):
        z = z.float()
        out.copy_(torch.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z).to(out.dtype))

    def linear_xielu(self, ctx, a, w, out, a_pos, a_neg):
        self.xielu(a.float() @ w.float().t(), out, a_pos, a_neg)

    def mingru(self, ctx, proj, cols, bias_z, bias_u, state, out):
        b = ctx.batch
        W = out.shape[1]
        cz, cu, cg = cols
        for r in range(b.num_requests):
            slot = int(b.slots[r])
            S = state[slot, :W].clone() if slot >= 0 else torch.zeros(W)
            for t in range(int(b.cu_q[r]), int(b.cu_q[r + 1])):
                z = torch.sigmoid(proj[t, cz:cz + W] + (bias_z if bias_z is not None else 0.0))
                u = proj[t, cu:cu + W] + (bias_u if bias_u is not None else 0.0)
                n = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
                S = (1 - z) * S + z * n
                g = proj[t, cg:cg + W]
                out[t] = (S * g * torch.sigmoid(g)).to(out.dtype)
            if slot >= 0:
                state[slot, :W] = S

    def conv_qkv_append(self, ctx, proj, bias, conv_w, taps, state, q_out, k_pool, v_pool, block_table, heads, kv_heads,
                        dim, vdim, q_weight, k_weight, eps, page_size, v_first_in=None, v_first_out=None, mix=0.0):
        b = ctx.batch
        T, C = proj.shape
        u = proj.float() + (bias.float() if bias is not None else 0.0)
        y = torch.zeros(T, C)
        keep = taps - 1
        for r in range(b.num_requests):
            t0, t1 = int(b.cu_q[r]), int(b.cu_q[r + 1])
            slot = int(b.slots[r])
            old = state[slot, :keep * C].reshape(keep, C).clone() if keep and slot >= 0 else torch.zeros(keep, C)
            rows = torch.cat([old, u[t0:t1]], 0)          # the kept rows, then the step's
            for j in range(taps):
                y[t0:t1] += rows[j:j + t1 - t0] * conv_w[:, j].float()
            if keep and slot >= 0:
                state[slot, :keep * C] = rows[-keep:].reshape(-1)
        nq, nk = heads * dim, kv_heads * dim

        def rms(v, w):
            return v if w is None else v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.float()

        q_out.copy_(rms(y[:, :nq].reshape(T, heads, dim), q_weight).to(q_out.dtype))
        k = rms(y[:, nq:nq + nk].reshape(T, kv_heads, dim), k_weight)
        v = y[:, nq + nk:]
        if v_first_out is not None:
            v_first_out.copy_(v)
        if v_first_in is not None:
            v = (1.0 - mix) * v + mix * v_first_in
        v = v.reshape(T, kv_heads, vdim)
        for t in range(T):
            pos = int(b.positions[t])
            page = int(block_table[int(b.token_req[t]), pos // page_size])
            if page >= 0:
                k_pool[page, :, pos % page_size, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, pos % page_size, :] = v[t].to(v_pool.dtype)

    # ---- a residual of several streams ----
    def streams_rmsnorm(self, x, in_w, weight, eps, out, rows=None):
        """rms(sum_s in_w[s] x[:, s]) * weight"""
        xs = x if rows is None else x[rows.long()]
        u = torch.einsum("s,tsd->td", in_w.float(), xs)
        out.copy_((u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))

    def streams_update(self, x, mix, out_w, y, next_in=None, norm_weight=None, eps=0.0, normed=None):
        """x[:, j] <- sum_s mix[s, j] x[:, s] + out_w[j] y, all j from the old streams"""
        S = x.shape[1]
        new = torch.einsum("sj,tsd->tjd", mix.float().reshape(S, S), x) + out_w.float()[None, :, None] * y[:, None, :]
        x.copy_(new)
        if next_in is not None:
            self.streams_rmsnorm(x, next_in, norm_weight, eps, normed)

    def qkv_bias_append(self, qkv, bias, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                        head_dim, value_dim, page_size):
        T = qkv.shape[0]
        x = qkv.float() + (bias.float() if bias is not None else 0.0)
        nq, nk = heads * head_dim, kv_heads * head_dim
        q_out.copy_(x[:, :nq].reshape(T, heads, head_dim).to(q_out.dtype))
        k = x[:, nq:nq + nk].reshape(T, kv_heads, head_dim)
        v = x[:, nq + nk:].reshape(T, kv_heads, value_dim)
        for t in range(T):
            pos = int(positions[t])
            page = int(block_table[int(token_req[t]), pos // page_size])
            if page >= 0:
                k_pool[page, :, pos % page_size, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, pos % page_size, :] = v[t].to(v_pool.dtype)

    # ---- the gated delta rule with a decay per key channel ----
    def delta_rule(self, ctx, proj, second, conv_w, a_log, dt_bias, norm_w, eps, state, heads, kv_heads, dim, vdim,
                   taps, out, decay_per_head=False, gate="sigmoid"):
        """decay_per_head: second = [decay logit per head | gate logits], dt_bias per head; gate: the
        activation of the gate's logit. Per request, token by token: the convolution over the kept last inputs and the new one,
        SiLU, unit vectors, S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; then
        o / rms(o) * norm_w * sigmoid(gate)."""
        b = ctx.batch
        H, G = heads, kv_heads
        C = 2 * G * dim + H * vdim
        n_state = H * dim * vdim
        cu, slots = b.cu_q.tolist(), b.slots.tolist()
        cw = conv_w.float()
        rate = torch.exp(a_log.float())
        for r, slot in enumerate(slots):
            if slot < 0:
                out[cu[r]:cu[r + 1]] = 0
                continue
            S = state[slot, :n_state].reshape(H, dim, vdim).clone()
            kept = state[slot, n_state:].reshape(taps - 1, C).clone()
            for t in range(cu[r], cu[r + 1]):
                x = proj[t, :C]
                window = torch.cat([kept, x[None, :]], 0)                   # [taps, C], oldest first
                a = (window * cw.t()).sum(0)
                a = a / (1.0 + torch.exp(-a))
                kept = window[1:]
                q = a[:G * dim].reshape(G, dim)
                k = a[G * dim:2 * G * dim].reshape(G, dim)
                v = a[2 * G * dim:].reshape(H, vdim)
                q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
                k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
                beta = torch.sigmoid(proj[t, C:C + H])
                if decay_per_head:
                    g = torch.exp(-rate * torch.nn.functional.softplus(second[t, :H] + dt_bias.float()))[:, None].expand(H, dim)
                    z = second[t, H:]
                else:
                    g = torch.exp(-rate[:, None] * torch.nn.functional.softplus(second[t, :H * dim] + dt_bias.float()).reshape(H, dim))
                    z = second[t, H * dim:]
                gate_v = (z * torch.sigmoid(z) if gate == "silu" else torch.sigmoid(z)).reshape(H, vdim)
                for n in range(H):
                    kk, qq = k[n // (H // G)], q[n // (H // G)]
                    S[n] = g[n][:, None] * S[n]
                    u = beta[n] * (v[n] - S[n].t() @ kk)
                    S[n] = S[n] + kk[:, None] * u[None, :]
                    o = S[n].t() @ qq
                    o = o / torch.sqrt((o * o).mean() + eps) * norm_w.float() * gate_v[n]
                    out[t, n * vdim:(n + 1) * vdim] = o.to(out.dtype)
            state[slot, :n_state] = S.reshape(-1)
            state[slot, n_state:] = kept.reshape(-1)

    # ---- the generalized delta rule ----
    def general_delta(self, ctx, proj, cols, zdec, w0, a0, decay_scale, norm_w, eps, state, heads, dim, vdim, out):
        """Per request, token by token: w = exp(-c sigmoid(zdec + w0)), a = sigmoid(logit + a0), u the
        unit key; S <- diag(w) S - (a u)(u^T S) + k v^T from the old S; o = S^T r; then per head
        o / rms(o) * norm_w * sigmoid(gate)."""
        b = ctx.batch
        H = heads
        cr, ck, cv, ca, cg = cols
        cu, slots = b.cu_q.tolist(), b.slots.tolist()
        for r_i, slot in enumerate(slots):
            if slot < 0:
                out[cu[r_i]:cu[r_i + 1]] = 0
                continue
            S = state[slot].reshape(H, dim, vdim).clone()
            for t in range(cu[r_i], cu[r_i + 1]):
                row = proj[t]
                r = row[cr:cr + H * dim].reshape(H, dim)
                k = row[ck:ck + H * dim].reshape(H, dim)
                v = row[cv:cv + H * vdim].reshape(H, vdim)
                a = torch.sigmoid(row[ca:ca + H * dim] + a0).reshape(H, dim)
                w = torch.exp(-decay_scale * torch.sigmoid(zdec[t, :H * dim] + w0)).reshape(H, dim)
                gate = torch.sigmoid(row[cg:cg + H * vdim]).reshape(H, vdim)
                u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
                for n in range(H):
                    S[n] = w[n][:, None] * S[n] - (a[n] * u[n])[:, None] * (u[n] @ S[n])[None, :] + k[n][:, None] * v[n][None, :]
                    o = S[n].t() @ r[n]
                    o = o / torch.sqrt((o * o).mean() + eps) * norm_w[n * vdim:(n + 1) * vdim] * gate[n]
                    out[t, n * vdim:(n + 1) * vdim] = o.to(out.dtype)
            state[slot] = S.reshape(-1)

    # ---- normed queries and keys; sublayers whose outputs are normed ----
    def qk_norm_rope_append(self, src, cols, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            dim, vdim, q_weight, k_weight, eps, rotary, page_size):
        """queries and keys normed per head (weights 32-bit; None: not), rotated, queries out, keys and
        the untouched value columns into their pages"""
        T = src.shape[0]
        cq, ck, cv = cols
        q = src[:, cq:cq + heads * dim].float().reshape(T, heads, dim)
        k = src[:, ck:ck + kv_heads * dim].float().reshape(T, kv_heads, dim)
        v = src[:, cv:cv + kv_heads * vdim].float().reshape(T, kv_heads, vdim)
        if q_weight is not None:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_weight.reshape(heads, dim)
        if k_weight is not None:
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_weight
        if rotary is not None:
            q, k = self._rotate(q, positions, rotary), self._rotate(k, positions, rotary)
        q_out.copy_(q.to(q_out.dtype))
        for t in range(T):
            pos = int(positions[t])
            page = int(block_table[int(token_req[t]), pos // page_size])
            if page >= 0:
                k_pool[page, :, pos % page_size, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, pos % page_size, :] = v[t].to(v_pool.dtype)

    @staticmethod
    def _unary(z, kind):
        if kind == "sigmoid":
            return torch.sigmoid(z)
        if kind == "silu":
            return z * torch.sigmoid(z)
        if kind == "relu2":
            return torch.relu(z) ** 2
        if kind == "tanh":
            return torch.tanh(z)
        raise ValueError(kind)

    def gate_mul(self, x, gate, kind="sigmoid"):
        x.copy_((x.float() * self._unary(gate.float(), kind)).to(x.dtype))

    def activation(self, z, out, kind):
        out.copy_(self._unary(z.float(), kind).to(out.dtype))

    def linear_act(self, ctx, a, w, out, kind):
        out.copy_(self._unary(a.float() @ w.float().t(), kind).to(out.dtype))

    def sublayer_merge(self, ys, branch_weights, eps, x=None, out=None, gate=None, gate_bias=None, weight=None,
                       branch_eps=None, rounded=None):
        """y = mean_b rms(y_b) w_b (or the one y); y *= sigmoid(gate + bias); x += rms(y) weight (or out = y)"""
        def rms(v, e):
            return v / torch.sqrt((v * v).mean(-1, keepdim=True) + e)
        if branch_weights is not None:
            be = eps if branch_eps is None else branch_eps
            y = sum(rms(yb, be) * wb for yb, wb in zip(ys, branch_weights)) / len(ys)
        else:
            y = ys[0]
        if gate is not None:
            y = y * torch.sigmoid(gate + (gate_bias if gate_bias is not None else 0.0))
        if x is None:
            out.copy_(y)
        else:
            x += rms(y, eps) * weight
            if rounded is not None:
                rounded.copy_(x.to(rounded.dtype))

    def latent_append(self, src, norm_w, eps, rank, rot, rotary, positions, token_req, block_table, pool, page_size):
        """rows [rms(src[:, :rank]) * w | rotate(src[:, rank:])] into their pages"""
        c = src[:, :rank]
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm_w.float()
        r = src[:, rank:rank + rot].clone()
        if rotary is not None:
            d = rotary.head_dim
            r[:, :d] = self._rotate(r[:, None, :d], positions, rotary)[:, 0]
        row = torch.cat([c, r], -1)
        for t in range(src.shape[0]):
            pos = int(positions[t])
            page = int(block_table[int(token_req[t]), pos // page_size])
            if page >= 0:
                pool[page, 0, pos % page_size, :] = row[t].to(pool.dtype)

    def latent_query_prepare(self, src, heads, dn, rot, rotary, positions, q_nope, q_lat):
        """unrotated query parts to q_nope, rotated parts (turned) to the last rot channels of q_lat"""
        T = src.shape[0]
        v = src.reshape(T, heads, dn + rot)
        q_nope.copy_(v[..., :dn].to(q_nope.dtype))
        r = v[..., dn:].clone()
        if rotary is not None:
            d = rotary.head_dim
            r[..., :d] = self._rotate(r[..., :d], positions, rotary)
        q_lat[..., q_lat.shape[2] - rot:] = r.to(q_lat.dtype)

    def latent_rows(self, src, heads, dn, rot, rank, rotary, positions, q_nope, q_lat, norm_w, eps, token_req,
                    block_table, pool, page_size):
        qw = heads * (dn + rot)
        self.latent_query_prepare(src[:, :qw], heads, dn, rot, rotary, positions, q_nope, q_lat)
        self.latent_append(src[:, qw:], norm_w, eps, rank, rot, rotary, positions, token_req, block_table, pool, page_size)

    def head_linear(self, a, w, out, n, k, transposed, tail=0):
        T, H = a.shape[:2]
        wf = w.float()
        for h in range(H):
            wh = wf[h * k:(h + 1) * k].t() if transposed else wf[h * n:(h + 1) * n]      # [n, k]
            out[:, h, :n] = (a[:, h, :k].float() @ wh.t()).to(out.dtype)
            if tail:
                out[:, h, n:n + tail] = a[:, h, k:k + tail].to(out.dtype)

    # garuda/src/runtime/mod.rs:99-107
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    # garuda/src/runtime/mod.rs:109-175
    def sample(self, logits, temperature, top_k, top_p, u, out, scratch):
        from .sampling_plain import candidates
        from .llama_plain import argmax_first
        for r in range(logits.shape[0]):
            row = logits[r].numpy()
            if float(temperature[r]) == 0.0:
                out[r] = argmax_first(row)
                continue
            cand = candidates(row, float(temperature[r]), int(top_k[r]), float(top_p[r]))
            total = np.float32(sum(np.float32(p) for _, p in cand))
            pick = cand[0][0]
            if total > 0:
                point = np.float32(np.float32(float(u[r])) * total)
                pick = cand[-1][0]
                for tok, p in cand:
                    point = np.float32(point - p)
                    if point <= 0:
                        pick = tok
                        break
            out[r] = pick
