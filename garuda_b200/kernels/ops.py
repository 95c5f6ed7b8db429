"""The kernel set of the product path: thin, checking wrappers around the CUDA
entry points. There is no other implementation behind them: without a CUDA
device or without the compiled library every call fails loudly.

Each method takes torch tensors that live on the device, checks dtypes, shapes
and contiguity, and launches on torch's current stream.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import c_void_p, c_int, c_float, c_longlong
from typing import Optional

import numpy as np
import torch

from ..csrc.build import load_kernel_lib

GB_F32, GB_BF16 = 0, 1
_TAG = {torch.float32: GB_F32, torch.bfloat16: GB_BF16}


class KernelError(RuntimeError):
    pass


def _tag(t: torch.Tensor, what: str) -> int:
    try:
        return _TAG[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_ERROR_WORD = None


def _error_word() -> torch.Tensor:
    global _ERROR_WORD
    if _ERROR_WORD is None:
        _ERROR_WORD = torch.zeros(4, dtype=torch.int32).pin_memory()
    return _ERROR_WORD


class PendingNorm:
    """An RMS norm of which only the first half has run, folded into the product that wrote the
    residual stream ``x``: ``values`` is ``x * weight`` in bfloat16 and ``sums`` ``[tiles, T]``
    holds partial sums of ``x^2`` per token. A product that takes it as its tokens multiplies
    its results by ``1/sqrt(sum / width + eps)`` (32-bit); ``materialize`` runs the norm part
    on ``x`` the ordinary way instead, for a consumer that cannot."""

    def __init__(self, values, sums, weight, eps, norm, x):
        self.values, self.sums, self.weight, self.eps, self.norm, self.x = values, sums, weight, float(eps), norm, x

    @property
    def shape(self):
        return self.values.shape

    @property
    def dtype(self):
        return self.values.dtype

    def materialize(self, ctx):
        return self.norm.forward(ctx, self.x)


class CudaOps:
    """Hand-written sm_100a kernels. ``tensor_cores=False`` keeps every matrix
    product and the attention on the plain 32-bit-arithmetic kernels (the true
    32-bit path uses them in any case)."""

    name = "cuda"

    def __init__(self, device="cuda:0", tensor_cores: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("garuda_b200 needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.core = load_kernel_lib("garuda_core")
        self._mixers = None
        self._state = None
        self._seq = None
        self._declare_core()
        # A word of pinned host memory that a kernel whose bounded wait ran out writes its code to (the
        # device reaches pinned host memory directly); ``failed_wait`` reads it without a copy.
        # The kernel libraries are loaded once per process, so the word is one per process as well.
        self.error_word = _error_word()
        self.tc = None
        if tensor_cores:
            from .tc import TensorCoreKernels
            self.tc = TensorCoreKernels(self)
        # whether products fold the norms around them in (``linear``'s ``emit_norm``); a test flips
        # it to compare the two ways
        self.folds_norms = self.tc is not None
        self._inv_freq = {}
        self._held_stream = None
        self.launches = 0
        from ..engine.batch import Workspace
        self.private_ws = Workspace(self.device)   # scratch for calls made outside a step

    def failed_wait(self) -> int:
        """The code of a bounded wait that ran out in a kernel which has finished by now, or 0.
        Costs nothing: call it where the host has just waited for a step's results. The full check
        (``tc.check_errors``) synchronises and clears."""
        return int(self.error_word[0])

    # ------------------------------------------------------------------ plumbing
    def _declare_core(self):
        L = self.core
        L.gb_last_error.restype = ctypes.c_char_p
        sig = {
            "gb_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
            "gb_embedding_copies": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
            "gb_scale_softcap": [c_void_p, c_longlong, c_float, c_float, c_void_p],
            "gb_layernorm": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
            "gb_residual_axpy": [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
            "gb_rms_add": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_int, c_int, c_void_p],
            "gb_gelu_gather_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_void_p],
            "gb_cast": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
            "gb_gated_act": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
            "gb_rmsnorm": [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
            "gb_rope_kv_append": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_int, c_void_p],
            "gb_rope_inplace": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
            "gb_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "gb_silu_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
            "gb_residual_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
            "gb_gemm_simple": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
            "gb_attention_simple": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                    c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
            "gb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p],
            "gb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                          c_void_p],
            "gb_sample_small_k": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_void_p],
        }
        for name, argtypes in sig.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = c_int

    @property
    def mixers(self):
        """The library of the latent-attention and routed-expert kernels, compiled and loaded when
        a model first needs it."""
        if self._mixers is None:
            L = load_kernel_lib("garuda_mixers")
            L.gb_last_error.restype = ctypes.c_char_p
            for name, argtypes in self._MIXER_SIGNATURES.items():
                fn = getattr(L, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            L.gb_moe_grouped_index_words.argtypes = [c_longlong, c_int]
            L.gb_moe_grouped_index_words.restype = c_longlong
            L.gb_moe_padded_rows.argtypes = [c_longlong, c_int]
            L.gb_moe_padded_rows.restype = c_longlong
            self._mixers = L
        return self._mixers

    @property
    def state_lib(self):
        """The library of the stream-residual and delta-rule kernels, compiled and loaded when a
        model first needs it."""
        if self._state is None:
            L = load_kernel_lib("garuda_state")
            L.gb_last_error.restype = ctypes.c_char_p
            for name, argtypes in self._STATE_SIGNATURES.items():
                fn = getattr(L, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            self._state = L
        return self._state

    @property
    def seq_lib(self):
        """The library of the post-norm, gated-recurrence and convolved-projection kernels, compiled
        and loaded when a model first needs it."""
        if self._seq is None:
            L = load_kernel_lib("garuda_seq")
            L.gb_last_error.restype = ctypes.c_char_p
            for name, argtypes in self._SEQ_SIGNATURES.items():
                fn = getattr(L, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            L.gb_mingru_scratch_floats.argtypes = [c_int, c_int, c_int]
            L.gb_mingru_scratch_floats.restype = c_longlong
            self._seq = L
        return self._seq

    _SEQ_SIGNATURES = {
        "gb_post_norm": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_void_p],
        "gb_group_gate_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "gb_xielu": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
        "gb_mingru": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                      c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "gb_conv_qkv": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_int, c_void_p],
        "gb_conv_state_shift": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                                c_void_p],
    }

    _STATE_SIGNATURES = {
        "gb_streams_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                               c_void_p],
        "gb_streams_update": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                              c_float, c_void_p, c_int, c_void_p],
        "gb_qkv_bias_append": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "gb_delta_prepare": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_void_p],
        "gb_delta_conv_state": [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "gb_delta_recurrence": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                c_int, c_void_p, c_void_p],
        "gb_delta_out": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_void_p],
        "gb_delta_decode": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p,
                            c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "gb_gdelta_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float,
                              c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "gb_gdelta_recurrence": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
        "gb_gdelta_decode": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float,
                             c_void_p, c_float, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_int,
                             c_void_p],
        "gb_qk_norm_rope_append": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                   c_void_p, c_int, c_int, c_void_p],
        "gb_gate_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "gb_unary_act": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "gb_sublayer_merge": [c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_float,
                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    }

    _MIXER_SIGNATURES = {
            "gb_latent_append": [c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
            "gb_head_gemm": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
            "gb_route_topk": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                              c_void_p, c_void_p],
            "gb_moe_gate_up": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_void_p, c_void_p],
            "gb_moe_down": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_float, c_void_p],
            "gb_moe_grouped": [c_void_p] * 6 + [c_int] * 7 + [c_float, c_float, c_int, c_int] + [c_void_p] * 4,
            "gb_moe_padded_prepare": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p],
            "gb_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
            "gb_grouped_gemm": [c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_longlong,
                                c_int, c_int, c_int, c_int, c_void_p],
            "gb_latent_query_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_void_p],
            "gb_latent_rows": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                               c_void_p],
    }

    def _stream(self):
        if self._held_stream is not None:
            return self._held_stream
        return torch.cuda.current_stream(self.device).cuda_stream

    @contextlib.contextmanager
    def on_current_stream(self):
        """Within the block every kernel is launched on the stream that is current now (asked
        for once, not per launch). The caller must not change the current stream inside."""
        outer = self._held_stream
        self._held_stream = torch.cuda.current_stream(self.device).cuda_stream
        try:
            yield
        finally:
            self._held_stream = outer

    def _check(self, lib, code: int, what: str, kernels: int = 1) -> None:
        if code != 0:
            raise KernelError(f"{what}: {lib.gb_last_error().decode()}")
        self.launches += kernels     # kernels of this library launched so far (not counting graph replays)

    def _on_device(self, *tensors):
        for t in tensors:
            if t is not None:
                _need(t.is_cuda, "kernel operands must live on the CUDA device")

    # ------------------------------------------------------------------ parts
    def inv_freq(self, rotary) -> torch.Tensor:
        """One frequency per pair of the head for a ``RotaryParams``: its own table if it has
        one, else ``1 / theta^(2i/head_dim)`` in 32-bit (garuda/src/simd/mod.rs:199). Made once
        per parameter set."""
        if rotary not in self._inv_freq:
            from ..parts.rotary import rotary_frequencies
            self._inv_freq[rotary] = torch.from_numpy(rotary_frequencies(rotary)).to(self.device)
        return self._inv_freq[rotary]

    def embedding(self, table, ids, out, scale: float = 1.0):
        """``out[t] = table[ids[t]] * scale`` in 32-bit; ``out [T, S, d]``: the row ``S`` times (a
        residual of several streams that all start as the embedding's output)."""
        self._on_device(table, ids, out)
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embedding: out must be contiguous float32")
        _need(ids.dtype == torch.int32, "embedding: ids must be int32")
        _need(table.is_contiguous() and table.shape[1] == out.shape[-1], "embedding: widths differ")
        T = ids.shape[0]
        _need(out.shape[0] >= T, "embedding: out has too few rows")
        copies = out.shape[1] if out.dim() == 3 else 1
        self._check(self.core, self.core.gb_embedding_copies(
            table.data_ptr(), _tag(table, "embedding table"), ids.data_ptr(), out.data_ptr(), T,
            table.shape[1], table.shape[0], float(scale), int(copies), self._stream()), "embedding")

    def scale_softcap(self, x, scale: float = 1.0, cap: float = 0.0):
        """``x <- x * scale``, then with ``cap`` > 0 ``x <- cap * tanh(x / cap)``; in place, 32-bit."""
        self._on_device(x)
        _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_softcap: contiguous float32")
        self._check(self.core, self.core.gb_scale_softcap(x.data_ptr(), x.numel(), float(scale), float(cap),
                                                          self._stream()), "scale_softcap")

    def rmsnorm(self, x, weight, eps, out, rows=None):
        self._on_device(x, weight, out, rows)
        _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: x must be contiguous float32")
        d = x.shape[1]
        _need(weight.numel() == d and out.shape[1] == d and out.is_contiguous(), "rmsnorm: widths differ")
        n = x.shape[0] if rows is None else rows.shape[0]
        _need(out.shape[0] == n, "rmsnorm: out has the wrong number of rows")
        if rows is not None:
            _need(rows.dtype == torch.int32, "rmsnorm: rows must be int32")
        self._check(self.core, self.core.gb_rmsnorm(
            x.data_ptr(), weight.data_ptr(), _tag(weight, "norm weight"), float(eps), out.data_ptr(),
            _tag(out, "rmsnorm out"), _ptr(rows), n, d, self._stream()), "rmsnorm")

    def linear(self, a, w, out, accumulate: bool = False, ctx=None, emit_norm=None, alpha: float = 1.0):
        """``out[M,N] (+)= a[M,K] @ w[N,K]^T``; accumulation is into a 32-bit ``out``, as
        ``out += alpha * product`` (``alpha``: a model's residual multiplier).

        ``emit_norm`` (with ``ctx``): the norm part that will be applied to ``out`` next. Where
        the kernel can, it folds that norm's first half into this product and returns a
        ``PendingNorm`` to hand to ``qkv_rope_append`` or ``linear_swiglu`` in place of the
        normed tensor; else it returns None and the norm runs as usual."""
        self._on_device(a, w, out)
        _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "linear: operands must be matrices")
        M, K = a.shape
        N = w.shape[0]
        if not (w.shape[1] == K and out.shape == (M, N)):       # the message is made only when it is needed
            _need(False, f"linear: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
        _need(a.dtype == w.dtype, "linear: a and w must have one dtype")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
        _need(accumulate or alpha == 1.0, "linear: a multiplier goes with accumulation only")
        if self.tc is not None and a.dtype == torch.bfloat16:
            pending = self._pending_for(ctx, emit_norm, out, accumulate) if alpha == 1.0 else None
            if self.tc.linear(a, w, out, accumulate, emit=pending, alpha=alpha):
                return pending
        self._check(self.core, self.core.gb_gemm_simple(
            a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _tag(a, "linear input"),
            _tag(out, "linear output"), int(accumulate), float(alpha), self._stream()), "linear")

    def _pending_for(self, ctx, norm, x, accumulate):
        """A ``PendingNorm`` with buffers for the product that adds into ``x``, or None."""
        if norm is None or ctx is None or not accumulate or x.dtype != torch.float32:
            return None
        fold = norm.fold() if hasattr(norm, "fold") else None
        T, d = x.shape
        tiles = self.tc.norm_tiles(T, d)
        if fold is None or not tiles:
            return None
        weight, eps = fold
        # two sets of buffers in turn: a block's second norm is pending while the first one's values are
        # still the operand of no kernel, but never more than two at a time
        turn = ctx.step_cache.get("pending_turn", 0) ^ 1
        ctx.step_cache["pending_turn"] = turn
        values = ctx.ws.get(f"pending_values_{turn}", (T, d), torch.bfloat16)
        sums = ctx.ws.get(f"pending_sums_{turn}", (tiles, T), torch.float32)
        return PendingNorm(values, sums, weight, eps, norm, x)

    def normed(self, ctx, h):
        """``h`` as a tensor: a ``PendingNorm`` is run as the ordinary norm."""
        return h.materialize(ctx) if isinstance(h, PendingNorm) else h

    def pack_gate_up(self, gate, up):
        """The layout ``linear_swiglu`` wants. With the tensor-core kernels: gate and
        up rows packed in groups of 64 (rows ``[128 g, 128 g + 64)`` are gate rows
        ``64 g ..``, the next 64 the matching up rows, zero rows padding the last
        group), so that a 128-row tile holds both values of 64 features. Without
        them: gate rows, then up rows."""
        F, K = gate.shape
        if self.tc is None or gate.dtype != torch.bfloat16:
            return torch.cat([gate, up], dim=0).contiguous()
        groups = (F + 63) // 64
        halves = []
        for m in (gate, up):
            padded = torch.zeros(groups * 64, K, dtype=m.dtype, device=m.device)
            padded[:F] = m
            halves.append(padded.view(groups, 64, K))
        packed = torch.stack(halves, dim=1).reshape(groups * 128, K).contiguous()
        packed.gb_group = 64
        return packed

    def linear_swiglu(self, ctx, h, w_gate_up, act):
        """``act[M,F] = silu(h @ gate^T) * (h @ up^T)``, the activation in 32-bit."""
        M, F = act.shape
        group = getattr(w_gate_up, "gb_group", 0)
        if isinstance(h, PendingNorm):
            if group == 64 and self.tc is not None and self.tc.linear_swiglu(h.values, w_gate_up, act, pending=h):
                return
            h = h.materialize(ctx)
        if (group == 64 and self.tc is not None and h.dtype == torch.bfloat16
                and self.tc.linear_swiglu(h, w_gate_up, act)):
            return
        tmp = ctx.ws.get("gate_up", (M, w_gate_up.shape[0]), torch.float32)
        self.linear(h, w_gate_up, tmp)
        self.silu_mul(tmp, act, group)

    def silu_mul(self, gate_up, out, group: int = 0):
        """``out[M,F] = silu(gate) * up``; ``gate_up`` rows are ``[gate | up]``, or with
        ``group`` 64 the packed layout of ``pack_gate_up``."""
        self._on_device(gate_up, out)
        M, F = out.shape
        width = 2 * group * ((F + group - 1) // group) if group else 2 * F
        _need(gate_up.shape == (M, width) and gate_up.is_contiguous() and out.is_contiguous(),
              f"silu_mul: gate_up must be [M, {width}] for out [M, {F}]")
        self._check(self.core, self.core.gb_silu_mul(
            gate_up.data_ptr(), _tag(gate_up, "silu_mul in"), out.data_ptr(), _tag(out, "silu_mul out"),
            M, F, group, width, self._stream()), "silu_mul")

    def residual_add(self, x, y):
        self._on_device(x, y)
        _need(x.dtype == torch.float32 and x.shape == y.shape and x.is_contiguous() and y.is_contiguous(),
              "residual_add: x must be contiguous float32 of y's shape")
        self._check(self.core, self.core.gb_residual_add(
            x.data_ptr(), y.data_ptr(), _tag(y, "residual_add y"), x.numel(), self._stream()), "residual_add")

    def qkv_rope_append(self, ctx, h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                        heads, kv_heads, head_dim, rotary, page_size):
        """``h @ w_qkv^T``, split into heads; queries and keys rotated (``rotary`` None:
        not), queries to ``q_out [T, heads, head_dim]``, keys and values into their
        pages. One kernel where the tensor-core product takes the shape, else the
        product in 32-bit followed by ``rope_kv_append``."""
        pending = h if isinstance(h, PendingNorm) else None
        if pending is not None:
            h = pending.values
            if self.tc is None or not self.tc.takes_qkv(h, w_qkv, q_out, head_dim):
                h, pending = pending.materialize(ctx), None
        self._on_device(h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table)
        T = h.shape[0]
        _need(w_qkv.shape == ((heads + 2 * kv_heads) * head_dim, h.shape[1]), "qkv_rope_append: weight shape")
        _need(q_out.is_contiguous() and q_out.shape == (T, heads, head_dim), "qkv_rope_append: q_out shape")
        if kv_heads:
            _need(k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.dtype == q_out.dtype
                  and tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), "qkv_rope_append: pool shape")
            _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "qkv_rope_append: block table")
        _need(positions.dtype == torch.int32 and token_req.dtype == torch.int32, "qkv_rope_append: int32 indices")
        if self.tc is not None and self.tc.takes_qkv(h, w_qkv, q_out, head_dim):
            table = None if rotary is None else self.rope_table(ctx, positions, rotary)
            self.tc.qkv_rope_append(h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads,
                                    kv_heads, head_dim, table, None if rotary is None else rotary.interleaved,
                                    page_size, pending=pending)
            return
        qkv = ctx.ws.get("qkv", (T, w_qkv.shape[0]), torch.float32)
        self.linear(h, w_qkv, qkv)
        self.rope_kv_append(qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            head_dim, rotary, page_size)

    def rope_table(self, ctx, positions, rotary):
        """``[T, head_dim / 2, 2]`` cosines and sines of every token's angles, made once per
        step (kept in the step's context) for every layer's fused projection to read."""
        half = rotary.head_dim // 2
        key = ("rope_table", rotary, positions.data_ptr(), positions.shape[0])
        cache = getattr(ctx, "step_cache", None)
        if cache is not None and key in cache:
            return cache[key]
        T = positions.shape[0]
        name = f"rope_table_{rotary.theta}_{rotary.head_dim}_{hash(rotary.inv_freq)}"
        out = ctx.ws.get(name, (T, half, 2), torch.float32)
        inv = self.inv_freq(rotary)
        code = self.core.gb_rope_table(positions.data_ptr(), inv.data_ptr(), out.data_ptr(), T, half, self._stream())
        self._check(self.core, code, "rope_table")
        if cache is not None:
            cache[key] = out
        return out

    def rope_kv_append(self, qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                       heads, kv_heads, head_dim, rotary, page_size):
        """Split ``qkv [T, (heads + 2 kv_heads) head_dim]``, rotate queries and keys
        (``rotary`` None: leave them), write queries to ``q_out [T, heads, head_dim]``
        and keys and values into their pages."""
        self._on_device(qkv, q_out, k_pool, v_pool, positions, token_req, block_table)
        T = qkv.shape[0]
        _need(qkv.stride(1) == 1 and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim,
              "rope_kv_append: qkv has the wrong width")
        _need(q_out.is_contiguous() and q_out.shape == (T, heads, head_dim), "rope_kv_append: q_out shape")
        _need(positions.dtype == torch.int32 and token_req.dtype == torch.int32, "rope_kv_append: int32 indices")
        if kv_heads:
            _need(k_pool.dtype == q_out.dtype and v_pool.dtype == q_out.dtype, "rope_kv_append: cache dtype")
            _need(k_pool.is_contiguous() and v_pool.is_contiguous() and
                  tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), "rope_kv_append: pool shape")
            _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "rope_kv_append: block table")
        inv = None
        inter = 0
        if rotary is not None:
            _need(rotary.head_dim == head_dim, "rope_kv_append: rotary is for another head_dim")
            inv = self.inv_freq(rotary)
            inter = int(rotary.interleaved)
        self._check(self.core, self.core.gb_rope_kv_append(
            qkv.data_ptr(), _tag(qkv, "qkv"), qkv.stride(0), q_out.data_ptr(), _ptr(k_pool), _ptr(v_pool),
            _tag(q_out, "q_out"), positions.data_ptr(), token_req.data_ptr(), _ptr(block_table),
            block_table.shape[1] if block_table is not None else 0, T, heads, kv_heads, head_dim,
            _ptr(inv), inter, page_size, self._stream()), "rope_kv_append")

    def rope_inplace(self, x, positions, rotary):
        """Rotate ``x [T, H, rotary.head_dim]`` (float32; rows and heads may be strided, so a
        view of every head's first channels will do) in place."""
        self._on_device(x, positions)
        _need(x.dtype == torch.float32 and x.dim() == 3 and x.stride(2) == 1 and x.stride(1) >= x.shape[2],
              "rope_inplace: x must be float32 [T, H, width] with unit stride along the width")
        T, H, hd = x.shape
        _need(hd == rotary.head_dim, "rope_inplace: the view is not as wide as the rotation")
        self._check(self.core, self.core.gb_rope_inplace(
            x.data_ptr(), x.stride(0), x.stride(1), T, H, hd, positions.data_ptr(),
            self.inv_freq(rotary).data_ptr(), int(rotary.interleaved), self._stream()), "rope_inplace")

    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out,
                        scale, window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1,
                        value_dim=None, softcap: float = 0.0, keep_first: int = 0, sink: bool = False,
                        sink_values=None, distance=None, chunk: int = 0):
        """``value_dim``: how many of a value row's first channels are the value (``out`` is then
        ``[T, Hq * value_dim]``); None: all ``hd``. A mixer whose keys and values are parts of one
        cached row passes the same pool for both and the narrower width; a value pool of its own may
        have rows of another width than the keys'. ``softcap`` c > 0: scores become ``c tanh(s / c)``.
        ``keep_first`` n: a windowed query also reads its request's first n positions. ``sink``: one
        is added to the softmax's denominator (an entry of score zero without a value).
        ``sink_values`` (32-bit ``[Hq]``): ``exp(sink_values[h])`` is added there instead, a learned
        number per head. ``distance = (r1, r2)`` (32-bit ``[Hq]`` each): ``r1[h] ln(1 + r2[h] (i - j))``
        is taken off the score of key ``j`` for the query at ``i``. ``chunk`` n: a query reads only
        the keys ``j <= i`` with ``floor(j / n) = floor(i / n)`` (no window then)."""
        self._on_device(q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, sink_values)
        r1, r2 = distance if distance is not None else (None, None)
        self._on_device(r1, r2)
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        v_hd = v_pool.shape[3]
        vd = v_hd if value_dim is None else int(value_dim)
        _need(q.is_contiguous() and out.is_contiguous() and out.shape == (T, Hq * vd), "attention: q/out shape")
        _need(q.dtype == k_pool.dtype == v_pool.dtype == out.dtype, "attention: one dtype for q, cache and out")
        _need(tuple(k_pool.shape[1:]) == (Hkv, page_size, hd) and tuple(v_pool.shape[:3]) == tuple(k_pool.shape[:3])
              and k_pool.is_contiguous() and v_pool.is_contiguous(), "attention: pool shape")
        _need(0 < vd <= v_hd, "attention: value_dim must be within the row")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: block table")
        for v in (sink_values, r1, r2):
            _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == Hq),
                  "attention: one float32 number per query head")
        _need(not chunk or not (window or keep_first), "attention: a chunked mask goes with no window")
        extras = sink_values is not None or distance is not None or chunk > 0
        plain = softcap == 0.0 and keep_first == 0 and not sink and v_hd == hd and not extras
        if (extras and self.tc is not None and q.dtype == torch.bfloat16 and self.tc.extras_attention(
                q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale, page_size, num_requests,
                max_q_len, max_kv_len, ws, vd, softcap, sink_values, r1, r2, chunk, window, keep_first, sink, min_q_len)):
            return
        if not plain and not extras and self.tc is not None and q.dtype == torch.bfloat16 and vd == v_hd and self.tc.capped_attention(
                q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale, window, page_size,
                num_requests, max_q_len, max_kv_len, ws, softcap, keep_first, sink, min_q_len):
            return
        if (plain and vd < hd and Hkv == 1 and window == 0 and self.tc is not None and q.dtype == torch.bfloat16
                and k_pool.data_ptr() == v_pool.data_ptr()
                and self.tc.latent_attention(q, k_pool, out, block_table, cu_q, kv_lens, vd, scale, page_size,
                                             num_requests, max_q_len, max_kv_len, ws)):
            return          # keys and values are parts of one cached row that every head reads
        if plain and vd == hd and self.tc is not None and q.dtype == torch.bfloat16 and self.tc.paged_attention(
                q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale, window, page_size,
                num_requests, max_q_len, max_kv_len, ws, min_q_len):
            return
        self._check(self.core, self.core.gb_attention_simple(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _tag(q, "attention q"),
            block_table.data_ptr(), block_table.shape[1], cu_q.data_ptr(), kv_lens.data_ptr(),
            token_req.data_ptr(), out.data_ptr(), T, Hq, Hkv, hd, v_hd, vd, float(scale), int(window),
            int(page_size), float(softcap), int(keep_first), int(bool(sink)), _ptr(sink_values), _ptr(r1), _ptr(r2),
            int(chunk), self._stream()), "attention")

    # ------------------------------------------------------------------ more norms and residual forms
    def layernorm(self, x, weight, bias, eps, out, rows=None):
        """``(x - mean) / sqrt(var + eps) * weight + bias`` per row (``bias`` may be None), 32-bit
        arithmetic, ``out`` in its own dtype; ``rows``: only these rows of ``x``."""
        self._on_device(x, weight, bias, out, rows)
        _need(x.dtype == torch.float32 and x.is_contiguous(), "layernorm: x must be contiguous float32")
        d = x.shape[1]
        _need(weight.numel() == d and out.shape[1] == d and out.is_contiguous(), "layernorm: widths differ")
        _need(bias is None or (bias.numel() == d and bias.dtype == weight.dtype), "layernorm: bias")
        n = x.shape[0] if rows is None else rows.shape[0]
        _need(out.shape[0] == n, "layernorm: out has the wrong number of rows")
        if rows is not None:
            _need(rows.dtype == torch.int32, "layernorm: rows must be int32")
        self._check(self.core, self.core.gb_layernorm(
            x.data_ptr(), weight.data_ptr(), _ptr(bias), _tag(weight, "norm weight"), float(eps), out.data_ptr(),
            _tag(out, "layernorm out"), _ptr(rows), n, d, self._stream()), "layernorm")

    def residual_axpy(self, x, y=None, alpha: float = 1.0, row=None):
        """``x[t] += alpha * y[t] + row`` on the 32-bit residual; ``y`` or ``row`` may be None."""
        self._on_device(x, y, row)
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "residual_axpy: x must be float32 [T, d]")
        T, d = x.shape
        _need(y is None or (y.shape == x.shape and y.is_contiguous()), "residual_axpy: y must have x's shape")
        _need(row is None or (row.numel() == d and row.is_contiguous()), "residual_axpy: row must be [d]")
        if y is None and row is None:
            return
        self._check(self.core, self.core.gb_residual_axpy(
            x.data_ptr(), _ptr(y), _tag(y, "residual_axpy y") if y is not None else GB_F32, float(alpha), _ptr(row),
            _tag(row, "residual_axpy row") if row is not None else GB_F32, T, d, self._stream()), "residual_axpy")

    def rms_add(self, x, y, weight, eps, alpha: float = 1.0):
        """``x[t] += alpha * y[t] / sqrt(mean(y[t]^2) + eps) * weight`` (x, y 32-bit)."""
        self._on_device(x, y, weight)
        _need(x.dtype == torch.float32 and y.dtype == torch.float32 and x.shape == y.shape and x.is_contiguous()
              and y.is_contiguous() and weight.numel() == x.shape[1], "rms_add: x and y float32 [T, d], weight [d]")
        self._check(self.core, self.core.gb_rms_add(
            x.data_ptr(), y.data_ptr(), weight.data_ptr(), _tag(weight, "rms_add weight"), float(eps), float(alpha),
            x.shape[0], x.shape[1], self._stream()), "rms_add")

    def gelu_gather_mul(self, z, table, ids, col0, out):
        """``out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j]``."""
        self._on_device(z, table, ids, out)
        T, dim = out.shape
        _need(z.shape == out.shape and z.is_contiguous() and out.is_contiguous() and table.is_contiguous()
              and ids.dtype == torch.int32, "gelu_gather_mul: shapes")
        self._check(self.core, self.core.gb_gelu_gather_mul(
            z.data_ptr(), _tag(z, "z"), table.data_ptr(), _tag(table, "table"), table.shape[1], int(col0),
            ids.data_ptr(), out.data_ptr(), _tag(out, "out"), T, dim, table.shape[0], self._stream()), "gelu_gather_mul")

    def cast(self, x, out):
        """``out = x`` rounded to ``out``'s dtype (x 32-bit)."""
        self._on_device(x, out)
        _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.numel() == out.numel(),
              "cast: float32 in, same size out")
        self._check(self.core, self.core.gb_cast(x.data_ptr(), out.data_ptr(), _tag(out, "cast out"), x.numel(),
                                                 self._stream()), "cast")

    # ------------------------------------------------------------------ gated feed-forwards
    GATE_ACTS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}

    def gated_act(self, gate_up, out, kind: str = "silu", limit: float = 0.0, group: int = 0):
        """``out[M,F] = act(gate, up)``: ``silu(g) u``, ``gelu_tanh(g) u`` or, clamped,
        ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``.
        ``gate_up`` rows are ``[gate | up]``, or with ``group`` 64 the layout of ``pack_gate_up``."""
        self._on_device(gate_up, out)
        M, F = out.shape
        width = 2 * group * ((F + group - 1) // group) if group else 2 * F
        _need(gate_up.shape == (M, width) and gate_up.is_contiguous() and out.is_contiguous(),
              f"gated_act: gate_up must be [M, {width}] for out [M, {F}]")
        self._check(self.core, self.core.gb_gated_act(
            gate_up.data_ptr(), _tag(gate_up, "gated_act in"), out.data_ptr(), _tag(out, "gated_act out"),
            M, F, group, width, self.GATE_ACTS[kind], float(limit), self._stream()), "gated_act")

    def linear_gated(self, ctx, h, w_gate_up, act, kind: str = "silu", limit: float = 0.0):
        """``act[M,F] = act(h @ gate^T, h @ up^T)``; ``w_gate_up`` from ``pack_gate_up``."""
        if kind == "silu":
            return self.linear_swiglu(ctx, h, w_gate_up, act)
        M, F = act.shape
        group = getattr(w_gate_up, "gb_group", 0)
        h = self.normed(ctx, h)
        if (group == 64 and self.tc is not None and h.dtype == torch.bfloat16
                and self.tc.linear_swiglu(h, w_gate_up, act, kind=self.GATE_ACTS[kind], limit=limit)):
            return
        tmp = ctx.ws.get("gate_up", (M, w_gate_up.shape[0]), torch.float32)
        self.linear(h, w_gate_up, tmp)
        self.gated_act(tmp, act, kind, limit, group)

    # ------------------------------------------------------------------ routed experts
    ROUTER_SCORES = {"softmax_chosen": 0, "sigmoid": 1, "softmax_all": 2}

    def route_topk(self, h, w_router, bias, top, ids, weights, score: str = "softmax_chosen"):
        """Router logits ``h @ w_router^T + bias`` in 32-bit; ``ids[T, top]`` the experts with the
        largest logits (descending), ``weights[T, top]`` the softmax over those logits only, or
        (``score`` "sigmoid") each chosen expert's ``sigmoid(logit)``, not renormalized, or
        (``"softmax_all"``) its share of the softmax over all experts' logits, not renormalized."""
        self._on_device(h, w_router, bias, ids, weights)
        T, K = h.shape
        E = w_router.shape[0]
        _need(h.is_contiguous() and w_router.is_contiguous() and w_router.shape[1] == K, "route_topk: shapes")
        _need(ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.shape == (T, top)
              and weights.shape == (T, top) and ids.is_contiguous() and weights.is_contiguous(), "route_topk: outputs")
        _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == E), "route_topk: a float32 bias")
        self._check(self.mixers, self.mixers.gb_route_topk(
            h.data_ptr(), _tag(h, "router input"), w_router.data_ptr(), _ptr(bias), _tag(w_router, "router"),
            T, E, K, int(top), self.ROUTER_SCORES[score], ids.data_ptr(), weights.data_ptr(), self._stream()), "route_topk")

    def moe_gate_up(self, h, w_gate_up, ids, act, kind: str, limit: float, in_scale=None):
        """``act[T, top, F]``: every token's gate/up products against its chosen experts'
        weights ``w_gate_up[E, 2F, K]`` (gate rows, then up rows), through the activation.
        ``in_scale [T, top]``: a factor on what goes into each chosen expert."""
        self._on_device(h, w_gate_up, ids, act)
        T, K = h.shape
        top = ids.shape[1]
        E, F2, _ = w_gate_up.shape
        _need(h.is_contiguous() and w_gate_up.is_contiguous() and act.is_contiguous() and h.dtype == w_gate_up.dtype
              and w_gate_up.shape[2] == K and act.shape == (T, top, F2 // 2), "moe_gate_up: shapes")
        self._check(self.mixers, self.mixers.gb_moe_gate_up(
            h.data_ptr(), _tag(h, "h"), w_gate_up.data_ptr(), _tag(w_gate_up, "w"), ids.data_ptr(), act.data_ptr(),
            _tag(act, "act"), T, top, F2 // 2, K, self.GATE_ACTS[kind], float(limit), _ptr(in_scale), self._stream()),
            "moe_gate_up")

    def moe_down(self, act, w_down, ids, weights, x, alpha: float = 1.0):
        """``x[t] += alpha * sum_j weights[t, j] * (act[t, j] @ w_down[ids[t, j]]^T)``; ``weights``
        None: all one."""
        self._on_device(act, w_down, ids, weights, x)
        T, top, F = act.shape
        E, N, _ = w_down.shape
        _need(act.is_contiguous() and w_down.is_contiguous() and w_down.shape[2] == F and x.shape == (T, N)
              and x.dtype == torch.float32 and x.is_contiguous(), "moe_down: shapes")
        self._check(self.mixers, self.mixers.gb_moe_down(
            act.data_ptr(), _tag(act, "act"), w_down.data_ptr(), _tag(w_down, "w"), ids.data_ptr(),
            _ptr(weights), x.data_ptr(), T, top, F, N, float(alpha), self._stream()), "moe_down")

    def pack_expert_gate_up(self, gates, ups):
        """The experts' gate and up matrices stacked, in the layout ``routed_feed_forward`` wants:
        ``[E, 2F, K]`` (an expert's gate rows, then its up rows), or, where the tensor-core products
        take the sizes, every expert packed as ``pack_gate_up`` packs: ``[E, 128 ceil(F / 64), K]``."""
        F, K = gates[0].shape
        if self.tc is not None and gates[0].dtype == torch.bfloat16 and K % 8 == 0 and F % 8 == 0 and len(gates) <= 4096:
            packed = torch.stack([self.pack_gate_up(g, u) for g, u in zip(gates, ups)]).contiguous()
            packed.gb_group = 64
            return packed
        return torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()

    #: (token, choice) pairs from which the routed experts run on the tcgen05 grouped product
    GROUPED_TC_PAIRS = 1024

    def routed_feed_forward(self, ctx, h, w_gate_up, w_down, ids, weights, x, kind: str, limit: float,
                            alpha: float = 1.0, scale_input: bool = False):
        """``x[t] += alpha * sum_j weights[t, j] * expert_{ids[t, j]}(h[t])`` with the experts'
        weights stacked: ``w_gate_up`` from ``pack_expert_gate_up``, ``w_down [E, N, F]``.
        ``scale_input``: the weight multiplies what goes into the expert instead,
        ``sum_j expert(weights[t, j] * h[t])``."""
        T, top = ids.shape
        E, N, F = w_down.shape
        K = h.shape[1]
        packed = getattr(w_gate_up, "gb_group", 0) == 64
        if packed and T * top >= self.GROUPED_TC_PAIRS and self._routed_tcgen05(ctx, h, w_gate_up, w_down, ids, weights,
                                                                               x, kind, limit, alpha, scale_input):
            return
        if packed:
            # on the tensor cores: pairs sorted by expert on the device, two grouped products, a weighted sum
            self._on_device(h, w_gate_up, w_down, ids, weights, x)
            _need(h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and ids.is_contiguous()
                  and weights.is_contiguous() and x.is_contiguous() and x.dtype == torch.float32
                  and tuple(w_gate_up.shape) == (E, 128 * ((F + 63) // 64), K) and x.shape == (T, N) and ids.dtype == torch.int32
                  and weights.dtype == torch.float32 and w_gate_up.dtype == w_down.dtype == torch.bfloat16,
                  "routed_feed_forward: shapes")
            L = self.mixers
            words = int(L.gb_moe_grouped_index_words(T * top, E))
            index = ctx.ws.get("expert_index", (words,), torch.int32)
            act = ctx.ws.get("expert_act", (T * top, F), torch.bfloat16)
            y = ctx.ws.get("expert_rows", (T * top, N), torch.float32)
            self._check(L, L.gb_moe_grouped(
                h.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), ids.data_ptr(), weights.data_ptr(), x.data_ptr(),
                T, top, E, F, K, N, self.GATE_ACTS[kind], float(limit), float(alpha), 1, int(scale_input), index.data_ptr(),
                act.data_ptr(), y.data_ptr(), self._stream()), "moe_grouped", 4)
            return
        act = ctx.ws.get("expert_act", (T, top, F), h.dtype)
        self.moe_gate_up(h, w_gate_up, ids, act, kind, limit, weights if scale_input else None)
        self.moe_down(act, w_down, ids, None if scale_input else weights, x, alpha)

    def _routed_tcgen05(self, ctx, h, w_gate_up, w_down, ids, weights, x, kind, limit, alpha, scale_input=False) -> bool:
        """Many pairs: sorted by expert into blocks of 128 rows (padding rows zero), then the two
        products on the tcgen05 many-token kernel with each block's expert read from a list."""
        T, top = ids.shape
        E, N, F = w_down.shape
        K = h.shape[1]
        L, tc = self.mixers, self.tc
        rows = int(L.gb_moe_padded_rows(T * top, E))
        blocks = rows // 128
        gu_rows = w_gate_up.shape[1]
        a = ctx.ws.get("expert_in", (rows, K), torch.bfloat16)
        act = ctx.ws.get("expert_act_padded", (rows, F), torch.bfloat16)
        if not (tc.lib.gb_gemm_tc_supported(a.data_ptr(), w_gate_up.data_ptr(), rows, F, K)
                and tc.lib.gb_gemm_tc_supported(act.data_ptr(), w_down.data_ptr(), rows, N, F)):
            return False
        self._on_device(h, w_gate_up, w_down, ids, weights, x)
        _need(h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and ids.is_contiguous()
              and weights.is_contiguous() and x.is_contiguous() and x.dtype == torch.float32 and x.shape == (T, N)
              and ids.dtype == torch.int32 and weights.dtype == torch.float32
              and h.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16, "routed_feed_forward: shapes")
        index = ctx.ws.get("expert_index_padded", (T * top + 2 * blocks,), torch.int32)
        y = ctx.ws.get("expert_rows_padded", (rows, N), torch.float32)
        self._check(L, L.gb_moe_padded_prepare(h.data_ptr(), ids.data_ptr(), T, top, E, K, gu_rows, N, index.data_ptr(),
                                               a.data_ptr(), weights.data_ptr() if scale_input else None,
                                               self._stream()), "moe_padded_prepare", 2)
        block_gu = index.data_ptr() + 4 * T * top
        block_dn = block_gu + 4 * blocks
        tc.grouped(a, w_gate_up, act, F, E, block_gu, 2, gate_act=self.GATE_ACTS[kind], gate_limit=limit)
        tc.grouped(act, w_down, y, N, E, block_dn, 0)
        self._check(L, L.gb_moe_combine(y.data_ptr(), index.data_ptr(), None if scale_input else weights.data_ptr(), x.data_ptr(), T, top, N,
                                        float(alpha), self._stream()), "moe_combine")
        return True

    # ------------------------------------------------------------------ attention over a cached latent
    def latent_append(self, src, norm_w, eps, rank, rot, rotary, positions, token_req, block_table, pool, page_size):
        """A step's cache rows ``[rms(src[:, :rank]) * norm_w | rotate(src[:, rank:rank + rot])]``
        written to their pages. ``src``: 32-bit rows (a view with any row stride); ``rotary``: a
        ``RotaryParams`` over the turned channels (pairs ``(2i, 2i + 1)``), or None."""
        self._on_device(src, norm_w, positions, token_req, block_table, pool)
        T = src.shape[0]
        _need(src.dtype == torch.float32 and src.stride(1) == 1 and src.shape[1] == rank + rot, "latent_append: src")
        _need(pool.is_contiguous() and tuple(pool.shape[1:]) == (1, page_size, rank + rot), "latent_append: pool shape")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "latent_append: block table")
        inv, dims = None, 0
        if rotary is not None:
            _need(rotary.interleaved and rotary.head_dim <= rot, "latent_append: pairs (2i, 2i + 1) within the rotated part")
            inv, dims = self.inv_freq(rotary), rotary.head_dim
        self._check(self.mixers, self.mixers.gb_latent_append(
            src.data_ptr(), src.stride(0), norm_w.data_ptr(), _tag(norm_w, "latent norm"), float(eps), int(rank),
            int(rot), int(dims), _ptr(inv), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], int(page_size), pool.data_ptr(), _tag(pool, "latent pool"), T, self._stream()),
            "latent_append")

    def latent_query_prepare(self, src, heads, dn, rot, rotary, positions, q_nope, q_lat):
        """From a step's 32-bit query rows ``src [T, heads * (dn + rot)]`` (a view with any row
        stride): the unrotated parts to ``q_nope [T, heads, dn]``, the rotated parts, turned at the
        tokens' positions, to the last ``rot`` channels of ``q_lat [T, heads, *]``."""
        self._on_device(src, positions, q_nope, q_lat)
        T = src.shape[0]
        _need(src.dtype == torch.float32 and src.stride(1) == 1 and src.shape[1] == heads * (dn + rot), "latent_query_prepare: src")
        _need(q_nope.is_contiguous() and q_lat.is_contiguous() and q_nope.dtype == q_lat.dtype
              and tuple(q_nope.shape) == (T, heads, dn) and q_lat.shape[:2] == (T, heads) and q_lat.shape[2] >= rot,
              "latent_query_prepare: outputs")
        inv, dims = None, 0
        if rotary is not None:
            _need(rotary.interleaved and rotary.head_dim <= rot, "latent_query_prepare: pairs (2i, 2i + 1) within the rotated part")
            inv, dims = self.inv_freq(rotary), rotary.head_dim
        self._check(self.mixers, self.mixers.gb_latent_query_prepare(
            src.data_ptr(), src.stride(0), int(heads), int(dn), int(rot), int(dims), _ptr(inv), positions.data_ptr(),
            q_nope.data_ptr(), q_lat.data_ptr(), _tag(q_lat, "q_lat"), q_lat.shape[2], T, self._stream()),
            "latent_query_prepare")

    def latent_rows(self, src, heads, dn, rot, rank, rotary, positions, q_nope, q_lat, norm_w, eps, token_req,
                    block_table, pool, page_size):
        """``latent_query_prepare`` and ``latent_append`` in one kernel, for a step's 32-bit rows
        ``src [T, heads * (dn + rot) + rank + rot]`` (a view with any row stride): queries first, then
        the latent and its key part."""
        self._on_device(src, positions, q_nope, q_lat, norm_w, token_req, block_table, pool)
        T = src.shape[0]
        _need(src.dtype == torch.float32 and src.stride(1) == 1 and src.shape[1] == heads * (dn + rot) + rank + rot,
              "latent_rows: src")
        _need(q_nope.is_contiguous() and q_lat.is_contiguous() and q_nope.dtype == q_lat.dtype == pool.dtype
              and tuple(q_nope.shape) == (T, heads, dn) and tuple(q_lat.shape) == (T, heads, rank + rot), "latent_rows: outputs")
        _need(pool.is_contiguous() and tuple(pool.shape[1:]) == (1, page_size, rank + rot), "latent_rows: pool shape")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "latent_rows: block table")
        inv, dims = None, 0
        if rotary is not None:
            _need(rotary.interleaved and rotary.head_dim <= rot, "latent_rows: pairs (2i, 2i + 1) within the rotated part")
            inv, dims = self.inv_freq(rotary), rotary.head_dim
        self._check(self.mixers, self.mixers.gb_latent_rows(
            src.data_ptr(), src.stride(0), int(heads), int(dn), int(rot), int(dims), _ptr(inv), positions.data_ptr(),
            q_nope.data_ptr(), q_lat.data_ptr(), norm_w.data_ptr(), _tag(norm_w, "latent norm"), float(eps), int(rank),
            token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], int(page_size), pool.data_ptr(),
            _tag(pool, "latent pool"), T, self._stream()), "latent_rows")

    def head_linear(self, a, w, out, n, k, transposed: bool, tail: int = 0):
        """One small product per head: ``out[t, h, :n] = a[t, h, :k] @ w_h^T`` and
        ``out[t, h, n:n + tail] = a[t, h, k:k + tail]``. ``a [T, H, >= k + tail]`` and ``out
        [T, H, >= n + tail]`` may be views (unit stride along the last axis). ``w`` is contiguous:
        ``[H * n, k]`` (``w_h`` = its rows ``h n ..``) or, ``transposed``, ``[H * k, n]`` (``w_h^T``
        = its rows ``h k ..``: the product with the transposed per-head matrix)."""
        self._on_device(a, w, out)
        T, H = a.shape[0], a.shape[1]
        _need(a.dim() == 3 and out.dim() == 3 and a.stride(2) == 1 and out.stride(2) == 1 and out.shape[:2] == (T, H)
              and a.shape[2] >= k + tail and out.shape[2] >= n + tail, "head_linear: a and out are [T, H, *] views")
        _need(w.is_contiguous() and tuple(w.shape) == ((H * k, n) if transposed else (H * n, k)), "head_linear: weight shape")
        if (self.tc is not None and not transposed and tail == 0 and a.dtype == w.dtype == out.dtype == torch.bfloat16
                and k % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) % 8 == 0 and a.data_ptr() % 16 == 0):
            # on the tensor cores: one grouped product, a group per head
            self._check(self.mixers, self.mixers.gb_grouped_gemm(
                a.data_ptr(), a.stride(0), a.stride(1), w.data_ptr(), n * k, out.data_ptr(), out.stride(0),
                out.stride(1), H, T, int(n), int(k), self._stream()), "grouped_gemm")
            return
        w_n, w_k = (1, n) if transposed else (k, 1)
        self._check(self.mixers, self.mixers.gb_head_gemm(
            a.data_ptr(), _tag(a, "a"), a.stride(0), a.stride(1), w.data_ptr(), _tag(w, "w"), n * k, w_n, w_k,
            out.data_ptr(), _tag(out, "out"), out.stride(0), out.stride(1), T, H, int(n), int(k), int(tail),
            self._stream()), "head_linear")

    # ------------------------------------------------------------------ a residual of several streams
    #: a stream write may compute the next sublayer's normed input in the same pass
    fuses_stream_reads = True

    def streams_rmsnorm(self, x, in_w, weight, eps, out, rows=None):
        """``out[r] = rms(sum_s in_w[s] x[row, s]) * weight`` for ``x [T, S, d]`` (32-bit); ``rows``:
        only these rows of ``x``."""
        self._on_device(x, in_w, weight, out, rows)
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3, "streams_rmsnorm: x must be float32 [T, S, d]")
        T, S, d = x.shape
        _need(in_w.dtype == torch.float32 and in_w.numel() == S and weight.numel() == d and out.shape[1] == d
              and out.is_contiguous(), "streams_rmsnorm: shapes")
        n = T if rows is None else rows.shape[0]
        _need(out.shape[0] == n and (rows is None or rows.dtype == torch.int32), "streams_rmsnorm: rows")
        L = self.state_lib
        self._check(L, L.gb_streams_rmsnorm(x.data_ptr(), in_w.data_ptr(), weight.data_ptr(), _tag(weight, "norm weight"),
                                            float(eps), out.data_ptr(), _tag(out, "streams_rmsnorm out"), _ptr(rows), n, S, d,
                                            self._stream()), "streams_rmsnorm")

    def streams_update(self, x, mix, out_w, y, next_in=None, norm_weight=None, eps: float = 0.0, normed=None):
        """``x[t, j] <- sum_s mix[s, j] x[t, s] + out_w[j] y[t]`` for all ``j`` at once (``x [T, S, d]``,
        ``y [T, d]``, 32-bit). With ``next_in``: also ``normed[t] = rms(sum_s next_in[s] x[t, s]) *
        norm_weight`` of the new streams, in the same pass."""
        self._on_device(x, mix, out_w, y, next_in, norm_weight, normed)
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3, "streams_update: x must be float32 [T, S, d]")
        T, S, d = x.shape
        _need(y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (T, d), "streams_update: y must be float32 [T, d]")
        _need(mix.dtype == torch.float32 and out_w.dtype == torch.float32 and mix.numel() == S * S and out_w.numel() == S
              and mix.is_contiguous(), "streams_update: weights")
        L = self.state_lib
        if next_in is None:
            self._check(L, L.gb_streams_update(x.data_ptr(), mix.data_ptr(), out_w.data_ptr(), y.data_ptr(), T, S, d, None,
                                               None, GB_F32, 0.0, None, GB_F32, self._stream()), "streams_update")
            return
        _need(next_in.dtype == torch.float32 and next_in.numel() == S and norm_weight.numel() == d
              and tuple(normed.shape) == (T, d) and normed.is_contiguous(), "streams_update: the next read")
        self._check(L, L.gb_streams_update(x.data_ptr(), mix.data_ptr(), out_w.data_ptr(), y.data_ptr(), T, S, d,
                                           next_in.data_ptr(), norm_weight.data_ptr(), _tag(norm_weight, "norm weight"),
                                           float(eps), normed.data_ptr(), _tag(normed, "normed"), self._stream()),
                    "streams_update")

    def qkv_bias_append(self, qkv, bias, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                        head_dim, value_dim, page_size):
        """Split ``qkv [T, heads * head_dim + kv_heads * (head_dim + value_dim)]`` (+ ``bias``):
        queries to ``q_out [T, heads, head_dim]``, keys (``head_dim`` wide) and values (``value_dim``
        wide) into their pages. Nothing is rotated."""
        self._on_device(qkv, bias, q_out, k_pool, v_pool, positions, token_req, block_table)
        T = qkv.shape[0]
        cols = heads * head_dim + kv_heads * (head_dim + value_dim)
        _need(qkv.is_contiguous() and qkv.shape[1] == cols, "qkv_bias_append: qkv has the wrong width")
        _need(bias is None or (bias.numel() == cols and bias.is_contiguous()), "qkv_bias_append: bias")
        _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, heads, head_dim), "qkv_bias_append: q_out shape")
        _need(k_pool.dtype == q_out.dtype == v_pool.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
              and tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
              and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim), "qkv_bias_append: pool shapes")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and positions.dtype == torch.int32
              and token_req.dtype == torch.int32, "qkv_bias_append: int32 indices")
        L = self.state_lib
        self._check(L, L.gb_qkv_bias_append(
            qkv.data_ptr(), _tag(qkv, "qkv"), _ptr(bias), _tag(bias, "bias") if bias is not None else GB_F32,
            q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _tag(q_out, "q_out"), positions.data_ptr(),
            token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], T, heads, kv_heads, head_dim,
            value_dim, page_size, self._stream()), "qkv_bias_append")

    # ------------------------------------------------------------------ gated delta rule with channel decay
    def delta_rule(self, ctx, proj, second, conv_w, a_log, dt_bias, norm_w, eps, state, heads, kv_heads, dim, vdim,
                   taps, out, decay_per_head: bool = False, gate: str = "sigmoid"):
        """The recurrent part of a delta-rule mixer for one step. ``proj [T, 2 G dim + H vdim + H]``
        (32-bit: q | k | v before their convolution, beta's logit), ``second [T, H dim + H vdim]``
        (32-bit: the decay's pre-activation, the output gate's logit), ``conv_w [2 G dim + H vdim,
        taps]``, ``state [slots, H dim vdim + (taps - 1) (2 G dim + H vdim)]`` (32-bit: S, then the
        kept last inputs of the convolution). ``out [T, H vdim]``: every head's read-out, divided by its
        root mean square, times ``norm_w`` and the gate. Advances the state of the batch's requests.
        ``decay_per_head``: one decay for all key channels of a head; ``second`` is then ``[T, H +
        H vdim]`` and ``dt_bias [H]``. ``gate``: ``sigmoid`` or ``silu`` of the gate's logit. ``proj``
        and ``second`` may be column ranges of one wider row (unit stride along a row)."""
        b = ctx.batch
        self._on_device(proj, second, conv_w, a_log, dt_bias, norm_w, state, out)
        T = proj.shape[0]
        H, G = int(heads), int(kv_heads)
        C = 2 * G * dim + H * vdim
        n_state = H * dim * vdim
        n_decay = H if decay_per_head else H * dim
        _need(gate in ("sigmoid", "silu"), "delta_rule: the gate is sigmoid or silu")
        silu_gate = int(gate == "silu")
        _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] == C + H, "delta_rule: proj")
        _need(second.dtype == torch.float32 and second.stride(1) == 1 and second.shape[1] == n_decay + H * vdim,
              "delta_rule: second")
        _need(conv_w.is_contiguous() and tuple(conv_w.shape) == (C, taps) and a_log.numel() == H and dt_bias.numel() == n_decay
              and norm_w.numel() == vdim and conv_w.dtype == a_log.dtype == dt_bias.dtype == norm_w.dtype, "delta_rule: weights")
        _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == n_state + (taps - 1) * C,
              "delta_rule: state")
        _need(out.is_contiguous() and tuple(out.shape) == (T, H * vdim), "delta_rule: out")
        L = self.state_lib
        stride = state.shape[1]
        conv_state = state.data_ptr() + 4 * n_state
        wt = _tag(conv_w, "delta_rule weights")
        if b.max_q_len == 1 and vdim <= 256:
            # single tokens: one kernel for everything but the shift of the kept inputs
            self._check(L, L.gb_delta_decode(
                proj.data_ptr(), proj.stride(0), second.data_ptr(), second.stride(0), conv_w.data_ptr(), wt, taps, conv_state,
                stride, a_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr(), float(eps), b.slots.data_ptr(),
                state.data_ptr(), stride, T, H, G, dim, vdim, out.data_ptr(), _tag(out, "delta_rule out"),
                int(decay_per_head), n_decay, silu_gate, self._stream()), "delta_decode")
        else:
            W = C + H * dim + H
            prep = ctx.ws.get("delta_prep", (T, W), torch.float32)
            o = ctx.ws.get("delta_o", (T, H * vdim), torch.float32)
            self._check(L, L.gb_delta_prepare(
                proj.data_ptr(), proj.stride(0), second.data_ptr(), second.stride(0), conv_w.data_ptr(), wt, taps, conv_state,
                stride, a_log.data_ptr(), dt_bias.data_ptr(), b.token_req.data_ptr(), b.cu_q.data_ptr(), b.slots.data_ptr(),
                prep.data_ptr(), W, T, H, G, dim, vdim, int(decay_per_head), self._stream()), "delta_prepare")
            self._check(L, L.gb_delta_recurrence(
                prep.data_ptr(), W, b.cu_q.data_ptr(), b.slots.data_ptr(), state.data_ptr(), stride, b.num_requests, H, G,
                dim, vdim, o.data_ptr(), self._stream()), "delta_recurrence")
            self._check(L, L.gb_delta_out(
                o.data_ptr(), second.data_ptr(), second.stride(0), n_decay, norm_w.data_ptr(), wt, float(eps), out.data_ptr(),
                _tag(out, "delta_rule out"), T, H, vdim, silu_gate, 0, self._stream()), "delta_out")
        self._check(L, L.gb_delta_conv_state(proj.data_ptr(), proj.stride(0), conv_state, stride, b.cu_q.data_ptr(),
                                             b.slots.data_ptr(), b.num_requests, C, taps, self._stream()), "delta_conv_state")

    # ------------------------------------------------------------------ the generalized delta rule
    def general_delta(self, ctx, proj, cols, zdec, w0, a0, decay_scale, norm_w, eps, state, heads, dim, vdim, out):
        """The recurrent part of a generalized-delta-rule mixer for one step. ``proj [T, P]`` (32-bit):
        the projected row; ``cols`` = the first columns of ``(r, k, v, removal logits, gate logits)`` in
        it (``H dim`` wide each, ``v`` and the gate ``H vdim``). ``zdec [T, H dim]`` (32-bit): the decay's
        pre-activation. Per head, with ``u`` the unit key: ``w = exp(-decay_scale sigmoid(zdec + w0))``,
        ``a = sigmoid(logit + a0)``, ``S <- diag(w) S - (a u)(u^T S) + k v^T``, ``o = S^T r``.
        ``state [slots, H dim vdim]`` (32-bit). ``out [T, H vdim]``: every head's read-out divided by
        its root mean square, times ``norm_w [H vdim]`` and the sigmoid of the gate. Advances the state
        of the batch's requests."""
        b = ctx.batch
        self._on_device(proj, zdec, w0, a0, norm_w, state, out)
        T, H = proj.shape[0], int(heads)
        HD, HV = H * dim, H * vdim
        col_r, col_k, col_v, col_a, col_g = (int(c) for c in cols)
        _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and zdec.dtype == torch.float32 and zdec.stride(1) == 1
              and zdec.shape[1] >= HD, "general_delta: float32 rows")
        _need(max(col_r + HD, col_k + HD, col_v + HV, col_a + HD, col_g + HV) <= proj.shape[1], "general_delta: columns")
        _need(all(t.dtype == torch.float32 and t.is_contiguous() for t in (w0, a0, norm_w)) and w0.numel() == HD
              and a0.numel() == HD and norm_w.numel() == HV, "general_delta: float32 vectors")
        _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == HD * vdim, "general_delta: state")
        _need(out.is_contiguous() and tuple(out.shape) == (T, HV), "general_delta: out")
        L = self.state_lib
        stride = state.shape[1]
        if b.max_q_len == 1 and vdim <= 256:
            self._check(L, L.gb_gdelta_decode(
                proj.data_ptr(), proj.stride(0), col_r, col_k, col_v, col_a, col_g, zdec.data_ptr(), zdec.stride(0),
                w0.data_ptr(), a0.data_ptr(), float(decay_scale), norm_w.data_ptr(), float(eps), b.slots.data_ptr(),
                state.data_ptr(), stride, T, H, dim, vdim, out.data_ptr(), _tag(out, "general_delta out"), self._stream()),
                "gdelta_decode")
            return
        W = 5 * HD + HV
        prep = ctx.ws.get("gdelta_prep", (T, W), torch.float32)
        o = ctx.ws.get("gdelta_o", (T, HV), torch.float32)
        self._check(L, L.gb_gdelta_prepare(
            proj.data_ptr(), proj.stride(0), col_r, col_k, col_v, col_a, zdec.data_ptr(), zdec.stride(0), w0.data_ptr(),
            a0.data_ptr(), float(decay_scale), prep.data_ptr(), W, T, H, dim, vdim, self._stream()), "gdelta_prepare")
        self._check(L, L.gb_gdelta_recurrence(
            prep.data_ptr(), W, b.cu_q.data_ptr(), b.slots.data_ptr(), state.data_ptr(), stride, b.num_requests, H, dim,
            vdim, o.data_ptr(), self._stream()), "gdelta_recurrence")
        gate = proj[:, col_g:col_g + HV]
        self._check(L, L.gb_delta_out(
            o.data_ptr(), gate.data_ptr(), proj.stride(0), 0, norm_w.data_ptr(), GB_F32, float(eps), out.data_ptr(),
            _tag(out, "general_delta out"), T, H, vdim, 0, 1, self._stream()), "delta_out")

    # ------------------------------------------------------------------ normed queries and keys; sublayers normed behind
    def qk_norm_rope_append(self, src, cols, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            dim, vdim, q_weight, k_weight, eps, rotary, page_size):
        """From a projected 32-bit row ``src [T, P]`` with ``cols = (q, k, v)`` the first columns of
        queries (``heads dim``), keys (``kv_heads dim``) and values (``kv_heads vdim``; the keys' own
        columns where the values are the keys as projected): queries and keys are divided by their root
        mean square per head (``q_weight [heads, dim]``, ``k_weight [dim]``, 32-bit; None: no norm),
        then rotated (``rotary``: a ``RotaryParams`` over ``dim``, or None); queries go to ``q_out
        [T, heads, dim]``, keys and the untouched values into their pages."""
        self._on_device(src, q_out, k_pool, v_pool, positions, token_req, block_table, q_weight, k_weight)
        T = src.shape[0]
        cq, ck, cv = (int(c) for c in cols)
        _need(src.dtype == torch.float32 and src.stride(1) == 1, "qk_norm_rope_append: a float32 row")
        _need(max(cq + heads * dim, ck + kv_heads * dim, cv + kv_heads * vdim) <= src.shape[1], "qk_norm_rope_append: columns")
        _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, heads, dim), "qk_norm_rope_append: q_out shape")
        _need(k_pool.dtype == q_out.dtype == v_pool.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
              and tuple(k_pool.shape[1:]) == (kv_heads, page_size, dim)
              and tuple(v_pool.shape[1:]) == (kv_heads, page_size, vdim), "qk_norm_rope_append: pool shapes")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and positions.dtype == torch.int32
              and token_req.dtype == torch.int32, "qk_norm_rope_append: int32 indices")
        _need(q_weight is None or (q_weight.dtype == torch.float32 and q_weight.is_contiguous()
                                   and q_weight.numel() == heads * dim), "qk_norm_rope_append: q_weight float32 [heads, dim]")
        _need(k_weight is None or (k_weight.dtype == torch.float32 and k_weight.is_contiguous()
                                   and k_weight.numel() == dim), "qk_norm_rope_append: k_weight float32 [dim]")
        inv, inter = None, 0
        if rotary is not None:
            _need(rotary.head_dim == dim, "qk_norm_rope_append: rotary is for another head width")
            inv, inter = self.inv_freq(rotary), int(rotary.interleaved)
        L = self.state_lib
        self._check(L, L.gb_qk_norm_rope_append(
            src.data_ptr(), src.stride(0), cq, ck, cv, q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
            _tag(q_out, "q_out"), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1],
            T, heads, kv_heads, dim, vdim, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv), inter, page_size,
            self._stream()), "qk_norm_rope_append")

    UNARY_ACTS = {"sigmoid": 0, "silu": 1, "relu2": 2, "tanh": 3}

    def gate_mul(self, x, gate, kind: str = "sigmoid"):
        """``x <- x * act(gate)`` in place; ``gate [T, n]`` 32-bit logits (a column range of a wider
        row will do), ``act`` = ``sigmoid`` or ``silu``."""
        self._on_device(x, gate)
        T, n = x.shape
        _need(x.is_contiguous() and gate.dtype == torch.float32 and tuple(gate.shape) == (T, n) and gate.stride(1) == 1,
              "gate_mul: x contiguous, gate float32 of its shape")
        _need(kind in ("sigmoid", "silu"), "gate_mul: sigmoid or silu")
        L = self.state_lib
        self._check(L, L.gb_gate_mul(x.data_ptr(), _tag(x, "gate_mul x"), gate.data_ptr(), gate.stride(0), T, n,
                                     self.UNARY_ACTS[kind], self._stream()), "gate_mul")

    def activation(self, z, out, kind: str):
        """``out = act(z)`` elementwise, 32-bit arithmetic; ``act`` = ``relu2`` (the square of
        relu), ``tanh``, ``sigmoid`` or ``silu``. Both may be column ranges of wider rows."""
        self._on_device(z, out)
        T, n = z.shape
        _need(tuple(out.shape) == (T, n) and z.stride(1) == 1 and out.stride(1) == 1, "activation: shapes")
        _need(kind in self.UNARY_ACTS, f"activation: unknown kind {kind!r}")
        L = self.state_lib
        self._check(L, L.gb_unary_act(z.data_ptr(), _tag(z, "activation in"), z.stride(0), out.data_ptr(),
                                      _tag(out, "activation out"), out.stride(0), T, n, self.UNARY_ACTS[kind],
                                      self._stream()), "activation")

    def linear_act(self, ctx, a, w, out, kind: str):
        """``out[M,N] = act(a[M,K] @ w[N,K]^T)``, the activation (see ``activation``) in 32-bit on the
        32-bit sums and rounded once: in the product's epilogue where the tensor-core kernel takes
        the shape, else a product into a 32-bit row and the activation kernel."""
        self._on_device(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        _need(w.shape[1] == K and tuple(out.shape) == (M, N) and a.dtype == w.dtype, "linear_act: shapes and dtypes")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_act: operands must be contiguous")
        _need(kind in self.UNARY_ACTS, f"linear_act: unknown kind {kind!r}")
        if self.tc is not None and a.dtype == torch.bfloat16 and self.tc.linear_act(a, w, out, kind):
            return
        z = ctx.ws.get("linear_act_z", (M, N), torch.float32)
        self.linear(a, w, z)
        self.activation(z, out, kind)

    def sublayer_merge(self, ys, branch_weights, eps, x=None, out=None, gate=None, gate_bias=None, weight=None,
                       branch_eps=None, rounded=None):
        """What stands between a sublayer's output and the residual where the output, not the input, is
        normed. ``ys``: one 32-bit ``[T, d]`` output, or several branches' with ``branch_weights`` (32-bit
        ``[d]`` each): ``y = mean_b rms(y_b) * w_b``. ``gate`` (32-bit logits ``[T, d]``, a column range
        will do) and ``gate_bias [d]``: ``y <- y * sigmoid(gate + gate_bias)``. Then ``x += rms(y) *
        weight`` (``x`` the 32-bit residual), or with ``out`` in place of ``x``: ``out = y``. ``rounded``
        (bfloat16 ``[T, d]``): also the new ``x`` rounded, the input of the sublayer that reads it next.
        One pass."""
        ys = list(ys)
        self._on_device(*ys, x, out, gate, gate_bias, weight, rounded)
        T, d = ys[0].shape
        _need(all(y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (T, d) for y in ys),
              "sublayer_merge: float32 [T, d] outputs")
        ws = None
        if branch_weights is not None:
            ws = list(branch_weights)
            _need(len(ws) == len(ys) and all(w.dtype == torch.float32 and w.is_contiguous() and w.numel() == d for w in ws),
                  "sublayer_merge: one float32 [d] weight per branch")
        _need(gate is None or (gate.dtype == torch.float32 and tuple(gate.shape) == (T, d) and gate.stride(1) == 1),
              "sublayer_merge: gate float32 [T, d]")
        _need(gate_bias is None or (gate_bias.dtype == torch.float32 and gate_bias.numel() == d), "sublayer_merge: gate_bias")
        target = x if x is not None else out
        _need(target is not None and target.dtype == torch.float32 and target.is_contiguous() and tuple(target.shape) == (T, d),
              "sublayer_merge: x or out float32 [T, d]")
        _need(x is None or (weight is not None and weight.dtype == torch.float32 and weight.numel() == d),
              "sublayer_merge: the norm's float32 weight")
        _need(rounded is None or (x is not None and rounded.dtype == torch.bfloat16 and rounded.is_contiguous()
                                  and tuple(rounded.shape) == (T, d)), "sublayer_merge: rounded bfloat16 [T, d] beside x")
        n = len(ys)
        y_ptrs = (c_void_p * n)(*[y.data_ptr() for y in ys])
        w_ptrs = (c_void_p * n)(*[w.data_ptr() for w in ws]) if ws is not None else None
        L = self.state_lib
        self._check(L, L.gb_sublayer_merge(
            y_ptrs, w_ptrs, n, 1.0 / n, float(eps if branch_eps is None else branch_eps), _ptr(gate),
            gate.stride(0) if gate is not None else 0, _ptr(gate_bias), _ptr(weight), float(eps), _ptr(x),
            None if x is not None else out.data_ptr(), _ptr(rounded), T, d, self._stream()), "sublayer_merge")

    # ------------------------------------------------------------------ a norm after the sum; gates per head; xIELU
    def post_norm(self, x, y, alpha, weight, eps, row=None, rounded=None):
        """``x <- rms(alpha * x + y + row) * weight`` in place on the 32-bit residual ``x [T, d]``; ``y``
        (32-bit ``[T, d]``) and ``row`` (32-bit ``[d]``) may be None. ``rounded`` (bfloat16 ``[T, d]``):
        also the new ``x`` rounded, the input of the sublayer that reads it next. One pass."""
        self._on_device(x, y, weight, row, rounded)
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "post_norm: x must be float32 [T, d]")
        T, d = x.shape
        _need(y is None or (y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (T, d)),
              "post_norm: y must be float32 of x's shape")
        _need(row is None or (row.dtype == torch.float32 and row.is_contiguous() and row.numel() == d), "post_norm: row float32 [d]")
        _need(weight.numel() == d and weight.is_contiguous(), "post_norm: weight [d]")
        _need(rounded is None or (rounded.dtype == torch.bfloat16 and rounded.is_contiguous() and tuple(rounded.shape) == (T, d)),
              "post_norm: rounded bfloat16 [T, d]")
        L = self.seq_lib
        self._check(L, L.gb_post_norm(x.data_ptr(), _ptr(y), _ptr(row), float(alpha), weight.data_ptr(),
                                      _tag(weight, "norm weight"), float(eps), _ptr(rounded), T, d, self._stream()), "post_norm")

    def group_gate_mul(self, x, gate, group: int):
        """``x[t, c] <- x[t, c] * sigmoid(gate[t, c // group])`` in place: one gate per head of
        ``group`` channels; ``gate [T, n / group]`` 32-bit logits (a column range of a wider row will do)."""
        self._on_device(x, gate)
        T, n = x.shape
        _need(x.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1 and group >= 1 and n % group == 0
              and tuple(gate.shape) == (T, n // group), "group_gate_mul: x contiguous [T, n], gate float32 [T, n / group]")
        L = self.seq_lib
        self._check(L, L.gb_group_gate_mul(x.data_ptr(), _tag(x, "group_gate_mul x"), gate.data_ptr(), gate.stride(0), T, n,
                                           int(group), self._stream()), "group_gate_mul")

    def xielu(self, z, out, a_pos: float, a_neg: float):
        """``out = a_pos z^2 + z / 2`` where ``z > 0``, ``a_neg (exp(z) - 1 - z) + z / 2`` elsewhere;
        32-bit arithmetic. Both may be column ranges of wider rows."""
        self._on_device(z, out)
        T, n = z.shape
        _need(tuple(out.shape) == (T, n) and z.stride(1) == 1 and out.stride(1) == 1, "xielu: shapes")
        L = self.seq_lib
        self._check(L, L.gb_xielu(z.data_ptr(), _tag(z, "xielu in"), z.stride(0), out.data_ptr(), _tag(out, "xielu out"),
                                  out.stride(0), T, n, float(a_pos), float(a_neg), self._stream()), "xielu")

    def linear_xielu(self, ctx, a, w, out, a_pos: float, a_neg: float):
        """``out[M,N] = xielu(a[M,K] @ w[N,K]^T)``, the activation in 32-bit on the 32-bit sums and
        rounded once: in the product's epilogue where the tensor-core kernel takes the shape, else a
        product into a 32-bit row and the activation kernel."""
        self._on_device(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        _need(w.shape[1] == K and tuple(out.shape) == (M, N) and a.dtype == w.dtype, "linear_xielu: shapes and dtypes")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_xielu: operands must be contiguous")
        if self.tc is not None and a.dtype == torch.bfloat16 and self.tc.linear_xielu(a, w, out, a_pos, a_neg):
            return
        z = ctx.ws.get("linear_act_z", (M, N), torch.float32)
        self.linear(a, w, z)
        self.xielu(z, out, a_pos, a_neg)

    # ------------------------------------------------------------------ a gated recurrence per channel
    def mingru(self, ctx, proj, cols, bias_z, bias_u, state, out):
        """The recurrent part of a minGRU mixer for one step. ``proj [T, P]`` (32-bit): the projected
        row; ``cols = (z, u, g)`` the first columns of the gate's logits, the candidate's pre-activation
        and the output gate's logits in it (``W`` wide each, ``W = out.shape[1]``). ``bias_z``,
        ``bias_u``: 32-bit ``[W]`` or None. Per channel: ``z = sigmoid(.)``, candidate ``u + 1/2`` where
        ``u >= 0`` and ``sigmoid(u)`` below, ``S <- (1 - z) S + z candidate``, ``out = S * silu(g)``.
        ``state [slots, >= W]`` (32-bit): a request's ``S``; advanced for the batch's requests."""
        b = ctx.batch
        self._on_device(proj, bias_z, bias_u, state, out)
        T, W = out.shape
        cz, cu, cg = (int(c) for c in cols)
        _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[0] == T
              and max(cz, cu, cg) + W <= proj.shape[1], "mingru: a float32 row with three column ranges")
        _need(all(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == W) for v in (bias_z, bias_u)),
              "mingru: float32 biases [W]")
        _need(state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= W, "mingru: state float32 [slots, W]")
        _need(out.is_contiguous(), "mingru: out must be contiguous")
        L = self.seq_lib
        R = b.num_requests
        need = int(L.gb_mingru_scratch_floats(R, W, int(b.max_q_len)))
        scratch = ctx.ws.get("mingru_parts", (need,), torch.float32) if need else None
        self._check(L, L.gb_mingru(proj.data_ptr(), proj.stride(0), cz, cu, cg, _ptr(bias_z), _ptr(bias_u), b.cu_q.data_ptr(),
                                   b.slots.data_ptr(), state.data_ptr(), state.stride(0), out.data_ptr(), _tag(out, "mingru out"),
                                   R, W, int(b.max_q_len), _ptr(scratch), self._stream()), "mingru", 2 if need else 1)

    # ------------------------------------------------------------------ a short convolution in front of attention
    def conv_qkv_append(self, ctx, proj, bias, conv_w, taps, state, q_out, k_pool, v_pool, block_table, heads, kv_heads,
                        dim, vdim, q_weight, k_weight, eps, page_size, v_first_in=None, v_first_out=None, mix: float = 0.0):
        """From a step's projected 32-bit rows ``proj [T, C]`` (``heads dim`` query, ``kv_heads dim`` key,
        ``kv_heads vdim`` value columns; ``bias [C]`` 32-bit or None is added): a causal convolution
        over time per channel (``conv_w [C, taps]`` 32-bit, the last column weighs the current token;
        zeros before a request's first token), queries and keys divided by their root mean square per
        head (``q_weight``, ``k_weight``: 32-bit ``[dim]``; None: no norm), values mixed with another
        layer's (``v <- (1 - mix) v + mix v_first_in``, 32-bit ``[T, kv_heads vdim]``) or written out
        for that (``v_first_out``); queries to ``q_out [T, heads, dim]``, keys and values into their
        pages. ``state [slots, (taps - 1) C]`` (32-bit) holds every request's last ``taps - 1``
        projected rows and is moved on."""
        b = ctx.batch
        self._on_device(proj, bias, conv_w, state, q_out, k_pool, v_pool, block_table, q_weight, k_weight, v_first_in, v_first_out)
        T = proj.shape[0]
        C = heads * dim + kv_heads * (dim + vdim)
        _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] == C, "conv_qkv_append: proj float32 [T, C]")
        _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C), "conv_qkv_append: bias")
        _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and tuple(conv_w.shape) == (C, taps),
              "conv_qkv_append: conv_w float32 [C, taps]")
        _need(taps == 1 or (state is not None and state.dtype == torch.float32 and state.stride(1) == 1
                            and state.shape[1] >= (taps - 1) * C), "conv_qkv_append: state float32 [slots, (taps - 1) C]")
        _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, heads, dim), "conv_qkv_append: q_out shape")
        _need(k_pool.dtype == q_out.dtype == v_pool.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
              and tuple(k_pool.shape[1:]) == (kv_heads, page_size, dim)
              and tuple(v_pool.shape[1:]) == (kv_heads, page_size, vdim), "conv_qkv_append: pool shapes")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "conv_qkv_append: block table")
        for v in (q_weight, k_weight):
            _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == dim), "conv_qkv_append: norm weights")
        for v in (v_first_in, v_first_out):
            _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and tuple(v.shape) == (T, kv_heads * vdim)),
                  "conv_qkv_append: shared values float32 [T, kv_heads vdim]")
        L = self.seq_lib
        st_ptr, st_stride = (state.data_ptr(), state.stride(0)) if state is not None else (None, 0)
        self._check(L, L.gb_conv_qkv(
            proj.data_ptr(), proj.stride(0), _ptr(bias), conv_w.data_ptr(), GB_F32, int(taps), st_ptr, st_stride,
            q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _tag(q_out, "q_out"), b.positions.data_ptr(),
            b.token_req.data_ptr(), b.cu_q.data_ptr(), b.slots.data_ptr(), block_table.data_ptr(), block_table.shape[1], T,
            heads, kv_heads, dim, vdim, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(v_first_in), _ptr(v_first_out),
            float(mix), int(page_size), self._stream()), "conv_qkv")
        if taps > 1:
            self._check(L, L.gb_conv_state_shift(proj.data_ptr(), proj.stride(0), _ptr(bias), int(taps), C, st_ptr, st_stride,
                                                 b.cu_q.data_ptr(), b.slots.data_ptr(), b.num_requests, self._stream()),
                        "conv_state_shift")

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        self._on_device(logits, out)
        _need(logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == torch.int32,
              "argmax: float32 logits, int32 out")
        R, V = logits.shape
        self._check(self.core, self.core.gb_argmax(logits.data_ptr(), out.data_ptr(), R, V, self._stream()),
                    "argmax")

    #: ``small_top_k`` may be said of rows that are greedy or have a top_k of 1 to this
    SMALL_TOP_K = 64

    def sample(self, logits, temperature, top_k, top_p, u, out, scratch, small_top_k: bool = False):
        """One token per row. ``temperature`` 0 is greedy; ``u`` is the row's uniform
        draw. ``scratch``: float32 ``[R, V]`` work space. ``small_top_k``: the caller knows
        that every row is greedy or has a top_k of 1 to ``SMALL_TOP_K`` (eight CTAs then share a
        row; the tokens are the same either way)."""
        self._on_device(logits, temperature, top_k, top_p, u, out, scratch)
        R, V = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: float32 logits")
        _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and u.dtype == torch.float32
              and top_k.dtype == torch.int32 and out.dtype == torch.int32, "sample: parameter dtypes")
        _need(scratch.dtype == torch.float32 and scratch.numel() >= R * V, "sample: scratch too small")
        fn = self.core.gb_sample_small_k if small_top_k else self.core.gb_sample
        self._check(self.core, fn(
            logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), u.data_ptr(),
            out.data_ptr(), scratch.data_ptr(), R, V, self._stream()), "sample")
