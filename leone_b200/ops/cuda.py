"""The kernel table: Python calls into the engine's own CUDA libraries.

Every call checks shapes, dtypes and contiguity on the host, then launches on
the current torch stream through a C entry point of ``csrc`` (loaded with
ctypes; compiled on first use by :mod:`leone_b200.csrc.build`).  There is no
other implementation behind these calls: without a CUDA device or without the
compiled libraries, construction raises.  The reference has the same split
between checked wrappers and raw entry points
(crates/leone-cuda/src/cuda.rs, crates/leone-cuda/src/ffi.rs).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import numpy as np
import torch

from ..csrc.build import ensure_built

_STATUS_TEXT = {
    1: "a token id outside the vocabulary reached the embedding kernel",
    2: "a token's block has no valid page in its block table",
    3: "a position outside the position table",
    4: "a bounded wait inside a kernel ran out",
    5: "a token names a sequence outside the batch",
}
_REFUSALS = {
    -1: "a size this kernel does not take",
    -2: "a pointer or stride that is not aligned as the kernel needs",
    -3: "a dtype this kernel does not take",
}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {t}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: refused — {_REFUSALS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


class PreparedMatrix:
    """A weight matrix ``[out, in]`` with what the kernels precompute for it."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self.tma = None           # tensor map for the tensor-core kernel, made on first use

    @property
    def shape(self):
        return self.weight.shape

    @property
    def dtype(self):
        return self.weight.dtype


class CudaOps:
    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError(
                "leone_b200 runs on a CUDA device only (there is no CPU path); "
                f"asked for device '{device}', torch.cuda.is_available() = {torch.cuda.is_available()}")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; device reports sm_{major}{minor}")
        self.dtype = dtype
        self.core = ctypes.CDLL(ensure_built("core"))
        self.fast = None
        self._pinned_stream = None
        if dtype == torch.bfloat16:
            from .fast import FastKernels
            self.fast = FastKernels(self.device)
        self.launches = 0
        self._sample_scratch = None
        self.status = None
        # LEONE_NO_PDL=1 launches every kernel fully serialised after its predecessor
        self.set_pdl(os.environ.get("LEONE_NO_PDL", "0") != "1")

    def set_pdl(self, enabled: bool) -> None:
        """Programmatic dependent launch: a kernel may start (and fetch weights) while its
        predecessor in the stream still runs; it waits before touching the step's data."""
        self._pdl = bool(enabled)
        # The kernels of the 'mixers' module call the same two instructions, but are launched without
        # the attribute unless LEONE_MIXERS_PDL=1: with it a decode step of the hybrid design measured
        # slower (1.15 ms against 1.04), a prompt step about the same (7.3 ms against 7.5).
        self._mixers_pdl = os.environ.get("LEONE_MIXERS_PDL", "0") == "1"
        self.core.leone_core_set_pdl(1 if enabled else 0)
        if self.__dict__.get("_mixers") is not None:
            self._mixers.leone_mixers_set_pdl(1 if enabled and self._mixers_pdl else 0)
        if self.fast is not None:
            self.fast.lib.leone_bf16_set_pdl(1 if enabled else 0)

    def bind_status(self, status: torch.Tensor) -> None:
        """The engine's status word; kernels with bounded waits report into it."""
        self.status = status
        if self.fast is not None:
            self.fast.status = status

    # -- helpers ------------------------------------------------------------------------
    def _stream(self):
        if self._pinned_stream is not None:        # (a handle of 0, the default stream, is a valid pin)
            return self._pinned_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def pin_stream(self, on: bool) -> None:
        """Between ``pin_stream(True)`` and ``pin_stream(False)`` every launch goes to the stream
        that was current at the first call: a step looks its stream up once, not once per launch."""
        handle = c_void_p(torch.cuda.current_stream(self.device).cuda_stream) if on else None
        self._pinned_stream = handle
        if self.fast is not None:
            self.fast.pin_stream(handle)

    def describe_status(self, word: int) -> str:
        return _STATUS_TEXT.get(word, "unknown status")

    # -- weights ------------------------------------------------------------------------
    def scratch_bytes(self) -> int:
        """Device memory the ops allocate for themselves beyond the runtime's named buffers."""
        return self.fast.scratch_bytes() if self.fast is not None else 0

    def prepare_matrix(self, w: torch.Tensor) -> PreparedMatrix:
        _need(w.dim() == 2 and w.is_contiguous(), "a weight matrix must be contiguous [out, in]")
        return PreparedMatrix(w)

    def prepare_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> PreparedMatrix:
        _need(gate.shape == up.shape, "gate and up matrices differ in shape")
        if self.fast is not None:
            return self.fast.prepare_gate_up(gate, up)
        m = PreparedMatrix(torch.cat([gate, up], dim=0).contiguous())
        m.gate_up_layout = "stacked"
        return m

    # -- kernels ------------------------------------------------------------------------
    def embedding(self, table, ids, out, status, scale: float = 1.0):
        n, hidden = out.shape
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embedding output must be fp32")
        _need(ids.dtype == torch.int32 and ids.numel() == n, "embedding ids must be int32 [N]")
        _need(table.shape[1] == hidden and table.is_contiguous(), "embedding table shape")
        self.launches += 1
        _check(self.core.leone_embedding(_dt(table.dtype), _ptr(table), _ptr(ids), _ptr(out), n,
                                         hidden, table.shape[0], c_float(scale), _ptr(status), self._stream()),
               "embedding")

    def logit_post(self, logits, scale: float = 1.0, soft_cap: Optional[float] = None):
        """In place: ``logits * scale``, then ``cap * tanh(. / cap)`` if a soft cap is given."""
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be contiguous fp32")
        _need(soft_cap is None or soft_cap > 0, "a soft cap must be positive")
        self.launches += 1
        _check(self.core.leone_logit_post(_ptr(logits), ctypes.c_longlong(logits.numel()), c_float(scale),
                                          c_float(soft_cap or 0.0), self._stream()), "logit_post")

    def rms_norm(self, x, weight, out, eps, rows=None):
        n_out, hidden = out.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == hidden,
              "rms_norm input must be contiguous fp32 [*, hidden]")
        _need(weight.numel() == hidden and out.is_contiguous(), "rms_norm weight/output shape")
        if rows is not None:
            _need(rows.dtype == torch.int32 and rows.numel() == n_out, "rms_norm rows must be int32")
        else:
            _need(x.shape[0] >= n_out, "rms_norm input has fewer rows than the output")
        self.launches += 1
        _check(self.core.leone_rms_norm(_ptr(x), _ptr(rows), _ptr(weight), _dt(weight.dtype),
                                        _ptr(out), _dt(out.dtype), n_out, hidden, c_float(eps),
                                        self._stream()), "rms_norm")

    def _gemm_simt(self, x, w, out, epilogue, residual):
        m, k = x.shape
        n = w.shape[0]
        self.launches += 1
        _check(self.core.leone_gemm_simt(_dt(x.dtype), epilogue, _ptr(x), _ptr(w), _ptr(out),
                                         _ptr(residual), m, n, k, x.stride(0), w.stride(0),
                                         out.stride(0), self._stream()), "gemm_simt")

    def linear_fuses_norm(self, n_tokens: int, w: PreparedMatrix) -> bool:
        """True if a product of ``n_tokens`` tokens with ``w`` can take part in a fused RMSNorm:
        as the product before the norm (``linear(..., norm_out=d)`` also leaves
        ``d.xn = bf16(out * d.weight)`` and the sums of ``out^2`` in ``d.ss``) or as the one
        after it (``linear(d.xn, ..., norm_in=d)`` scales its rows by the norm's factor)."""
        wt = w.weight
        # (a gate/up pair takes part only in the interleaved layout of the fused gated epilogue)
        return (self.fast is not None and self.fast.fuses_norm(n_tokens, wt.shape[0], wt.shape[1])
                and getattr(w, "gate_up_layout", "interleaved16") == "interleaved16"
                and wt.dtype == torch.bfloat16
                and wt.shape[0] % 8 == 0 and wt.shape[1] % 8 == 0 and wt.stride(0) % 8 == 0
                and wt.data_ptr() % 16 == 0)

    def norm_parts(self, n_tokens: int, n: int) -> int:
        """Rows of the ``ss`` buffer a product of ``n_tokens`` tokens with ``n`` outputs fills for
        the norm after it."""
        return self.fast.norm_parts(n_tokens, n)

    def _norm_args(self, m, w, norm_in, norm_out):
        ni = no = None
        if norm_in is not None:
            d = norm_in
            _need(self.linear_fuses_norm(m, w) and d.ss.dtype == torch.float32 and d.ss.is_contiguous()
                  and d.ss.shape == (d.parts, m), "linear: norm_in layout")
            ni = (d.ss, d.parts, d.eps)
        if norm_out is not None:
            d = norm_out
            _need(self.linear_fuses_norm(m, w) and d.weight.dtype == torch.float32 and d.weight.is_contiguous()
                  and d.weight.numel() == w.out_features and d.xn.dtype == torch.bfloat16
                  and d.xn.shape == (m, w.out_features) and d.xn.stride(1) == 1
                  and d.ss.dtype == torch.float32 and d.ss.is_contiguous()
                  and d.ss.shape == (self.norm_parts(m, w.out_features), m), "linear: norm_out layout")
            no = (d.xn, d.weight, d.ss)
        return ni, no

    def linear(self, x, w: PreparedMatrix, out, residual=None, norm_in=None, norm_out=None):
        """``out = x @ w.T`` (+ ``residual``).  ``out`` in x's dtype, or fp32 (then a fp32
        ``residual`` may be added; it may be ``out`` itself).  ``norm_in`` / ``norm_out``: see
        :meth:`linear_fuses_norm`."""
        m, k = x.shape
        _need(k == w.in_features and out.shape == (m, w.out_features), "linear: shapes do not chain")
        _need(x.dtype == w.dtype and x.stride(1) == 1 and out.stride(1) == 1, "linear: dtype/stride")
        if residual is not None:
            _need(out.dtype == torch.float32 and residual.dtype == torch.float32
                  and residual.shape == out.shape and residual.stride() == out.stride(),
                  "linear: a residual needs fp32 output of the same layout")
            epilogue = 2
        elif out.dtype == torch.float32 and x.dtype != torch.float32:
            epilogue = 1
        else:
            _need(out.dtype == x.dtype, "linear: output dtype")
            epilogue = 0
        if m == 0:
            return
        if norm_in is not None or norm_out is not None:
            _need(norm_out is None or epilogue in (1, 2), "linear: norm_out needs fp32 output")
            ni, no = self._norm_args(m, w, norm_in, norm_out)
            _need(self.fast.linear(x, w, out, epilogue, residual, ni, no), "linear: fused norm off the tensor-core path")
            self.launches += 1
            return
        if self.fast is not None and self.fast.linear(x, w, out, epilogue, residual):
            self.launches += 1
            return
        self._gemm_simt(x, w.weight, out, epilogue, residual)

    def linear_swiglu(self, x, w_gate_up: PreparedMatrix, out, norm_in=None, gate_shape=None):
        """``out = silu(x @ gate.T) * (x @ up.T)`` for a matrix from ``prepare_gate_up``.
        ``gate_shape = (slope, limit, shift)``: ``g' sigmoid(slope g') (u' + shift)`` with
        ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)`` (``limit`` may be ``inf``)."""
        m = x.shape[0]
        inter = w_gate_up.out_features // 2
        _need(out.shape == (m, inter) and out.dtype == x.dtype and out.is_contiguous(),
              "linear_swiglu: output shape")
        _need(gate_shape is None or (len(gate_shape) == 3 and gate_shape[1] > 0), "linear_swiglu: gate shape")
        if m == 0:
            return
        if norm_in is not None:
            ni, _ = self._norm_args(m, w_gate_up, norm_in, None)
            _need(self.fast.linear_swiglu(x, w_gate_up, out, ni, gate_shape),
                  "linear_swiglu: fused norm off the tensor-core path")
            self.launches += 1
            return
        if self.fast is not None and self.fast.linear_swiglu(x, w_gate_up, out, None, gate_shape):
            self.launches += 1
            return
        _need(getattr(w_gate_up, "gate_up_layout", None) == "stacked", "gate/up layout")
        scratch = self._scratch("gate_up", m, 2 * inter, x.dtype)
        self._gemm_simt(x, w_gate_up.weight, scratch, 0, None)
        self.launches += 1
        if gate_shape is None:
            _check(self.core.leone_swiglu(_dt(x.dtype), _ptr(scratch), _ptr(out), m, inter,
                                          self._stream()), "swiglu")
        else:
            slope, limit, shift = gate_shape
            _check(self.core.leone_gated_act(_dt(x.dtype), _ptr(scratch), _ptr(out), m, inter, c_float(slope),
                                             c_float(limit), c_float(shift), self._stream()), "gated_act")

    def convert(self, src, out):
        """``out = src`` elementwise, ``src`` fp32, ``out`` fp32 or the run dtype (same shape)."""
        _need(src.dtype == torch.float32 and src.is_contiguous() and out.is_contiguous()
              and src.shape == out.shape, "convert: layout")
        self.launches += 1
        _check(self.core.leone_convert(_dt(out.dtype), _ptr(src), _ptr(out), ctypes.c_longlong(src.numel()),
                                       self._stream()), "convert")

    def swiglu(self, gate_up, out):
        m, two_i = gate_up.shape
        _need(out.shape == (m, two_i // 2) and gate_up.is_contiguous() and out.is_contiguous(),
              "swiglu shapes")
        self.launches += 1
        _check(self.core.leone_swiglu(_dt(gate_up.dtype), _ptr(gate_up), _ptr(out), m, two_i // 2,
                                      self._stream()), "swiglu")

    _scratch_bufs = None

    def _scratch(self, name, rows, cols, dtype):
        if self._scratch_bufs is None:
            self._scratch_bufs = {}
        key = (name, cols, dtype)
        buf = self._scratch_bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            if buf is not None:
                self._scratch_bufs[("retired", id(buf))] = buf     # a captured graph may still use it
            buf = torch.empty((max(rows, 64), cols), dtype=dtype, device=self.device)
            self._scratch_bufs[key] = buf
        return buf[:rows]

    def qk_norm_rope_write(self, ctx, qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, table,
                           rotary_dim, cache, pairing="half_split"):
        """``pairing``: which elements of a head form rotation pair ``i``: ``(i, i + rotary_dim/2)``
        ("half_split") or ``(2i, 2i + 1)`` ("adjacent")."""
        _need(pairing in ("half_split", "adjacent"), f"rotary pairing '{pairing}'")
        n = qkv.shape[0]
        _need(qkv.is_contiguous() and qkv.shape[1] == (n_q + 2 * n_kv) * d, "qkv layout")
        w_dtype = 0
        if q_norm_w is not None:
            _need(k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype
                  and q_norm_w.numel() == d and k_norm_w.numel() == d, "q/k norm weights")
            w_dtype = _dt(q_norm_w.dtype)
        max_pos = 0
        if table is not None:
            _need(table.dtype == torch.float32 and table.is_contiguous() and table.dim() == 3
                  and table.shape[1] * 2 == rotary_dim and table.shape[2] == 2, "rotary table layout")
            max_pos = table.shape[0]
        if cache is not None:
            kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
            _need(kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype
                  and kp.shape[1] == n_kv and kp.shape[3] == d and kp.shape[2] == cache.page_tokens,
                  "cache pool layout")
            _need(bt.dtype == torch.int32 and bt.is_contiguous(), "block table")
            pool_args = (_ptr(bt), bt.shape[1], bt.shape[0], _ptr(kp), _ptr(vp), kp.shape[0],
                         cache.page_tokens)
        else:
            pool_args = (c_void_p(0), 0, 0, c_void_p(0), c_void_p(0), 0, 0)
        self.launches += 1
        _check(self.core.leone_qk_norm_rope_write(
            _dt(qkv.dtype), _ptr(qkv), n, n_q, n_kv, d, _ptr(q_norm_w), _ptr(k_norm_w), w_dtype,
            c_float(eps), _ptr(table), rotary_dim, max_pos, _ptr(ctx.positions),
            _ptr(ctx.seq_of_token), pool_args[0], pool_args[1], pool_args[2], pool_args[3],
            pool_args[4], pool_args[5], pool_args[6], 1 if pairing == "adjacent" else 0, _ptr(ctx.status),
            self._stream()), "qk_norm_rope_write")

    def can_fuse_decode(self, ctx, qkv, n_q, n_kv, d) -> bool:
        """True if the attention kernel can do the q/k norm, rotation and cache write itself
        for this step (then ``qk_norm_rope_write`` is not called and ``attention`` gets
        ``fuse``: q_w, k_w (fp32 [d] or None), eps, rope ([positions, d/2, 2] fp32 or None),
        write_cache, and optionally pairing ("half_split" or "adjacent"))."""
        return self.fast is not None and self.fast.decode_fusable(ctx, qkv.dtype, n_q, n_kv, d, qkv.stride(0))

    def attention(self, ctx, qkv, out, n_q, n_kv, d, scale, window, cache, fuse=None):
        n = qkv.shape[0]
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        _need(out.shape == (n, n_q * d) and out.is_contiguous() and out.dtype == qkv.dtype,
              "attention output layout")
        _need(kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype
              and kp.shape[1] == n_kv and kp.shape[3] == d, "cache pool layout")
        if self.fast is not None and self.fast.attention(ctx, qkv, out, n_q, n_kv, d, scale,
                                                         window, cache, fuse):
            self.launches += 1
            return
        _need(fuse is None, "the any-size attention kernel needs q/k norm and cache write done before")
        self.launches += 1
        _check(self.core.leone_attention_generic(
            _dt(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp),
            _ptr(bt), bt.shape[1], _ptr(ctx.seq_of_token), _ptr(ctx.positions), n, n_q, n_kv, d,
            c_float(scale), int(window or 0), cache.page_tokens, kp.shape[0], bt.shape[0],
            _ptr(ctx.status), self._stream()), "attention_generic")

    _MASKS = {"causal": 0, "window": 1, "chunk": 2}
    _WEIGHTS = {"softmax": 0, "softmax_plus_one": 1, "sigmoid": 2}

    def attention_prepare(self, ctx, qkv, n_q, n_kv, dk, dv, norm, q_w, k_w, eps, freqs, pairing, cache):
        """Norm (``None``, ``"per_head"`` or ``"whole"``; fp32 weights) and rotation (fp32
        ``freqs`` per pair or None) of q and k in place, and the step's keys and values into
        their pages (``csrc/attention_masked.cu``).  Row layout ``[q heads x dk | k heads x dk |
        v heads x dv]``."""
        n = qkv.shape[0]
        _need(qkv.stride(1) == 1 and qkv.shape[1] == (n_q + n_kv) * dk + n_kv * dv, "attention_prepare: qkv layout")
        mode = {None: 0, "per_head": 1, "whole": 2}[norm]
        if mode:
            want = (dk, dk) if mode == 1 else (n_q * dk, n_kv * dk)
            _need(q_w is not None and k_w is not None and q_w.dtype == torch.float32 and k_w.dtype == torch.float32
                  and q_w.is_contiguous() and k_w.is_contiguous() and (q_w.numel(), k_w.numel()) == want,
                  "attention_prepare: norm weights")
        rot = 0
        if freqs is not None:
            _need(freqs.dtype == torch.float32 and freqs.is_contiguous() and 2 * freqs.numel() <= dk,
                  "attention_prepare: frequencies")
            rot = 2 * freqs.numel()
        _need(pairing in ("half_split", "adjacent"), f"rotary pairing '{pairing}'")
        if cache is not None:
            kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
            _need(vp is not None and kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype == vp.dtype
                  and kp.shape[1] == n_kv and kp.shape[2] == cache.page_tokens and kp.shape[3] == dk
                  and vp.shape[3] == dv and bt.dtype == torch.int32 and bt.is_contiguous(), "attention_prepare: cache layout")
            pool_args = (_ptr(bt), bt.shape[1], bt.shape[0], _ptr(kp), _ptr(vp), kp.shape[0], cache.page_tokens)
        else:
            pool_args = (c_void_p(0), 0, ctx.n_seqs, c_void_p(0), c_void_p(0), 0, 0)
        self.launches += 1
        _check(self.mixers.leone_attention_prepare(
            _dt(qkv.dtype), _ptr(qkv), qkv.stride(0), n, n_q, n_kv, dk, dv, mode, _ptr(q_w), _ptr(k_w), c_float(eps),
            _ptr(freqs), rot, 1 if pairing == "adjacent" else 0, _ptr(ctx.positions), _ptr(ctx.seq_of_token),
            *pool_args, _ptr(ctx.status), self._stream()), "attention_prepare")

    def attention_masked(self, ctx, qkv, out, n_q, n_kv, dk, dv, scale, mask, mask_size, weights, bias, cache):
        """Attention with a mask (``"causal"``, ``"window"``, ``"chunk"`` of ``mask_size``) and a
        weight rule (``"softmax"``, ``"softmax_plus_one"``, ``"sigmoid"`` with a fp32 ``bias`` per
        head) over key pages of ``dk`` and value pages of ``dv`` elements."""
        n = qkv.shape[0]
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        _need(out.shape == (n, n_q * dv) and out.is_contiguous() and out.dtype == qkv.dtype and qkv.stride(1) == 1,
              "attention_masked: output layout")
        _need(vp is not None and kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype == vp.dtype
              and kp.shape[1] == n_kv and kp.shape[3] == dk and vp.shape[3] == dv, "attention_masked: cache layout")
        _need(mask in self._MASKS and weights in self._WEIGHTS, f"attention_masked: mask '{mask}' / weights '{weights}'")
        if weights == "sigmoid":
            _need(bias is not None and bias.dtype == torch.float32 and bias.numel() == n_q and bias.is_contiguous(),
                  "attention_masked: bias")
        self.launches += 1
        if self.fast is not None and self.attention_masked_tiled(ctx, qkv, out, n_q, n_kv, dk, dv, scale, mask,
                                                                 mask_size, weights, bias, cache):
            return
        _check(self.mixers.leone_attention_masked(
            _dt(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp), _ptr(bt),
            bt.shape[1], _ptr(ctx.seq_of_token), _ptr(ctx.positions), n, n_q, n_kv, dk, dv, c_float(scale),
            self._MASKS[mask], int(mask_size), self._WEIGHTS[weights], _ptr(bias), cache.page_tokens, kp.shape[0],
            bt.shape[0], _ptr(ctx.status), self._stream()), "attention_masked")

    def attention_masked_tiled(self, ctx, qkv, out, n_q, n_kv, dk, dv, scale, mask, mask_size, weights, bias, cache) -> bool:
        """The tensor-core form of :meth:`attention_masked` (``csrc/attention_masked_mma.cu``) where
        there is one for these sizes: bfloat16, key and value widths multiples of 16 up to 128, up
        to 64 query heads per KV head (16 in a decode step, whose keys are also split over blocks
        until the SMs are busy)."""
        decode = bool(ctx.decode_only)
        # prompt portions with head sizes 64 and 128: the tcgen05 prompt kernel takes the rule as a parameter
        if (dk == dv and not decode and getattr(ctx, "q_start", None) is not None
                and os.environ.get("LEONE_NO_MASKED_TC", "0") != "1"
                and self.fast.attention_rules(ctx, qkv, out, n_q, n_kv, dk, scale, mask_size if mask == "window" else 0,
                                              mask_size if mask == "chunk" else 0, self._WEIGHTS[weights], bias, cache)):
            return True
        if (qkv.dtype != torch.bfloat16 or os.environ.get("LEONE_NO_MASKED_MMA", "0") == "1"
                or getattr(ctx, "q_start", None) is None
                or not self.mixers.leone_attention_masked_mma_supported(n_q, n_kv, dk, dv, 1 if decode else 0)
                or qkv.stride(0) % 8 or out.stride(0) % 2):
            return False
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        splits, partial = 1, None
        if decode:
            keys = min(int(mask_size), ctx.max_ctx_len) if mask != "causal" else ctx.max_ctx_len
            tiles = -(-keys // 32) + 1                # the decode form's tiles hold 32 keys, a block has four warps
            splits = max(1, min(64, tiles // 8, (3 * 148) // max(ctx.n_seqs * n_kv, 1)))
            if splits > 1:
                self.mixers.leone_attention_masked_mma_scratch.restype = ctypes.c_longlong
                need = int(self.mixers.leone_attention_masked_mma_scratch(ctx.n_seqs, n_kv, dv, splits))
                partial = self._scratch("masked_partial", -(-need // 64), 64, torch.float32)
                self.launches += 1
        _check(self.mixers.leone_attention_masked_mma(
            _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp), _ptr(bt), bt.shape[1],
            _ptr(ctx.q_start), _ptr(ctx.ctx_len), ctx.n_seqs, 1 if decode else int(ctx.max_q_len), n_q, n_kv, dk, dv,
            c_float(scale), self._MASKS[mask], int(mask_size), self._WEIGHTS[weights], _ptr(bias), cache.page_tokens,
            kp.shape[0], 1 if decode else 0, splits, _ptr(partial), _ptr(ctx.status), self._stream()),
            "attention_masked_mma")
        return True

    # -- mixers and feed-forwards of the 'mixers' module (compiled when a model first needs it) ----
    @property
    def mixers(self):
        lib = self.__dict__.get("_mixers")
        if lib is None:
            lib = self.__dict__["_mixers"] = ctypes.CDLL(ensure_built("mixers"))
            lib.leone_mixers_set_pdl(1 if self._pdl and self._mixers_pdl else 0)
        return lib

    def rms_norm_pair(self, x, w_a, w_b, out_a, out_b, eps):
        """Two RMS norms (weights ``w_a``, ``w_b``, one eps) of the same fp32 rows in one pass."""
        n, width = out_a.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape == (n, width), "rms_norm_pair input")
        _need(out_b.shape == out_a.shape and out_a.dtype == out_b.dtype and out_a.is_contiguous()
              and out_b.is_contiguous() and w_a.dtype == w_b.dtype and w_a.numel() == width == w_b.numel(),
              "rms_norm_pair outputs/weights")
        self.launches += 1
        _check(self.mixers.leone_rms_norm_pair(_ptr(x), _ptr(w_a), _ptr(w_b), _dt(w_a.dtype), _ptr(out_a), _ptr(out_b),
                                               _dt(out_a.dtype), n, width, c_float(eps), self._stream()), "rms_norm_pair")

    def relu_squared(self, t):
        """In place: ``max(t, 0)^2``."""
        _need(t.is_contiguous(), "relu_squared needs a contiguous tensor")
        self.launches += 1
        _check(self.mixers.leone_relu_squared(_dt(t.dtype), _ptr(t), ctypes.c_longlong(t.numel()), self._stream()),
               "relu_squared")

    def linear_per_head(self, a, a_head_stride, w, c, c_head_stride, heads, k, n):
        """``c[t, h*c_head_stride : +n] = a[t, h*a_head_stride : +k] @ w[h].T`` for every head;
        ``w``: ``[heads, n, k]`` contiguous."""
        m = a.shape[0]
        _need(c.shape[0] == m and a.dtype == c.dtype == w.dtype and a.stride(1) == 1 and c.stride(1) == 1
              and w.is_contiguous() and tuple(w.shape) == (heads, n, k), "linear_per_head layout")
        _need((heads - 1) * a_head_stride + k <= a.shape[1] and (heads - 1) * c_head_stride + n <= c.shape[1],
              "linear_per_head: heads run past a row")
        self.launches += 1
        _check(self.mixers.leone_gemm_batched(_dt(a.dtype), _ptr(a), _ptr(w), _ptr(c), m, n, k, a.stride(0), k,
                                              c.stride(0), ctypes.c_longlong(a_head_stride),
                                              ctypes.c_longlong(n * k), ctypes.c_longlong(c_head_stride), heads,
                                              self._stream()), "linear_per_head")

    def linear_attention(self, ctx, proj, out, state, decay, heads, dim, vdim, q_off, k_off, v_off, chunk=0):
        """The decaying-state recurrence over the step's tokens (``csrc/linear_attention.cu``).
        ``chunk`` > 0: prompt portions are cut into chunks of that many tokens that run side by side."""
        n = proj.shape[0]
        _need(proj.stride(1) == 1 and out.dtype == torch.float32 and out.is_contiguous()
              and out.shape == (n, heads * vdim), "linear_attention layout")
        _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim)
              and decay.dtype == torch.float32 and decay.numel() == heads, "linear_attention state/decay")
        n_chunks, chunk_state = 0, None
        if chunk > 0:
            n_chunks = int(sum(-(-int(q) // chunk) for q in ctx.q_lens))
            chunk_state = self._scratch("linattn_chunks", n_chunks, heads * dim * vdim, torch.float32)
        self.launches += 1 if chunk == 0 else 3
        _check(self.mixers.leone_linear_attention(
            _dt(proj.dtype), _ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(out), out.stride(0), _ptr(state),
            _ptr(ctx.q_start), _ptr(ctx.slot_ids), _ptr(decay), ctx.n_seqs, heads, dim, vdim, state.shape[0], chunk,
            n_chunks, _ptr(chunk_state), _ptr(ctx.status), self._stream()), "linear_attention")

    def gate_norm(self, o, weight, gate, out, eps):
        """``out = rms_norm(o) * weight * sigmoid(gate)``; ``o`` fp32, ``gate`` a column slice."""
        n, width = o.shape
        _need(o.dtype == torch.float32 and o.is_contiguous() and out.shape == o.shape and out.is_contiguous()
              and gate.shape == o.shape and gate.stride(1) == 1 and gate.dtype == out.dtype
              and weight.numel() == width, "gate_norm layout")
        self.launches += 1
        _check(self.mixers.leone_gate_norm(_dt(out.dtype), _ptr(o), n, width, _ptr(weight), _dt(weight.dtype), _ptr(gate),
                                           gate.stride(0), _ptr(out), c_float(eps), self._stream()), "gate_norm")

    def latent_prepare(self, ctx, proj, q_abs, heads, dim, rot_dim, rank, norm_w, eps, freqs, magnitude, pairing,
                       cache, q_off, dkv_off):
        """Cache rows [normed latent | rotated shared key part] of the step's tokens and the
        rotated query parts (``csrc/attention_latent.cu``).  ``freqs``: fp32 per pair, or None."""
        n = proj.shape[0]
        dk = rank + rot_dim
        _need(proj.stride(1) == 1 and q_abs.is_contiguous() and q_abs.shape == (n, heads * dk)
              and q_abs.dtype == proj.dtype and norm_w.numel() == rank, "latent_prepare layout")
        rot_dims = 0
        if freqs is not None:
            _need(freqs.dtype == torch.float32 and freqs.is_contiguous(), "latent_prepare frequencies")
            rot_dims = 2 * freqs.numel()
        if cache is not None:
            kp, bt = cache.k_pool, cache.block_table
            _need(cache.v_pool is None and kp.is_contiguous() and kp.dtype == proj.dtype and kp.shape[1] == 1
                  and kp.shape[2] == cache.page_tokens and kp.shape[3] == dk and bt.dtype == torch.int32
                  and bt.is_contiguous(), "latent cache layout")
            pool_args = (_ptr(bt), bt.shape[1], bt.shape[0], _ptr(kp), kp.shape[0], cache.page_tokens)
        else:
            pool_args = (c_void_p(0), 0, ctx.n_seqs, c_void_p(0), 0, 0)
        self.launches += 1
        _check(self.mixers.leone_latent_prepare(
            _dt(proj.dtype), _ptr(proj), proj.stride(0), q_off, dkv_off, _ptr(q_abs), n, heads, dim, rot_dim, rank,
            _ptr(norm_w), _dt(norm_w.dtype), c_float(eps), _ptr(freqs), rot_dims, c_float(magnitude),
            1 if pairing == "adjacent" else 0, _ptr(ctx.positions), _ptr(ctx.seq_of_token), pool_args[0],
            pool_args[1], pool_args[2], pool_args[3], pool_args[4], pool_args[5], _ptr(ctx.status), self._stream()),
            "latent_prepare")

    def attention_latent(self, ctx, q_abs, out, cache, heads, dk, dv, scale, window, sink=None, gate=None):
        """Softmax attention of ``q_abs [n, heads*dk]`` over cache rows of ``dk`` elements whose
        first ``dv`` are the value; ``sink``: per head or None; ``gate``: ``[n, >= heads]`` or None."""
        n = q_abs.shape[0]
        kp, bt = cache.k_pool, cache.block_table
        _need(q_abs.is_contiguous() and out.is_contiguous() and out.shape == (n, heads * dv) and out.dtype == q_abs.dtype
              and kp.dtype == q_abs.dtype and kp.is_contiguous() and kp.shape[3] == dk and kp.shape[1] == 1,
              "attention_latent layout")
        if gate is not None:
            _need(gate.dtype == q_abs.dtype and gate.stride(1) == 1 and gate.shape[0] == n and gate.shape[1] >= heads,
                  "attention_latent gate")
        if sink is not None:
            _need(sink.numel() == heads and sink.is_contiguous(), "attention_latent sink")
        self.launches += 1
        if (q_abs.dtype == torch.bfloat16 and os.environ.get("LEONE_NO_LATENT_MMA", "0") != "1"
                and self.mixers.leone_attention_latent_mma_supported(dk, dv)):
            # few tokens (decode): a token's keys are split over blocks until the SMs are busy
            groups = -(-heads // 16)
            keys = min(int(window), ctx.max_ctx_len) if window else ctx.max_ctx_len
            splits = max(1, min(16, -(-keys // 64), 148 // max(n * groups, 1)))
            partial = None
            if splits > 1:
                partial = self._scratch("latent_partial", n * groups * splits * 16, dv + 2, torch.float32)
                self.launches += 1
            _check(self.mixers.leone_attention_latent_mma(
                _ptr(q_abs), _ptr(out), _ptr(kp), _ptr(bt), bt.shape[1], _ptr(ctx.seq_of_token), _ptr(ctx.positions),
                n, heads, dk, dv, c_float(scale), int(window or 0), _ptr(sink), 0 if sink is None else _dt(sink.dtype),
                _ptr(gate), 0 if gate is None else gate.stride(0), cache.page_tokens, kp.shape[0], bt.shape[0],
                splits, _ptr(partial), 1 if os.environ.get("LEONE_NO_SHARED_KEY_TILES", "0") == "1" else 0,
                _ptr(ctx.status), self._stream()), "attention_latent_mma")
            return
        _check(self.mixers.leone_attention_latent(
            _dt(q_abs.dtype), _ptr(q_abs), _ptr(out), _ptr(kp), _ptr(bt), bt.shape[1], _ptr(ctx.seq_of_token),
            _ptr(ctx.positions), n, heads, dk, dv, c_float(scale), int(window or 0), _ptr(sink),
            0 if sink is None else _dt(sink.dtype), _ptr(gate), 0 if gate is None else gate.stride(0),
            cache.page_tokens, kp.shape[0], bt.shape[0], _ptr(ctx.status), self._stream()), "attention_latent")

    def experts_route(self, x, w_router, chosen, weight, top, softmax=False, renormalize=False, groups=1,
                      groups_kept=None, weight_scale=1.0, bias=None, experts=None, correction=None):
        """Router logits as an fp32 product (bfloat16 operands multiply exactly in fp32), then the
        scores and the ``top`` best experts of every token (``csrc/experts.cu``), optionally among
        the experts of the ``groups_kept`` best of ``groups`` groups only; the weights times
        ``weight_scale``.  ``softmax``: False (sigmoid scores), True (softmax over all experts) or
        ``"chosen"`` (the logits are ranked, the weights are the softmax over the chosen ones).
        ``bias``: fp32 ``[experts]`` added to the logits.  ``correction``: fp32 ``[experts]`` added to the scores
        for the choice (and the groups' worth) only; the weights are the scores without it.  ``experts``: the router matrix's first so
        many rows are experts; further rows are other per-token logits that ride in the same product.
        Returns the fp32 logits ``[n, rows]`` (valid until the next call)."""
        n, width = x.shape
        if not isinstance(w_router, PreparedMatrix):
            w_router = self.prepare_matrix(w_router)
        rows = w_router.out_features
        experts = rows if experts is None else int(experts)
        _need(chosen.dtype == torch.int32 and weight.dtype == torch.float32 and chosen.numel() == n * top
              and weight.numel() == n * top and 0 < experts <= rows, "experts_route layout")
        for b in (bias, correction):
            _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == experts),
                  "experts_route bias/correction")
        _need(correction is None or softmax != "chosen", "experts_route: a correction needs scores")
        logits = self._scratch("router_logits", n, rows, torch.float32)
        self.linear(x, w_router, logits)
        self.launches += 1
        mode = 2 if softmax == "chosen" else (1 if softmax else 0)
        _check(self.mixers.leone_experts_select(_ptr(logits), logits.stride(0), _ptr(bias), _ptr(correction), n, experts, top, mode,
                                                1 if renormalize else 0, int(groups), int(groups_kept or groups),
                                                c_float(weight_scale), _ptr(chosen), _ptr(weight), self._stream()),
               "experts_select")
        return logits

    # -- short convolutions with state, the minGRU recurrence, pooled-window attention --------------
    def short_conv(self, ctx, x, weight, state, out, add_input=False, update_state=False, activation=None):
        """``out_t = (x_t if add_input) + sum_j weight[:, j] x_(t - taps + 1 + j)`` on every channel,
        inputs before the step from ``state`` (fp32 ``[slots, taps - 1, channels]``), which is not
        changed (``csrc/short_conv.cu``) unless ``update_state``, which is for steps in which every
        sequence brings one token: the kernel then leaves the state as :meth:`short_conv_state`
        would.  ``weight``: fp32 ``[channels, taps]``.  ``activation``: ``None`` or ``"silu"`` on the result."""
        _need(activation in (None, "silu"), f"short_conv: activation '{activation}'")
        _need(not update_state or ctx.decode_only, "short_conv: update_state is for steps of one token a sequence")
        n, channels = out.shape
        taps = weight.shape[1]
        _need(x.shape == (n, channels) and x.stride(1) == 1 and out.stride(1) == 1 and weight.dtype == torch.float32
              and weight.is_contiguous() and weight.shape[0] == channels, "short_conv layout")
        _need(taps == 1 or (state.dtype == torch.float32 and state.is_contiguous()
                            and tuple(state.shape[1:]) == (taps - 1, channels)), "short_conv state")
        self.launches += 1
        _check(self.mixers.leone_short_conv(
            _dt(x.dtype), _dt(out.dtype), _ptr(x), x.stride(0), _ptr(weight), _ptr(state), _ptr(out), out.stride(0),
            _ptr(ctx.q_start), _ptr(ctx.seq_of_token), _ptr(ctx.slot_ids), n, channels, taps,
            (1 if add_input else 0) | (2 if activation == "silu" else 0), 1 if update_state else 0, ctx.n_seqs, state.shape[0] if state is not None else 0, _ptr(ctx.status),
            self._stream()), "short_conv")

    def short_conv_state(self, ctx, x, state):
        """The state after the step: the last ``taps - 1`` rows of ``x`` of every sequence (older
        state rows move up where the step brought fewer).  Runs after every reader of the state."""
        keep, channels = state.shape[1], state.shape[2]
        _need(x.shape[1] >= channels and x.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous(),
              "short_conv_state layout")
        if keep == 0:
            return
        self.launches += 1
        _check(self.mixers.leone_short_conv_state(
            _dt(x.dtype), _ptr(x), x.stride(0), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.slot_ids), ctx.n_seqs,
            channels, keep + 1, state.shape[0], _ptr(ctx.status), self._stream()), "short_conv_state")

    def min_gru(self, ctx, proj, z_bias, x_bias, state, out, out_scale=1.0, chunk=0):
        """``S_t = (1 - z) S_(t-1) + z c`` per channel with ``z = sigmoid(pz + bz)``, ``u = px + bx``,
        ``c = u + 1/2`` where ``u >= 0`` else ``sigmoid(u)``; ``out_t = out_scale * S_t * silu(pg)``.
        ``proj``: rows ``[pz | px | pg]``; ``state``: fp32 ``[slots, width]``.  ``chunk`` > 0: the
        step's tokens are cut into chunks of that many that run side by side."""
        n, width = out.shape
        _need(proj.shape == (n, 3 * width) and proj.stride(1) == 1 and out.stride(1) == 1
              and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width, "min_gru layout")
        for b in (z_bias, x_bias):
            _need(b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.numel() == width), "min_gru bias")
        n_chunks, chunk_args = 0, (c_void_p(0),) * 5
        if chunk > 0:
            cuts = ctx.__dict__.setdefault("_token_chunks", {})      # the cut is the same for every layer of the step
            if chunk not in cuts:
                first, last, seq_start = [], [], [0]
                for a, q in zip(np.cumsum(ctx.q_lens) - ctx.q_lens, ctx.q_lens):
                    for c0 in range(0, int(q), chunk):
                        first.append(int(a) + c0)
                        last.append(int(a) + min(c0 + chunk, int(q)))
                    seq_start.append(len(first))
                cuts[chunk] = (len(first), torch.tensor(first + last + seq_start, dtype=torch.int32).to(self.device))
            n_chunks, meta = cuts[chunk]
            sums = self._scratch("min_gru_chunks", 2 * n_chunks, width, torch.float32)
            chunk_args = (_ptr(meta), _ptr(meta[n_chunks:]), _ptr(meta[2 * n_chunks:]), _ptr(sums), _ptr(sums[n_chunks:]))
        self.launches += 1 if n_chunks == 0 else 3
        _check(self.mixers.leone_min_gru(
            _dt(proj.dtype), _dt(out.dtype), _ptr(proj), proj.stride(0), 0, width, 2 * width, _ptr(z_bias), _ptr(x_bias),
            _ptr(state), _ptr(out), out.stride(0), _ptr(ctx.q_start), _ptr(ctx.slot_ids), ctx.n_seqs, width,
            state.shape[0], c_float(out_scale), n_chunks, *chunk_args, _ptr(ctx.status), self._stream()), "min_gru")

    def scale_rows(self, a, gate, scale=1.0):
        """In place: ``a[t, :] *= scale * sigmoid(gate[t])``; ``gate``: one fp32 logit per row (a
        column of a wider matrix is fine) or ``None``."""
        n, cols = a.shape
        _need(a.stride(1) == 1 and (gate is None or (gate.dtype == torch.float32 and gate.shape[0] == n)), "scale_rows layout")
        self.launches += 1
        _check(self.mixers.leone_scale_rows(_dt(a.dtype), _ptr(a), a.stride(0), n, cols, _ptr(gate),
                                            0 if gate is None else gate.stride(0), c_float(scale), self._stream()),
               "scale_rows")

    def add_scaled(self, x, y, scale=1.0):
        """In place: ``x += scale * y`` (both fp32, same shape)."""
        _need(x.dtype == torch.float32 and y.dtype == torch.float32 and x.shape == y.shape and x.is_contiguous()
              and y.is_contiguous(), "add_scaled layout")
        self.launches += 1
        _check(self.mixers.leone_add_scaled(_ptr(x), _ptr(y), ctypes.c_longlong(x.numel()), c_float(scale),
                                            self._stream()), "add_scaled")

    def attention_pooled_prepare(self, ctx, proj, q_out, n_q, n_kv, dk, dv, conv_w, conv_state, freqs, pairing,
                                 magnitude, unit_norm, eps, cache, update_state=False):
        """Per token, in fp32: the short convolution of the projected row ``[q | k | v]`` (weights
        fp32 ``[cols, taps]`` or None; earlier inputs from ``conv_state``), the rotation of q and k,
        the unit RMS norm of every q and k head, q into ``q_out``, k and v into their pages
        (``csrc/attention_pooled.cu``)."""
        n = proj.shape[0]
        cols = (n_q + n_kv) * dk + n_kv * dv
        _need(proj.stride(1) == 1 and proj.shape[1] == cols and q_out.shape == (n, n_q * dk) and q_out.stride(1) == 1,
              "attention_pooled_prepare layout")
        taps = 0
        if conv_w is not None:
            taps = conv_w.shape[1]
            _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == cols
                  and (taps == 1 or (conv_state is not None and conv_state.dtype == torch.float32
                                     and conv_state.is_contiguous() and tuple(conv_state.shape[1:]) == (taps - 1, cols))),
                  "attention_pooled_prepare convolution")
        rot = 0
        if freqs is not None:
            _need(freqs.dtype == torch.float32 and freqs.is_contiguous() and 2 * freqs.numel() <= dk,
                  "attention_pooled_prepare frequencies")
            rot = 2 * freqs.numel()
        _need(pairing in ("half_split", "adjacent"), f"rotary pairing '{pairing}'")
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        _need(vp is not None and kp.is_contiguous() and vp.is_contiguous() and kp.dtype == q_out.dtype == vp.dtype
              and kp.shape[1] == n_kv and kp.shape[2] == cache.page_tokens and kp.shape[3] == dk and vp.shape[3] == dv
              and bt.dtype == torch.int32 and bt.is_contiguous(), "attention_pooled_prepare cache layout")
        self.launches += 1
        _check(self.mixers.leone_attention_pooled_prepare(
            _dt(proj.dtype), _dt(q_out.dtype), _ptr(proj), proj.stride(0), n, n_q, n_kv, dk, dv, _ptr(conv_w), taps,
            _ptr(conv_state), 1 if (update_state and ctx.decode_only) else 0, _ptr(freqs), rot, 1 if pairing == "adjacent" else 0, c_float(magnitude),
            1 if unit_norm else 0, c_float(eps), _ptr(q_out), q_out.stride(0), _ptr(ctx.positions),
            _ptr(ctx.seq_of_token), _ptr(ctx.q_start), _ptr(ctx.slot_ids),
            conv_state.shape[0] if conv_state is not None else 0, _ptr(bt), bt.shape[1], bt.shape[0],
            _ptr(kp) if cache.writes else c_void_p(0), _ptr(vp) if cache.writes else c_void_p(0), kp.shape[0],
            cache.page_tokens, _ptr(ctx.status), self._stream()), "attention_pooled_prepare")

    @staticmethod
    def _pooled_args(tokens, blocks, n_kv, dk, dv, pool):
        kp, vp, bt = tokens.k_pool, tokens.v_pool, tokens.block_table
        kb, vb, pt = blocks.k_pool, blocks.v_pool, blocks.block_table
        rows = kb.shape[2]
        _need(kp.is_contiguous() and vp.is_contiguous() and kb.is_contiguous() and vb.is_contiguous()
              and kp.dtype == vp.dtype == kb.dtype == vb.dtype and kp.shape[1] == n_kv == kb.shape[1]
              and kp.shape[3] == dk == kb.shape[3] and vp.shape[3] == dv == vb.shape[3]
              and blocks.page_tokens == tokens.page_tokens and blocks.tokens_per_row == pool
              and rows == -(-tokens.page_tokens // pool) and bt.dtype == torch.int32 and pt.dtype == torch.int32
              and bt.is_contiguous() and pt.is_contiguous() and bt.shape[0] == pt.shape[0], "pooled attention cache layout")
        return (_ptr(kp), _ptr(vp), _ptr(bt), bt.shape[1], kp.shape[0], tokens.page_tokens,
                _ptr(kb), _ptr(vb), _ptr(pt), pt.shape[1], kb.shape[0], rows)

    def attention_pool_blocks(self, ctx, tokens, blocks, n_kv, dk, dv, pool):
        """Every block of ``pool`` positions that one of the step's tokens ends gets its mean key
        and mean value (over the rows as the token cache holds them) in the cache of blocks."""
        args = self._pooled_args(tokens, blocks, n_kv, dk, dv, pool)
        self.launches += 1
        _check(self.mixers.leone_attention_pool_blocks(
            _dt(tokens.k_pool.dtype), *args, _ptr(ctx.positions), _ptr(ctx.seq_of_token), ctx.n_tokens, ctx.n_seqs,
            n_kv, dk, dv, pool, _ptr(ctx.status), self._stream()), "attention_pool_blocks")

    def attention_pooled(self, ctx, q, out, tokens, blocks, n_q, n_kv, dk, dv, scale, window, pool, out_scale=1.0):
        """Softmax attention of every token over the last ``window`` cached keys and the mean keys
        of all blocks of ``pool`` positions that lie wholly before that window; ``out`` times
        ``out_scale``."""
        n = q.shape[0]
        _need(q.shape[1] == n_q * dk and q.stride(1) == 1 and out.shape == (n, n_q * dv) and out.stride(1) == 1
              and out.dtype == q.dtype == tokens.k_pool.dtype, "attention_pooled layout")
        args = self._pooled_args(tokens, blocks, n_kv, dk, dv, pool)
        self.launches += 1
        if self.fast is not None and self.attention_pooled_tiled(ctx, q, out, args, n_q, n_kv, dk, dv, scale, window,
                                                                 pool, out_scale):
            return
        _check(self.mixers.leone_attention_pooled(
            _dt(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), *args, _ptr(ctx.seq_of_token),
            _ptr(ctx.positions), n, n_q, n_kv, dk, dv, c_float(scale), int(window), int(pool), c_float(out_scale),
            ctx.n_seqs, _ptr(ctx.status), self._stream()), "attention_pooled")

    def attention_pooled_tiled(self, ctx, q, out, args, n_q, n_kv, dk, dv, scale, window, pool, out_scale) -> bool:
        """The tensor-core form of :meth:`attention_pooled`: the masked attention of
        ``csrc/attention_masked_mma.cu`` with its mask of a window and pooled blocks before it, for
        the sizes that kernel takes (bfloat16, key and value widths multiples of 16 up to 128).  A
        decode step's members (block rows, then token rows) are split over blocks until the SMs are busy."""
        decode = bool(ctx.decode_only)
        if q.dtype != torch.bfloat16 or getattr(ctx, "q_start", None) is None:
            return False
        # prompt portions with head sizes 64 and 128 and values as wide as keys: the tcgen05 prompt kernel
        if (not decode and dk == dv and os.environ.get("LEONE_NO_POOLED_TC", "0") != "1"
                and self.fast.attention_pooled_window(ctx, q, out, args, n_q, n_kv, dk, scale, window, pool, out_scale)):
            return True
        if (os.environ.get("LEONE_NO_POOLED_MMA", "0") == "1"
                or not self.mixers.leone_attention_masked_mma_supported(n_q, n_kv, dk, dv, 1 if decode else 0)
                or q.stride(0) % 8 or out.stride(0) % 2):
            return False
        splits, partial = 1, None
        if decode:
            longest = int(ctx.max_ctx_len)
            tiles = -(-min(int(window), longest) // 32) + 1 + -(-(max(longest - int(window), 0) // int(pool)) // 32)
            splits = max(1, min(64, tiles // 8, (3 * 148) // max(ctx.n_seqs * n_kv, 1)))
            if splits > 1:
                self.mixers.leone_attention_masked_mma_scratch.restype = ctypes.c_longlong
                need = int(self.mixers.leone_attention_masked_mma_scratch(ctx.n_seqs, n_kv, dv, splits))
                partial = self._scratch("masked_partial", -(-need // 64), 64, torch.float32)
                self.launches += 1
        _check(self.mixers.leone_attention_pooled_mma(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), *args, _ptr(ctx.q_start), _ptr(ctx.ctx_len), ctx.n_seqs,
            1 if decode else int(ctx.max_q_len), n_q, n_kv, dk, dv, c_float(scale), int(window), int(pool),
            c_float(out_scale), 1 if decode else 0, splits, _ptr(partial), _ptr(ctx.status), self._stream()),
            "attention_pooled_mma")
        return True

    # -- the norm of a sublayer's output, elementwise gates, mixed-head attention, the gated delta rule ----
    def zero(self, t):
        """``t = 0`` (a contiguous tensor)."""
        _need(t.is_contiguous(), "zero needs a contiguous tensor")
        self.launches += 1
        _check(self.mixers.leone_zero(_ptr(t), ctypes.c_longlong(t.numel() * t.element_size()), self._stream()), "zero")

    def rms_norm_add(self, dst, a, w_a, eps, b=None, w_b=None, coef=1.0, accumulate=True, rounded=None, then=None):
        """``dst (+)= coef * (rms_norm(a) * w_a [+ rms_norm(b) * w_b])``: fp32 rows, each source normed over
        its own row; ``rounded``: also the new ``dst`` in another dtype (the stream for its next reader).
        ``then``: a weight; the combination is itself RMS-normed with it (same eps) before it is added."""
        n, width = dst.shape
        _need(dst.dtype == torch.float32 and dst.is_contiguous() and a.dtype == torch.float32 and a.is_contiguous()
              and a.shape == dst.shape and w_a.numel() == width and w_a.is_contiguous(), "rms_norm_add layout")
        if b is not None:
            _need(b.dtype == torch.float32 and b.is_contiguous() and b.shape == dst.shape and w_b is not None
                  and w_b.numel() == width and w_b.dtype == w_a.dtype and w_b.is_contiguous(), "rms_norm_add second source")
        if rounded is not None:
            _need(rounded.shape == dst.shape and rounded.is_contiguous(), "rms_norm_add rounded copy")
        if then is not None:
            _need(then.numel() == width and then.dtype == w_a.dtype and then.is_contiguous() and width <= 12000,
                  "rms_norm_add: the norm after the combination")
        self.launches += 1
        _check(self.mixers.leone_rms_norm_add(
            _ptr(dst), _ptr(a), _ptr(w_a), _ptr(b), _ptr(w_b if b is not None else None), _dt(w_a.dtype), n, width,
            c_float(coef), c_float(eps), 1 if accumulate else 0, _ptr(rounded),
            0 if rounded is None else _dt(rounded.dtype), _ptr(then), self._stream()), "rms_norm_add")

    def gate_rows(self, a, gate, act="sigmoid"):
        """In place: ``a[t, c] *= act(gate[t, c])`` (``"sigmoid"`` or ``"silu"``); both in one dtype."""
        n, cols = a.shape
        _need(gate.shape == a.shape and gate.dtype == a.dtype and a.stride(1) == 1 and gate.stride(1) == 1
              and act in ("sigmoid", "silu"), "gate_rows layout")
        self.launches += 1
        _check(self.mixers.leone_gate_rows(_dt(a.dtype), _ptr(a), a.stride(0), _ptr(gate), gate.stride(0), n, cols,
                                           1 if act == "silu" else 0, self._stream()), "gate_rows")

    def gelu_gate(self, z, rows, offset, out):
        """``out[t, c] = gelu_tanh(z[t, c]) * rows[t, offset + c]``; ``z`` and ``rows`` fp32."""
        n, cols = out.shape
        _need(z.dtype == torch.float32 and rows.dtype == torch.float32 and z.shape == (n, cols) and z.stride(1) == 1
              and rows.stride(1) == 1 and rows.shape[0] == n and 0 <= offset and offset + cols <= rows.shape[1]
              and out.stride(1) == 1, "gelu_gate layout")
        self.launches += 1
        _check(self.mixers.leone_gelu_gate(_dt(out.dtype), _ptr(z), z.stride(0), _ptr(rows), rows.stride(0), int(offset),
                                           _ptr(out), out.stride(0), n, cols, self._stream()), "gelu_gate")

    def attention_mixed_heads(self, ctx, q, out, cache, n_q, n_kv, dk, dv, scale, temp, cap, mix, sink, mask, mask_size):
        """Softmax attention whose scores are mixed across heads before the softmax
        (``csrc/attention_mixed_heads.cu``): ``raw_g = q_g . k * scale * temp_g``, soft-capped at ``cap``,
        ``s_h = sum_g mix[h, g] raw_g``, a sink per head in the denominator.  ``temp``, ``mix``, ``sink``: fp32
        or None; ``cap``: a float or None.  ``q``: ``[n, >= n_q * dk]`` (the heads' queries first in a row)."""
        n = q.shape[0]
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        _need(out.shape == (n, n_q * dv) and out.is_contiguous() and out.dtype == q.dtype and q.stride(1) == 1
              and q.shape[1] >= n_q * dk, "attention_mixed_heads: output layout")
        _need(vp is not None and kp.is_contiguous() and vp.is_contiguous() and kp.dtype == q.dtype == vp.dtype
              and kp.shape[1] == n_kv and kp.shape[3] == dk and vp.shape[3] == dv, "attention_mixed_heads: cache layout")
        _need(mask in self._MASKS, f"attention_mixed_heads: mask '{mask}'")
        for v, count in ((temp, n_q), (mix, n_q * n_q), (sink, n_q)):
            _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == count),
                  "attention_mixed_heads: per-head constants")
        size = int(mask_size or 0)
        if self.attention_mixed_heads_tiled(ctx, q, out, cache, n_q, n_kv, dk, dv, scale, temp, cap, mix, sink, mask, size):
            return
        # steps of few tokens: a token's key tiles are dealt to several blocks
        keys = min(size, ctx.max_ctx_len) if mask != "causal" and size else ctx.max_ctx_len
        splits = max(1, min(32, -(-keys // 32), 296 // max(n, 1)))
        partial = None
        if splits > 1:
            partial = self._scratch("mixed_heads_partial", n * splits, n_q * (dv + 2), torch.float32)
            self.launches += 1
        self.launches += 1
        _check(self.mixers.leone_attention_mixed_heads(
            _dt(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(partial), _ptr(kp), _ptr(vp), _ptr(bt),
            bt.shape[1], _ptr(ctx.seq_of_token), _ptr(ctx.positions), n, n_q, n_kv, dk, dv, c_float(scale), _ptr(temp),
            c_float(cap or 0.0), _ptr(mix), _ptr(sink), self._MASKS[mask], size, cache.page_tokens, kp.shape[0],
            bt.shape[0], splits, _ptr(ctx.status), self._stream()), "attention_mixed_heads")

    def attention_mixed_heads_tiled(self, ctx, q, out, cache, n_q, n_kv, dk, dv, scale, temp, cap, mix, sink, mask, size) -> bool:
        """The tensor-core form of :meth:`attention_mixed_heads` (``csrc/attention_mixed_heads_mma.cu``) for
        prompt portions in bfloat16 where the sizes allow; False if it does not apply.  The step's rows are
        cut into tiles of 16 consecutive rows of one sequence (the cut is the same for every layer)."""
        if (q.dtype != torch.bfloat16 or ctx.decode_only or ctx.max_q_len < 8 or q.stride(0) % 8 or q.data_ptr() % 16
                or os.environ.get("LEONE_NO_MIXED_MMA", "0") == "1"):
            return False
        groups, smem = c_int(0), c_int(0)
        if not self.mixers.leone_attention_mixed_heads_mma_plan(n_q, n_kv, dk, dv, ctypes.byref(groups), ctypes.byref(smem)):
            return False
        tiles = ctx.__dict__.get("_row_tiles")
        if tiles is None:
            rows, at = [], 0
            for s, n in enumerate(ctx.q_lens):
                for r0 in range(0, int(n), 16):
                    rows += [s, at + r0, min(16, int(n) - r0)]
                at += int(n)
            tiles = ctx.__dict__["_row_tiles"] = (len(rows) // 3, torch.tensor(rows, dtype=torch.int32).to(self.device))
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        self.launches += 1
        _check(self.mixers.leone_attention_mixed_heads_mma(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp), _ptr(bt), bt.shape[1], _ptr(ctx.positions),
            _ptr(tiles[1]), tiles[0], n_q, n_kv, dk, dv, c_float(scale), _ptr(temp), c_float(cap or 0.0), _ptr(mix),
            _ptr(sink), self._MASKS[mask], size, cache.page_tokens, kp.shape[0], bt.shape[0], _ptr(ctx.status),
            self._stream()), "attention_mixed_heads_mma")
        return True

    def gated_delta(self, ctx, act, raw, out, state, a_log, dt_bias, heads, kv_heads, dim, vdim, q_off, k_off, v_off,
                    a_off, b_off, q_scale):
        """The gated delta rule over the step's tokens (``csrc/gated_delta.cu``).  ``act``: fp32 rows with the
        activations of q, k (``kv_heads x dim``) and v (``heads x vdim``) at their offsets; ``raw``: fp32 rows with
        one decay logit and one beta logit per head at ``a_off`` / ``b_off``; ``state``: fp32 ``[slots, heads,
        dim, vdim]``; ``out``: fp32 ``[n, heads * vdim]``."""
        n = act.shape[0]
        _need(act.dtype == torch.float32 and raw.dtype == torch.float32 and act.stride(1) == 1 and raw.stride(1) == 1
              and raw.shape[0] == n and out.dtype == torch.float32 and out.is_contiguous()
              and out.shape == (n, heads * vdim), "gated_delta layout")
        _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim)
              and a_log.dtype == torch.float32 and a_log.numel() == heads and dt_bias.dtype == torch.float32
              and dt_bias.numel() == heads, "gated_delta state/constants")
        self.launches += 1
        _check(self.mixers.leone_gated_delta(
            _ptr(act), act.stride(0), q_off, k_off, v_off, _ptr(raw), raw.stride(0), a_off, b_off, _ptr(a_log),
            _ptr(dt_bias), c_float(q_scale), _ptr(out), out.stride(0), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.slot_ids),
            ctx.n_seqs, heads, kv_heads, dim, vdim, state.shape[0], _ptr(ctx.status), self._stream()), "gated_delta")

    def group_gate_norm(self, o, weight, gate, out, eps, heads, vdim, act="sigmoid"):
        """``out[t, h, :] = rms_norm(o[t, h, :]) * weight * act(gate[t, h, :])``: every head normed on its own,
        one weight ``[vdim]`` for all; ``o`` and ``gate`` fp32 (``gate`` may be None)."""
        n = o.shape[0]
        _need(o.dtype == torch.float32 and o.stride(1) == 1 and o.shape[1] == heads * vdim and out.shape == o.shape
              and out.stride(1) == 1 and weight.numel() == vdim and weight.is_contiguous()
              and act in ("sigmoid", "silu"), "group_gate_norm layout")
        _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == o.shape),
              "group_gate_norm gate")
        self.launches += 1
        _check(self.mixers.leone_group_gate_norm(
            _dt(out.dtype), _ptr(o), o.stride(0), n, heads, vdim, _ptr(weight), _dt(weight.dtype), _ptr(gate),
            0 if gate is None else gate.stride(0), 1 if act == "silu" else 0, _ptr(out), out.stride(0), c_float(eps),
            self._stream()), "group_gate_norm")

    def experts_forward(self, x, w_gate, w_up, w_down, chosen, weight, top, scale_input, hidden, rt, identity=0,
                        fresh=False):
        """``hidden += sum over each token's chosen experts``; scratch comes from ``rt``.
        ``w_gate`` None: ungated experts, ``W_down max(W_up a, 0)^2``.  ``identity``: choices past the last
        expert (that many) are experts without tensors whose output is their input.  ``fresh``: ``hidden`` is
        written, not added to."""
        n, width = x.shape
        experts, ff = w_up.shape[0], w_up.shape[1]
        _need(x.stride(1) == 1 and (w_gate is None or (w_gate.is_contiguous() and w_gate.shape == w_up.shape))
              and w_up.is_contiguous() and w_down.is_contiguous()
              and tuple(w_up.shape) == (experts, ff, width) and tuple(w_down.shape) == (experts, width, ff)
              and w_up.dtype == x.dtype and hidden.dtype == torch.float32 and hidden.is_contiguous()
              and hidden.shape == (n, width), "experts_forward layout")
        _need(w_gate is not None or not scale_input, "experts_forward: ungated experts are weighted at their output")
        pairs = n * top
        cap = rt.max_tokens * top
        offsets = rt.flat_buffer("experts_offsets", experts + 1, torch.int32)
        order = rt.flat_buffer("experts_order", pairs, torch.int32, reserve=cap)
        act = rt.flat_buffer("experts_act", pairs * ff, x.dtype, reserve=cap * ff)
        pair_out = rt.flat_buffer("experts_pair_out", pairs * width, torch.float32, reserve=cap * width)
        self.launches += 4
        _check(self.mixers.leone_experts_forward(
            _dt(x.dtype), _ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(w_down), _ptr(chosen), _ptr(weight), n,
            width, ff, experts, top, 1 if scale_input else 0, _ptr(offsets), _ptr(order), _ptr(act), _ptr(pair_out),
            _ptr(hidden), 0 if os.environ.get("LEONE_NO_EXPERT_MMA", "0") == "1" else 1, int(identity),
            1 if fresh else 0, self._stream()), "experts_forward")

    def sample(self, logits, temperature, seeds, positions, out):
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(temperature.dtype == torch.float32 and seeds.dtype == torch.int64
              and positions.dtype == torch.int64 and out.dtype == torch.int32, "sample arguments")
        _need(temperature.numel() >= rows and seeds.numel() >= rows and positions.numel() >= rows
              and out.numel() >= rows, "sample argument lengths")
        self.launches += 1
        _check(self.core.leone_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(seeds),
                                      _ptr(positions), _ptr(out), self._stream()), "sample")

    def sample_slots(self, logits, slot_ids, records, out):
        """One token per row with the row's temperature, seed and position taken from the slot
        record of its request (``records``: int64 ``[slots, 8]`` on the device, see
        :mod:`leone_b200.cache.slots`)."""
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(slot_ids.dtype == torch.int32 and slot_ids.numel() >= rows and records.dtype == torch.int64
              and records.is_contiguous() and records.shape[1] == 8 and out.dtype == torch.int32
              and out.numel() >= rows, "sample_slots arguments")
        self.launches += 1
        _check(self.core.leone_sample_slots(_ptr(logits), rows, vocab, _ptr(slot_ids), _ptr(records), _ptr(out),
                                            self._stream()), "sample_slots")

    def penalize(self, logits, entries, penalties):
        """Penalties from the decode history, in place: ``entries`` lists (row, token, occurrences
        in the row's window, DRY penalty), each (row, token) once; ``penalties[row]`` holds the
        row's repetition, presence and frequency factors (``csrc/sampling_pipeline.cu``)."""
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(len(penalties) == rows and all(0 <= e[0] < rows for e in entries), "penalize: rows")
        dev = self.device
        ints = torch.tensor([[e[0] for e in entries], [e[1] for e in entries], [e[2] for e in entries]],
                            dtype=torch.int32, device=dev)
        dry = torch.tensor([e[3] for e in entries], dtype=torch.float64, device=dev)
        per_row = torch.tensor([[p.repetition for p in penalties], [p.presence for p in penalties],
                                [p.frequency for p in penalties]], dtype=torch.float64, device=dev)
        self.launches += 1
        _check(self.core.leone_penalize(_ptr(logits), vocab, len(entries), _ptr(ints[0]), _ptr(ints[1]),
                                        _ptr(ints[2]), _ptr(dry), _ptr(per_row[0]), _ptr(per_row[1]),
                                        _ptr(per_row[2]), self._stream()), "penalize")

    def sample_truncated(self, logits, temperatures, seeds, positions, stages, want_probs: bool = False,
                         maximum_surprise=None, rows=None, out=None):
        """Rows that sample through truncation stages: ``stages`` is a list of (stage number,
        value) applied in order to every row (``csrc/sampling_pipeline.cu``).  ``rows``: which
        rows of ``logits`` take part (default: all); their ids are written to ``out`` at the same
        row numbers (``out``: int32 device tensor with a place per logits row; default: a new
        one).  Returns ``out`` (and the fp64 distribution the draws were made from, one row per
        participating row).  ``maximum_surprise`` (one per participating row): Mirostat's filter
        after the stages; the drawn tokens' probabilities before that filter are returned too
        (fp64 device tensor).  A row whose logits are all non-finite gets the id -1."""
        import ctypes
        n_rows, vocab = logits.shape
        members = list(range(n_rows)) if rows is None else [int(r) for r in rows]
        count = len(members)
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(count == len(temperatures) == len(seeds) == len(positions), "one temperature, seed and position a row")
        _need(all(0 <= r < n_rows for r in members) and len(set(members)) == count, "rows must be distinct rows of the logits")
        _need(all(t > 0 for t in temperatures), "truncation stages need a temperature")
        self.core.leone_sample_truncated_scratch.restype = ctypes.c_longlong
        need = int(self.core.leone_sample_truncated_scratch(count, vocab))
        if self._sample_scratch is None or self._sample_scratch.numel() < need:
            self._sample_scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        dev = self.device
        t = torch.tensor(temperatures, dtype=torch.float64, device=dev)
        sd = torch.tensor(np.array([s_ & 0xFFFF_FFFF_FFFF_FFFF for s_ in seeds], dtype=np.uint64).view(np.int64),
                          device=dev)
        pos = torch.tensor(positions, dtype=torch.int64, device=dev)
        row_map = None if rows is None else torch.tensor(members, dtype=torch.int32, device=dev)
        if out is None:
            out = torch.empty(n_rows, dtype=torch.int32, device=dev)
        _need(out.dtype == torch.int32 and out.numel() >= n_rows and out.is_contiguous(), "out: int32, a place per logits row")
        probs = torch.empty((count, vocab), dtype=torch.float64, device=dev) if want_probs else None
        mu = chosen = None
        if maximum_surprise is not None:
            _need(len(maximum_surprise) == count, "one maximum surprise a row")
            mu = torch.tensor([float(m) for m in maximum_surprise], dtype=torch.float64, device=dev)
            chosen = torch.zeros(count, dtype=torch.float64, device=dev)
        n = len(stages)
        types = (ctypes.c_int * max(n, 1))(*[int(a) for a, _ in stages])
        values = (ctypes.c_double * max(n, 1))(*[float(b) for _, b in stages])
        self.launches += 1
        _check(self.core.leone_sample_truncated(_ptr(logits), count, vocab, _ptr(t), _ptr(sd), _ptr(pos), n,
                                                types, values, _ptr(self._sample_scratch), _ptr(out),
                                                _ptr(probs), _ptr(mu), _ptr(chosen), _ptr(row_map), self._stream()),
               "sample_truncated")
        result = (out,) + ((probs,) if want_probs else ()) + ((chosen,) if mu is not None else ())
        return result if len(result) > 1 else out

    def decode_advance(self, token_ids, positions, ctx_len, sample_pos, sampled, history, counter,
                       slot_ids=None, records=None):
        """Feeds the sampled ids back as the next step's inputs.  Either ``sample_pos`` (int64 per
        row) is advanced, or, with ``slot_ids`` and ``records``, each request's slot record."""
        n = token_ids.numel()
        _need(history.dtype == torch.int32 and history.shape[1] == n and counter.dtype == torch.int32,
              "decode_advance arguments")
        if records is not None:
            _need(sample_pos is None and slot_ids is not None and slot_ids.dtype == torch.int32
                  and records.dtype == torch.int64 and records.shape[1] == 8, "decode_advance: slot records")
        else:
            _need(sample_pos is not None and sample_pos.dtype == torch.int64, "decode_advance: sample positions")
        self.launches += 1
        _check(self.core.leone_decode_advance(_ptr(token_ids), _ptr(positions), _ptr(ctx_len),
                                              _ptr(sample_pos), _ptr(sampled), _ptr(history),
                                              _ptr(counter), n, history.shape[0], _ptr(slot_ids), _ptr(records),
                                              self._stream()),
               "decode_advance")
