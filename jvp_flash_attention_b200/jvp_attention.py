"""Drop-in mirror of ``jvp_flash_attention.jvp_attention`` backed by libjvpfa.so (CUDA, sm_100a).

Same public names as the reference module (jvp_flash_attention/jvp_attention.py): ``JVPAttn`` with
``fwd`` (:2915) and ``fwd_dual`` (:2972), ``attention`` (:3229), ``MASK_CONST`` and
``MIN_SEQUENCE_LENGTH`` (:48-51). Differences, all supersets of the reference behaviour:

* the tangent output takes part in autograd: ``backward`` receives the upstream gradients of both
  the primal and the tangent output and returns gradients for q, k, v and their tangents (the
  reference ignores the second gradient and returns None for the tangents, :3081, :3226);
* masks follow ``F.scaled_dot_product_attention`` semantics: a float mask is added after scaling
  and may contain ``-inf``; any mask broadcastable to (Z, H, N, N) is accepted without a copy;
* there is no Triton, no dispatch to another backend and no CPU path: without the CUDA library,
  or on CPU tensors, calls raise.

Second derivatives: Hessian-vector products work in reverse-over-forward form (the gradient of a directional derivative
taken with ``fwd_dual`` / ``dual``: the tangent output is part of the autograd graph); differentiating the backward itself
(``create_graph=True`` through these functions) is not supported and raises.

Failure detection: every device-side wait in the kernels is bounded; one that gives up records a code in a status
word and the kernel runs to its end. Each call enqueues a copy of that word to pinned host memory behind its
kernels, and the next call on the same stream (without synchronising) or ``check()`` (which synchronises the
device) raises ``_lib.JvpfaError`` with status ``ERR_DEVICE_TIMEOUT``; the results of the call that timed out are
undefined. Errors the reference reports as Python exceptions (jvp_attention.py:2550, 2574, 3111) keep their types.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.autograd.forward_ad as fwAD
from torch import Tensor
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from . import _lib

MASK_CONST = -100.0          # jvp_attention.py:48-50; kept for callers that build {0, MASK_CONST} masks
MIN_SEQUENCE_LENGTH = 32     # jvp_attention.py:51


def _validate(q: Tensor, k: Tensor, v: Tensor, attn_mask: Optional[Tensor], dropout_p: float, causal: bool,
              verify_attn_mask: bool) -> None:
    """Argument checks with the reference's exception types (jvp_attention.py:2550-2586, 2632-2656)."""
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError(f"dropout_p must be in [0, 1), got {dropout_p}")
    if dropout_p != 0.0 and not _lib.dropout_supported(q.dtype, q.shape[-1]):
        # the reference refuses every dropout_p != 0 with this exception (jvp_attention.py:2550-2551); here dropout exists
        # wherever the tensor-core kernels run (head dimensions that are multiples of 8: up to 128 in fp16 / bf16, 64 in fp32)
        raise NotImplementedError("Dropout is not currently supported in JVP attention.")
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must have shape (Z, H, N_CTX, HEAD_DIM)"
    Z, H, N_CTX, HEAD_DIM_Q = q.shape
    HEAD_DIM_K, HEAD_DIM_V = k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V, (
        "JVP attention requires HEAD_DIM_Q == HEAD_DIM_K == HEAD_DIM_V"
        f" but got HEAD_DIM_Q={HEAD_DIM_Q}, HEAD_DIM_K={HEAD_DIM_K}, HEAD_DIM_V={HEAD_DIM_V}")
    assert k.shape == q.shape and v.shape == q.shape, "JVP attention is self-attention: q, k, v must share one shape"
    assert q.dtype == k.dtype == v.dtype, "q, k, v must share one dtype"
    assert q.dtype in (torch.float16, torch.bfloat16, torch.float32), f"unsupported dtype {q.dtype}"
    if not q.is_cuda:
        raise RuntimeError("jvp_flash_attention_b200 runs on CUDA tensors only (there is no CPU path)")
    if causal and attn_mask is not None:
        raise ValueError("Causal attention does not support an attention mask.")
    if attn_mask is not None and verify_attn_mask:
        assert attn_mask.dim() == 4, "The provided attention mask must have 4 dimensions (Z, H, N_CTX, N_CTX)."
        ok = all(ms in (1, fs) for ms, fs in zip(attn_mask.shape, (Z, H, N_CTX, N_CTX)))
        assert ok, "The provided attention mask must be broadcastable to (Z, H, N_CTX, N_CTX)."
        assert attn_mask.dtype == torch.bool or attn_mask.dtype.is_floating_point, (
            "The attention mask must be of the dtype bool or a floating-point dtype.")
        if attn_mask.dtype == torch.bool:
            assert attn_mask.any(dim=(-1, -2)).all(), "The attention mask cannot be all False for any head."
        else:
            assert not torch.isnan(attn_mask).any(), "The attention mask cannot contain NaNs."


def _draw_seed(dropout_p: float, dropout_seed) -> int:
    """The seed of the dropout pattern: the caller's, or 63 bits from torch's CPU generator (so ``torch.manual_seed``
    makes runs repeatable, and no device synchronisation is needed)."""
    if dropout_p == 0.0:
        return 0
    if dropout_seed is not None:
        return int(dropout_seed)
    return int(torch.randint(0, 2 ** 63 - 1, (), dtype=torch.int64).item())


def _mask_for_kernel(attn_mask: Optional[Tensor], q: Tensor) -> Optional[Tensor]:
    """Returns the mask in an element type the kernels read (bool, q.dtype-compatible or fp32)."""
    if attn_mask is None:
        return None
    m = attn_mask
    if m.dtype == torch.bool:
        return m
    if m.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        m = m.to(torch.float32)
    return m


class _DualAttention(Function):
    """(q, k, v, tq, tk, tv) -> (o, to, lse2, mu[, mask summary]); autograd through o and to."""

    @staticmethod
    def forward(q, k, v, tq, tk, tv, attn_mask, causal, sm_scale, dropout_p=0.0, dropout_seed=0):
        B, H, N, D = q.shape
        mask_c = _lib.make_mask(attn_mask, B, H, N)
        summary = _lib.mask_summary(mask_c, attn_mask, B, H, N) if attn_mask is not None else None
        o, to, lse2, mu = _lib.fwd(q, k, v, tq, tk, tv, mask_c, summary, causal, sm_scale, dropout_p, dropout_seed)
        if summary is None:
            summary = torch.empty(0, dtype=torch.uint8, device=q.device)
        return o, to, lse2, mu, summary

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        q, k, v, tq, tk, tv, attn_mask, causal, sm_scale, dropout_p, dropout_seed = inputs
        o, to, lse2, mu, summary = outputs
        ctx.mark_non_differentiable(lse2, mu, summary)
        ctx.save_for_backward(q, k, v, tq, tk, tv, o, to, lse2, mu, summary)
        ctx.attn_mask = attn_mask
        ctx.causal = causal
        ctx.sm_scale = sm_scale
        ctx.dropout = (dropout_p, dropout_seed)
        ctx.set_materialize_grads(False)    # an output the loss does not use arrives as None, not as a tensor of zeros

    @staticmethod
    @once_differentiable      # the gradients come from kernels: differentiating them again raises instead of returning zeros
    def backward(ctx, go, gto, _g_lse, _g_mu, _g_summary):
        q, k, v, tq, tk, tv, o, to, lse2, mu, summary = ctx.saved_tensors
        B, H, N, D = q.shape
        if go is None and gto is None:
            return (None,) * 11
        mask_c = _lib.make_mask(ctx.attn_mask, B, H, N)
        summ = summary if summary.numel() > 0 else None
        if gto is None:
            # Nothing flows back through the tangent output (a tangent that is only used as a detached target, or not at
            # all): the primal-only backward -- what the reference's backward always is (jvp_attention.py:3081, 3226) --
            # gives dq, dk, dv with half the tile products, and the tangent inputs get no gradient.
            dq, dk, dv = _lib.bwd(q, k, v, None, None, None, o, None, lse2, mu, go, None, mask_c, summ, ctx.causal,
                                  ctx.sm_scale, dropout_p=ctx.dropout[0], dropout_seed=ctx.dropout[1])
            return dq, dk, dv, None, None, None, None, None, None, None, None
        if go is None:
            go = torch.zeros_like(o)
        dq, dk, dv, dtq, dtk, dtv = _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, go, gto, mask_c, summ,
                                              ctx.causal, ctx.sm_scale, dropout_p=ctx.dropout[0], dropout_seed=ctx.dropout[1])
        return dq, dk, dv, dtq, dtk, dtv, None, None, None, None, None


class _PrimalAttention(Function):
    """(q, k, v) -> (o, lse2): the primal-only entry; backward gives dq, dk, dv."""

    @staticmethod
    def forward(q, k, v, attn_mask, causal, sm_scale, dropout_p=0.0, dropout_seed=0):
        B, H, N, D = q.shape
        mask_c = _lib.make_mask(attn_mask, B, H, N)
        summary = _lib.mask_summary(mask_c, attn_mask, B, H, N) if attn_mask is not None else None
        o, _, lse2, mu = _lib.fwd(q, k, v, None, None, None, mask_c, summary, causal, sm_scale, dropout_p, dropout_seed)
        if summary is None:
            summary = torch.empty(0, dtype=torch.uint8, device=q.device)
        return o, lse2, mu, summary

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        q, k, v, attn_mask, causal, sm_scale, dropout_p, dropout_seed = inputs
        o, lse2, mu, summary = outputs
        ctx.mark_non_differentiable(lse2, mu, summary)
        ctx.save_for_backward(q, k, v, o, lse2, mu, summary)
        ctx.attn_mask = attn_mask
        ctx.causal = causal
        ctx.sm_scale = sm_scale
        ctx.dropout = (dropout_p, dropout_seed)

    @staticmethod
    @once_differentiable
    def backward(ctx, go, _g_lse, _g_mu, _g_summary):
        q, k, v, o, lse2, mu, summary = ctx.saved_tensors
        B, H, N, D = q.shape
        mask_c = _lib.make_mask(ctx.attn_mask, B, H, N)
        summ = summary if summary.numel() > 0 else None
        dq, dk, dv = _lib.bwd(q, k, v, None, None, None, o, None, lse2, mu, go, None, mask_c, summ, ctx.causal,
                              ctx.sm_scale, dropout_p=ctx.dropout[0], dropout_seed=ctx.dropout[1])
        return dq, dk, dv, None, None, None, None, None


class JVPAttn:
    """JVP (Jacobian-vector product) attention; mirrors the reference class of the same name."""

    @staticmethod
    def fwd(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None = None, dropout_p: float = 0.0,
            causal: bool = False, sm_scale: float | None = None, warp_specialize: bool = True, USE_TMA: bool = True,
            verify_attn_mask: bool = True, dropout_seed: int | None = None) -> Tensor:
        """Primal-only attention (jvp_attention.py:2915-2970). ``warp_specialize`` and ``USE_TMA`` are
        accepted for signature compatibility and ignored. ``dropout_p`` > 0 (every shape the tensor-core kernels take; the
        reference refuses it) drops attention probabilities with a pattern drawn from ``dropout_seed``, or from torch's
        CPU generator when no seed is given."""
        _validate(q, k, v, attn_mask, dropout_p, causal, verify_attn_mask)
        # strided views are read in place where the kernels can (``_lib.as_input``); the reference copies them (:2950)
        q, k, v = (_lib.as_input(t) for t in (q, k, v))
        if sm_scale is None:
            sm_scale = q.shape[-1] ** -0.5
        o, _, _, _ = _PrimalAttention.apply(q, k, v, _mask_for_kernel(attn_mask, q), bool(causal), float(sm_scale),
                                            float(dropout_p), _draw_seed(dropout_p, dropout_seed))
        return o

    @staticmethod
    def fwd_dual(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None = None, dropout_p: float = 0.0,
                 causal: bool = False, sm_scale: float | None = None, warp_specialize: bool = True,
                 USE_TMA: bool = True, verify_attn_mask: bool = True, dropout_seed: int | None = None) -> Tensor:
        """Attention on forward-mode dual tensors (jvp_attention.py:2972-3063): works inside
        ``fwAD.dual_level()`` and under ``torch.func.jvp``; the result is a dual tensor whose tangent is
        the JVP. Inputs without a tangent contribute a zero tangent; if no input is dual this is ``fwd``."""
        q_p, q_t = fwAD.unpack_dual(q)
        k_p, k_t = fwAD.unpack_dual(k)
        v_p, v_t = fwAD.unpack_dual(v)
        if q_t is None and k_t is None and v_t is None:
            return JVPAttn.fwd(q, k, v, attn_mask, dropout_p, causal, sm_scale, warp_specialize, USE_TMA,
                               verify_attn_mask, dropout_seed)
        q_t = torch.zeros_like(q_p) if q_t is None else q_t
        k_t = torch.zeros_like(k_p) if k_t is None else k_t
        v_t = torch.zeros_like(v_p) if v_t is None else v_t
        # ``dual`` validates, and inside torch.compile switches to the opaque operators (the reference routes its
        # compiled dual call through its custom op in the same place, jvp_attention.py:3014-3041)
        o, to = JVPAttn.dual(q_p, k_p, v_p, q_t, k_t, v_t, attn_mask=attn_mask, causal=causal, sm_scale=sm_scale,
                             verify_attn_mask=verify_attn_mask, dropout_p=dropout_p, dropout_seed=dropout_seed)
        return fwAD.make_dual(o, to)

    @staticmethod
    def dual(q: Tensor, k: Tensor, v: Tensor, q_t: Tensor, k_t: Tensor, v_t: Tensor, attn_mask: Tensor | None = None,
             causal: bool = False, sm_scale: float | None = None, verify_attn_mask: bool = True, dropout_p: float = 0.0,
             dropout_seed: int | None = None):
        """Explicit-tangent form: returns ``(o, to)`` as ordinary tensors, both connected to autograd
        (gradients reach q, k, v and the three tangents). No reference counterpart; this is what
        ``fwd_dual`` calls once it has unpacked the dual tensors."""
        if torch.compiler.is_compiling():
            # inside torch.compile: the opaque operator pair of compile_op.py (no data-dependent checks in a graph)
            from .compile_op import attn_fwd_dual
            if sm_scale is None:
                sm_scale = q.shape[-1] ** -0.5
            if dropout_p != 0.0 and dropout_seed is None:
                raise RuntimeError("inside torch.compile dropout needs an explicit dropout_seed")
            o, to, _, _ = attn_fwd_dual(q, k, v, q_t, k_t, v_t, _mask_for_kernel(attn_mask, q), float(sm_scale),
                                        bool(causal), float(dropout_p), int(dropout_seed or 0))
            return o, to
        _validate(q, k, v, attn_mask, dropout_p, causal, verify_attn_mask)
        # strided views are read in place where the kernels can; the reference copies them (jvp_attention.py:3007)
        q, k, v, q_t, k_t, v_t = (_lib.as_input(t) for t in (q, k, v, q_t, k_t, v_t))
        if sm_scale is None:
            sm_scale = q.shape[-1] ** -0.5
        o, to, _, _, _ = _DualAttention.apply(q, k, v, q_t, k_t, v_t, _mask_for_kernel(attn_mask, q), bool(causal),
                                              float(sm_scale), float(dropout_p), _draw_seed(dropout_p, dropout_seed))
        return o, to


attention = JVPAttn.fwd


def check(device=None) -> None:
    """Synchronises ``device`` (default: the current CUDA device) and raises ``_lib.JvpfaError`` if a bounded
    device-side wait gave up in any call since the last check."""
    _lib.read_status(device)
