"""Opaque ``torch.library`` operators so that ``torch.compile`` can carry the attention call through a graph.

Counterpart of the reference's ``jvp_flash_attention::attn_fwd_dual_triton`` custom op and its fake
(jvp_flash_attention/jvp_attention.py:2247-2427), extended with a registered backward: the reference's compiled
path has no autograd (its op is called under ``no_grad``, :2677-2692), here gradients flow through both outputs.
``JVPAttn.dual`` switches to these operators while a graph is being compiled; eager calls keep using the
``autograd.Function`` in ``jvp_attention.py``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib


@torch.library.custom_op("jvp_flash_attention_b200::attn_fwd_dual", mutates_args=())
def attn_fwd_dual(q: Tensor, k: Tensor, v: Tensor, q_t: Tensor, k_t: Tensor, v_t: Tensor, mask: Optional[Tensor],
                  sm_scale: float, causal: bool, dropout_p: float = 0.0,
                  dropout_seed: int = 0) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    B, H, N, D = q.shape
    mask_c = _lib.make_mask(mask, B, H, N)
    summary = _lib.mask_summary(mask_c, mask, B, H, N) if mask is not None else None
    o, o_t, lse2, mu = _lib.fwd(q, k, v, q_t, k_t, v_t, mask_c, summary, causal, sm_scale, dropout_p, dropout_seed)
    return o, o_t, lse2, mu


@attn_fwd_dual.register_fake
def _(q, k, v, q_t, k_t, v_t, mask, sm_scale, causal, dropout_p=0.0, dropout_seed=0):
    B, H, N, D = q.shape
    stats = q.new_empty((B, H, N), dtype=torch.float32)
    return torch.empty_like(q), torch.empty_like(q), stats, torch.empty_like(stats)


@torch.library.custom_op("jvp_flash_attention_b200::attn_bwd_dual", mutates_args=())
def attn_bwd_dual(q: Tensor, k: Tensor, v: Tensor, q_t: Tensor, k_t: Tensor, v_t: Tensor, o: Tensor, o_t: Tensor,
                  lse2: Tensor, mu: Tensor, go: Tensor, go_t: Tensor, mask: Optional[Tensor], sm_scale: float,
                  causal: bool, dropout_p: float = 0.0,
                  dropout_seed: int = 0) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    B, H, N, D = q.shape
    mask_c = _lib.make_mask(mask, B, H, N)
    summary = _lib.mask_summary(mask_c, mask, B, H, N) if mask is not None else None
    return _lib.bwd(q, k, v, q_t, k_t, v_t, o.contiguous(), o_t.contiguous(), lse2, mu, go, go_t, mask_c, summary,
                    causal, sm_scale, dropout_p=dropout_p, dropout_seed=dropout_seed)


@attn_bwd_dual.register_fake
def _(q, k, v, q_t, k_t, v_t, o, o_t, lse2, mu, go, go_t, mask, sm_scale, causal, dropout_p=0.0, dropout_seed=0):
    return tuple(torch.empty_like(q) for _ in range(6))


@torch.library.custom_op("jvp_flash_attention_b200::attn_bwd_primal", mutates_args=())
def attn_bwd_primal(q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse2: Tensor, mu: Tensor, go: Tensor, mask: Optional[Tensor],
                    sm_scale: float, causal: bool, dropout_p: float = 0.0,
                    dropout_seed: int = 0) -> Tuple[Tensor, Tensor, Tensor]:
    """Backward through the primal output only (nothing flows back through the tangent output): dq, dk, dv."""
    B, H, N, D = q.shape
    mask_c = _lib.make_mask(mask, B, H, N)
    summary = _lib.mask_summary(mask_c, mask, B, H, N) if mask is not None else None
    return _lib.bwd(q, k, v, None, None, None, o.contiguous(), None, lse2, mu, go, None, mask_c, summary, causal, sm_scale,
                    dropout_p=dropout_p, dropout_seed=dropout_seed)


@attn_bwd_primal.register_fake
def _(q, k, v, o, lse2, mu, go, mask, sm_scale, causal, dropout_p=0.0, dropout_seed=0):
    return tuple(torch.empty_like(q) for _ in range(3))


def _setup_context(ctx, inputs, output):
    q, k, v, q_t, k_t, v_t, mask, sm_scale, causal, dropout_p, dropout_seed = inputs
    o, o_t, lse2, mu = output
    ctx.save_for_backward(q, k, v, q_t, k_t, v_t, o, o_t, lse2, mu)
    ctx.mask, ctx.sm_scale, ctx.causal, ctx.dropout = mask, sm_scale, causal, (dropout_p, dropout_seed)
    ctx.set_materialize_grads(False)


def _backward(ctx, go, go_t, _g_lse, _g_mu):
    q, k, v, q_t, k_t, v_t, o, o_t, lse2, mu = ctx.saved_tensors
    if go is None and go_t is None:
        return (None,) * 11
    if go_t is None:   # nothing flows back through the tangent output: the primal-only backward, no tangent-input gradients
        dq, dk, dv = attn_bwd_primal(q, k, v, o, lse2, mu, go, ctx.mask, ctx.sm_scale, ctx.causal, ctx.dropout[0], ctx.dropout[1])
        return (dq, dk, dv, None, None, None, None, None, None, None, None)
    go = torch.zeros_like(o) if go is None else go
    grads = attn_bwd_dual(q, k, v, q_t, k_t, v_t, o, o_t, lse2, mu, go, go_t, ctx.mask, ctx.sm_scale, ctx.causal,
                          ctx.dropout[0], ctx.dropout[1])
    return (*grads, None, None, None, None, None)


attn_fwd_dual.register_autograd(_backward, setup_context=_setup_context)
