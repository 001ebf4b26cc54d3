"""CPU oracle for dual (JVP) attention: forward outputs O, tO and the six input gradients.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; it is the checker and
the timed CPU baseline, never the thing that is shipped. The product path
(``jvp_flash_attention_b200``) never imports this module and fails loudly without its CUDA library.

Two independent statements of the same mathematics live here:

``sdpa_jvp_oracle``
    The construction the reference's own validator uses (tests/test_jvp_attention.py:548-561 for
    the dual-level form, :595-601 for the ``torch.func.jvp`` form): ``F.scaled_dot_product_attention``
    forced to ``SDPBackend.MATH``, differentiated in forward mode with ``torch.func.jvp`` and in
    reverse mode with autograd. It is run in fp64 on the fp64 upcast of the already-rounded inputs,
    and the loss is ``sum(O*gO) + sum(tO*gtO)`` so that gradients flow through BOTH outputs. The
    arithmetic lives in PyTorch (third party, pinned by the reference as ``torch>=2.8.0``,
    pyproject.toml:26); this is the oracle the stated tolerances refer to.

``closed_form_oracle``
    A numpy fp64 restatement, head by head, of what the reference's kernels compute
    (jvp_flash_attention/jvp_attention.py:244-247 scores and tangent scores, :312-333 and :1041-1044
    online softmax / tangent accumulation / epilogue, :1419 delta, :1514-1572 dK/dV, :1666-1716 dQ),
    extended with the gradient through the tangent output, which the reference does not implement
    (jvp_attention.py:3081 ignores the second incoming gradient, :3226 returns None for the tangent
    inputs). Mask semantics follow SDPA (additive after scaling, -inf allowed, boolean True = keep),
    not the reference's "add before scaling / MASK_CONST" quirk (jvp_attention.py:250-262).

Pinning: ``closed_form_oracle`` is checked against ``sdpa_jvp_oracle`` and against outputs of the
reference's own Triton kernels run under the Triton CPU interpreter (tests/golden/make_golden.py
wrote those outputs; tests/test_oracle.py compares). The reference holds no golden vectors of its
own. Gradients with respect to the tangent output and the tangent inputs are pinned by
``sdpa_jvp_oracle`` only: the reference cannot produce them (parity unpinned on the reference side).
"""
from __future__ import annotations

import math
import time
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

GRAD_NAMES = ("dq", "dk", "dv", "dtq", "dtk", "dtv")


# --------------------------------------------------------------------------------------------
# primary oracle: SDPA-MATH + torch.func.jvp + autograd (reference validator's construction)
# --------------------------------------------------------------------------------------------
def sdpa_jvp_oracle(q, k, v, tq, tk, tv, gO=None, gtO=None, attn_mask=None, causal=False, sm_scale=None,
                    dtype=torch.float64):
    """Returns dict(O, tO, dq, dk, dv, dtq, dtk, dtv) computed on CPU in ``dtype``.

    Follows tests/test_jvp_attention.py:548-561, 595-601 (SDPA under SDPBackend.MATH on dual
    inputs), with the loss extended by ``sum(tO*gtO)``. Gradients are skipped when gO is None.
    """
    up = lambda t: t.detach().to("cpu").to(dtype)
    args = [up(t).requires_grad_(gO is not None) for t in (q, k, v, tq, tk, tv)]
    mask = None
    if attn_mask is not None:
        mask = attn_mask.detach().to("cpu")
        if mask.dtype != torch.bool:
            mask = mask.to(dtype)

    def fn(a, b, c):
        return F.scaled_dot_product_attention(a, b, c, attn_mask=mask, is_causal=causal, scale=sm_scale)

    with sdpa_kernel(SDPBackend.MATH):
        O, tO = torch.func.jvp(fn, tuple(args[:3]), tuple(args[3:]))
    out = {"O": O.detach(), "tO": tO.detach()}
    if gO is not None:
        loss = (O * up(gO)).sum() + (tO * up(gtO)).sum()
        grads = torch.autograd.grad(loss, args)
        out.update({n: g.detach() for n, g in zip(GRAD_NAMES, grads)})
    return out


# --------------------------------------------------------------------------------------------
# dropout pattern: Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11), keyed by the
# 64-bit seed, counter (q >> 1, k >> 1, batch*head unit, 0); the four 32-bit outputs of one call belong to the 2 x 2
# block of elements (q, k), index (q & 1) * 2 + (k & 1). An element is kept when its number is >= p * 2^32.
# --------------------------------------------------------------------------------------------
def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox4x32 with 10 rounds on uint32 numpy arrays; returns the four output words."""
    M0, M1, W0, W1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), 0x9E3779B9, 0xBB67AE85
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32) for c in (c0, c1, c2, c3))
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c0.astype(np.uint64)
        p1 = M1 * c2.astype(np.uint64)
        hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), p0.astype(np.uint32)
        hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), p1.astype(np.uint32)
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint32(k0), lo1, hi0 ^ c3 ^ np.uint32(k1), lo0
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def dropout_threshold(p: float) -> int:
    """The 32-bit threshold of the keep test ``number >= threshold`` for drop probability p."""
    return min(0xFFFFFFFF, max(0, int(round(p * 4294967296.0))))


def dropout_keep(seed: int, unit: int, N: int, p: float) -> np.ndarray:
    """(N, N) array of 0.0 / 1.0: which attention probabilities of (batch, head) unit ``unit`` survive dropout."""
    half = (N + 1) // 2
    qp, kp = np.meshgrid(np.arange(half, dtype=np.uint32), np.arange(half, dtype=np.uint32), indexing="ij")
    words = philox4x32_10(qp, kp, np.full_like(qp, unit), np.zeros_like(qp), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    full = np.empty((2 * half, 2 * half), dtype=np.uint32)
    for i in range(2):
        for j in range(2):
            full[i::2, j::2] = words[i * 2 + j]
    return (full[:N, :N] >= np.uint32(dropout_threshold(p))).astype(np.float64)


# --------------------------------------------------------------------------------------------
# second oracle: closed-form numpy restatement, one (batch, head) slice at a time
# --------------------------------------------------------------------------------------------
def _closed_form_head(q, k, v, tq, tk, tv, gO, gtO, bias, s, keep=None):
    """One head in numpy fp64. ``bias`` is an (N, N) additive matrix (0 / -inf / finite) or None. ``keep`` is an (N, N)
    dropout matrix (0 for dropped probabilities, 1 / (1 - p) for kept ones) applied after the softmax, or None."""
    S = s * (q @ k.T)                                   # jvp_attention.py:244 (qk), scaled
    if bias is not None:
        S = S + bias
    m = S.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    E = np.exp(S - m)
    l = E.sum(axis=-1, keepdims=True)
    dead = l == 0.0                                     # fully masked rows: outputs and grads are 0
    P = E / np.where(dead, 1.0, l)                      # jvp_attention.py:1371-1375 (l := 1)
    lse = (m + np.log(np.where(dead, 1.0, l)))[:, 0]
    lse = np.where(dead[:, 0], -np.inf, lse)
    tS = s * (tq @ k.T + q @ tk.T)                      # jvp_attention.py:245-247 (t_qk)
    mu = (P * tS).sum(axis=-1, keepdims=True)           # jvp_attention.py:330-331 (mu accumulation)
    tP = P * (tS - mu)
    Pd, tPd = (P, tP) if keep is None else (P * keep, tP * keep)   # dropout acts on the probabilities that reach V
    O = Pd @ v                                          # jvp_attention.py:333 (acc)
    tO = tPd @ v + Pd @ tv                              # jvp_attention.py:1041-1044 (epilogue)
    out = {"O": O, "tO": tO, "lse": lse, "mu": mu[:, 0]}
    if gO is None:
        return out
    A = gtO @ v.T
    X = gO @ v.T + gtO @ tv.T
    if keep is not None:
        A, X = A * keep, X * keep
    a = (gtO * O).sum(axis=-1, keepdims=True)
    dtS = P * (A - a)                                   # gradient w.r.t. the tangent scores
    dP = X + A * (tS - mu) - a * tS
    delta = (gO * O).sum(-1, keepdims=True) + (gtO * tO).sum(-1, keepdims=True) - a * mu  # :1419 when gtO == 0
    dS = P * (dP - delta)                               # jvp_attention.py:1557 (dsT)
    out.update(
        dq=s * (dS @ k + dtS @ tk),                     # jvp_attention.py:1708 (+ tangent term)
        dk=s * (dS.T @ q + dtS.T @ tq),                 # jvp_attention.py:1564
        dv=Pd.T @ gO + tPd.T @ gtO,                     # jvp_attention.py:1552
        dtq=s * (dtS @ k),
        dtk=s * (dtS.T @ q),
        dtv=Pd.T @ gtO,
        delta=delta[:, 0],
        a=a[:, 0],
    )
    return out


def _as_np64(t):
    if isinstance(t, torch.Tensor):
        return t.detach().to("cpu").to(torch.float64).numpy()
    return np.asarray(t, dtype=np.float64)


def closed_form_oracle(q, k, v, tq, tk, tv, gO=None, gtO=None, attn_mask=None, causal=False, sm_scale=None,
                       slices: Optional[Sequence[tuple]] = None, dropout_p: float = 0.0, dropout_seed: int = 0):
    """Closed-form fp64 oracle. Returns a dict of numpy arrays shaped like the inputs (plus the
    per-row statistics ``lse``, ``mu`` and, with gradients, ``delta`` and ``a``).

    ``slices`` = iterable of (b, h) pairs restricts the work to those heads; the returned arrays
    then have shape (len(slices), N, D) in that order (used for the large configurations).

    ``dropout_p`` > 0 applies dropout to the attention probabilities with the keep pattern of ``dropout_keep``
    (a counter-based generator keyed by the seed and the element's position, so that any implementation can
    regenerate it); the reference only sketches this (jvp_attention.py:105-133) and refuses dropout_p != 0 (:2550).
    """
    qn, kn, vn, tqn, tkn, tvn = (_as_np64(t) for t in (q, k, v, tq, tk, tv))
    gOn = _as_np64(gO) if gO is not None else None
    gtOn = _as_np64(gtO) if gtO is not None else None
    B, H, N, D = qn.shape
    s = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
    mask = None
    if attn_mask is not None:
        mt = attn_mask.detach().to("cpu") if isinstance(attn_mask, torch.Tensor) else torch.as_tensor(attn_mask)
        if mt.dtype == torch.bool:
            mask = np.where(mt.numpy(), 0.0, -np.inf)
        else:
            mask = mt.to(torch.float64).numpy()
        mask = np.broadcast_to(mask, (B, H, N, N))
    tri = np.where(np.tril(np.ones((N, N), dtype=bool)), 0.0, -np.inf) if causal else None
    pairs = list(slices) if slices is not None else [(b, h) for b in range(B) for h in range(H)]
    res = {}
    for idx, (b, h) in enumerate(pairs):
        bias = None
        if mask is not None:
            bias = mask[b, h]
        if tri is not None:
            bias = tri if bias is None else bias + tri
        keep = None
        if dropout_p > 0.0:
            keep = dropout_keep(dropout_seed, b * H + h, N, dropout_p) / (1.0 - dropout_p)
        r = _closed_form_head(qn[b, h], kn[b, h], vn[b, h], tqn[b, h], tkn[b, h], tvn[b, h],
                              None if gOn is None else gOn[b, h], None if gtOn is None else gtOn[b, h], bias, s, keep)
        for name, val in r.items():
            res.setdefault(name, []).append(val)
    out = {name: np.stack(vals) for name, vals in res.items()}
    if slices is None:
        out = {name: val.reshape((B, H) + val.shape[1:]) for name, val in out.items()}
    return out


# --------------------------------------------------------------------------------------------
# synthetic inputs of the benchmark configurations (seeded; stand in for any dataset)
# --------------------------------------------------------------------------------------------
def make_inputs(B, H, N, D, dtype=torch.float32, seed=42, scale=1.0, device="cpu"):
    """Eight i.i.d. N(0,1)*scale tensors (q, k, v, tq, tk, tv, gO, gtO) from one CPU generator,
    as in tests/test_jvp_attention.py:276-306 (seed 42), rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    ts = [(torch.randn(B, H, N, D, generator=g) * scale).to(dtype) for _ in range(8)]
    return [t.to(device) for t in ts]


def make_bool_mask(B, N, keep=0.9, seed=1042):
    """(B,1,N,N) Bernoulli keep mask with the diagonal forced True."""
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(B, 1, N, N, generator=g) < keep
    return m | torch.eye(N, dtype=torch.bool)


def make_block_sparse_mask(B, N, block=128, density=0.25, seed=1042):
    """(B,1,N,N) mask of block x block tiles kept with the given density, diagonal tiles kept."""
    g = torch.Generator().manual_seed(seed)
    nb = N // block
    blk = (torch.rand(B, 1, nb, nb, generator=g) < density) | torch.eye(nb, dtype=torch.bool)
    return blk.repeat_interleave(block, -1).repeat_interleave(block, -2)


def make_additive_mask(B, N, dtype=torch.float32, drop=0.1, seed=1042):
    """(B,1,N,N) N(0,1) additive mask with a fraction ``drop`` of -inf entries, diagonal finite."""
    g = torch.Generator().manual_seed(seed)
    m = torch.randn(B, 1, N, N, generator=g)
    d = (torch.rand(B, 1, N, N, generator=g) < drop) & ~torch.eye(N, dtype=torch.bool)
    m[d] = float("-inf")
    return m.to(dtype)


# --------------------------------------------------------------------------------------------
# timed CPU baseline: the reference's CPU-runnable path on the host cores
# --------------------------------------------------------------------------------------------
def time_cpu_reference_path(B, H, N, D, causal=False, dtype=torch.float32, n_slices=1, repeats=1, seed=0):
    """Times SDPA-MATH + torch.func.jvp + autograd (six grads, loss through both outputs) on
    ``n_slices`` (b,h) slices of an (B,H,N,D) problem and returns (seconds per slice, threads).

    SDPA-MATH materialises the N x N matrices per head, so large shapes are timed per slice and
    scaled by the caller. Same construction as tests/test_jvp_attention.py:548-561, 595-601.
    """
    g = torch.Generator().manual_seed(seed)
    ts = [torch.randn(1, n_slices, N, D, generator=g).to(dtype) for _ in range(8)]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        sdpa_jvp_oracle(*ts, causal=causal, dtype=dtype)
        best = min(best, time.perf_counter() - t0)
    return best / n_slices, torch.get_num_threads()
