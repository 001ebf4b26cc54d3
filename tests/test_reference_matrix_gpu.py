"""The reference's own validation matrix on the CUDA path.

``tests/test_jvp_attention.py`` of the reference (a script, not a pytest module) walks batch 2, 12 heads of dimension
64 over sequence lengths 32 ... 2048, three mask types and causal / non-causal, in three dtypes, and compares the primal
output, the tangent output and the q, k, v gradients of a mean-squared loss on the primal output with SDPA-MATH
(tests/test_jvp_attention.py:515-667, shapes :225-236, masks :337-392 with 10 % of the entries attended, loss
:400-410). The same cases run here against the fp64 oracle, with seeded N(0,1) tensors of those shapes:

* outputs: max abs error <= 2e-2 (fp16 / bf16), <= 1e-4 (fp32) -- the reference allows 4e-3 / 3.2e-2 / 2.35e-2. The
  sparse masks of this matrix (10 % attended) leave some rows with two or three keys, whose tangent outputs reach
  magnitude 7: there the bound is two steps of the output type at the tensor's largest value (bf16: up to 6e-2) and, for
  fp32 (three bf16 products per product), 3e-5 of the largest value;
* gradients of the reference's loss: <= 5e-4 absolute (its own gradient tolerance, :526-527) and, because such
  gradients are of the order 1e-5 and an absolute bound says little, <= 2 % (fp32: 0.1 %) of the largest oracle entry;
  the upstream gradient the oracle gets is the one autograd hands to the backward (rounded to the tensors' type).
"""
import numpy as np
import pytest
import torch
import torch.autograd.forward_ad as fwAD

from oracle.jvp_attention_oracle import closed_form_oracle

pytestmark = pytest.mark.gpu
MASK_PROB = 0.9      # tests/test_jvp_attention.py: rand > mask_prob is attended
TOL = {torch.float16: 2e-2, torch.bfloat16: 2e-2, torch.float32: 1e-4}
REL = {torch.float16: 2e-2, torch.bfloat16: 2e-2, torch.float32: 1e-3}


def _mask(kind, B, H, N, dtype):
    from jvp_flash_attention_b200.jvp_attention import MASK_CONST
    if kind in ("none", "causal"):
        return None
    g = torch.Generator().manual_seed(1042)
    keep = torch.rand(B, H, N, N, generator=g) > MASK_PROB
    if kind == "boolean":
        return keep
    return torch.where(keep, 0.0, MASK_CONST).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kind", ["none", "causal", "boolean", "additive"])
@pytest.mark.parametrize("N", [32, 64, 128, 256, 512, 1024, 2048])
def test_reference_validation_matrix(N, kind, dtype):
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    dev = torch.device("cuda:0")
    B, H, D = 2, 12, 64
    g = torch.Generator().manual_seed(42)
    q, tq, k, tk, v, tv, target = [torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(7)]
    mask = _mask(kind, B, H, N, dtype)
    causal = kind == "causal"
    dq, dk, dv = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    with fwAD.dual_level():
        out = JVPAttn.fwd_dual(fwAD.make_dual(dq, tq.to(dev)), fwAD.make_dual(dk, tk.to(dev)), fwAD.make_dual(dv, tv.to(dev)),
                               attn_mask=None if mask is None else mask.to(dev), causal=causal, verify_attn_mask=False)
        O, tO = fwAD.unpack_dual(out)
        loss = (O.float() - target.to(dev).float()).square().mean()
        (gO,) = torch.autograd.grad(loss, O, retain_graph=True)     # what the backward is handed, in the tensors' type
        grads = torch.autograd.grad(loss, (dq, dk, dv))
    torch.cuda.synchronize()
    _lib.read_status(dev)
    # the oracle on a few (b, h) slices (all of them for short sequences); upstream gradient of the loss taken at the
    # computed output, so that the comparison is about the backward pass
    rng = np.random.default_rng(N)
    slices = [(b, h) for b in range(B) for h in range(H)] if N <= 128 else \
        [(0, 0), (B - 1, H - 1), (int(rng.integers(0, B)), int(rng.integers(0, H)))]
    pick = lambda t: torch.stack([t[b, h] for b, h in slices]).unsqueeze(1)        # (slices, 1, N, .) on the host
    ref = closed_form_oracle(*[pick(t) for t in (q, k, v, tq, tk, tv)], pick(gO.cpu().double()), pick(torch.zeros_like(q)).double(),
                             attn_mask=None if mask is None else pick(mask), causal=causal)
    ref = {n: a[:, 0] for n, a in ref.items() if n in ("O", "tO", "dq", "dk", "dv")}
    take = lambda t: torch.stack([t[b, h] for b, h in slices]).double().cpu()
    for name, got in (("O", O.detach()), ("tO", tO.detach())):
        r = torch.from_numpy(ref[name])
        top = float(r.abs().max())
        allowed = max(TOL[dtype], 3e-5 * top if dtype == torch.float32 else
                      2.0 * 2.0 ** (np.floor(np.log2(top)) - (7 if dtype == torch.bfloat16 else 10)))
        err = float((take(got) - r).abs().max())
        assert err <= allowed, (name, err, allowed, top)
    for name, got in zip(("dq", "dk", "dv"), grads):
        r = torch.from_numpy(ref[name])
        err = float((take(got) - r).abs().max())
        # (fp16 stores these 1e-6-sized gradients as subnormals, in steps of 2^-24: four steps are allowed)
        floor = 4 * 2.0 ** -24 if dtype == torch.float16 else 1e-9
        assert err <= 5e-4 and err <= max(REL[dtype] * float(r.abs().max()), floor), (name, err, float(r.abs().max()))
