"""Dropout on the attention probabilities (every shape the tensor-core kernels take). The reference sketches it
(jvp_attention.py:105-133) but refuses dropout_p != 0 (:2550); here the keep pattern is a counter-based function of
(seed, batch*head unit, query, key) that the forward, the three backward kernels and the CPU oracle all regenerate."""
import numpy as np
import pytest
import torch
import torch.autograd.forward_ad as fwAD

from oracle.jvp_attention_oracle import GRAD_NAMES, closed_form_oracle, dropout_keep, make_bool_mask, make_inputs
from test_parity_gpu import TOL, _compare

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def test_keep_pattern_matches_the_oracle_bit_for_bit(dev):
    """q = k = 0 makes every probability 1/N and v = identity turns the output into the dropped-out probabilities, so the
    kernel's keep pattern can be read off the output and compared with the oracle's generator."""
    from jvp_flash_attention_b200.jvp_attention import attention
    B, H, N, D, p, seed = 2, 3, 128, 128, 0.3, 987654321987
    z = torch.zeros(B, H, N, D, device=dev, dtype=torch.float16)
    v = torch.eye(N, D, device=dev, dtype=torch.float16).expand(B, H, N, D).contiguous()
    o = attention(z, z, v, dropout_p=p, dropout_seed=seed)
    got = (o.float() > 0).cpu().numpy()
    for b in range(B):
        for h in range(H):
            want = dropout_keep(seed, b * H + h, N, p) > 0
            assert np.array_equal(got[b, h], want), (b, h)
    kept = got.mean()
    assert abs(kept - (1 - p)) < 0.01
    assert torch.allclose(o[o > 0].float(), torch.tensor(1.0 / (N * (1 - p))), rtol=2e-3)


@pytest.mark.parametrize("dtype,B,H,N,D,causal,p", [
    (torch.bfloat16, 2, 3, 200, 64, True, 0.1),
    (torch.float16, 1, 2, 256, 128, False, 0.5),
    (torch.float16, 2, 2, 333, 64, True, 0.25),
    (torch.bfloat16, 1, 2, 512, 128, True, 0.2),
    (torch.bfloat16, 2, 2, 256, 72, False, 0.15),     # padded head dimensions
    (torch.float16, 1, 3, 130, 40, True, 0.3),
    (torch.float32, 1, 2, 256, 64, True, 0.25),       # fp32 as three bf16 products
    (torch.float32, 2, 1, 97, 24, False, 0.1),
])
def test_dual_forward_and_backward_with_dropout(dev, dtype, B, H, N, D, causal, p):
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    seed = 1000 + N
    ts = make_inputs(B, H, N, D, dtype=dtype, seed=N, scale=0.5 if dtype == torch.bfloat16 else 1.0)
    q, k, v, tq, tk, tv, gO, gtO = [t.to(dev) for t in ts]
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, tq, tk, tv)]
    with fwAD.dual_level():
        out = JVPAttn.fwd_dual(*[fwAD.make_dual(leaves[i], leaves[i + 3]) for i in range(3)], causal=causal, dropout_p=p,
                               dropout_seed=seed)
        O, tO = fwAD.unpack_dual(out)
        grads = torch.autograd.grad((O * gO).sum() + (tO * gtO).sum(), leaves)
    torch.cuda.synchronize()
    _lib.read_status(dev)
    ref = closed_form_oracle(*ts, causal=causal, dropout_p=p, dropout_seed=seed)
    got = {"O": O.detach(), "tO": tO.detach(), **dict(zip(GRAD_NAMES, grads))}
    _compare({n: t.double().cpu() for n, t in got.items()}, ref, TOL[dtype])


def test_dropout_with_mask_primal_only_and_determinism(dev):
    from jvp_flash_attention_b200.jvp_attention import attention
    B, H, N, D, p = 2, 2, 192, 64, 0.3
    q, k, v, _, _, _, gO, _ = make_inputs(B, H, N, D, dtype=torch.float16, seed=4)
    mask = make_bool_mask(B, N, keep=0.7)
    leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    o = attention(*leaves, attn_mask=mask.to(dev), dropout_p=p, dropout_seed=5)
    grads = torch.autograd.grad((o * gO.to(dev)).sum(), leaves)
    z = torch.zeros_like(q)
    ref = closed_form_oracle(q, k, v, z, z, z, gO, z, attn_mask=mask, dropout_p=p, dropout_seed=5)
    got = {"O": o.detach().double().cpu(), **{n: g.double().cpu() for n, g in zip(("dq", "dk", "dv"), grads)}}
    _compare(got, ref, TOL[torch.float16], names=("O", "dq", "dk", "dv"))
    o2 = attention(*leaves, attn_mask=mask.to(dev), dropout_p=p, dropout_seed=5)
    o3 = attention(*leaves, attn_mask=mask.to(dev), dropout_p=p, dropout_seed=6)
    assert torch.equal(o, o2) and not torch.equal(o, o3)
    torch.manual_seed(11)
    a = attention(*leaves, dropout_p=p)              # seed drawn from torch's CPU generator
    torch.manual_seed(11)
    b = attention(*leaves, dropout_p=p)
    assert torch.equal(a, b)


def test_dropout_inside_torch_compile(dev):
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    ts = [t.to(dev) for t in make_inputs(1, 2, 128, 64, dtype=torch.bfloat16, seed=9, scale=0.5)]

    def fn(q, k, v, tq, tk, tv, go, gto):
        o, to = JVPAttn.dual(q, k, v, tq, tk, tv, causal=True, dropout_p=0.2, dropout_seed=77)
        return (o * go).sum() + (to * gto).sum(), o, to

    def run(f):
        leaves = [t.clone().requires_grad_(True) for t in ts[:6]]
        loss, o, to = f(*leaves, ts[6], ts[7])
        return o.detach(), to.detach(), torch.autograd.grad(loss, leaves)

    o1, t1, g1 = run(fn)
    o2, t2, g2 = run(torch.compile(fn, fullgraph=True))
    assert torch.equal(o1, o2) and torch.equal(t1, t2) and all(torch.equal(a, b) for a, b in zip(g1, g2))
