"""Edge cases of the CUDA path against the oracle: tiny and ragged sequences with masks, head dimensions on the padded
kernels, many small (batch, head) units, mask layouts (broadcast, strided, mask type different from the input type),
primal-only calls with masks, and long causal sequences through a prefix property."""
import math

import pytest
import torch

from oracle.jvp_attention_oracle import (GRAD_NAMES, closed_form_oracle, make_additive_mask, make_bool_mask, make_inputs)
from test_parity_gpu import TOL, _compare, _run_cuda          # helpers of the parity tests (same directory)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("N", [1, 2, 7, 33, 65, 129])
def test_tiny_sequences(dev, dtype, N):
    ts = make_inputs(2, 3, N, 64, dtype=dtype, seed=100 + N)
    for causal in (False, True):
        got = _run_cuda(ts, dev, causal=causal)
        _compare(got, closed_form_oracle(*ts, causal=causal), TOL[dtype])


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 8), (torch.float16, 24), (torch.bfloat16, 40), (torch.float16, 120),
                                     (torch.float32, 8), (torch.float32, 24), (torch.float32, 56)])
def test_head_dimensions_on_the_padded_kernels(dev, dtype, D):
    ts = make_inputs(1, 2, 160, D, dtype=dtype, seed=D, scale=0.5 if dtype == torch.bfloat16 else 1.0)
    got = _run_cuda(ts, dev, causal=True)
    _compare(got, closed_form_oracle(*ts, causal=True), TOL[dtype])


@pytest.mark.parametrize("kind", ["bool", "additive"])
@pytest.mark.parametrize("dtype,N", [(torch.bfloat16, 200), (torch.float16, 77), (torch.float32, 150)])
def test_masks_on_ragged_sequences(dev, dtype, N, kind):
    B, H, D = 2, 2, 64
    ts = make_inputs(B, H, N, D, dtype=dtype, seed=N, scale=0.5 if dtype == torch.bfloat16 else 1.0)
    mask = make_bool_mask(B, N, keep=0.7) if kind == "bool" else make_additive_mask(B, N, dtype=torch.float32)
    got = _run_cuda(ts, dev, attn_mask=mask)              # a float32 mask with 16-bit inputs, too
    _compare(got, closed_form_oracle(*ts, attn_mask=mask), TOL[dtype])


def test_mask_layouts(dev):
    """Masks broadcast over the batch only / the heads only, and a transposed (non-contiguous) mask."""
    B, H, N, D = 2, 3, 128, 64
    ts = make_inputs(B, H, N, D, dtype=torch.float16, seed=77)
    g = torch.Generator().manual_seed(5)
    base = torch.rand(B, H, N, N, generator=g) > 0.3
    base |= torch.eye(N, dtype=torch.bool)
    for mask in (base[:1], base[:, :1], base.transpose(-1, -2), base[:1, :1].expand(B, H, N, N)):
        got = _run_cuda(ts, dev, attn_mask=mask)
        _compare(got, closed_form_oracle(*ts, attn_mask=mask.expand(B, H, N, N)), TOL[torch.float16])


def test_many_small_units(dev):
    """301 (batch, head) units of one row tile each: the block order's last group is a partial one."""
    B, H, N, D = 7, 43, 96, 64
    ts = make_inputs(B, H, N, D, dtype=torch.float16, seed=301)
    got = _run_cuda(ts, dev, causal=True)
    slices = [(0, 0), (6, 42), (3, 17), (6, 40), (6, 41)]
    _compare(got, closed_form_oracle(*ts, causal=True, slices=slices), TOL[torch.float16], slices)


def test_primal_only_with_masks(dev):
    from jvp_flash_attention_b200.jvp_attention import attention
    B, H, N, D = 2, 2, 192, 128
    for dtype, mask in ((torch.bfloat16, make_bool_mask(B, N, keep=0.6)), (torch.float32, make_additive_mask(B, N, dtype=torch.float32))):
        q, k, v, _, _, _, gO, _ = make_inputs(B, H, N, 64 if dtype == torch.float32 else D, dtype=dtype, seed=8, scale=0.5)
        leaves = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
        o = attention(*leaves, attn_mask=mask.to(dev))
        grads = torch.autograd.grad((o * gO.to(dev)).sum(), leaves)
        z = torch.zeros_like(q)
        ref = closed_form_oracle(q, k, v, z, z, z, gO, z, attn_mask=mask)
        got = {"O": o.detach().double().cpu(), **{n: g.double().cpu() for n, g in zip(("dq", "dk", "dv"), grads)}}
        _compare(got, ref, TOL[dtype], names=("O", "dq", "dk", "dv"))


def test_long_causal_sequence_prefix_property(dev):
    """N = 16384, D = 128, causal: a query's outputs depend only on its prefix, and the kernels visit a row's key tiles
    in the same order whatever comes after, so the first 4096 rows of the long run equal the 4096-row run bit for bit;
    one (b, h) slice of the short run is checked against the oracle."""
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    B, H, N, D, P = 1, 2, 16384, 128, 4096
    g = torch.Generator(device=dev).manual_seed(3)
    q, k, v, tq, tk, tv = [torch.randn(B, H, N, D, device=dev, dtype=torch.float16, generator=g) for _ in range(6)]
    O, tO = JVPAttn.dual(q, k, v, tq, tk, tv, causal=True)
    Op, tOp = JVPAttn.dual(*[t[:, :, :P].contiguous() for t in (q, k, v, tq, tk, tv)], causal=True)
    torch.cuda.synchronize()
    _lib.read_status(dev)
    assert torch.isfinite(O).all() and torch.isfinite(tO).all()
    assert torch.equal(O[:, :, :P], Op) and torch.equal(tO[:, :, :P], tOp)
    cpu = [t[:, :1, :P].cpu() for t in (q, k, v, tq, tk, tv)]
    ref = closed_form_oracle(*cpu, causal=True)
    _compare({"O": Op[:, :1].double().cpu(), "tO": tOp[:, :1].double().cpu()}, ref, TOL[torch.float16], names=("O", "tO"))
