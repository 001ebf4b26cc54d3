"""CPU tests of the oracle: the closed-form restatement against the SDPA-MATH + torch.func.jvp
construction of the reference's validator, and both against the committed golden vectors."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle.jvp_attention_oracle import (GRAD_NAMES, closed_form_oracle, make_additive_mask, make_block_sparse_mask,
                                         make_bool_mask, make_inputs, sdpa_jvp_oracle)

GOLDEN = Path(__file__).resolve().parent / "golden"


def _cases():
    B, N = 2, 256
    return {
        "none": {},
        "causal": {"causal": True},
        "bool": {"attn_mask": make_bool_mask(B, N)},
        "block_sparse": {"attn_mask": make_block_sparse_mask(B, N, block=128)},
        "additive_inf": {"attn_mask": make_additive_mask(B, N, dtype=torch.float64)},
    }


@pytest.mark.parametrize("case", ["none", "causal", "bool", "block_sparse", "additive_inf"])
def test_closed_form_matches_sdpa_oracle(case):
    kw = _cases()[case]
    ts = [t.double() for t in make_inputs(2, 3, 256, 32, dtype=torch.bfloat16, seed=3)]
    ref = sdpa_jvp_oracle(*ts, **kw)
    got = closed_form_oracle(*ts, **kw)
    for name in ("O", "tO") + GRAD_NAMES:
        err = np.abs(got[name] - ref[name].numpy()).max()
        assert np.isfinite(got[name]).all()
        assert err < 1e-11, (case, name, err)


def test_closed_form_slices_and_scale():
    ts = [t.double() for t in make_inputs(2, 2, 64, 16, seed=5)]
    full = closed_form_oracle(*ts, causal=True, sm_scale=0.3)
    part = closed_form_oracle(*ts, causal=True, sm_scale=0.3, slices=[(1, 0), (0, 1)])
    ref = sdpa_jvp_oracle(*ts, causal=True, sm_scale=0.3)
    for name in ("O", "tO") + GRAD_NAMES:
        assert np.allclose(part[name][0], full[name][1, 0]) and np.allclose(part[name][1], full[name][0, 1])
        assert np.abs(full[name] - ref[name].numpy()).max() < 1e-11


def test_fully_masked_rows_give_zero():
    ts = [t.double() for t in make_inputs(1, 1, 32, 16, seed=9)]
    mask = torch.ones(1, 1, 32, 32, dtype=torch.bool)
    mask[0, 0, 5, :] = False
    out = closed_form_oracle(*ts, attn_mask=mask)
    assert np.all(out["O"][0, 0, 5] == 0) and np.all(out["tO"][0, 0, 5] == 0) and np.all(out["dq"][0, 0, 5] == 0)
    assert out["lse"][0, 0, 5] == -np.inf
    assert all(np.isfinite(out[n]).all() for n in ("O", "tO") + GRAD_NAMES)


def test_golden_sdpa_cfg1():
    """The CPU reference configuration (fp32 B=2 H=4 N=128 D=64, seed 42) against the stored outputs."""
    g = np.load(GOLDEN / "sdpa_cfg1.npz")
    ts = make_inputs(2, 4, 128, 64, dtype=torch.float32, seed=42)
    chk = np.array([float(sum(t.double().sum() for t in ts)), float(sum((t.double() ** 2).sum() for t in ts))])
    assert np.allclose(chk, g["input_checksum"], rtol=1e-12), "seeded inputs differ from the ones the fixture was made from"
    got = closed_form_oracle(*ts)
    for name in ("O", "tO") + GRAD_NAMES:
        err = np.abs(got[name][:, :, ::5, :] - g[name]).max()
        assert err < 5e-6, (name, err)   # fixture stored as fp32


@pytest.mark.parametrize("case", ["none", "causal", "bool"])
def test_golden_reference_interpreter(case):
    """Outputs of the reference's own kernels (Triton CPU interpreter, fp32 with fp32 products)."""
    g = np.load(GOLDEN / f"reference_interp_{case}.npz")
    ts = [torch.from_numpy(g[n]) for n in ("q", "k", "v", "tq", "tk", "tv", "gO")]
    kw = {}
    if case == "causal":
        kw["causal"] = True
    if case == "bool":
        kw["attn_mask"] = torch.from_numpy(g["mask"])
    got = closed_form_oracle(*ts, gtO=torch.zeros_like(ts[0]), **kw)
    for name in ("O", "tO", "dq", "dk", "dv"):
        err = np.abs(got[name] - g[name]).max()
        assert err < 2e-5, (case, name, err)
