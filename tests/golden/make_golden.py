"""Writes the golden fixtures of this folder. Run once in a container that holds the reference
checkout (its path in the REFERENCE_ROOT environment variable); the fixtures travel, the reference does not.

reference_interp_*.npz
    Inputs and outputs of the reference's own Triton kernels (jvp_flash_attention/jvp_attention.py,
    pointer variant) executed by the Triton CPU interpreter (TRITON_INTERPRET=1) on fp32
    (1, 2, 64, 32) tensors: O, tO from ``JVPAttn.fwd_dual`` under ``fwAD.dual_level`` and dq, dk, dv
    of ``sum(O * gO)`` (the reference has no gradient through tO). Cases: no mask, causal, boolean mask.
sdpa_cfg1.npz
    The primary oracle (SDPA-MATH + torch.func.jvp + autograd, fp64) on the CPU reference
    configuration fp32 B=2 H=4 N=128 D=64, seed 42: O, tO and the six gradients, every 5th row.
"""
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(os.environ["REFERENCE_ROOT"])
sys.path.insert(0, str(REPO))

import numpy as np
import torch
import torch.autograd.forward_ad as fwAD

from oracle.jvp_attention_oracle import make_inputs, sdpa_jvp_oracle


def reference_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_jvp_attention", REF / "jvp_flash_attention" / "jvp_attention.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    B, H, N, D = 1, 2, 64, 32
    q, k, v, tq, tk, tv, gO, gtO = make_inputs(B, H, N, D, dtype=torch.float32, seed=7)
    g = torch.Generator().manual_seed(1042)
    bm = (torch.rand(B, H, N, N, generator=g) < 0.7) | torch.eye(N, dtype=torch.bool)
    for name, kw in (("none", {}), ("causal", {"causal": True}), ("bool", {"attn_mask": bm})):
        with fwAD.dual_level():
            qd, kd, vd = [fwAD.make_dual(a.clone(), b.clone()) for a, b in ((q, tq), (k, tk), (v, tv))]
            for t in (qd, kd, vd):
                t.requires_grad_(True)
            out = ref.JVPAttn.fwd_dual(qd, kd, vd, **kw)
            O, tO = fwAD.unpack_dual(out)
            (O * gO).sum().backward()
            arrays = dict(q=q, k=k, v=v, tq=tq, tk=tk, tv=tv, gO=gO, O=O.detach(), tO=tO.detach(), dq=qd.grad,
                          dk=kd.grad, dv=vd.grad)
        if "attn_mask" in kw:
            arrays["mask"] = bm
        np.savez_compressed(HERE / f"reference_interp_{name}.npz", **{n: t.numpy() for n, t in arrays.items()})
        print("wrote", name)


def sdpa_cfg1():
    ts = make_inputs(2, 4, 128, 64, dtype=torch.float32, seed=42)
    out = sdpa_jvp_oracle(*ts)
    sub = {n: t[:, :, ::5, :].numpy().astype(np.float32) for n, t in out.items()}
    sub["input_checksum"] = np.array([float(sum(t.double().sum() for t in ts)), float(sum((t.double() ** 2).sum() for t in ts))])
    np.savez_compressed(HERE / "sdpa_cfg1.npz", **sub)
    print("wrote sdpa_cfg1")


if __name__ == "__main__":
    sdpa_cfg1()
    reference_cases()
