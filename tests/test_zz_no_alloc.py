"""GPU test of jvpfa_bwd_noalloc, the backward entry point for callers that cannot allocate device
memory (a plug-in inside a process whose memory pool already owns the GPU's memory, or a
latency-critical path that must stay clear of cudaMalloc's device-wide synchronisation).

It is called through the C ABI twice in a row and must reproduce what the ordinary entry point
(jvpfa_bwd, with a caller-provided workspace) returns for the same inputs: the two run the same
kernels, so the results are required to agree within the tolerance of the other GPU tests (2e-2 for
16-bit inputs; in practice they are bit-identical). Collected last on purpose (file name), so that a
failure here cannot hide the other tests in a run that stops at the first failure.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bwd_args(_lib, tensors, outs, o, to, lse2, mu, causal, s):
    q, k, v, tq, tk, tv, go, gto = tensors
    B, H, N, D = q.shape
    a = _lib.BwdArgs()
    a.B, a.H, a.N, a.D = B, H, N, D
    a.dtype, a.causal, a.sm_scale = _lib.dtype_code(q.dtype), int(causal), float(s)
    a.mask = _lib.make_mask(None, B, H, N)
    a.mask_summary = None
    a.q, a.k, a.v, a.tq, a.tk, a.tv = (t.data_ptr() for t in (q, k, v, tq, tk, tv))
    a.o, a.to, a.lse2, a.mu = o.data_ptr(), to.data_ptr(), lse2.data_ptr(), mu.data_ptr()
    a.go, a.gto = go.data_ptr(), gto.data_ptr()
    a.dq, a.dk, a.dv, a.dtq, a.dtk, a.dtv = (t.data_ptr() for t in outs)
    a.workspace, a.workspace_bytes = None, 0      # ignored by the allocation-free entry point
    return a


@pytest.mark.parametrize("dtype,B,H,N,D,causal", [
    (torch.bfloat16, 2, 4, 1024, 128, True),     # tensor-core kernels
    (torch.float32, 1, 2, 200, 64, False),       # CUDA-core kernels
])
def test_noalloc_backward_matches_ordinary_entry_point(dtype, B, H, N, D, causal):
    from jvp_flash_attention_b200 import _lib
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    L = _lib.lib()
    g = torch.Generator(device=dev).manual_seed(17)
    tensors = [torch.randn(B, H, N, D, device=dev, dtype=dtype, generator=g) * 0.5 for _ in range(8)]
    q, k, v, tq, tk, tv, go, gto = tensors
    s = 1.0 / math.sqrt(D)
    mask_c = _lib.make_mask(None, B, H, N)
    o, to, lse2, mu = _lib.fwd(q, k, v, tq, tk, tv, mask_c, None, causal, s)
    want = _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, go, gto, mask_c, None, causal, s)
    torch.cuda.synchronize()
    _lib.read_status(dev)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    stream = _lib.stream_ptr(dev)
    status = torch.full((1,), -1, dtype=torch.int32, device=dev)
    for call in range(2):                            # two calls in a row share the one scratch array
        outs = [torch.full_like(q, float("nan")) for _ in range(6)]
        a = _bwd_args(_lib, tensors, outs, o, to, lse2, mu, causal, s)
        rc = L.jvpfa_bwd_noalloc(C.byref(a), C.c_void_p(status.data_ptr()), stream)
        assert rc == _lib.OK, L.jvpfa_error_string(rc)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a device-side wait gave up"
        for name, got, ref in zip(("dq", "dk", "dv", "dtq", "dtk", "dtv"), outs, want):
            assert torch.isfinite(got).all(), (call, name)
            err = float((got.float() - ref.float()).abs().max())
            assert err <= tol, (call, name, err)


def test_noalloc_rejects_problems_beyond_its_scratch():
    from jvp_flash_attention_b200 import _lib
    L = _lib.lib()
    a = _lib.BwdArgs()
    a.B, a.H, a.N, a.D, a.dtype = 8, 16, 4096, 128, _lib.BF16      # 524288 rows > 262144
    assert L.jvpfa_bwd_noalloc(C.byref(a), None, None) == _lib.ERR_NO_ALLOC_LIMIT
    assert L.jvpfa_bwd_noalloc(None, None, None) == _lib.ERR_BAD_ARG
