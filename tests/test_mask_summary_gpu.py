"""The mask summary pre-pass (``jvpfa_mask_summary``): per 64x64 tile the "anything kept" / "anything that needs the mask"
flags, and for boolean masks the mask packed into 64-bit words by query row and by key row. Checked against torch for
contiguous, broadcast, transposed and ragged masks (the contiguous ones take the direct-load kernel, the others the
generic one). No reference counterpart: the reference reads the mask element-wise in every tile
(jvp_attention.py:250-262)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def _pack64(x):
    """x [..., 64] bool -> int64 words with bit c = x[..., c]."""
    w = 1 << torch.arange(63, device=x.device, dtype=torch.int64)
    lo = (x[..., :63].to(torch.int64) * w).sum(-1)
    return lo + torch.where(x[..., 63], torch.tensor(-2 ** 63, device=x.device), torch.tensor(0, device=x.device))


def _expected(kept, masked, N):
    """kept / masked: [planes, N, N] bool. Returns flags [planes, n64, n64], row words [planes, n64, n_pad], column words."""
    planes = kept.shape[0]
    n64 = (N + 63) // 64
    n_pad = 64 * n64
    kp = torch.zeros(planes, n_pad, n_pad, dtype=torch.bool, device=kept.device)
    mp = torch.zeros_like(kp)
    kp[:, :N, :N] = kept
    mp[:, :N, :N] = masked
    t = lambda x: x.view(planes, n64, 64, n64, 64)
    flags = t(kp).any(4).any(2).to(torch.uint8) + 2 * t(mp).any(4).any(2).to(torch.uint8)
    rows = _pack64(kp.view(planes, n_pad, n64, 64)).permute(0, 2, 1).contiguous()          # [plane][key tile][query]
    cols = _pack64(kp.view(planes, n64, 64, n_pad).permute(0, 1, 3, 2)).contiguous()        # [plane][query tile][key]
    return flags, rows, cols


@pytest.mark.parametrize("B,H,N,layout", [
    (2, 1, 192, "head_broadcast"),
    (1, 2, 64, "full"),
    (2, 3, 130, "full"),            # rows of 130 bytes: not 16-byte aligned, generic kernel
    (1, 2, 208, "full"),            # 16-byte aligned rows, ragged last tile
    (1, 1, 1100, "batch_head_broadcast"),
    (2, 2, 256, "transposed"),
    (1, 2, 2048, "full"),
])
def test_boolean_mask_summary_matches_torch(dev, B, H, N, layout):
    from jvp_flash_attention_b200 import _lib
    g = torch.Generator(device=dev).manual_seed(N)
    Bm = 1 if layout == "batch_head_broadcast" else B
    Hm = 1 if layout in ("head_broadcast", "batch_head_broadcast") else H
    m = torch.rand(Bm, Hm, N, N, device=dev, generator=g) > 0.6
    m[..., : min(N, 64), : min(N, 64)] = True                     # one tile that needs no mask
    if N > 128:
        m[..., 64:128, :64] = False                               # one tile with nothing kept
    given = m.transpose(-1, -2).contiguous().transpose(-1, -2) if layout == "transposed" else m
    mc = _lib.make_mask(given, B, H, N)
    out = _lib.mask_summary(mc, given, B, H, N)
    torch.cuda.synchronize()
    planes, n64 = Bm * Hm, (N + 63) // 64
    n_pad = 64 * n64
    fb = (planes * n64 * n64 + 255) // 256 * 256
    bb = planes * n64 * n_pad * 8
    assert out.numel() == fb + 2 * bb + planes * n64 * n64 * 4
    flags = out[: planes * n64 * n64].view(planes, n64, n64)
    rows = out[fb: fb + bb].view(torch.int64).view(planes, n64, n_pad)
    cols = out[fb + bb: fb + 2 * bb].view(torch.int64).view(planes, n64, n_pad)
    mm = m.reshape(planes, N, N)
    want_flags, want_rows, want_cols = _expected(mm, ~mm, N)
    assert torch.equal(flags, want_flags)
    assert torch.equal(rows, want_rows)
    assert torch.equal(cols, want_cols)


@pytest.mark.parametrize("N", [200, 130, 1024])     # 130: rows that are not 16-byte multiples take the generic kernel
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_additive_mask_summary_flags(dev, dtype, N):
    from jvp_flash_attention_b200 import _lib
    B, H = 1, 2
    g = torch.Generator(device=dev).manual_seed(3)
    r = torch.rand(B, H, N, N, device=dev, generator=g)
    m = torch.where(r > 0.5, 0.0, -100.0)
    m = torch.where(r > 0.9, float("-inf"), m).to(dtype)
    m[..., :64, :64] = 0.0                                          # needs no mask
    m[..., 64:128, :64] = float("-inf")                             # nothing kept
    m[..., :64, 64:128] = -0.0                                      # negative zero is zero
    mc = _lib.make_mask(m, B, H, N)
    out = _lib.mask_summary(mc, m, B, H, N)
    torch.cuda.synchronize()
    planes, n64 = B * H, (N + 63) // 64
    flags = out[: planes * n64 * n64].view(planes, n64, n64)
    mm = m.reshape(planes, N, N).float()
    want_flags, _, _ = _expected(mm != float("-inf"), mm != 0, N)
    assert torch.equal(flags & 3, want_flags)      # (bit 2 marks two-valued tiles of contiguous masks)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_additive_two_valued_tiles(dev, dtype):
    """Contiguous additive masks: the bit words mark the +-0 entries, and a tile whose other entries all carry one value is
    flagged two-valued (bit 2) with that value in the tile values; a tile with two different biases is not."""
    from jvp_flash_attention_b200 import _lib
    B, H, N = 1, 2, 256
    g = torch.Generator(device=dev).manual_seed(8)
    r = torch.rand(B, H, N, N, device=dev, generator=g)
    m = torch.where(r > 0.7, 0.0, -100.0)
    m[..., :64, 64:128] = torch.where(r[..., :64, 64:128] > 0.5, 0.0, float("-inf"))   # 0 / -inf
    m[..., 64:128, 64:128] = torch.where(r[..., 64:128, 64:128] > 0.5, -1.0, -2.0)       # two biases, no zeros
    m[..., 128:192, :64] = torch.where(r[..., 128:192, :64] > 0.5, 0.0, -3.5)
    m[..., 128, 5] = -7.0                                                                # a third value
    m = m.to(dtype)
    mc = _lib.make_mask(m, B, H, N)
    out = _lib.mask_summary(mc, m, B, H, N)
    torch.cuda.synchronize()
    planes, n64 = B * H, N // 64
    fb = (planes * n64 * n64 + 255) // 256 * 256
    bb = planes * n64 * N * 8
    flags = out[: planes * n64 * n64].view(planes, n64, n64)
    rows = out[fb: fb + bb].view(torch.int64).view(planes, n64, N)
    cols = out[fb + bb: fb + 2 * bb].view(torch.int64).view(planes, n64, N)
    vals = out[fb + 2 * bb: fb + 2 * bb + planes * n64 * n64 * 4].view(torch.float32).view(planes, n64, n64)
    mm = m.reshape(planes, N, N).float()
    _, want_rows, want_cols = _expected(mm == 0, mm != 0, N)
    assert torch.equal(rows, want_rows) and torch.equal(cols, want_cols)
    two = (flags & 4) != 0
    assert two[:, 0, 0].all() and vals[:, 0, 0].eq(-100.0).all()
    assert two[:, 0, 1].all() and torch.isinf(vals[:, 0, 1]).all() and (flags[:, 0, 1] & 3).eq(3).all()
    assert not two[:, 1, 1].any()
    assert not two[:, 2, 0].any()
    assert two[:, 3, 3].all() and vals[:, 3, 3].eq(-100.0).all()
