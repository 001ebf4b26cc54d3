"""GPU test of the end-to-end JVP training step (bench_dit.py) on a small model: with this library's attention
and with SDPA-MATH the step must give the same loss and the same parameter gradients (head dimension 72, i.e.
the zero-padded tensor-core path in bf16 and the CUDA-core path in fp32)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _grads(impl, dtype, dev):
    import bench_dit
    torch.manual_seed(0)
    model = bench_dit.DiT(depth=2, hidden=144, heads=2, impl=impl).to(dev, dtype)
    g = torch.Generator(device=dev).manual_seed(1)
    mk = lambda: torch.randn(2, 64, 32, device=dev, dtype=dtype, generator=g)
    x, tx, target, target_t = mk(), mk(), mk(), mk()
    t = torch.rand(2, device=dev, generator=g) * 1000
    out, tout = torch.func.jvp(lambda inp: model(inp, t), (x,), (tx,))
    loss = F.mse_loss(out.float(), target.float()) + F.mse_loss(tout.float(), target_t.float())
    loss.backward()
    return float(loss.detach()), {n: p.grad.float().clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("dtype,rel", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_dit_jvp_step_matches_sdpa(dtype, rel):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    loss_a, grads_a = _grads("jvpfa", dtype, dev)
    loss_b, grads_b = _grads("sdpa", dtype, dev)
    assert abs(loss_a - loss_b) <= rel * abs(loss_b)
    for name, ga in grads_a.items():
        gb = grads_b[name]
        err = float((ga - gb).norm() / (gb.norm() + 1e-12))
        assert err <= rel, (name, err)
    from jvp_flash_attention_b200 import _lib
    _lib.read_status(dev)
