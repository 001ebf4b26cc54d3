"""Failure detection on the GPU: a bounded device-side wait that runs out must surface as a Python exception.

No GPU is faulted, trapped or hung: the library's self-test kernel waits on a barrier that nothing arrives on with a
budget of two milliseconds, gives up, records the wait's id in the status word and returns normally.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def test_wait_that_runs_out_is_reported_once(dev):
    from jvp_flash_attention_b200 import _lib, check
    check(dev)                                              # clean start
    out = _lib.selftest_timeout(dev, budget_us=2000)
    torch.cuda.synchronize()
    first, second, us_first, us_second = out.tolist()
    assert first == 0 and second == 0                       # both waits gave up
    assert 1500 <= us_first <= 200000                       # the first one after its budget ...
    assert us_second < us_first and us_second <= 1000       # ... the second one on the short path of a failed CTA
    with pytest.raises(_lib.JvpfaError) as err:
        check(dev)
    assert err.value.status == _lib.ERR_DEVICE_TIMEOUT and "wait id 177" in str(err.value)
    check(dev)                                              # reported once, then clear


def test_next_call_on_the_stream_raises_without_synchronising(dev):
    from jvp_flash_attention_b200 import _lib, attention, check
    check(dev)
    q = torch.randn(1, 2, 128, 64, device=dev, dtype=torch.bfloat16)
    attention(q, q, q)                                      # makes sure the stream has a workspace
    _lib.selftest_timeout(dev, budget_us=2000)
    torch.cuda.synchronize()                                # the status copy has landed in pinned host memory
    with pytest.raises(_lib.JvpfaError) as err:
        attention(q, q, q)
    assert err.value.status == _lib.ERR_DEVICE_TIMEOUT
    o = attention(q, q, q)                                  # the error was consumed: the library works again
    torch.cuda.synchronize()
    check(dev)
    assert torch.isfinite(o).all()


def test_streams_have_their_own_workspace(dev):
    """Two backward calls on different streams must not share scratch (the per-row statistics live in it)."""
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    g = torch.Generator(device=dev).manual_seed(5)
    sets = [[torch.randn(2, 4, 512, 64, device=dev, dtype=torch.bfloat16, generator=g) * 0.5 for _ in range(8)]
            for _ in range(2)]

    def run(ts):
        leaves = [t.clone().requires_grad_(True) for t in ts[:6]]
        O, tO = JVPAttn.dual(*leaves, causal=True)
        return torch.autograd.grad([O, tO], leaves, [ts[6], ts[7]])

    ref = [run(ts) for ts in sets]                          # one after the other on the default stream
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(dev) for _ in range(2)]
    got = [None, None]
    for _ in range(3):                                      # interleaved on two streams
        for i, st in enumerate(streams):
            st.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(st):
                got[i] = run(sets[i])
    torch.cuda.synchronize()
    assert len({k[1] for k in _lib._workspaces if k[0] == dev.index}) >= 3
    for r, g_ in zip(ref, got):
        assert all(torch.equal(a, b) for a, b in zip(r, g_))
    _lib.read_status(dev)
