"""Multi-rank host logic on CPU: two gloo ranks shard the (batch, head) axis, each computes its slice
with the CPU oracle, and the gathered result equals the unsharded one; max-over-ranks timing reduces
as the benchmark does."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jvp_flash_attention_b200.sharding import shard_bh, shard_bounds


def test_shard_bounds_cover_everything():
    for units in (1, 7, 64, 128):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = shard_bounds(units, world, r)
                seen += list(range(lo, hi))
            assert seen == list(range(units))
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.jvp_attention_oracle import closed_form_oracle, make_inputs
    ts = make_inputs(2, 3, 32, 16, dtype=torch.float32, seed=1)
    mine = [shard_bh(t, world, rank) for t in ts]
    out = closed_form_oracle(*mine, causal=True)
    local = torch.from_numpy(np.concatenate([out["O"], out["dk"]], axis=-1)).float()   # (1, units, N, 2D)
    sizes = [shard_bounds(6, world, r) for r in range(world)]
    bufs = [torch.empty(1, hi - lo, 32, 32) for lo, hi in sizes]
    dist.all_gather(bufs, local) if len({b.shape for b in bufs}) == 1 else None
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        q.put((torch.cat(bufs, dim=1).numpy(), float(t)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_unsharded():
    from oracle.jvp_attention_oracle import closed_form_oracle, make_inputs
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, tmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ts = make_inputs(2, 3, 32, 16, dtype=torch.float32, seed=1)
    full = closed_form_oracle(*ts, causal=True)
    ref = np.concatenate([full["O"], full["dk"]], axis=-1).reshape(1, 6, 32, 32)
    assert np.abs(gathered - ref).max() < 1e-6
    assert tmax == 2.0
