#!/usr/bin/env python
"""End-to-end JVP training step of a random-init diffusion transformer that uses this library's attention.

The fifth benchmark configuration: 28 blocks, hidden 1152, 16 heads (head dimension 72), MLP ratio 4, 256 tokens
per sample, LayerNorm + adaLN-Zero conditioning, bf16; global batch 256 split data-parallel (32 per GPU at 8 GPUs);
one step = ``torch.func.jvp`` of the model with respect to its N(0,1) input along an N(0,1) tangent, an MSE loss on
the primal and on the tangent output, backward, gradient all-reduce with NCCL, AdamW update. The model is not part
of the reference (its README only shows loss curves); attention goes through ``JVPAttn.fwd_dual`` exactly as the
reference's README tells its users to call it inside ``torch.func.jvp``.

    python bench_dit.py [--gpus N] [--steps K] [--warmup W] [--depth 28] [--hidden 1152] [--heads 16] [--tokens 256]
                        [--per-gpu-batch 32] [--attention jvpfa|sdpa]

``--attention sdpa`` swaps in ``F.scaled_dot_product_attention`` forced to the MATH backend (the reference's own
comparison point) for an A/B on the same box. N > 1: launch with ``python -m torch.distributed.run``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def modulate(x, shift, scale):
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class LayerNorm(nn.Module):
    """LayerNorm without affine parameters, written out in elementary ops: under forward-mode AD on CUDA the fused
    bf16 ``F.layer_norm`` hands back a float32 result, which the following bf16 linear layer rejects."""

    def __init__(self, eps=1e-6):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        mean = xf.mean(dim=-1, keepdim=True)
        var = xf.var(dim=-1, unbiased=False, keepdim=True)
        return ((xf - mean) * torch.rsqrt(var + self.eps)).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, hidden, heads, impl):
        super().__init__()
        self.heads, self.impl = heads, impl
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.proj = nn.Linear(hidden, hidden)

    def forward(self, x):
        B, N, C = x.shape
        qkv = self.qkv(x).reshape(B, N, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        q, k, v = qkv[0], qkv[1], qkv[2]        # strided views of the fused projection; the kernels read them in place
        if self.impl == "jvpfa":
            from jvp_flash_attention_b200.jvp_attention import JVPAttn
            o = JVPAttn.fwd_dual(q, k, v, verify_attn_mask=False)
        else:
            from torch.nn.attention import SDPBackend, sdpa_kernel
            with sdpa_kernel(SDPBackend.MATH):
                o = F.scaled_dot_product_attention(q, k, v)
        return self.proj(o.transpose(1, 2).reshape(B, N, C))


class Block(nn.Module):
    def __init__(self, hidden, heads, mlp_ratio, impl):
        super().__init__()
        self.norm1 = LayerNorm()
        self.attn = Attention(hidden, heads, impl)
        self.norm2 = LayerNorm()
        self.fc1 = nn.Linear(hidden, mlp_ratio * hidden)
        self.fc2 = nn.Linear(mlp_ratio * hidden, hidden)
        self.ada = nn.Linear(hidden, 6 * hidden)

    def forward(self, x, c):
        sa, ca, ga, sm, cm, gm = self.ada(F.silu(c)).chunk(6, dim=1)
        x = x + ga.unsqueeze(1) * self.attn(modulate(self.norm1(x), sa, ca))
        h = self.fc2(F.gelu(self.fc1(modulate(self.norm2(x), sm, cm)), approximate="tanh"))
        return x + gm.unsqueeze(1) * h


class DiT(nn.Module):
    def __init__(self, depth=28, hidden=1152, heads=16, mlp_ratio=4, in_dim=32, impl="jvpfa"):
        super().__init__()
        self.embed = nn.Linear(in_dim, hidden)
        self.t_embed = nn.Sequential(nn.Linear(256, hidden), nn.SiLU(), nn.Linear(hidden, hidden))
        self.blocks = nn.ModuleList([Block(hidden, heads, mlp_ratio, impl) for _ in range(depth)])
        self.norm = LayerNorm()
        self.ada = nn.Linear(hidden, 2 * hidden)
        self.head = nn.Linear(hidden, in_dim)

    @staticmethod
    def timestep_embedding(t, dim=256):
        half = dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
        args = t.float()[:, None] * freqs[None]
        return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)

    def forward(self, x, t):
        c = self.t_embed(self.timestep_embedding(t).to(x.dtype))
        x = self.embed(x)
        for blk in self.blocks:
            x = blk(x, c)
        shift, scale = self.ada(F.silu(c)).chunk(2, dim=1)
        return self.head(modulate(self.norm(x), shift, scale))


def jvp_training_step(model, opt, x, tx, t, target, target_t, world):
    """One step: JVP forward, MSE on primal + tangent, backward, gradient all-reduce, optimizer update."""
    out, tout = torch.func.jvp(lambda inp: model(inp, t), (x,), (tx,))
    loss = F.mse_loss(out.float(), target.float()) + F.mse_loss(tout.float(), target_t.float())
    opt.zero_grad(set_to_none=True)
    loss.backward()
    if world > 1:
        import torch.distributed as dist
        grads = [p.grad for p in model.parameters() if p.grad is not None]
        flat = torch._utils._flatten_dense_tensors(grads)
        dist.all_reduce(flat)
        flat.div_(world)
        for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
            g.copy_(f)
    opt.step()
    return loss.detach()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--depth", type=int, default=28)
    ap.add_argument("--hidden", type=int, default=1152)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--per-gpu-batch", type=int, default=32)
    ap.add_argument("--attention", choices=("jvpfa", "sdpa"), default="jvpfa")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # one JSON line on stdout: NCCL prints its version banner to file descriptor 1 from native code
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)                      # same initial weights on every rank
    model = DiT(args.depth, args.hidden, args.heads, impl=args.attention).to(dev, torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    B, N = args.per_gpu_batch, args.tokens
    mk = lambda *s: torch.randn(*s, device=dev, dtype=torch.bfloat16, generator=g)
    x, tx, target, target_t = mk(B, N, 32), mk(B, N, 32), mk(B, N, 32), mk(B, N, 32)
    t = torch.rand(B, device=dev, generator=g) * 1000

    def sync():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        loss = jvp_training_step(model, opt, x, tx, t, target, target_t, world)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = jvp_training_step(model, opt, x, tx, t, target, target_t, world)
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        tms = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(tms, op=torch.distributed.ReduceOp.MAX)
        ms = float(tms)
    if args.attention == "jvpfa":
        from jvp_flash_attention_b200 import _lib
        _lib.read_status(dev)
    if rank == 0:
        n_params = sum(p.numel() for p in model.parameters())
        os.write(json_fd, (json.dumps({
            "metric": "DiT JVP training step, samples/s", "value": B * world / (ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "dtype": "bf16", "data": "synthetic", "loss": float(loss),
            "config": {"workload": f"DiT depth={args.depth} hidden={args.hidden} heads={args.heads} "
                                   f"(head dim {args.hidden // args.heads}) tokens={N}, torch.func.jvp + MSE on primal and "
                                   "tangent + backward + NCCL all-reduce + AdamW", "attention": args.attention,
                       "global_batch": B * world, "parameters": n_params}}) + "\n").encode())
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
