#!/usr/bin/env python
"""Benchmark of the JVP attention hot path: dual forward + dual backward, in algorithmic TFLOP/s.

One "step" = one dual forward and one dual backward over one batch of synthetic inputs
(B=8, H=16, N=4096, D=128, causal; N(0,1) inputs, tangents and upstream gradients) per GPU.
Algorithmic FLOPs per step = 42 * B * H * N^2 * D / 2 (matmul FLOPs only, causal halved: 12 for the
dual forward, 30 for the backward; recomputed or padded work is not counted).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|fp16] [--impl reference]

N > 1 is launched with torch.distributed.run, one rank per GPU; every rank takes the same per-GPU
workload (weak scaling, independent (batch, head) units, no collective on the attention path), the
timed region is bracketed by a barrier and a device synchronize, the device time is reduced with MAX
over ranks, and rank 0 prints one JSON line.

``--impl reference`` times the reference's CPU-runnable path (SDPA-MATH + torch.func.jvp + autograd,
as in the reference's validator) on the host cores for the same metric and configuration, each step
a bounded sample of (batch, head) slices.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=8, H=16, N=4096, D=128, causal=True)
METRIC = "JVP fwd+bwd attention TFLOP/s/GPU & % tensor peak, N=4096 D=128, 1-8 GPUs"
NOMINAL_DENSE_TFLOPS = 2250.0


def algorithmic_flops(B, H, N, D, causal):
    f = B * H * N * N * D * (0.5 if causal else 1.0)
    return 12.0 * f, 30.0 * f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML on a background thread."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz, self._stop, self._thread, self.ok = None, threading.Event(), None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def _reason_names(self, mask: int):
        nv = self.nv
        table = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        return {name for name, bit in table.items() if mask & bit}

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                self.reasons |= self._reason_names(int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# ------------------------------------------------------------------------------------------------
def run_reference(args, rank):
    if rank != 0:
        return
    from oracle.jvp_attention_oracle import sdpa_jvp_oracle
    w = WORKLOAD
    slices = args.ref_slices
    g = torch.Generator().manual_seed(0)
    ts = [torch.randn(1, slices, w["N"], w["D"], generator=g) for _ in range(8)]
    fwd_f, bwd_f = algorithmic_flops(1, slices, w["N"], w["D"], w["causal"])
    for _ in range(args.warmup):
        sdpa_jvp_oracle(*ts, causal=w["causal"], dtype=torch.float32)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sdpa_jvp_oracle(*ts, causal=w["causal"], dtype=torch.float32)
    dt = time.perf_counter() - t0
    value = (fwd_f + bwd_f) * args.steps / dt / 1e12
    sample = (f"{slices} of {w['B'] * w['H']} (batch, head) slices per step, fp32, SDPA-MATH + torch.func.jvp + autograd "
              f"(six gradients through both outputs)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"dual fwd+bwd attention B={w['B']} H={w['H']} N={w['N']} D={w['D']} causal, CPU reference path",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# CUDA arm
# ------------------------------------------------------------------------------------------------
def run_cuda(args, rank, world, local_rank):
    import torch.distributed as dist
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # rank 0 prints exactly one JSON line on stdout: NCCL writes its version banner to file descriptor 1 from native
    # code, so everything else written to it during the run goes to stderr and the line goes to the saved descriptor
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = dict(WORKLOAD)
    if args.batch:
        w["B"] = args.batch
    B, H, N, D, causal = w["B"], w["H"], w["N"], w["D"], w["causal"]
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    s = D ** -0.5
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, tq, tk, tv, gO, gtO = [torch.randn(B, H, N, D, device=dev, dtype=dtype, generator=g) for _ in range(8)]
    mask_c = _lib.make_mask(None, B, H, N)
    fwd_f, bwd_f = algorithmic_flops(B, H, N, D, causal)
    step_f = fwd_f + bwd_f

    def step():
        o, to, lse2, mu = _lib.fwd(q, k, v, tq, tk, tv, mask_c, None, causal, s)
        return _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, gO, gtO, mask_c, None, causal, s)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        return ms

    # ---- device-resident timing (the `value`) ----
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.read_status(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    _lib.read_status(dev)
    ms_step = ms_total / args.steps
    value = step_f * world / (ms_step * 1e-3) / 1e12

    # ---- per-kernel durations, same steps, events on the launching stream ----
    _lib.kernel_timing(True)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    kt = _lib.kernel_timing(False)
    kernels = {name: {"ms_per_launch": (ms / n if n else None), "launches": n} for name, (ms, n) in kt.items()}
    bwd_names = ("bwd_q", "bwd_k", "bwd_v")
    bwd_ms = sum(kt[n][0] for n in bwd_names)
    bwd_launches = sum(kt[n][1] for n in bwd_names)
    peak_burst, peak_sustained, peak_kind = measured_peaks()
    # dominant kernel: the backward family kernel (one template, three launches per step); algorithmic FLOPs per
    # launch = a third of the backward's 30*B*H*N^2*D/2
    ach = (bwd_f / 3.0) / ((bwd_ms / max(bwd_launches, 1)) * 1e-3) / 1e12 if bwd_launches else None
    roofline = {"bound": "tensor", "kernel": "bwd_sm100_kernel (families Q, K, V)", "achieved": ach, "peak": peak_sustained,
                "unit": "TFLOP/s", "frac": (ach / peak_sustained if ach else None), "peak_kind": f"{peak_kind} sustained bf16 cuBLAS",
                # DRAM bytes per backward-family launch: ncu capture of the B=2 case (profiles/bwd_fwd_sm100_full_set_small.md:
                # 321.9 / 320.9 / 251.3 MB read+write for families Q / K / V), scaled by B/2 -- traffic grows with the
                # number of (batch, head) units, every unit's tensors are read from HBM once per launch
                "traffic": (321.9e6 + 320.9e6 + 251.3e6) / 3.0 * (B / 2.0), "traffic_unit": "bytes per launch",
                "fwd_kernel": {"achieved": fwd_f / (kt["fwd"][0] / max(kt["fwd"][1], 1) * 1e-3) / 1e12 if kt["fwd"][1] else None}}
    if roofline["fwd_kernel"]["achieved"]:
        roofline["fwd_kernel"]["frac"] = roofline["fwd_kernel"]["achieved"] / peak_sustained

    # ---- end to end through the public API with host buffers ----
    e2e = None
    if not args.no_e2e:
        host_in = [torch.empty(B, H, N, D, dtype=dtype).pin_memory() for _ in range(8)]
        for hbuf, src in zip(host_in, (q, k, v, tq, tk, tv, gO, gtO)):
            hbuf.copy_(src)
        host_out = [torch.empty(B, H, N, D, dtype=dtype).pin_memory() for _ in range(8)]
        # Three streams, inputs double-buffered on the device: the copy-in of step i+1 and the copy-out of step
        # i-1 overlap the kernels of step i, as a caller that streams batches through the public API would do.
        dev_in = [[torch.empty(B, H, N, D, dtype=dtype, device=dev) for _ in range(8)] for _ in range(2)]
        s_main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of this buffer set have arrived
        ev_free = [torch.cuda.Event() for _ in range(2)]   # kernels that read this buffer set are done
        ev_out = torch.cuda.Event()
        state = {"i": 0}

        def e2e_step():
            i = state["i"]
            cur = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_free[cur])
                for d_, h_ in zip(dev_in[cur], host_in):
                    d_.copy_(h_, non_blocking=True)
                ev_in[cur].record(s_in)
            s_main.wait_event(ev_in[cur])
            leaves = [t.detach().requires_grad_(True) for t in dev_in[cur][:6]]
            O, tO = JVPAttn.dual(*leaves, causal=causal, verify_attn_mask=False)
            grads = torch.autograd.grad([O, tO], leaves, [dev_in[cur][6], dev_in[cur][7]])
            ev_free[cur].record(s_main)
            results = (O.detach(), tO.detach(), *grads)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[cur])
                for h_, d_ in zip(host_out, results):
                    d_.record_stream(s_out)
                    h_.copy_(d_, non_blocking=True)
                ev_out.record(s_out)
            state["i"] = i + 1

        for _ in range(3):
            e2e_step()
        barrier()
        n_e2e = max(4, args.steps // 2)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        s_main.wait_event(ev_out)       # the last copy-out ends the timed region
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        nbytes = 8 * B * H * N * D * q.element_size()
        e2e = {"value": step_f * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e, "steps": n_e2e,
               "note": "JVPAttn.dual + autograd.grad; every step copies its 8 input tensors from pinned host memory and "
                       "O, tO and the six gradients back to pinned host memory inside the timed region; copies run on "
                       "their own streams and overlap the kernels of the neighbouring steps"}
        del host_in, host_out, dev_in

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle.jvp_attention_oracle import sdpa_jvp_oracle
        gcpu = torch.Generator().manual_seed(0)
        ts = [torch.randn(1, 1, N, D, generator=gcpu) for _ in range(8)]
        sdpa_jvp_oracle(*ts, causal=causal, dtype=torch.float32)  # warm-up
        done, t0 = 0, time.perf_counter()
        while done < 32 and (time.perf_counter() - t0 < 10.0 or done < 2):
            sdpa_jvp_oracle(*ts, causal=causal, dtype=torch.float32)
            done += 1
        dt = time.perf_counter() - t0
        f1, b1 = algorithmic_flops(1, 1, N, D, causal)
        cpu_baseline = {"value": (f1 + b1) * done / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                        "kind": "port", "sample": f"{done} (batch, head) slices of the workload, fp32, SDPA-MATH + "
                        "torch.func.jvp + autograd on the host cores", "seconds": dt}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"dual fwd+bwd attention, per GPU B={B} H={H} N={N} D={D} causal {args.dtype}, "
                                   "fully masked key tiles skipped; batch x head units sharded over GPUs, no collective",
                       "global_batch": B * world, "l2": "inputs larger than L2 (8 tensors of 134 MB per step)",
                       "flops_per_step_per_gpu": step_f},
            "per_gpu_tflops": value / world,
            "frac_of_nominal_dense_peak": value / world / NOMINAL_DENSE_TFLOPS,
            "frac_of_measured_peak": value / world / peak_burst,
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": 5 * args.steps, "clocks": clocks.summary(),
        }
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", choices=("bf16", "fp16"), default="bf16")
    ap.add_argument("--impl", choices=("cuda", "reference"), default="cuda")
    ap.add_argument("--ref-slices", type=int, default=2, help="(batch, head) slices per step of the reference arm")
    ap.add_argument("--batch", type=int, default=None, help="override B of the workload (small profiler captures only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nnodes=1 --nproc-per-node N "
                         "--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...")
    run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
