#!/usr/bin/env python
"""Benchmark of the JVP attention hot path: dual forward + dual backward, in algorithmic TFLOP/s.

One "step" = one dual forward and one dual backward over the whole problem B=8, H=16, N=4096, D=128, causal
(N(0,1) inputs, tangents and upstream gradients). Algorithmic FLOPs per step = 42 * B * H * N^2 * D / 2 (matmul
FLOPs only, causal halved: 12 for the dual forward, 30 for the backward; recomputed or padded work is not counted).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype bf16|fp16] [--impl reference]

N > 1 is launched with torch.distributed.run, one rank per GPU. The 128 (batch, head) units of the one problem are
independent, so they are sliced over the ranks (16 per GPU at N = 8; strong scaling, no collective on the attention
path); the timed region is bracketed by a barrier and a device synchronize, the device time is reduced with MAX over
ranks, `value` = the whole problem's FLOPs over that time, and rank 0 prints one JSON line. The same line carries a
`weak` record (every rank runs the full problem, as a fixed per-GPU workload) and an `fp16` record.

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
        self.index, self.period, self.samples, self.reasons, self.power = index, period_s, [], set(), []
        self.max_mhz, self._stop, self._thread, self.ok = None, threading.Event(), None, False
        self.in_kernel_mhz = None
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
                self.power.append(self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable",
                    "sm_mhz_in_kernel": self.in_kernel_mhz}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "power_w_median": statistics.median(self.power) if self.power else None,
                "power_w_max": max(self.power) if self.power else None,
                # cycles per microsecond counted on an SM beside the timed kernels (NVML's figure is sampled between them)
                "sm_mhz_in_kernel": self.in_kernel_mhz}


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
def host_threads(requested):
    """Threads of the CPU arm: all host cores unless told otherwise (torch.distributed.run exports OMP_NUM_THREADS=1,
    which would otherwise leave the CPU arm on one core)."""
    n = requested if requested and requested > 0 else (os.cpu_count() or 1)
    torch.set_num_threads(n)
    return torch.get_num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle.jvp_attention_oracle import sdpa_jvp_oracle
    cores = host_threads(args.ref_threads)
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
              f"(six gradients through both outputs), {cores} host threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"dual fwd+bwd attention B={w['B']} H={w['H']} N={w['N']} D={w['D']} causal, CPU reference path",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU incumbent: the reference's own Triton kernels on this GPU (a child process, so that a failure there cannot
# take the benchmark down). Reads the copy of the reference package under baseline/_ref.
# ------------------------------------------------------------------------------------------------
INCUMBENT_SHAPES = (
    # name, dtype (None = the benchmark's), B, H, N, D, causal, mask   (the reference's published tables: B=2 H=12 N=2048
    # D=64, masks of shape (B,H,N,N) with 10 % of the entries kept, tests/test_jvp_attention.py:309-394)
    ("readme_shape_bf16", "bf16", 2, 12, 2048, 64, False, None),
    ("readme_shape_fp16", "fp16", 2, 12, 2048, 64, False, None),
    ("readme_shape_fp32", "fp32", 2, 12, 2048, 64, False, None),
    ("readme_shape_bf16_causal", "bf16", 2, 12, 2048, 64, True, None),
    ("readme_shape_bf16_boolean_mask", "bf16", 2, 12, 2048, 64, False, "boolean"),
    ("readme_shape_bf16_additive_mask", "bf16", 2, 12, 2048, 64, False, "additive"),
    ("headline_shape", None, 8, 16, 4096, 128, True, None),
)


def _time_ms(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _peak_mb(fn):
    """Device memory one call allocates beyond what is held before it (outputs included), as the reference's benchmark
    reports it (tests/test_jvp_attention.py:116-143), in MB."""
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    out = fn()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated()
    del out
    return (peak - before) / 1e6


def run_incumbent_child(args):
    """Child process: times the reference's dual forward (JVPAttn.fwd_dual under fwAD.dual_level) and its primal-only
    backward through its stock code path, and this library's kernels on the same shapes; prints one JSON object."""
    import torch.autograd.forward_ad as fwAD
    out = {"shapes": {}}
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "jvp_flash_attention")):
        print(json.dumps({"unavailable": "reference-on-B200: unavailable (no copy of the reference under baseline/_ref)"}))
        return
    sys.path.insert(0, ref_dir)
    try:
        from jvp_flash_attention.jvp_attention import JVPAttn as RefAttn
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"unavailable": f"reference-on-B200: unavailable (import failed: {type(exc).__name__}: {exc})"[:400]}))
        return
    from jvp_flash_attention_b200 import _lib
    dev = torch.device("cuda", 0)
    dtypes = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
    only = set(args.incumbent_shapes.split(",")) if args.incumbent_shapes else None
    for name, dt_name, B, H, N, D, causal, mask_kind in INCUMBENT_SHAPES:
        if only is not None and name not in only:
            continue
        dt_name = dt_name or args.dtype
        dtype = dtypes[dt_name]
        rec = {"B": B, "H": H, "N": N, "D": D, "causal": causal, "dtype": dt_name, "mask": mask_kind}
        g = torch.Generator(device=dev).manual_seed(7)
        q, k, v, tq, tk, tv, go = [torch.randn(B, H, N, D, device=dev, dtype=dtype, generator=g) for _ in range(7)]
        mask = None
        if mask_kind is not None:   # the reference benchmark's masks: every entry kept with probability 0.1
            keep = torch.rand(B, H, N, N, device=dev, generator=g) > 0.9
            mask = keep if mask_kind == "boolean" else torch.where(keep, 0.0, -100.0).to(dtype)
        fwd_f, bwd_f = algorithmic_flops(B, H, N, D, causal)
        iters = 5 if N >= 4096 else 20
        try:
            def ref_fwd():
                with fwAD.dual_level():
                    o = RefAttn.fwd_dual(fwAD.make_dual(q, tq), fwAD.make_dual(k, tk), fwAD.make_dual(v, tv), attn_mask=mask,
                                         causal=causal)
                    return fwAD.unpack_dual(o)
            o_ref, to_ref = ref_fwd()
            torch.cuda.synchronize()
            rec["ref_dual_fwd_ms"] = _time_ms(ref_fwd, iters)
            rec["ref_dual_fwd_peak_mb"] = _peak_mb(ref_fwd)
            ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
            o2 = RefAttn.fwd(ql, kl, vl, attn_mask=mask, causal=causal)

            def ref_bwd():
                return torch.autograd.grad(o2, (ql, kl, vl), go, retain_graph=True)
            g_ref = ref_bwd()
            torch.cuda.synchronize()
            rec["ref_primal_bwd_ms"] = _time_ms(ref_bwd, iters)
        except Exception as exc:  # noqa: BLE001
            rec["ref_error"] = f"{type(exc).__name__}: {exc}"[:400]
            out["shapes"][name] = rec
            continue
        s = D ** -0.5
        mask_c = _lib.make_mask(mask, B, H, N)
        summ = _lib.mask_summary(mask_c, mask, B, H, N) if mask is not None else None

        def ours_fwd():   # what a forward call through the public API launches: the mask pre-pass, then the kernel
            sm = _lib.mask_summary(mask_c, mask, B, H, N) if mask is not None else None
            return _lib.fwd(q, k, v, tq, tk, tv, mask_c, sm, causal, s)
        o, to, lse2, mu = ours_fwd()
        rec["ours_dual_fwd_ms"] = _time_ms(ours_fwd, iters)
        rec["ours_dual_fwd_peak_mb"] = _peak_mb(ours_fwd)
        if mask is not None:
            rec["ours_mask_prepass_ms"] = _time_ms(lambda: _lib.mask_summary(mask_c, mask, B, H, N), iters)
        o1, _, lse1, mu1 = _lib.fwd(q, k, v, None, None, None, mask_c, summ, causal, s)
        gours = _lib.bwd(q, k, v, None, None, None, o1, None, lse1, mu1, go, None, mask_c, summ, causal, s)
        rec["ours_primal_bwd_ms"] = _time_ms(
            lambda: _lib.bwd(q, k, v, None, None, None, o1, None, lse1, mu1, go, None, mask_c, summ, causal, s), iters)
        rec["ours_dual_bwd_ms"] = _time_ms(
            lambda: _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, go, go, mask_c, summ, causal, s), iters)
        rec["ref_dual_fwd_tflops"] = fwd_f / rec["ref_dual_fwd_ms"] / 1e9
        rec["ours_dual_fwd_tflops"] = fwd_f / rec["ours_dual_fwd_ms"] / 1e9
        rec["fwd_speedup"] = rec["ref_dual_fwd_ms"] / rec["ours_dual_fwd_ms"]
        rec["primal_bwd_speedup"] = rec["ref_primal_bwd_ms"] / rec["ours_primal_bwd_ms"]
        # the two implementations against each other (not a parity gate: the reference multiplies P V in TF32)
        rec["max_abs_diff"] = {"O": float((o.float() - o_ref.float()).abs().max()),
                               "tO": float((to.float() - to_ref.float()).abs().max()),
                               "dq": float((gours[0].float() - g_ref[0].float()).abs().max()),
                               "dk": float((gours[1].float() - g_ref[1].float()).abs().max()),
                               "dv": float((gours[2].float() - g_ref[2].float()).abs().max())}
        out["shapes"][name] = rec
        del q, k, v, tq, tk, tv, go, o, to, o_ref, to_ref
        torch.cuda.empty_cache()
    _lib.read_status(dev)
    out["note"] = ("reference = jvp_flash_attention (Triton) run unmodified from baseline/_ref on this GPU: JVPAttn.fwd_dual "
                   "under fwAD.dual_level (dual forward) and autograd through JVPAttn.fwd (its backward covers the primal "
                   "output only); ours = this library on the same tensors, dual forward / primal-only backward / dual backward")
    print(json.dumps(out))


def gpu_incumbent_record(args, timeout_s=420):
    import subprocess
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "gpu-incumbent", "--dtype", args.dtype]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"reference-on-B200: unavailable (child process did not finish within {timeout_s} s)"}
    for ln in reversed(r.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                return json.loads(ln)
            except json.JSONDecodeError:
                break
    tail = (r.stderr or r.stdout or "").strip().splitlines()[-1:] or [""]
    return {"unavailable": f"reference-on-B200: unavailable (child exit code {r.returncode}: {tail[0][:300]})"}


def dit_record(timeout_s=300):
    """The end-to-end configuration (bench_dit.py: DiT JVP training step, 32 samples on this GPU) with this library's
    attention and, for an A/B on the same box, with SDPA forced to its MATH backend; child processes."""
    import subprocess
    rec = {}
    for impl in ("jvpfa", "sdpa"):
        cmd = [sys.executable, os.path.join(ROOT, "bench_dit.py"), "--steps", "6", "--warmup", "3", "--attention", impl]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, cwd=ROOT)
            line = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
            d = json.loads(line[-1])
            rec[impl] = {"ms_per_step": d["ms_per_step"], "samples_per_s": d["value"], "loss": d["loss"]}
        except Exception as exc:  # noqa: BLE001
            rec[impl] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    if "ms_per_step" in rec.get("jvpfa", {}) and "ms_per_step" in rec.get("sdpa", {}):
        rec["speedup_vs_sdpa_math"] = rec["sdpa"]["ms_per_step"] / rec["jvpfa"]["ms_per_step"]
    rec["workload"] = ("DiT 28 blocks, hidden 1152, 16 heads of 72, 256 tokens, bf16, 32 samples: torch.func.jvp + MSE on "
                       "primal and tangent + backward + AdamW")
    return rec


# ------------------------------------------------------------------------------------------------
# CUDA arm
# ------------------------------------------------------------------------------------------------
def run_cuda(args, rank, world, local_rank):
    import torch.distributed as dist
    from jvp_flash_attention_b200 import _lib
    from jvp_flash_attention_b200.jvp_attention import JVPAttn
    from jvp_flash_attention_b200.sharding import shard_bounds

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
    units = B * H
    lo, hi = shard_bounds(units, world, rank)          # this rank's slice of the flattened (batch, head) axis
    U = hi - lo
    s = D ** -0.5
    peak_burst, peak_sustained, peak_kind = measured_peaks()

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

    probe_stream = torch.cuda.Stream(dev)

    def make_inputs(n_units, dtype, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return [torch.randn(1, n_units, N, D, device=dev, dtype=dtype, generator=g) for _ in range(8)]

    def timed_steps(ts, steps, warmup, sampler=None):
        """Device time per step of dual forward + dual backward on resident inputs, MAX over ranks."""
        q, k, v, tq, tk, tv, gO, gtO = ts
        n_units = q.shape[1]
        mask_c = _lib.make_mask(None, 1, n_units, N)

        def step():
            o, to, lse2, mu = _lib.fwd(q, k, v, tq, tk, tv, mask_c, None, causal, s)
            return _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, gO, gtO, mask_c, None, causal, s)

        for _ in range(warmup):
            step()
        barrier()
        _lib.read_status(dev)
        we0, we1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        we0.record()
        step()
        we1.record()
        torch.cuda.synchronize()
        est_ms = we0.elapsed_time(we1)                 # length of one step, to size the clock probe
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.__enter__()
        barrier()
        probe = None
        if sampler is not None:
            # the SM clock the kernels actually get: a one-thread probe beside them for about the length of the region
            probe = _lib.sm_clock_probe(probe_stream, int(min(900000, max(2000, steps * est_ms * 1000 * 0.9))))
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        if sampler is not None:
            sampler.__exit__(None, None, None)
            probe_stream.synchronize()
            sampler.in_kernel_mhz = float(probe.item())
        ms = max_over_ranks(e0.elapsed_time(e1)) / steps
        _lib.read_status(dev)
        return ms

    fwd_f, bwd_f = algorithmic_flops(1, units, N, D, causal)          # the whole problem
    step_f = fwd_f + bwd_f
    warmup = max(args.warmup, 3)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16

    # ---- device-resident timing of this rank's slice (the `value`) ----
    ts = make_inputs(U, dtype, 1234 + rank)
    clocks = ClockSampler(physical_gpu_index(local_rank))
    ms_step = timed_steps(ts, args.steps, warmup, clocks)
    value = step_f / (ms_step * 1e-3) / 1e12

    # ---- per-kernel durations of the same steps: caller-owned events recorded between the launches ----
    q, k, v, tq, tk, tv, gO, gtO = ts
    mask_c = _lib.make_mask(None, 1, U, N)
    # one set of events per step, read after the last step: no synchronisation (and so no idle GPU) between the steps
    ev_f = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    for group in ev_f + marks:
        for e in group:
            e.record()                                 # creates the underlying CUDA events
    names = ("fwd", "bwd_preprocess", "bwd_q", "bwd_k", "bwd_v")
    acc = dict.fromkeys(names, 0.0)
    for i in range(args.steps):
        o = torch.empty_like(q)                        # warm allocator: the forward's outputs come from its cache
        del o
        ev_f[i][0].record()
        o, to, lse2, mu = _lib.fwd(q, k, v, tq, tk, tv, mask_c, None, causal, s)
        ev_f[i][1].record()
        _lib.bwd(q, k, v, tq, tk, tv, o, to, lse2, mu, gO, gtO, mask_c, None, causal, s, marks=marks[i])
    torch.cuda.synchronize()
    for i in range(args.steps):
        acc["fwd"] += ev_f[i][0].elapsed_time(ev_f[i][1])
        for j, nme in enumerate(names[1:]):
            acc[nme] += marks[i][j].elapsed_time(marks[i][j + 1])
    kernels = {nme: {"ms_per_launch": acc[nme] / args.steps, "launches": args.steps} for nme in names}
    lfwd_f, lbwd_f = algorithmic_flops(1, U, N, D, causal)            # this rank's slice
    fam_ms = (acc["bwd_q"] + acc["bwd_k"] + acc["bwd_v"]) / (3.0 * args.steps)
    # dominant kernel: the backward family kernel (one template, three launches per step); algorithmic FLOPs per
    # launch = a third of the backward's 30 * units * N^2 * D / 2
    ach = (lbwd_f / 3.0) / (fam_ms * 1e-3) / 1e12
    fwd_ach = lfwd_f / (acc["fwd"] / args.steps * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "bwd_sm100_kernel (families Q, K, V)", "achieved": ach, "peak": peak_burst,
                "unit": "TFLOP/s", "frac": ach / peak_burst, "peak_kind": f"{peak_kind} burst bf16 cuBLAS",
                "frac_sustained": ach / peak_sustained, "frac_nominal": ach / NOMINAL_DENSE_TFLOPS,
                "executed_over_algorithmic": 1.6, "achieved_executed": ach * 1.6,
                # DRAM bytes per backward-family launch from an ncu capture of 32 (batch, head) units (321.9 / 320.9 /
                # 251.3 MB read+write for families Q / K / V), scaled by the units of this launch: every unit's tensors
                # are read from HBM once per launch, so the traffic grows in proportion
                "traffic": (321.9e6 + 320.9e6 + 251.3e6) / 3.0 * (U / 32.0), "traffic_unit": "bytes per launch",
                "fwd_kernel": {"achieved": fwd_ach, "frac": fwd_ach / peak_burst, "frac_sustained": fwd_ach / peak_sustained}}

    # ---- the other 16-bit type (the headline configuration is stated in fp16, the target line in bf16) ----
    other = torch.float16 if dtype == torch.bfloat16 else torch.bfloat16
    other_name = "fp16" if other == torch.float16 else "bf16"
    del ts, q, k, v, tq, tk, tv, gO, gtO, o, to
    ts_o = make_inputs(U, other, 4321 + rank)
    ms_o = timed_steps(ts_o, max(4, args.steps // 2), 3)
    other_rec = {"value": step_f / (ms_o * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_o, "dtype": other_name}
    del ts_o

    # ---- weak scaling beside it: every rank runs the full problem (a fixed per-GPU workload) ----
    weak = None
    if world > 1 and not args.no_weak:
        ts_w = make_inputs(units, dtype, 99 + rank)
        ms_w = timed_steps(ts_w, max(4, args.steps // 2), 3)
        weak = {"value": step_f * world / (ms_w * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_w,
                "scaling": "weak", "global_batch": B * world,
                "note": "every rank runs the full B x H problem; aggregate over ranks"}
        del ts_w

    # ---- end to end through the public API with host buffers (this rank's slice) ----
    e2e = None
    if not args.no_e2e:
        ts = make_inputs(U, dtype, 1234 + rank)
        host_in = [torch.empty(1, U, N, D, dtype=dtype).pin_memory() for _ in range(8)]
        for hbuf, src in zip(host_in, ts):
            hbuf.copy_(src)
        del ts
        host_out = [torch.empty(1, U, N, D, dtype=dtype).pin_memory() for _ in range(8)]
        # Three streams, inputs double-buffered on the device: the copy-in of step i+1 and the copy-out of step
        # i-1 overlap the kernels of step i, as a caller that streams batches through the public API would do.
        dev_in = [[torch.empty(1, U, N, D, dtype=dtype, device=dev) for _ in range(8)] for _ in range(2)]
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
        n_e2e = max(8, args.steps)     # (the first copy-in and the last copy-out are not overlapped: amortise them)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        s_main.wait_event(ev_out)       # the last copy-out ends the timed region
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        nbytes = 8 * U * N * D * 2
        e2e = {"value": step_f / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e, "steps": n_e2e,
               "note": "JVPAttn.dual + autograd.grad on this rank's slice; every step copies its 8 input tensors from "
                       "pinned host memory and O, tO and the six gradients back to pinned host memory inside the timed "
                       "region (bytes are per rank); copies run on their own streams and overlap the kernels of the "
                       "neighbouring steps. The limiter is the host link, not a kernel: all ranks of a node share host "
                       "memory and PCIe root bandwidth"}
        del host_in, host_out, dev_in
        _lib.read_status(dev)

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle.jvp_attention_oracle import sdpa_jvp_oracle
        cores = host_threads(args.ref_threads)
        gcpu = torch.Generator().manual_seed(0)
        tsc = [torch.randn(1, 1, N, D, generator=gcpu) for _ in range(8)]
        sdpa_jvp_oracle(*tsc, causal=causal, dtype=torch.float32)  # warm-up
        done, t0 = 0, time.perf_counter()
        while done < 32 and (time.perf_counter() - t0 < 10.0 or done < 2):
            sdpa_jvp_oracle(*tsc, causal=causal, dtype=torch.float32)
            done += 1
        dt = time.perf_counter() - t0
        f1, b1 = algorithmic_flops(1, 1, N, D, causal)
        cpu_baseline = {"value": (f1 + b1) * done / dt / 1e12, "unit": "TFLOP/s", "cores": cores,
                        "kind": "port", "sample": f"{done} (batch, head) slices of the workload, fp32, SDPA-MATH + "
                        "torch.func.jvp + autograd on the host cores", "seconds": dt}

    # ---- the reference's own GPU kernels on this box (rank 0, N = 1 only) ----
    incumbent = None
    if rank == 0 and world == 1 and not args.no_incumbent:
        torch.cuda.empty_cache()
        incumbent = gpu_incumbent_record(args)

    # ---- the end-to-end model configuration (rank 0, N = 1 only) ----
    dit = None
    if rank == 0 and world == 1 and not args.no_dit:
        torch.cuda.empty_cache()
        dit = dit_record()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": f"dual fwd+bwd attention, one problem B={B} H={H} N={N} D={D} causal {args.dtype}, "
                                   f"fully masked key tiles skipped; its {units} (batch, head) units sliced over the "
                                   f"GPUs ({U} per GPU), no collective",
                       "global_batch": B, "units_per_gpu": U,
                       "l2": f"inputs larger than L2 (8 tensors of {U * N * D * 2 / 1e6:.0f} MB per GPU and step)",
                       "flops_per_step": step_f},
            "per_gpu_tflops": value / world,
            "frac_of_nominal_dense_peak": value / world / NOMINAL_DENSE_TFLOPS,
            "frac_of_measured_peak": value / world / peak_burst,
            "frac_of_measured_sustained_peak": value / world / peak_sustained,
            "roofline": roofline, "kernels": kernels, other_name: other_rec, "weak": weak,
            "cpu_baseline": cpu_baseline, "gpu_incumbent": incumbent, "dit": dit, "e2e": e2e,
            "gpu_launches": 5 * args.steps, "clocks": clocks.summary(),
            # time x clock: millions of SM cycles per step at the clock counted beside the kernels (power-cap noise drops out)
            "mcycles_per_step": (ms_step * clocks.in_kernel_mhz / 1e3) if clocks.in_kernel_mhz else None,
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
    ap.add_argument("--dtype", choices=("bf16", "fp16", "fp32"), default="bf16")
    ap.add_argument("--impl", choices=("cuda", "reference", "gpu-incumbent"), default="cuda")
    ap.add_argument("--ref-slices", type=int, default=2, help="(batch, head) slices per step of the reference arm")
    ap.add_argument("--ref-threads", type=int, default=0, help="host threads of the CPU arm (default: all cores)")
    ap.add_argument("--batch", type=int, default=None, help="override B of the workload (small profiler captures only)")
    ap.add_argument("--incumbent-shapes", default="", help="comma-separated subset of the GPU-incumbent shapes")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-weak", action="store_true")
    ap.add_argument("--no-incumbent", action="store_true")
    ap.add_argument("--no-dit", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "gpu-incumbent":
        run_incumbent_child(args)
        return
    if args.dtype == "fp32":
        raise SystemExit("--dtype fp32 is for --impl gpu-incumbent only")
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nnodes=1 --nproc-per-node N "
                         "--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...")
    run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
