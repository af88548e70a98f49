#!/usr/bin/env python
"""Benchmark of the WUSH hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line.  The headline `value` is the fused transform+quantize throughput in
algorithmic GB/s (MXFP4, per-group WUSH matrices, 16384 tokens x 14336 channels per GPU, inputs
resident in HBM); `e2e` is the same pass through the public op with host buffers (pinned H2D of
the activations and D2H of codes+scales inside the timed region).  `roofline` covers the quantize
kernel, `cpu_baseline` times the CPU restatement of the reference's torch quantizer on a bounded
sample.  `extra` carries the other two kernels of the path when they are built.

With --impl reference the reference's CPU path (the oracle port; the reference is pure Python
and needs its own checkout to import) is timed on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, HIDDEN, GROUP = 16384, 14336, 32
BYTES_PER_ELEM_MX = 2.0 + 0.5 + 1.0 / 32.0


def algorithmic_bytes(tokens: int, hidden: int, group: int = GROUP) -> float:
    """x read once (2 B), codes written (0.5 B), one scale byte per group, matrix read once."""
    return tokens * hidden * (2.0 + 0.5 + 1.0 / group) + group * hidden * 2.0


def measured_peaks() -> tuple[dict, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only queries) from a thread while
    the timed region runs; falls back to no samples when NVML is unavailable."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period, self.samples, self.mask = index, period_s, [], 0
        self.stop = threading.Event()
        self.max_mhz = None
        self.thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                try:
                    idx = int(visible.split(",")[self.index])
                except ValueError:
                    idx = self.index
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def _poll(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.mask |= nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                pass
            time.sleep(self.period)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for bit, n in self.REASONS.items() if self.mask & bit), "samples": len(s)}


# ------------------------------------------------------------------------------------------
# CPU leg (oracle port) -- also the whole of --impl reference
# ------------------------------------------------------------------------------------------

def cpu_quant_throughput(sample_rows: int, hidden: int, repeats: int = 1) -> dict:
    """Time the CPU restatement of block_transform + rtn_xxfp4 on `sample_rows` rows of the
    benchmark workload; GB/s uses the same algorithmic byte count as the GPU kernel."""
    import numpy as np
    import torch
    from oracle import synth, torch_port
    x = synth.activations(sample_rows, hidden, seed=0)
    mat = torch.from_numpy(synth.wush_matrix(hidden, GROUP)).to(torch.bfloat16)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    torch_port.fused_transform_quant(x[:32], mat, "mxfp4")          # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        torch_port.fused_transform_quant(x, mat, "mxfp4")
        best = min(best, time.perf_counter() - t0)
    gbs = algorithmic_bytes(sample_rows, hidden) / best / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_rows} of {TOKENS} rows x {hidden} channels, MXFP4 WUSH, torch CPU float64 "
                      f"restatement of block_transform + rtn_xxfp4, best of {repeats}: {best:.2f} s",
            "seconds": best}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 512
    times = []
    res = None
    for i in range(args.warmup + args.steps):
        res = cpu_quant_throughput(rows, HIDDEN, repeats=1)
        if i >= args.warmup:
            times.append(res["seconds"])
    sec = sum(times) / len(times)
    gbs = algorithmic_bytes(rows, HIDDEN) / sec / 1e9
    res.pop("seconds")
    res["value"] = gbs
    line = {
        "impl": "reference", "metric": "fused_transform_quant_GBps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * TOKENS / rows,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(args.gpus), "cpu_baseline": res,
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU torch path of the reference restated in oracle/torch_port.py; each step is a "
                f"{rows}-row sample of the workload, ms_per_step is scaled to the full {TOKENS} rows",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int) -> dict:
    return {"workload": f"fused WUSH transform + MXFP4 quantize, {TOKENS} tokens x {HIDDEN} channels bf16 per GPU, "
                        f"per-group 32x32 matrices, N(0,1) + 0.5% outlier channels x50 (seeded)",
            "tokens_per_gpu": TOKENS, "hidden": HIDDEN, "group": GROUP, "format": "mxfp4",
            "l2_policy": "inputs (470 MB) and outputs (125 MB) larger than the 126 MB L2, no flush needed",
            "parallelism": f"rows sharded over {n_gpus} GPU(s), no collective",
            "baseline_metric": "MXFP4 W4A4 GEMM TFLOPS + fused transform-quant GB/s; Hessian tok/s @1/2/4/8"}


# ------------------------------------------------------------------------------------------
# GPU leg
# ------------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from oracle import synth
    from wush_b200 import qutlass_ops as ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # inputs: every rank its own shard of rows (different seed), same matrices
    x_host = synth.activations(TOKENS, HIDDEN, seed=100 + rank).pin_memory()
    mat = synth.to_bf16_tensor(synth.wush_matrix(HIDDEN, GROUP)).to(dev)
    x = x_host.to(dev)
    alg = algorithmic_bytes(TOKENS, HIDDEN)

    def step():
        return ops.fused_quantize_mx_wush_op(x, mat, "abs_max", False)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    clock_summary = clocks.summary()

    # kernel-only duration: events directly around each launch on the launching stream
    from wush_b200 import _lib
    lib = _lib.load()
    q = torch.empty(TOKENS, HIDDEN // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(TOKENS, HIDDEN // GROUP, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    k0.record()
    for _ in range(args.steps):
        rc = lib.wush_fused_quantize_mx(x.data_ptr(), mat.data_ptr(), HIDDEN, q.data_ptr(), sf.data_ptr(),
                                        HIDDEN // GROUP, 0, TOKENS, HIDDEN, 0, stream)
        assert rc == 0, rc
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / args.steps

    # end to end: pinned host activations in, codes + scales back to pinned host memory
    q_host = torch.empty(TOKENS, HIDDEN // 2, dtype=torch.uint8).pin_memory()
    sf_host = torch.empty(TOKENS, HIDDEN // GROUP, dtype=torch.uint8).pin_memory()

    def e2e_step():
        xd = x_host.to(dev, non_blocking=True)
        qd, sd, _ = ops.fused_quantize_mx_wush_op(xd, mat, "abs_max", False)
        q_host.copy_(qd, non_blocking=True)
        sf_host.copy_(sd.view(torch.uint8)[:TOKENS, : HIDDEN // GROUP], non_blocking=True)

    e2e_ms = float("nan")
    if not args.kernel_only:
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)

    times = torch.tensor([ms, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, kernel_ms = (float(v) for v in times.tolist())

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        value = world * alg * args.steps / (ms * 1e-3) / 1e9
        e2e_value = world * alg * args.steps / (e2e_ms * 1e-3) / 1e9
        achieved = alg / (kernel_ms * 1e-3) / 1e9
        cpu = cpu_quant_throughput(512, HIDDEN, repeats=2) if (world == 1 and not args.kernel_only) else None
        if cpu:
            cpu.pop("seconds", None)
        line = {
            "metric": "fused_transform_quant_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": q_host.numel() + sf_host.numel(), "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "kernel": "fused_quantize_kernel<MX>", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": alg,
                         "kernel_ms": kernel_ms, "traffic": None},
            "cpu_baseline": cpu,
            "clocks": clock_summary,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS, help="rows per GPU of the quantize workload")
    ap.add_argument("--hidden", type=int, default=HIDDEN, help="channels of the quantize workload")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time only the kernel launches (no end-to-end or CPU leg); used for profiler captures")
    args = ap.parse_args()
    globals()["TOKENS"], globals()["HIDDEN"] = args.tokens, args.hidden
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
