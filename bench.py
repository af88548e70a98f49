#!/usr/bin/env python
"""Benchmark of the WUSH hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line.  The headline `value` is the fused transform+quantize throughput in
algorithmic GB/s (MXFP4, per-group WUSH matrices, 16384 tokens x 14336 channels per GPU, inputs
resident in HBM); `e2e` is the same pass through the public host-buffer entry point (pinned H2D of
the activations and D2H of codes+scales inside the timed region, chunked and overlapped).  `roofline` covers the quantize
kernel, `cpu_baseline` times the CPU restatement of the reference's torch quantizer on a bounded
sample.  The other parts of the metric are top-level objects of the same line, each with its own value,
roofline fraction, clock summary and a `parity` object (sampled outputs of the timed configuration checked
against the float64 oracle inside the run): `quant_nvfp4`, `gemm` (MXFP4 GEMM at 8192^3), `gemm_nvfp4`,
`decode` (the decoder-layer shape grid with M from 1 to 8192), `hessian` / `hessian_14336` (262144 calibration
tokens sharded over the GPUs and combined over NVLink), `sweep` (GPTQ column sweep of one 4096 x 4096 layer),
`layer_4096` (one whole layer: calibration, sweep, real-quant forward, next to the CPU pseudo-quantizer) and, on
several GPUs, `block_70b` (the seven linears of a hidden-8192 decoder block with column-sharded weights).  A parity
failure makes the run exit non-zero.  `extra` repeats the same objects with their long-form fields.

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

    def __init__(self, index: int, period_s: float = 0.02):
        # One sample when the region is entered (the warm-up steps have just run), one every `period_s` from a
        # thread, one when the region is left.  NVML queries take driver-wide locks: polled every half millisecond
        # by eight ranks at once they slowed every rank's kernel launches (the 8-GPU Hessian job took 0.86 ms in the
        # benchmark against 0.57 ms without the sampler), hence the long period and rank 0 only when there are
        # several ranks.
        self.index, self.period, self.samples, self.mask = index, period_s, [], 0
        self.stop = threading.Event()
        self.max_mhz = None
        self.thread = None
        self.enabled = int(os.environ.get("RANK", "0")) == 0

    def _sample(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            self.mask |= self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            pass

    def __enter__(self):
        if not self.enabled:
            return self
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
            self._sample()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def _poll(self):
        while not self.stop.wait(self.period):
            self._sample()

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
            self._sample()

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
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(args.gpus), "cpu_baseline": res,
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "sample_rows_per_step": rows,
        "ms_per_full_workload_extrapolated": sec * 1e3 * TOKENS / rows,
        "note": "CPU torch path of the reference restated in oracle/torch_port.py; each step is a "
                f"{rows}-row sample of the {TOKENS}-row workload and ms_per_step is the time of that sample "
                "(throughput in GB/s does not depend on the sample size: rows are independent)",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int) -> dict:
    return {"workload": f"fused WUSH transform + MXFP4 quantize, {TOKENS} tokens x {HIDDEN} channels bf16 per GPU, "
                        f"per-group 32x32 matrices, N(0,1) + 0.5% outlier channels x50 (seeded)",
            "tokens_per_gpu": TOKENS, "hidden": HIDDEN, "group": GROUP, "format": "mxfp4",
            "l2_policy": f"inputs ({TOKENS * HIDDEN * 2 / 1e6:.0f} MB) and outputs ({TOKENS * HIDDEN * 0.53125 / 1e6:.0f} MB) "
                         "against a 126 MB L2: larger than L2 at the default size, so no flush between iterations",
            "parallelism": f"rows sharded over {n_gpus} GPU(s), no collective",
            "launch": "the K timed steps (K calls of the public op) are captured into one CUDA graph and replayed",
            "baseline_metric": "MXFP4 W4A4 GEMM TFLOPS + fused transform-quant GB/s; Hessian tok/s @1/2/4/8"}


# ------------------------------------------------------------------------------------------
# GPU leg
# ------------------------------------------------------------------------------------------

GEMM_M = GEMM_N = GEMM_K = 8192
HESS_TOKENS, HESS_HIDDEN = 128 * 2048, 4096
FP4_NOMINAL_TFLOPS = 9000.0      # NVIDIA's dense FP4 figure for B200 (the 2:4-sparse figure is twice that)
PARITY_FAILURES: list = []       # sections whose in-run parity check failed: the run exits non-zero


def _capture_steps(fn, steps: int, torch):
    """`steps` calls of fn captured into one CUDA graph (the Python and dispatcher time of a call is of the
    order of the kernels timed here, so an eager loop leaves the GPU waiting for the host).  Returns a callable
    that replays the graph, or None when capture is not possible."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()                                   # allocator and lazy initialisation outside the capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(steps):
                fn()
        return graph.replay
    except Exception as exc:                       # noqa: BLE001 - fall back to the eager loop
        sys.stderr.write(f"bench: CUDA graph capture failed ({exc}); timing an eager loop\n")
        torch.cuda.synchronize()
        return None


def _time_steps(fn, steps: int, torch, graph: bool = False) -> float:
    """Average milliseconds per call, CUDA events on the launching stream."""
    replay = _capture_steps(fn, steps, torch) if graph else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    if replay is not None:
        replay()
    else:
        for _ in range(steps):
            fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _parity(name: str, err: float, tol: float, what: str) -> dict:
    ok = bool(err <= tol)
    if not ok:
        PARITY_FAILURES.append(name)
    return {"max_rel": float(err), "tol": tol, "ok": ok, "what": what}


def _sample_rows(rows: int, n: int):
    import numpy as np
    fixed = [0, 1, 127, 128, rows - 129, rows - 1]
    rng = np.random.default_rng(rows)
    return np.unique(np.concatenate([np.array(fixed) % rows, rng.choice(rows, size=max(0, n - len(fixed)), replace=False)]))


def quant_parity(x_host, mat_np, q, sf, fmt: str, torch) -> dict:
    """Codes and scale bytes of sampled rows of the timed output against the oracle quantizer."""
    import numpy as np
    from oracle import synth
    from oracle import wush_oracle as wo
    g = 32 if fmt == "mxfp4" else 16
    idx = _sample_rows(x_host.shape[0], 32)
    ref = wo.fused_transform_quant(synth.bf16_to_f64(x_host[idx]), mat_np, fmt)
    keep = ~np.isnan(ref["fake_quant"]).any(axis=1)
    t = torch.from_numpy(idx).to(q.device)
    fold = lambda p: np.where(wo.unpack_e2m1_codes(p) == 8, 0, wo.unpack_e2m1_codes(p))
    bad_q = float(np.mean(fold(q[t].cpu().numpy()[keep]) != fold(ref["e2m1"][keep])))
    bad_s = float(np.mean(sf.view(torch.uint8)[t].cpu().numpy()[keep][:, : x_host.shape[1] // g] != ref["scale_quant"][keep]))
    return _parity("quant_" + fmt, max(bad_q, bad_s), 1e-4,
                   f"fraction of differing codes / scale bytes on {int(keep.sum())} sampled rows of the timed output vs "
                   f"the float64 oracle (budget: rounding-boundary ties)")


def bench_quant_nv(args, dev, torch, ops, peaks, peak_kind) -> dict:
    """The quantize kernel in its NVFP4 form (groups of 16, E4M3 scales, tensor scale 10) on the benchmark shape."""
    from oracle import synth
    from wush_b200 import _lib
    x_host = synth.activations(TOKENS, HIDDEN, seed=100)
    mat_np = synth.wush_matrix(HIDDEN, 16)
    x, mat = x_host.to(dev), synth.to_bf16_tensor(mat_np).to(dev)
    gs = torch.tensor([10.0], device=dev)
    lib = _lib.load()
    q = torch.empty(TOKENS, HIDDEN // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(TOKENS, HIDDEN // 16, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        rc = lib.wush_fused_quantize_nv(x.data_ptr(), mat.data_ptr(), HIDDEN, gs.data_ptr(), q.data_ptr(), sf.data_ptr(),
                                        HIDDEN // 16, 0, TOKENS, HIDDEN, 0, stream)
        assert rc == 0, rc

    for _ in range(3):
        launch()
    with ClockSampler(dev.index) as clocks:
        ms = _time_steps(launch, args.steps, torch)
    alg = algorithmic_bytes(TOKENS, HIDDEN, 16)
    gbs = alg / (ms * 1e-3) / 1e9
    return {"metric": "fused_transform_quant_nvfp4_GBps", "value": gbs, "unit": "GB/s", "ms_per_step": ms,
            "frac": gbs / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind} HBM copy bandwidth",
            "algorithmic_bytes_per_launch": alg, "gpu_launches": args.steps,
            "parity": quant_parity(x_host, mat_np, q, sf, "nvfp4", torch), "clocks": clocks.summary()}


def bench_gemm(args, dev, torch, ops, peaks, peak_kind, fmt: str = "mx") -> dict:
    """W4A4 GEMM at 8192^3: operands produced by the fused quantize kernel from Gaussian activations /
    N(0, 0.02^2) weights with a shared Hadamard transform, scales written directly in the blocked layout."""
    import numpy as np
    from oracle import synth
    from oracle import wush_oracle as wo
    from wush_b200 import _lib
    g = 32 if fmt == "mx" else 16
    name = "mxfp4" if fmt == "mx" else "nvfp4"
    gen = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(GEMM_M, GEMM_K, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(GEMM_N, GEMM_K, generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    had = synth.to_bf16_tensor(synth.hadamard_matrix(g)).to(dev)
    gs = torch.tensor([10.0], device=dev) if fmt == "nv" else None
    xq, xs = ops._quantize(x, had, fmt, gs, sf_layout=_lib.SF_BLOCKED)
    wq, wsf = ops._quantize(w, had, fmt, gs, sf_layout=_lib.SF_BLOCKED)
    a_val = 1.0 / 9.0 if fmt == "mx" else 1.0 / 100.0
    alpha = torch.tensor([a_val], device=dev)
    del x, w
    fn = lambda: ops.matmul_fp4_blocked(xq, wq, xs.view(-1), wsf.view(-1), alpha, fmt)
    for _ in range(3):
        y = fn()
    with ClockSampler(dev.index) as clocks:
        ms = _time_steps(fn, args.steps, torch, graph=True)
    flops = 2.0 * GEMM_M * GEMM_N * GEMM_K
    tflops = flops / (ms * 1e-3) / 1e12
    peak4 = 4.0 * peaks["bf16_tflops"]
    # parity on sampled rows x columns of the timed output: the oracle dequantizes the same codes and scales
    ra, rb = _sample_rows(GEMM_M, 24), _sample_rows(GEMM_N, 40)
    ta, tb = torch.from_numpy(ra).to(dev), torch.from_numpy(rb).to(dev)
    xs_rm = unblock_scales(xs.view(-1), GEMM_M, GEMM_K // g, torch)
    ws_rm = unblock_scales(wsf.view(-1), GEMM_N, GEMM_K // g, torch)
    want = wo.fp4_gemm(xq[ta].cpu().numpy(), xs_rm[ta].cpu().numpy(), wq[tb].cpu().numpy(), ws_rm[tb].cpu().numpy(), a_val, name)
    got = y[ta][:, tb].double().cpu().numpy()
    par = _parity("gemm_" + name, float(np.linalg.norm(got - want) / np.linalg.norm(want)), 1e-2,
                  f"relative Frobenius error of {len(ra)} x {len(rb)} sampled outputs of the timed GEMM vs the float64 oracle")
    res = {"metric": f"{name}_w4a4_gemm_TFLOPS", "value": tflops, "unit": "TFLOP/s", "ms_per_step": ms,
           "config": {"workload": f"{name.upper()} GEMM M=N=K={GEMM_M}, bf16 out, operands from the fused quantize kernel"},
           "gpu_launches": args.steps,
           "roofline": {"bound": "tensor", "kernel": f"fp4_gemm_pair_kernel<{fmt.upper()}>", "achieved": tflops, "peak": peak4,
                        "unit": "TFLOP/s", "frac": tflops / peak4,
                        "peak_kind": f"4 x {peak_kind} bf16 burst (no FP4 figure was measured)",
                        "frac_of_nominal_dense_fp4": tflops / FP4_NOMINAL_TFLOPS, "traffic": None},
           "parity": par, "clocks": clocks.summary()}
    if fmt == "mx":
        res["cublaslt"] = cublaslt_fp4(args, torch, xq, wq, xs, wsf, y, flops)
    return res


def unblock_scales(blocked, rows: int, groups: int, torch):
    """Blocked (128 x 4 tiles) scale bytes -> row-major [rows, groups] (index arithmetic of the layout definition)."""
    r = torch.arange(rows, device=blocked.device)[:, None]
    gidx = torch.arange(groups, device=blocked.device)[None, :]
    cols4 = (groups + 3) // 4
    off = ((r // 128) * cols4 + gidx // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + gidx % 4
    return blocked.view(torch.uint8)[off]


def cublaslt_fp4(args, torch, xq, wq, xs, wsf, y_ours, flops) -> dict:
    """Same-box comparator: cuBLASLt's block-scaled FP4 GEMM through torch on the same operands (1 GPU, local
    memory).  Reported next to ours; a failure to run is recorded, not fatal."""
    try:
        import torch.nn.functional as F
        a = xq.view(torch.float4_e2m1fn_x2)
        b = wq.view(torch.float4_e2m1fn_x2).t()
        sa, sb = xs.view(-1).view(torch.float8_e8m0fnu), wsf.view(-1).view(torch.float8_e8m0fnu)
        kind, sw = F.ScalingType.BlockWise1x32, F.SwizzleType.SWIZZLE_32_4_4
        fn = lambda: F.scaled_mm(a, b, sa, kind, sb, kind, swizzle_a=sw, swizzle_b=sw, output_dtype=torch.bfloat16)
        for _ in range(3):
            y = fn()
        ms = _time_steps(fn, args.steps, torch, graph=True)
        ref = y.float() * (1.0 / 9.0)
        rel = float((y_ours.float() - ref).norm() / ref.norm())
        return {"TFLOPS": flops / (ms * 1e-3) / 1e12, "ms_per_step": ms, "rel_diff_to_ours": rel,
                "how": "torch.nn.functional.scaled_mm, BlockWise1x32 E8M0 scales, SWIZZLE_32_4_4, bf16 out"}
    except Exception as exc:                       # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


DECODE_SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]      # (N, K) of the decoder layer
DECODE_M = [1, 16, 128, 1024, 8192]


def bench_decode(args, dev, torch, ops, peaks, peak_kind) -> dict:
    """MXFP4 GEMM over the decoder-layer shapes of a hidden-4096 / FFN-14336 model for M from 1 to 8192.  Device
    time per call with the calls replayed from a CUDA graph.  For M <= 16 the roofline is HBM (the weights are
    streamed once), from 1024 on the tensor cores; in between neither is approached.  Parity: every (N, K) at
    M = 1 and 16 against the float64 oracle on all outputs."""
    import numpy as np
    from oracle import wush_oracle as wo
    grid, worst = {}, 0.0
    gen = torch.Generator(device=dev).manual_seed(17)
    peak4 = 4.0 * peaks["bf16_tflops"]
    for (n, k) in DECODE_SHAPES:
        wq = torch.randint(0, 256, (n, k // 2), generator=gen, device=dev, dtype=torch.uint8)
        wsf = torch.randint(118, 126, (n, k // 32), generator=gen, device=dev, dtype=torch.uint8)
        wsb = ops.to_blocked(wsf).view(-1)
        alpha = torch.tensor([1.0 / 9.0], device=dev)
        # consecutive calls read different copies of the weights, 256 MB in total (twice the L2), as the layers of
        # a model would: the small-M numbers are HBM numbers, not L2 numbers
        copies = [(wq, wsb)] + [(wq.clone(), wsb.clone()) for _ in range(int(np.ceil(2.56e8 / (n * k * 0.53125))) - 1)]
        for m in DECODE_M:
            xq = torch.randint(0, 256, (m, k // 2), generator=gen, device=dev, dtype=torch.uint8)
            xsf = torch.randint(122, 130, (m, k // 32), generator=gen, device=dev, dtype=torch.uint8)
            xsb = ops.to_blocked(xsf).view(-1)
            turn = [0]

            def fn():
                wq_i, wsb_i = copies[turn[0] % len(copies)] if m <= 128 else copies[0]
                turn[0] += 1
                return ops.matmul_fp4_blocked(xq, wq_i, xsb, wsb_i, alpha, "mx")
            for _ in range(3):
                fn()
            turn[0] = 0
            y = fn()                       # the parity check below reads the product with the first copy
            steps = 20 if m <= 1024 else 10
            us = _time_steps(fn, steps, torch, graph=True) * 1e3
            wbytes = n * k / 2 + n * k / 32 + m * k / 2 + m * k / 32 + 2.0 * m * n
            ent = {"us": us, "GBps": wbytes / us / 1e3, "TFLOPS": 2.0 * m * n * k / us / 1e6}
            if m <= 16:
                ent["frac_hbm"] = ent["GBps"] / peaks["hbm_gbs"]
                want = wo.fp4_gemm(xq.cpu().numpy(), xsf.cpu().numpy(), wq.cpu().numpy(), wsf.cpu().numpy(), 1.0 / 9.0, "mxfp4")
                got = y.double().cpu().numpy()
                worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            elif m >= 1024:
                ent["frac_tensor"] = ent["TFLOPS"] / peak4
            grid[f"N{n}_K{k}_M{m}"] = ent
    return {"metric": "mxfp4_decoder_shape_gemm_us", "unit": "us per call (device, graph replay)", "grid": grid,
            "value": grid["N4096_K4096_M1"]["us"],
            "config": {"workload": "MXFP4 GEMM, (N,K) of a hidden-4096 / FFN-14336 decoder layer x M in {1,16,128,1024,8192}, "
                                   "random codes, E8M0 scales within 2^-9..2^2; one launch per call (M <= 4: matrix-vector "
                                   "kernel on the CUDA cores; above: tcgen05 GEMM, K split inside a cluster); for M <= 128 "
                                   "successive calls read different weight copies (256 MB in rotation, twice the L2)"},
            "peak_kind": f"frac_hbm of {peak_kind} copy bandwidth (weights + activations + output once); frac_tensor of 4 x "
                         f"{peak_kind} bf16 burst",
            "gpu_launches": sum(5 + (20 if m <= 1024 else 10) for _ in DECODE_SHAPES for m in DECODE_M),   # warm-ups + replayed graph
            "parity": _parity("decode", worst, 1e-2, "worst relative Frobenius error over the four (N,K) at M = 1 and 16, all "
                                                      "outputs vs the float64 oracle")}


SHARD_M, SHARD_N, SHARD_K = 32768, 8192, 8192      # 16 x 2048 tokens through one hidden-8192 projection


def bench_sharded_gemm(args, dev, torch, dist, world, barrier) -> dict:
    """MXFP4 linear layer with the weight rows sharded over the ranks (70B-shape projection: 32768 tokens,
    8192 -> 8192): GEMM with the peer-store epilogue (the all-gather of the output columns happens inside the
    kernel) next to the local GEMM + NCCL all-gather baseline.  Activations are replicated.  Parity: the two paths
    must give the same bits on every rank, and this rank's columns must equal the unsharded kernel's."""
    from oracle import synth
    from wush_b200 import _lib
    from wush_b200 import qutlass_ops as ops
    from wush_b200.sharded import ColumnShardedFP4Linear, shard_bounds
    rank = dist.get_rank() if world > 1 else 0
    g = torch.Generator(device=dev).manual_seed(11)
    had = synth.to_bf16_tensor(synth.hadamard_matrix(32)).to(dev)
    x = torch.randn(SHARD_M, SHARD_K, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    xq, xs = ops._quantize(x, had, "mx", None, sf_layout=_lib.SF_BLOCKED)
    del x
    c0, c1 = shard_bounds(SHARD_N, world, rank)
    w = (torch.randn(c1 - c0, SHARD_K, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    wq, wsf = ops._quantize(w, had, "mx", None)
    del w
    res, outs = {}, {}
    for name, peer in (("fused", True), ("nccl", False)):
        layer = ColumnShardedFP4Linear(wq, wsf[: c1 - c0, : SHARD_K // 32], SHARD_N, "mx", 1.0 / 9.0, max_tokens=SHARD_M,
                                       peer=peer)
        for _ in range(3):
            layer.forward(xq, xs.view(-1))
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = layer.forward(xq, xs.view(-1))
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name + "_ms"] = float(t.item())
        res[name + "_path"] = "peer-store epilogue" if layer.fused else ("NCCL all-gather" if world > 1 else "local")
        outs[name] = out[::257].clone()            # every 257th row: 128 rows spread over all row blocks
        if name == "nccl":
            local = ops.matmul_fp4_blocked(xq, wq, xs.view(-1), layer.ws, layer.alpha, "mx")[::257]
            same_cols = bool(torch.equal(outs["fused"][:, c0:c1], local))
        del layer
    bad = torch.tensor([0 if (torch.equal(outs["fused"], outs["nccl"]) and same_cols) else 1], device=dev)
    if world > 1:
        dist.all_reduce(bad)
    flops = 2.0 * SHARD_M * SHARD_N * SHARD_K
    gather_bytes = SHARD_M * (SHARD_N - (c1 - c0)) * 2          # what every rank must receive
    return {"metric": "column_sharded_mxfp4_linear_TFLOPS", "value": flops / (res["fused_ms"] * 1e-3) / 1e12,
            "unit": "TFLOP/s", "ms_per_step": res["fused_ms"], **res,
            "nccl_baseline_TFLOPS": flops / (res["nccl_ms"] * 1e-3) / 1e12,
            "config": {"workload": f"MXFP4 linear M={SHARD_M} K={SHARD_K} N={SHARD_N}, weight rows sharded over {world} "
                                   f"GPUs, activations replicated, complete bf16 output on every rank"},
            "gather_bytes_per_rank": gather_bytes,
            "nvlink_floor_ms": gather_bytes / 770e9 * 1e3, "gpu_launches": 2 * args.steps, "scaling": "strong",
            "parity": _parity("sharded", float(bad.item()), 0.0, "ranks on which the fused output differs from the NCCL "
                              "all-gather output or from the unsharded kernel on this rank's columns (128 sampled rows)")}


SWEEP_ROWS, SWEEP_COLS, SWEEP_CALIB = 4096, 4096, 32768


def bench_sweep(args, dev, torch) -> dict:
    """Column sweep of one 4096 x 4096 layer (MXFP4, WUSH transforms, second moment from 16 x 2048 synthetic
    calibration tokens): round-to-nearest (all blocks in one kernel launch) and GPTQ (block after block).
    Every rank sweeps its own layer: layers are independent, there is no collective."""
    from oracle import synth
    from wush_b200 import gptq
    from wush_b200.hessian import accumulate_hessian
    x = synth.activations(SWEEP_CALIB, SWEEP_COLS, seed=400).to(dev)
    h = accumulate_hessian(torch.zeros(SWEEP_COLS, SWEEP_COLS, device=dev), x)
    h /= SWEEP_CALIB
    del x
    w = synth.weights(SWEEP_ROWS, SWEEP_COLS, seed=401).to(dev)
    out = {}
    with ClockSampler(dev.index) as clocks:
        for name, rtn, reps in (("rtn", True, 3), ("gptq", False, 1)):
            gptq.gptq_babai_sweep(w, h, "mxfp4", "wush", force_rtn=rtn)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(reps):
                gptq.gptq_babai_sweep(w, h, "mxfp4", "wush", force_rtn=rtn)
            torch.cuda.synchronize()
            out[name + "_ms_per_layer"] = (time.perf_counter() - t0) * 1e3 / reps
    nb = SWEEP_COLS // 32
    return {"metric": "column_sweep_weight_rows_per_s", "value": SWEEP_ROWS / (out["rtn_ms_per_layer"] * 1e-3),
            "unit": "rows/s", **out,
            "config": {"workload": f"W {SWEEP_ROWS}x{SWEEP_COLS} bf16 N(0,0.02^2), MXFP4, WUSH transforms, H from "
                                   f"{SWEEP_CALIB} synthetic tokens; host wall clock incl. Cholesky and all torch ops"},
            "gpu_launches": 4 * (1 + nb), "clocks": clocks.summary(),
            "note": "value is the round-to-nearest sweep; gptq_ms_per_layer is the "
            "sequential nearest-plane sweep (one wush_gptq_block_step launch per 32-column block)"}


def cpu_sweep_throughput() -> dict:
    """The oracle's restatement of gptq_babai_outer (round-to-nearest, WUSH transforms) on a bounded sample:
    all 4096 input channels, 256 of the 4096 weight rows (rows are independent; the Cholesky factorization
    of H is a fixed cost paid in both arms)."""
    import numpy as np
    from oracle import synth
    from oracle import wush_oracle as wo
    rows = 256
    x = synth.bf16_to_f64(synth.activations(4096, SWEEP_COLS, seed=400))
    h = x.T @ x / x.shape[0]
    w = synth.bf16_to_f64(synth.weights(rows, SWEEP_COLS, seed=401))
    t0 = time.perf_counter()
    wo.gptq_babai_outer(w, h, "mxfp4", "wush", True)
    sec = time.perf_counter() - t0
    return {"value": rows / sec, "unit": "rows/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{rows} of {SWEEP_ROWS} weight rows, all {SWEEP_COLS} channels, round-to-nearest sweep in "
                      f"NumPy float64 (BLAS threads as configured): {sec:.2f} s"}


def bench_hessian(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind, HESS_HIDDEN=HESS_HIDDEN) -> dict:
    """GPTQ Hessian over 128 x 2048 calibration tokens, tokens sharded over the ranks; the ranks are combined over
    NVLink (peer-memory / NVSwitch reduce kernel) panel by panel while later tiles are still being multiplied, then
    the mirror image is rebuilt.  Parity: sampled 256 x 256 blocks of the timed result against a float64
    accumulation of the same seeded shards (summed over the ranks), and all ranks must hold the same bits."""
    from wush_b200.hessian import DistributedHessian
    local = HESS_TOKENS // world
    g = torch.Generator(device=dev).manual_seed(200 + rank)
    outl = torch.randperm(HESS_HIDDEN, generator=torch.Generator().manual_seed(1))[: int(0.005 * HESS_HIDDEN)].to(dev)
    x = torch.empty(local, HESS_HIDDEN, device=dev, dtype=torch.bfloat16)
    for r0 in range(0, local, 16384):          # generate in slices: the fp32 temporary stays small
        blk = torch.randn(min(16384, local - r0), HESS_HIDDEN, generator=g, device=dev, dtype=torch.float32)
        blk[:, outl] *= 50.0
        x[r0:r0 + blk.shape[0]] = blk.to(torch.bfloat16)
    del blk
    events: list = []
    info = {}
    marks: list = []
    if args.timeline and world > 1:
        # CUDA events around every cross-GPU combine (barrier, reduce, barrier, mirror) on the stream it runs on
        from wush_b200 import hessian as hz
        inner = hz._PeerBuffers.combine

        def combine(self, hidden, a, b, channel, **kw):
            st = torch.cuda.current_stream(self.flat.device)
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record(st)
            inner(self, hidden, a, b, channel, **kw)
            ev[1].record(st)
            marks.append((channel, a, b, ev))
        hz._PeerBuffers.combine = combine

    def job():
        dh = DistributedHessian(HESS_HIDDEN, dev)
        dh.profile = events
        dh.accumulate_overlapped(x)
        h = dh.finalize()
        info["path"] = ("multimem (NVSwitch) reduce" if dh._peer is not None and dh._peer.mc_ptr else
                        "peer-memory reduce" if dh._peer is not None else ("NCCL all-reduce" if world > 1 else "single GPU"))
        dh.release()          # peer-memory buffers go back to the pool for the next job
        return h

    # enough jobs for a timed region of several milliseconds at any number of GPUs (a job shrinks with the shard)
    steps = (5 if HESS_HIDDEN <= 4096 else 3) * (1 if world == 1 else 4 if HESS_HIDDEN <= 4096 else 2)
    steps = max(1, min(steps, max(args.steps, 1) * 4))
    for _ in range(2):
        job()
    barrier()
    del events[:]
    del marks[:]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for _ in range(steps):
            h = job()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1) / steps
    timeline = None
    if marks:
        per_job = len(marks) // steps
        last = marks[-per_job:]
        timeline = {"combines_of_the_last_job": [{"stream": "side (overlaps the next panel's accumulation)" if ch == 0 else "main (tail)",
                                                   "tiles": [a, b], "us": ev[0].elapsed_time(ev[1]) * 1e3} for ch, a, b, ev in last],
                    "accumulate_end_to_tail_combine_start_us": events[-1][1].elapsed_time(last[-1][3][0]) * 1e3}
    # the accumulation launches of the timed jobs themselves (events around them on the launching stream)
    kms = sum(a.elapsed_time(b) for a, b in events) / max(1, len(events))
    t = torch.tensor([ms, kms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, kms = (float(v) for v in t.tolist())

    # ---- parity of the timed result --------------------------------------------------------------------
    nb = HESS_HIDDEN // 256
    blocks = sorted({(0, 0), (nb - 1, 0), (nb - 1, nb - 1), (nb // 2, nb // 3), (nb // 3, nb // 3)})
    worst = 0.0
    for bi, bj in blocks:
        xi = x[:, bi * 256:(bi + 1) * 256].double()
        xj = x[:, bj * 256:(bj + 1) * 256].double()
        want = xi.t() @ xj                       # float64 on this rank's tokens
        if world > 1:
            dist.all_reduce(want)
        want /= HESS_TOKENS
        got = h[bi * 256:(bi + 1) * 256, bj * 256:(bj + 1) * 256].double()
        worst = max(worst, float((got - want).abs().max() / want.abs().max()))
        if not torch.equal(h[bj * 256:(bj + 1) * 256, bi * 256:(bi + 1) * 256], h[bi * 256:(bi + 1) * 256, bj * 256:(bj + 1) * 256].t()):
            worst = float("inf")                 # the mirror image must be exact
    if world > 1:
        # every rank must hold the same bits: compare a bit-level checksum of the whole matrix
        cs = h.view(torch.int32).to(torch.int64).sum().reshape(1)
        lo, hi = cs.clone(), cs.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if int(lo.item()) != int(hi.item()):
            worst = float("inf")
        w = torch.tensor([worst], dtype=torch.float64, device=dev)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        worst = float(w.item())
    tri_flops = float(local) * HESS_HIDDEN * (HESS_HIDDEN + 1)
    ach = tri_flops / (kms * 1e-3) / 1e12
    # a job of tens of milliseconds runs power-capped: compare with the sustained bf16 figure there
    long_job = ms > 20.0
    peak = peaks["bf16_tflops_sustained"] if long_job else peaks["bf16_tflops"]
    from wush_b200.hessian import tile_panels, token_segments
    segments = len(token_segments(local))
    launches_per_job = segments + 1
    return {"metric": "hessian_tokens_per_s", "value": HESS_TOKENS / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms,
            "scaling": "strong", "steps": steps,
            "config": {"workload": f"H = X^T X / N over {HESS_TOKENS} tokens (128 x 2048), hidden {HESS_HIDDEN}, bf16 "
                                   f"in / fp32 out, {local} tokens per GPU; ranks combined by: {info.get('path')}"},
            "combine_path": info.get("path"), "timeline": timeline,
            "gpu_launches": steps * launches_per_job,
            "roofline": {"bound": "tensor", "kernel": "hessian_pair_kernel", "achieved": ach, "peak": peak,
                         "unit": "TFLOP/s", "frac": ach / peak,
                         "peak_kind": f"of {peak_kind} (bf16 {'sustained: the job runs tens of ms' if long_job else 'burst'})",
                         "algorithmic_flops_per_launch": tri_flops, "kernel_ms": kms,
                         "note": "flops of one triangle incl. diagonal, T*C*(C+1); the full-square equivalent is twice that; "
                                 "kernel_ms = CUDA events around the accumulation launches inside the timed jobs",
                         "traffic": None},
            "parity": _parity(f"hessian_{HESS_HIDDEN}", worst, 1e-5, f"max-abs error / max-abs value over {len(blocks)} sampled "
                              "256 x 256 blocks of the timed result vs a float64 accumulation of the same shards; mirror "
                              "exact; all ranks bit-identical"),
            "clocks": clocks.summary()}


def bench_layer_4096(args, dev, torch) -> dict:
    """The reference's CPU-runnable case on the GPU: one 4096 x 4096 layer, second moment from 16 x 2048 calibration
    tokens, MXFP4 round-to-nearest sweep with WUSH transforms, then the real-quant forward of 2048 tokens (fused
    transform + quantize, FP4 GEMM).  Next to it the CPU pseudo-quantizer (the oracle) on a bounded sample: the sweep
    of 64 weight rows and the activation quantizer + float64 product for the same 64 output features, whose result
    is also the parity check of the GPU layer."""
    import numpy as np
    from oracle import synth
    from oracle import wush_oracle as wo
    from wush_b200 import gptq
    from wush_b200.hessian import DistributedHessian
    from wush_b200.linear import FPQuantConfig, FPQuantDtype, FPQuantLinear
    hidden, tokens = 4096, 2048
    calib = [synth.activations(2048, hidden, seed=500 + i).to(dev) for i in range(16)]
    w = synth.weights(hidden, hidden, seed=520)
    x = synth.activations(tokens, hidden, seed=530)
    wd, xd = w.to(dev), x.to(dev)

    def calibrate():
        dh = DistributedHessian(hidden, dev, peer=False)
        for c in calib:
            dh.update(c[None])
        return dh.finalize()

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            out = fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / reps, out

    with ClockSampler(dev.index) as clocks:
        t_h, h = timed(calibrate, 3)
        t_s, res = timed(lambda: gptq.gptq_babai_sweep(wd, h, "mxfp4", "wush", force_rtn=True), 3)
        entry = gptq.export_realquant({k: res[k] for k in ("transform_basis", "qweight", "scale_quant", "global_scale")}, "mxfp4")
        layer = FPQuantLinear(hidden, hidden, FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, transform_init="wush"),
                              bias=False, device=dev)
        layer.load_quantized(entry["qweight"], entry["scales"], entry["forward_hadamard_matrix"],
                             entry["weight_global_scale"], entry["act_global_scale"])
        y = layer(xd)
        t_f = _time_steps(lambda: layer(xd), 20, torch, graph=True)
    # ---- CPU pseudo-quantizer on a sample, same transforms -------------------------------------------------
    rows = np.sort(np.random.default_rng(0).choice(hidden, size=64, replace=False))
    t = res["transform_basis"].double().cpu().numpy()
    h64 = h.double().cpu().numpy()
    t0 = time.perf_counter()
    ref_w = wo.gptq_babai_outer(synth.bf16_to_f64(w)[rows], h64, "mxfp4", "wush", True, transform_fn=lambda b, basis, yy: t[b])
    cpu_sweep = time.perf_counter() - t0
    t0 = time.perf_counter()
    ref_x = wo.fused_transform_quant(synth.bf16_to_f64(x), wo.transform_to_matrix(t), "mxfp4")["fake_quant"]
    want = ref_x @ ref_w["fake_quant"].T
    cpu_fwd = time.perf_counter() - t0
    got = y.double().cpu().numpy()[:, rows]
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    code_bad = float(np.mean(wo.unpack_e2m1_codes(res["qweight"].cpu().numpy()[rows]) != ref_w["codes"]))
    scale_ok = bool(np.array_equal(res["scale_quant"].view(torch.uint8).cpu().numpy()[rows], ref_w["scale_quant"]))
    par = _parity("layer_4096", rel if scale_ok and code_bad <= 1e-3 else float("inf"), 1e-2,
                  "relative Frobenius error of 2048 x 64 sampled outputs of the real-quant layer vs the CPU pseudo-quantizer "
                  "(oracle sweep + oracle activation quantizer + float64 product); weight scale bytes identical, codes "
                  f"differing on {code_bad:.1e} of the sampled elements")
    return {"metric": "layer_4096_quantize_and_forward_ms", "value": t_h + t_s + t_f, "unit": "ms", "ms_per_step": t_h + t_s + t_f,
            "hessian_ms": t_h, "sweep_ms": t_s, "forward_ms": t_f,
            "forward_TFLOPS": 2.0 * tokens * hidden * hidden / (t_f * 1e-3) / 1e12,
            "config": {"workload": "W 4096 x 4096 bf16 N(0, 0.02^2); X 2048 x 4096 bf16 N(0,1) with 0.5 % outlier channels x 50; "
                                   "16 x 2048 calibration tokens; MXFP4, group 32, round-to-nearest sweep, WUSH transforms"},
            "cpu_baseline": {"value": (cpu_sweep * hidden / 64 + cpu_fwd * hidden / 64) * 1e3, "unit": "ms (extrapolated to all 4096 "
                             "output features)", "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": f"64 of 4096 weight rows: sweep {cpu_sweep:.2f} s, activation quantizer + product "
                                       f"{cpu_fwd:.2f} s (NumPy float64)"},
            "gpu_launches": 3 * (16 + 6) + 22, "parity": par, "clocks": clocks.summary()}


BLOCK_TOKENS, BLOCK_SEQ = 16 * 2048, 2048


def bench_block(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind) -> dict:
    """The seven W4A4 linears (plus attention, norms, SwiGLU) of one decoder block of a hidden-8192 / 64-head /
    8-KV-head / FFN-28672 model on 16 x 2048 tokens, weights column-sharded over the GPUs, FP4 codes exchanged
    through NVLink by the copy engines while the other micro-batch multiplies.  Parity: the first sequence of the
    timed configuration against a step-by-step restatement (dequantized codes, fp32 matmuls) of the whole block
    computed on every rank with the unsharded weights."""
    import torch.nn.functional as F
    from oracle import synth
    from wush_b200.block import BlockConfig, ShardedDecoderBlock, quantize_block_weights
    from wush_b200.gptq import dequantize
    from wush_b200 import qutlass_ops as ops
    cfg = BlockConfig()
    H, FF, d = cfg.hidden, cfg.ffn, cfg.head_dim
    kv = cfg.n_kv_heads * d
    gen = torch.Generator(device=dev).manual_seed(31)           # the same weights on every rank
    shapes = {"q": (H, H), "k": (kv, H), "v": (kv, H), "o": (H, H), "gate": (FF, H), "up": (FF, H), "down": (H, FF)}
    had = synth.to_bf16_tensor(synth.hadamard_matrix(32))
    transforms = {"attn_in": synth.to_bf16_tensor(synth.wush_matrix(H, 32, seed=41)), "o": had,
                  "mlp_in": synth.to_bf16_tensor(synth.wush_matrix(H, 32, seed=42)),
                  "down": synth.to_bf16_tensor(synth.wush_matrix(FF, 32, seed=43))}
    qw = {}
    for name, (r, c) in shapes.items():
        w = (torch.randn(r, c, generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        qw.update(quantize_block_weights(cfg, {name: w}, transforms, dev))
        del w
    gammas = (torch.ones(H, dtype=torch.bfloat16), torch.ones(H, dtype=torch.bfloat16))
    hs = H // world
    h_full0 = torch.randn(BLOCK_SEQ, H, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)   # sequence 0
    h = torch.randn(BLOCK_TOKENS, hs, generator=torch.Generator(device=dev).manual_seed(50 + rank), device=dev,
                    dtype=torch.float32).to(torch.bfloat16)
    h[:BLOCK_SEQ] = h_full0[:, rank * hs:(rank + 1) * hs]
    blk = ShardedDecoderBlock(cfg, qw, transforms, gammas, BLOCK_SEQ, BLOCK_TOKENS, dev, micro_batches=int(os.environ.get("WUSH_B200_BLOCK_MICRO_BATCHES", "2")) if world > 1 else 1)

    # ---- parity on sequence 0 (before the timed loop changes h) ---------------------------------------------
    first = blk.forward(h.clone())[:BLOCK_SEQ].float()

    def linear(x, t, names):
        q, sf = ops._quantize(x.contiguous(), t.to(dev), "mx", None)
        xd = dequantize(q, sf[: x.shape[0], : x.shape[1] // 32], "mxfp4")
        outs = []
        for nme in names:
            wd = dequantize(*qw[nme], "mxfp4")
            outs.append((xd @ wd.t()).to(torch.bfloat16))
            del wd
        return outs

    def norm(x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)).to(torch.bfloat16)

    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    hr = h_full0.clone()
    q_, k_, v_ = linear(norm(hr), transforms["attn_in"], ("q", "k", "v"))
    sh = lambda t, nh: t.view(1, BLOCK_SEQ, nh, d).transpose(1, 2)
    o = F.scaled_dot_product_attention(sh(q_, cfg.n_heads), sh(k_, cfg.n_kv_heads), sh(v_, cfg.n_kv_heads), is_causal=True,
                                       enable_gqa=True)
    hr = linear(o.transpose(1, 2).reshape(BLOCK_SEQ, -1), had, ("o",))[0] + hr
    g_, u_ = linear(norm(hr), transforms["mlp_in"], ("gate", "up"))
    want = (linear(F.silu(g_) * u_, transforms["down"], ("down",))[0] + hr)[:, rank * hs:(rank + 1) * hs].float()
    torch.backends.cuda.matmul.allow_tf32 = old_tf32
    err = torch.stack([(first - want).norm() ** 2, want.norm() ** 2])
    if world > 1:
        dist.all_reduce(err)
    rel = float((err[0] / err[1]).sqrt())
    del want, first, hr, g_, u_, q_, k_, v_, o

    steps = max(2, min(args.steps, 8))
    for _ in range(2):
        blk.forward(h)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for _ in range(steps):
            blk.forward(h)
        e1.record()
        barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    lin_flops = 2.0 * BLOCK_TOKENS * (H * (H + 2 * kv) + H * H + 3 * H * FF)
    code_bytes = BLOCK_TOKENS * (3 * H + FF) * (0.5 + 1.0 / 32) * (world - 1) / world       # received per rank
    return {"metric": "w4a4_decoder_block_forward_ms", "value": ms, "unit": "ms per block", "ms_per_step": ms,
            "higher_is_better": False, "scaling": "strong", "steps": steps,
            "linear_TFLOPS": lin_flops / (ms * 1e-3) / 1e12,
            "frac_of_nominal_dense_fp4_per_gpu": lin_flops / (ms * 1e-3) / 1e12 / world / FP4_NOMINAL_TFLOPS,
            "model_forward_ms_80_blocks": 80 * ms,
            "nvlink_bytes_received_per_rank": code_bytes, "nvlink_floor_ms": code_bytes / 770e9 * 1e3,
            "config": {"workload": f"one decoder block, hidden {H}, {cfg.n_heads} heads / {cfg.n_kv_heads} KV heads, FFN {FF}, "
                                   f"{BLOCK_TOKENS // BLOCK_SEQ} x {BLOCK_SEQ} tokens, MXFP4 W4A4 (per-group WUSH matrices on "
                                   f"the q/k/v, gate/up and down inputs, Hadamard on the o_proj input), weight rows of all "
                                   f"seven linears sharded over {world} GPU(s); attention = torch SDPA on local heads; "
                                   f"embedding and lm_head (not quantized in the reference) are not part of it"},
            "gpu_launches": steps * 8 * (2 if world > 1 else 1),
            "parity": _parity("block_70b", rel, 1e-2, "relative Frobenius error of the block output on the first sequence vs a "
                              "step-by-step fp32 restatement with the unsharded weights (all ranks)"),
            "clocks": clocks.summary()}


def _compact(sec: dict) -> dict:
    """The figures of a section a reader of the one-line record needs."""
    out = {k: sec[k] for k in ("metric", "value", "unit", "ms_per_step", "combine_path", "fused_ms", "nccl_ms",
                               "rtn_ms_per_layer", "gptq_ms_per_layer", "frac", "linear_TFLOPS",
                               "frac_of_nominal_dense_fp4_per_gpu", "model_forward_ms_80_blocks", "hessian_ms", "sweep_ms",
                               "forward_ms") if k in sec}
    if "roofline" in sec:
        out["frac"] = sec["roofline"]["frac"]
        out["peak_kind"] = sec["roofline"]["peak_kind"]
        if "frac_of_nominal_dense_fp4" in sec["roofline"]:
            out["frac_of_nominal_dense_fp4"] = sec["roofline"]["frac_of_nominal_dense_fp4"]
        if "kernel_ms" in sec["roofline"]:
            out["kernel_ms"] = sec["roofline"]["kernel_ms"]
    if "parity" in sec:
        out["parity"] = {k: sec["parity"][k] for k in ("max_rel", "tol", "ok")}
    if "clocks" in sec:
        out["clocks"] = sec["clocks"]
    if "cublaslt" in sec:
        out["cublaslt_TFLOPS"] = sec["cublaslt"].get("TFLOPS", sec["cublaslt"].get("unavailable"))
    if "grid" in sec:
        out["grid_us"] = {k: round(v["us"], 2) for k, v in sec["grid"].items()}
        out["frac_hbm"] = {k: round(v["frac_hbm"], 3) for k, v in sec["grid"].items() if "frac_hbm" in v}
    return out


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from oracle import synth
    from wush_b200 import _lib
    from wush_b200 import qutlass_ops as ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL prints its version banner on stdout when the first communicator is made: stdout is for the JSON line
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks, peak_kind = measured_peaks()
    warmup = max(args.warmup, 3)

    single = {"gemm": lambda: bench_gemm(args, dev, torch, ops, peaks, peak_kind),
              "gemm_nv": lambda: bench_gemm(args, dev, torch, ops, peaks, peak_kind, "nv"),
              "quant_nv": lambda: bench_quant_nv(args, dev, torch, ops, peaks, peak_kind),
              "decode": lambda: bench_decode(args, dev, torch, ops, peaks, peak_kind),
              "sharded": lambda: bench_sharded_gemm(args, dev, torch, dist, world, barrier),
              "sweep": lambda: bench_sweep(args, dev, torch),
              "layer": lambda: bench_layer_4096(args, dev, torch),
              "block": lambda: bench_block(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind),
              "hessian": lambda: bench_hessian(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind,
                                               HESS_HIDDEN=args.hess_hidden)}
    if args.only in single:
        res = single[args.only]()
        if rank == 0:
            res.update({"n_gpus": world, "only": args.only, "data": "synthetic"})
            print(json.dumps(res), flush=True)
        if world > 1:
            dist.destroy_process_group()
        if PARITY_FAILURES:
            raise SystemExit(f"parity check failed: {PARITY_FAILURES}")
        return

    # ---- fused transform + quantize: every rank its own shard of rows, same matrices -------------
    x_host = synth.activations(TOKENS, HIDDEN, seed=100 + rank).pin_memory()
    mat_np = synth.wush_matrix(HIDDEN, GROUP)
    mat = synth.to_bf16_tensor(mat_np).to(dev)
    x = x_host.to(dev)
    alg = algorithmic_bytes(TOKENS, HIDDEN)

    def step():
        return ops.fused_quantize_mx_wush_op(x, mat, "abs_max", False)

    for _ in range(warmup):
        out = step()
    # the K timed steps are one CUDA graph: K calls of the public op, replayed with one launch
    replay = _capture_steps(step, args.steps, torch)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record()
        if replay is not None:
            replay()
        else:
            for _ in range(args.steps):
                step()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)

        # kernel-only duration: events directly around the launches on the launching stream
        lib = _lib.load()
        q = torch.empty(TOKENS, HIDDEN // 2, dtype=torch.uint8, device=dev)
        sf = torch.empty(TOKENS, HIDDEN // GROUP, dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream().cuda_stream

        def launch():
            rc = lib.wush_fused_quantize_mx(x.data_ptr(), mat.data_ptr(), HIDDEN, q.data_ptr(), sf.data_ptr(),
                                            HIDDEN // GROUP, 0, TOKENS, HIDDEN, 0, stream)
            assert rc == 0, rc

        kernel_ms = _time_steps(launch, args.steps, torch)
    clock_summary = clocks.summary()
    quant_par = quant_parity(x_host, mat_np, out[0], out[1], "mxfp4", torch)
    del out

    # end to end: pinned host activations in, codes + scales back to pinned host memory
    e2e_ms = float("nan")
    q_host = torch.empty(TOKENS, HIDDEN // 2, dtype=torch.uint8).pin_memory()
    sf_host = torch.empty(TOKENS, HIDDEN // GROUP, dtype=torch.uint8).pin_memory()
    if not args.kernel_only:
        # the public host-buffer entry point: row chunks, upload / kernel / download overlapped on three streams
        from wush_b200.host_stream import HostQuantizer
        hq = HostQuantizer(HIDDEN, mat, "mx", chunk_rows=2048, device=dev)

        def e2e_step():
            hq(x_host, q_host, sf_host)

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
        hq.synchronize()
        if not (torch.equal(q_host, q.cpu()) and torch.equal(sf_host, sf.cpu())):
            PARITY_FAILURES.append("e2e")       # the host-buffer pass must give the bytes of the single launch

    times = torch.tensor([ms, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, kernel_ms = (float(v) for v in times.tolist())
    del x, q, sf, x_host, q_host, sf_host

    extra = {}
    if not args.kernel_only and args.only == "all":
        extra["gemm"] = single["gemm"]()
        extra["hessian"] = bench_hessian(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind)
        extra["hessian_14336"] = bench_hessian(args, dev, torch, dist, rank, world, barrier, peaks, peak_kind, HESS_HIDDEN=14336)
        if world == 1:
            # single-GPU paths: measured once, not again at every N of a scaling run
            extra["quant_nvfp4"] = single["quant_nv"]()
            extra["gemm_nvfp4"] = single["gemm_nv"]()
            extra["decode"] = single["decode"]()
            extra["sweep"] = single["sweep"]()
            extra["layer_4096"] = single["layer"]()
        else:
            extra["sharded"] = single["sharded"]()
        extra["block_70b"] = single["block"]()

    if rank == 0:
        value = world * alg * args.steps / (ms * 1e-3) / 1e9
        e2e_value = world * alg * args.steps / (e2e_ms * 1e-3) / 1e9
        achieved = alg / (kernel_ms * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.kernel_only and args.only == "all":
            cpu = cpu_quant_throughput(512, HIDDEN, repeats=2)
            cpu.pop("seconds", None)
            extra["gemm"]["cpu_baseline"] = cpu_gemm_throughput()
            extra["hessian"]["cpu_baseline"] = cpu_hessian_throughput()
            extra["sweep"]["cpu_baseline"] = cpu_sweep_throughput()
        launches = args.steps + sum(v.get("gpu_launches", 0) for v in extra.values())
        line = {
            "metric": "fused_transform_quant_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": TOKENS * HIDDEN * 2,
                    "d2h_bytes_per_step": TOKENS * HIDDEN // 2 + TOKENS * HIDDEN // GROUP,
                    "ms_per_step": e2e_ms / args.steps,
                    "path": "wush_b200.host_stream.HostQuantizer: pinned host buffers, 2048-row chunks, upload / "
                            "kernel / download overlapped on three streams"},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "kernel": "fused_quantize_kernel<MX>", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": alg,
                         "kernel_ms": kernel_ms, "traffic": quant_traffic_bytes(TOKENS, HIDDEN)},
            "cpu_baseline": cpu,
            "clocks": clock_summary,
            "parity": {k: quant_par[k] for k in ("max_rel", "tol", "ok")},
        }
        for name, sec in extra.items():
            line[name] = _compact(sec)
        line["parity_failures"] = list(PARITY_FAILURES)
        line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if PARITY_FAILURES:
        raise SystemExit(f"parity check failed: {PARITY_FAILURES}")


# DRAM bytes per launch of the quantize kernel: dram__bytes_read.sum + dram__bytes_write.sum of the ncu
# capture summarised in profiles/fused_quantize_mx_8192x8192.md (134.78 MB + 18.4 MB for 8192 x 8192),
# scaled by elements to the launched shape.  In that small case about half of the 35.7 MB output is still
# dirty in L2 when the kernel ends, so the write part under-counts what a 125 MB output writes back.
def quant_traffic_bytes(tokens: int, hidden: int) -> float:
    return (134.78e6 + 18.4e6) * (tokens * hidden) / (8192.0 * 8192.0)


def cpu_gemm_throughput() -> dict:
    """CPU restatement of the reference GEMM semantics (dequantize both operands, fp32 matmul) on a
    bounded sample of the 8192^3 workload."""
    import torch
    from oracle import torch_port
    m, n, k = 2048, 8192, GEMM_K
    g = torch.Generator().manual_seed(3)
    a = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    b = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    sa = torch.randint(120, 130, (m, k // 32), generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 130, (n, k // 32), generator=g, dtype=torch.uint8)
    torch.set_num_threads(os.cpu_count() or 1)
    torch_port.fp4_gemm(a[:32], sa[:32], b[:32], sb[:32], 1.0, "mxfp4")
    t0 = time.perf_counter()
    torch_port.fp4_gemm(a, sa, b, sb, 1.0 / 9.0, "mxfp4")
    sec = time.perf_counter() - t0
    return {"value": 2.0 * m * n * k / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"M={m}, N={n} of the 8192^3 problem (K full), dequantize + fp32 matmul on CPU: {sec:.2f} s"}


def cpu_hessian_throughput() -> dict:
    """WUSH.update arithmetic on CPU (fp32, the Triton launch replaced by addmm) for a few sequences."""
    import torch
    from oracle import synth, torch_port
    torch.set_num_threads(os.cpu_count() or 1)
    seqs, tok = 25, 2048
    xs = [synth.activations(tok, HESS_HIDDEN, seed=300 + i) for i in range(seqs)]
    h, n = torch.zeros(HESS_HIDDEN, HESS_HIDDEN), 0
    n = torch_port.hessian_update(h, n, xs[0][None])
    t0 = time.perf_counter()
    for x in xs[1:]:
        n = torch_port.hessian_update(h, n, x[None])
    sec = time.perf_counter() - t0
    return {"value": (seqs - 1) * tok / sec, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{seqs - 1} of 128 sequences of {tok} tokens, hidden {HESS_HIDDEN}, fp32 running-mean update on CPU: "
                      f"{sec:.2f} s"}


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
    ap.add_argument("--only", default="all", choices=["all", "quant", "quant_nv", "gemm", "gemm_nv", "decode", "hessian", "sweep", "sharded", "block", "layer"],
                    help="run one section only (profiler captures of a single kernel on a small case)")
    ap.add_argument("--gemm-size", type=int, default=GEMM_M, help="M = N = K of the GEMM section")
    ap.add_argument("--hess-tokens", type=int, default=HESS_TOKENS)
    ap.add_argument("--hess-hidden", type=int, default=HESS_HIDDEN)
    ap.add_argument("--timeline", action="store_true",
                    help="Hessian section on several GPUs: also report CUDA-event durations of every cross-GPU combine")
    args = ap.parse_args()
    g = globals()
    g["TOKENS"], g["HIDDEN"] = args.tokens, args.hidden
    g["GEMM_M"] = g["GEMM_N"] = g["GEMM_K"] = args.gemm_size
    g["HESS_TOKENS"] = args.hess_tokens
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
