#!/usr/bin/env python
"""Benchmark of the cleave tensor hot path on B200.

Headline metric: f32 GEMM TFLOP/s at M = N = K = 8192 (algorithmic flops 2*M*N*K, not counting the
3x of the TF32 split), one problem per GPU per step.  With N GPUs every rank multiplies its own
8192^3 problem (independent units, no collective: weak scaling), launched as
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
Rank 0 prints ONE JSON line.

  value     whole-job TFLOP/s, operands resident in HBM when the timed region starts
            (each step = operand split pre-pass + tcgen05 GEMM kernel)
  e2e       the same metric through the C ABI with HOST buffers: per step both operands are
            copied from pinned host memory, multiplied, and C is copied back
  roofline  the tcgen05 kernel alone (CUDA events around each launch on the launching stream)
            against the 3xTF32-effective tensor peak
  cpu_baseline  the CPU oracle (restatement of the reference's loop) on a bounded row slice of the
            same problem: all host threads, and one thread (the reference itself is single-threaded)
  mlp_fwd_bwd   the second half of the metric, "MLP fwd+bwd samples/s vs host CPU" (configuration 2):
            device-resident and end-to-end samples/s, its own roofline and its own CPU baseline; the same
            record is repeated under roofline / cpu_baseline / e2e as `mlp_fwd_bwd`
  sharded   the workloads that shard over GPUs, run by the same ranks after the headline: batched
            64 x 4096^3 by batch index, 16384^3 by row blocks, data-parallel MLP training at global batch
            32768 (fused exchange kernel and NCCL); at N = 1 the same workloads on one rank, so every
            N > 1 line has its one-GPU time from the same series of runs
  secondary the linear-regression step in GB/s (configuration 1)

`--impl reference` times the reference's CPU arithmetic (the oracle; the reference itself is Rust +
MLIR and cannot be built here) on the same workload, each step a bounded row slice.
Inputs are seeded synthetic data (the workload is defined by shapes and distributions).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192          # headline size; --size overrides it for profiling captures only
FLOPS = 2.0 * M * N * K
# DRAM traffic of one tcgen05 GEMM kernel launch at 8192^3: not measured by this program (it needs a
# profiler) but taken from a one-pass ncu capture of it at full size (dram__bytes_read.sum +
# dram__bytes_write.sum).  The record names the capture, so a value that no longer matches the kernel shows.
NCU_TRAFFIC = {"bytes_per_launch": 4.633e9 + 268.3e6,
               "kernel": "gemm_3xtf32_pair_kernel<0, 1, 32> (256x256 tiles on CTA pairs, K-block 32, 3 stages, "
                         "tile-rows in groups of 8)",
               "summary": "profiles/gemm_3xtf32_pair_kernel_8192cubed_group_size_and_traffic.md"}
NCU_TRAFFIC_BYTES_PER_LAUNCH = NCU_TRAFFIC["bytes_per_launch"]
NOMINAL_TF32_DENSE_TFLOPS = 1125.0   # datasheet, dense (half the 2:4-sparse figure), at the 1965 MHz boost clock


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs.  nvidia-smi needs a moment to
    start, so the sampler is started early and `stop(t0, t1)` keeps the samples stamped inside [t0, t1]
    (`time.time()` values around the timed region)."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "20"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self, t0: float | None = None, t1: float | None = None) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        self.f.seek(0)
        import datetime
        sm, mx, reasons, total = [], [], set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            total += 1
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, cmax = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if t0 is not None and not (t0 - 0.02 <= stamp <= t1 + 0.02):
                continue
            sm.append(clk)
            mx.append(cmax)
            for nm, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_outside_window": total - len(sm), "reasons": sorted(reasons)}


def cpu_gemm_sample(a: np.ndarray, b: np.ndarray, target_s: float = 10.0, threads: int | None = None):
    """Times the oracle GEMM on a row slice of the problem sized for ~target_s of CPU work."""
    from oracle import ref
    # torchrun exports OMP_NUM_THREADS=1; use every core we may unless a thread count is asked for
    ref.set_num_threads(threads if threads else _host_threads())
    rows = 8 if threads == 1 else 32
    t0 = time.perf_counter()
    ref.matmul_rows(a, b, 0, rows)
    dt = time.perf_counter() - t0
    rows = int(max(8, min(a.shape[0], rows * target_s / max(dt, 1e-3))))
    rows -= rows % 8
    t0 = time.perf_counter()
    ref.matmul_rows(a, b, 0, rows)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * b.shape[0] * b.shape[1] / dt / 1e12
    return tflops, rows, dt, ref.num_threads()


def headline_config(world: int) -> dict:
    """The workload description, identical in both arms (`--impl reference` times the same problem)."""
    return {"workload": f"f32 GEMM C=A*B, M=N=K={M}, uniform[-1,1), row-major; one problem per GPU per step",
            "l2": f"operands {M * K * 4 >> 20} MiB each (L2 is 126 MB)", "parallelism": f"replicas x{world}"}


def run_reference(args):
    """Reference arm: the CPU restatement of cleave's matmul loop, all host threads, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from cleave_b200 import workloads
    from oracle import ref
    ref.set_num_threads(_host_threads())
    a, b = workloads.gemm_inputs(M, N, K)
    rows = 64
    for _ in range(max(args.warmup, 1)):
        ref.matmul_rows(a, b, 0, rows)
    t0 = time.perf_counter()
    for i in range(args.steps):
        ref.matmul_rows(a, b, (i * rows) % (M - rows), rows)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": f"f32 GEMM TFLOP/s ({M}^3)", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": ref.num_threads(), "kind": "port",
                         "sample": f"{rows} of {M} rows of the product per step, {args.steps} steps; the reference's CPU "
                                   "arithmetic as restated by the oracle (the Rust + MLIR reference cannot be built "
                                   "here), OpenMP over rows"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


MLP_DIMS = (4096, 1024, 4096, 1024)   # batch, d_in, d_hid, d_out of configuration 2
MLP_GEMM_FLOPS = 5 * 2.0 * 4096 * 4096 * 1024   # two forward products, dZ1, dW2, dW1
# streaming passes of the step if nothing were fused: bias adds 128 + 32 MiB, tanh 128, sigmoid 32, MSE + dY 48,
# sigmoid' 48, tanh' 192, column sums 80 (read + write bytes)
MLP_STREAM_BYTES_UNFUSED = 688 * (1 << 20)


def mlp_record(cb, torch, L, peaks, peaks_kind, do_cpu=True, do_e2e=True, steps=30):
    """Configuration 2, "MLP fwd+bwd samples/s vs host CPU": batch 4096, 1024 -> 4096 (tanh) -> 1024 (sigmoid),
    MSE, all weight and bias gradients.  Returns {value.., roofline, cpu_baseline, e2e}."""
    from cleave_b200 import autodiff, linalg, workloads
    from cleave_b200._lib import c_f32p
    batch, d_in, d_hid, d_out = MLP_DIMS
    X, W1, b1, W2, b2, T = workloads.mlp_inputs()
    net = autodiff.MLP2(d_in, d_hid, d_out)
    net.load(W1, b1, W2, b2)
    tX, tT = linalg.Tensor(X), linalg.Tensor(T)
    loss_dev = linalg.Tensor.zero(1)
    for _ in range(3):
        net.forward_backward(tX, tT, loss_out=loss_dev)
    cb.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = L.cleave_cuda_kernel_launches()
    L.cleave_cuda_profile_begin()
    e0.record()
    for i in range(steps):
        net.forward_backward(tX, tT, loss_out=loss_dev)     # the loss stays on the device ...
        if (i + 1) % 10 == 0:
            loss = loss_dev[0]                                # ... and is read back as a training loop logs it
    e1.record()
    e1.synchronize()
    cnt = ctypes.c_int32(0)
    gemm_ms = L.cleave_cuda_profile_end(ctypes.byref(cnt)) / steps
    launches = (L.cleave_cuda_kernel_launches() - l0) / steps
    ms = e0.elapsed_time(e1) / steps
    tensor_peak = peaks["bf16_tflops_sustained"] / 6.0     # a step is a long sequence of kernels: sustained basis
    rec = {"metric": "MLP fwd+bwd samples/s", "value": batch / (ms * 1e-3), "unit": "samples/s", "ms_per_step": ms,
           "steps": steps, "loss": loss, "gpu_launches_per_step": launches,
           "config": "batch 4096, 1024->4096 tanh->1024 sigmoid, MSE vs uniform[0,1) targets, Xavier weights, f32; loss "
                     "read back every 10 steps",
           "roofline": {"bound": "tensor", "achieved": MLP_GEMM_FLOPS / (ms * 1e-3) / 1e12, "peak": tensor_peak,
                        "unit": "TFLOP/s", "frac": MLP_GEMM_FLOPS / (ms * 1e-3) / 1e12 / tensor_peak,
                        "frac_of_burst_basis": MLP_GEMM_FLOPS / (ms * 1e-3) / 1e12 / (peaks["bf16_tflops"] / 6.0),
                        "gemm_kernels_ms_per_step": gemm_ms,
                        "other_kernels_ms_per_step": max(ms - gemm_ms, 0.0),
                        "stream_bytes_unfused": MLP_STREAM_BYTES_UNFUSED,
                        "peak_basis": f"{peaks_kind} bf16_tflops_sustained / 2 (tf32) / 3 (split); 5 GEMMs x 34.36 GFLOP "
                                      "per step are the algorithmic work, the streaming passes ride in the remainder",
                        "traffic": None}}
    # ---- end to end: every step uploads that step's inputs (X and T, pinned host memory) on the copy engine,
    # runs forward + backward and reads the loss back on the host; two input sets alternate so step i's compute
    # overlaps step i+1's upload.
    if do_e2e:
        nX, nT = X.size, T.size
        pins = [L.cleave_cuda_host_alloc(4 * n) for n in (nX, nT)]
        if not all(pins):
            cb._lib.raise_last_error("pinned host allocation")
        hX = np.ctypeslib.as_array(ctypes.cast(pins[0], c_f32p), shape=(nX,))
        hT = np.ctypeslib.as_array(ctypes.cast(pins[1], c_f32p), shape=(nT,))
        hX[:] = X.ravel()
        hT[:] = T.ravel()
        sets = [(tX, tT), (linalg.Tensor.empty(batch, d_in), linalg.Tensor.empty(batch, d_out))]

        def up(k):
            if L.cleave_cuda_upload_async_f32(sets[k][0]._h, hX.ctypes.data_as(c_f32p), nX) != 0 or \
                    L.cleave_cuda_upload_async_f32(sets[k][1]._h, hT.ctypes.data_as(c_f32p), nT) != 0:
                cb._lib.raise_last_error("upload_async")

        def run(n):
            up(0)
            for i in range(n):
                if i + 1 < n:
                    up((i + 1) & 1)
                last = net.forward_backward(sets[i & 1][0], sets[i & 1][1])    # returns the loss: a host read
            return last

        run(3)
        L.cleave_cuda_transfers_sync()
        e0.record()
        e2e_loss = run(steps)
        e1.record()
        e1.synchronize()
        L.cleave_cuda_transfers_sync()
        e2e_ms = e0.elapsed_time(e1) / steps
        rec["e2e"] = {"value": batch / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": 4 * (nX + nT), "d2h_bytes_per_step": 4, "steps": steps, "loss": e2e_loss,
                      "mode": "one library call per kernel"}
        # The same loop with the step captured once per input set and replayed (one launch call per step): uploads go
        # to the set the other graph reads, the host waits for a set's upload before it replays that set's graph, and
        # reads the loss (a device-to-host read, which waits for the step) every step.
        try:
            graphs = [cb.StepGraph(lambda k=k: net.forward_backward(sets[k][0], sets[k][1], loss_out=loss_dev))
                      for k in (0, 1)]

            def run_graphs(n):
                up(0)
                last = None
                for i in range(n):
                    L.cleave_cuda_transfers_sync()          # step i's inputs have landed
                    if i + 1 < n:
                        up((i + 1) & 1)
                    graphs[i & 1].replay()
                    last = loss_dev[0]                       # host read: waits for the step
                return last

            run_graphs(3)
            L.cleave_cuda_transfers_sync()
            e0.record()
            g_loss = run_graphs(steps)
            e1.record()
            e1.synchronize()
            L.cleave_cuda_transfers_sync()
            g_ms = e0.elapsed_time(e1) / steps
            for g in graphs:
                g.close()
            if g_ms < e2e_ms and abs(g_loss - e2e_loss) <= 1e-6 * abs(e2e_loss):
                rec["e2e"].update({"value": batch / (g_ms * 1e-3), "ms_per_step": g_ms, "loss": g_loss,
                                   "mode": "step captured once per input set (cleave_cuda_graph_*) and replayed",
                                   "call_by_call_ms_per_step": e2e_ms})
            else:
                rec["e2e"]["graph_replay_ms_per_step"] = g_ms
        except Exception as e:   # noqa: BLE001 - an extra; the call-by-call figure above stands
            rec["e2e"]["graph_replay_error"] = f"{type(e).__name__}: {e}"[:200]
            torch.cuda.synchronize()
        del sets
        for p in pins:
            L.cleave_cuda_host_free(p)
    # ---- the same step captured once into a CUDA graph through the library's own entry points and replayed: the
    # same 11 kernels without the launch gaps between them
    rec["graph"] = None
    try:
        g = cb.StepGraph(lambda: net.forward_backward(tX, tT, loss_out=loss_dev))
        for _ in range(3):
            g.replay()
        cb.sync()
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        e1.synchronize()
        gms = e0.elapsed_time(e1) / steps
        rec["graph"] = {"ms_per_step": gms, "samples_per_s": batch / (gms * 1e-3), "loss": loss_dev[0],
                        "gemm_tflops": MLP_GEMM_FLOPS / (gms * 1e-3) / 1e12,
                        "note": "one forward+backward step captured (cleave_cuda_graph_begin / _end) and replayed"}
        g.close()
    except Exception as e:   # noqa: BLE001 - the graph leg is an extra; the eager figure above is the record
        rec["graph"] = {"error": f"{type(e).__name__}: {e}"[:200]}
        torch.cuda.synchronize()
    del net, tX, tT
    # ---- the reference's CPU arithmetic for the same step (oracle), on this box's host cores
    if do_cpu:
        from oracle import ref
        ref.set_num_threads(_host_threads())
        t0 = time.perf_counter()
        r = ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
        dt = time.perf_counter() - t0
        cores = ref.num_threads()
        ref.set_num_threads(1)
        sl = 64
        t0 = time.perf_counter()
        ref.mlp2_fwd_bwd(X[:sl], W1, b1, W2, b2, T[:sl])
        dt1 = time.perf_counter() - t0
        ref.set_num_threads(_host_threads())
        rec["cpu_baseline"] = {"value": batch / dt, "unit": "samples/s", "cores": cores, "kind": "port",
                               "sample": f"one full forward+backward step of configuration 2 ({dt:.1f} s), the oracle's "
                                         "restatement of the reference loops, OpenMP over rows",
                               "loss": float(r["loss"]),
                               "single_thread": {"value": sl / dt1, "unit": "samples/s", "cores": 1,
                                                 "sample": f"a {sl}-sample batch slice ({dt1:.1f} s); the reference "
                                                           "itself runs on one thread"}}
    return rec


def secondary_configs(cb, torch, peaks):
    """Linear-regression step (configuration 1)."""
    from cleave_b200 import autodiff, linalg, workloads
    out = {}
    L = cb.lib()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # --- linear regression 1,048,576 x 16.  One operand set is 72 MiB and would sit in the 126 MB L2,
    # so four distinct sets are used in rotation (288 MiB touched per rotation).
    sets = []
    for i in range(4):
        X, y, _w = workloads.linreg_inputs() if i == 0 else (workloads.normal(50 + i, 1 << 20, 16),
                                                             workloads.normal(60 + i, 1 << 20), None)
        sets.append((linalg.Tensor(X), linalg.Tensor(y)))
    tw = linalg.Tensor(np.zeros(16, np.float32))
    for tX, ty in sets:
        autodiff.linreg_step(tX, ty, tw)
    rot = 3
    L.cleave_cuda_profile_begin()
    e0.record()
    for _ in range(rot):
        for tX, ty in sets:
            autodiff.linreg_step(tX, ty, tw)
    e1.record()
    e1.synchronize()
    cnt = ctypes.c_int32(0)
    kms = L.cleave_cuda_profile_end(ctypes.byref(cnt)) / max(cnt.value, 1)
    ms = e0.elapsed_time(e1) / (rot * len(sets))
    loss, _g, _p = autodiff.linreg_step(sets[0][0], sets[0][1], tw)
    nbytes = 4.0 * ((1 << 20) * 16 + 2 * (1 << 20))
    # the same sweep with the loss left on the device and the outputs reused: steps queue without a host wait
    loss_dev, g_dev, p_dev = linalg.Tensor.zero(1), linalg.Tensor.empty(16), linalg.Tensor.empty(1 << 20)
    for tX, ty in sets:
        autodiff.linreg_step(tX, ty, tw, loss_out=loss_dev, grad_out=g_dev, pred_out=p_dev)
    e0.record()
    for _ in range(rot):
        for tX, ty in sets:
            autodiff.linreg_step(tX, ty, tw, loss_out=loss_dev, grad_out=g_dev, pred_out=p_dev)
    e1.record()
    e1.synchronize()
    ms_dev = e0.elapsed_time(e1) / (rot * len(sets))
    out["linreg_step"] = {"gb_per_s": nbytes / (ms * 1e-3) / 1e9, "ms_per_step": ms, "loss": loss,
                          "kernel_ms": kms, "kernel_gb_per_s": nbytes / (kms * 1e-3) / 1e9,
                          "kernel_hbm_frac": nbytes / (kms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "device_resident_ms": ms_dev, "device_resident_gb_per_s": nbytes / (ms_dev * 1e-3) / 1e9,
                          "device_resident_hbm_frac": nbytes / (ms_dev * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "note": "ms_per_step is the synchronous API call (output allocation, the kernel, the loss read "
                                  "back, a stream sync); kernel_* is the kernel alone (event pair per call); device_resident_* "
                                  "is the call that leaves the loss on the device, 12 steps queued back to back",
                          "config": "X 1048576x16 N(0,1), loss + dL/dw in one sweep; 4 operand sets in rotation"}
    return out


def _host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _setup_single(local: int = 0):
    import torch

    import cleave_b200 as cb
    from cleave_b200 import dp
    torch.cuda.set_device(local)
    L = cb.lib()
    if L.cleave_cuda_init(local) != 0:
        cb._lib.raise_last_error("init")
    dp.use_torch_stream()
    return torch, cb, L


def _time_ms(torch, fn, iters: int, warmup: int = 3) -> float:
    """Average device time of fn() over `iters` back-to-back calls (CUDA events on the library's stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def run_ops(args):
    """Streaming operators and reductions at configuration-2 sizes: achieved GB/s (algorithmic bytes)
    against the measured HBM copy bandwidth.  Each operator runs over four distinct operand sets in
    rotation (64 MiB per tensor, 768 MiB touched per rotation, so nothing is served from the 126 MB
    L2) inside ONE event pair, 5 rotations per measurement."""
    torch, cb, L = _setup_single()
    from cleave_b200 import linalg, nn, workloads
    peaks, kind = measured_peaks()
    rows, cols = args.ops_rows, 4096
    n = rows * cols
    R = 4
    A = [linalg.Tensor(workloads.normal(11 + i, rows, cols)) for i in range(R)]
    B = [linalg.Tensor(workloads.normal(21 + i, rows, cols) + np.float32(3.0)) for i in range(R)]
    Y = [nn.tanh(a) for a in A]
    W = [linalg.Tensor(workloads.normal(31 + i, n)) for i in range(R)]
    bias = linalg.Tensor(workloads.normal(13, cols))
    cases = {
        "add": (lambda i: A[i] + B[i], 12 * n), "mul": (lambda i: A[i] * B[i], 12 * n),
        "div": (lambda i: A[i] / B[i], 12 * n), "neg": (lambda i: -A[i], 8 * n),
        "relu": (lambda i: nn.relu(A[i]), 8 * n), "sigmoid": (lambda i: nn.sigmoid(A[i]), 8 * n),
        "tanh": (lambda i: nn.tanh(A[i]), 8 * n), "exp": (lambda i: nn.exp(Y[i]), 8 * n),
        "tanh_bwd": (lambda i: nn.tanh_bwd(Y[i], B[i]), 12 * n),
        "sigmoid_bwd": (lambda i: nn.sigmoid_bwd(Y[i], B[i]), 12 * n),
        "bias_tanh": (lambda i: nn.bias_act(A[i], bias, "tanh"), 8 * n),
        "sgd": (lambda i: nn.sgd_step(W[i], B[i].reshape(n), 1e-9), 12 * n),
        "fill": (lambda i: linalg.Tensor.zero(n), 4 * n),
        "colsum": (lambda i: nn.colsum(A[i]), 4 * n),
        # scalar-returning: every call ends with a device->host read of the result and a stream sync
        "sum": (lambda i: nn.sum(A[i]), 4 * n), "max_of": (lambda i: nn.max_of(A[i]), 4 * n),
        "mse_fwd_bwd": (lambda i: nn.mse(Y[i], B[i]), 12 * n),
    }
    # the same reduction kernel with its result left on the device (no host wait per call): what the
    # kernel alone achieves, next to the synchronous scalar-returning entry above
    dev_out = linalg.Tensor.empty(1)
    stream = ctypes.c_void_p(L.cleave_cuda_get_stream() or 0)

    def sum_dev(i):
        if L.cleave_cuda_sum_noalloc_f32(ctypes.c_void_p(A[i].data_ptr), n, ctypes.c_void_p(dev_out.data_ptr),
                                         stream) != 0:
            cb._lib.raise_last_error("sum_noalloc")
    cases["sum_device_result"] = (sum_dev, 4 * n)
    loss_dev = linalg.Tensor.zero(1)
    # the loss kernel with its result left on the device: loss + gradient with respect to the pre-activation
    cases["mse_sigmoid_bwd_device_result"] = (lambda i: nn.mse_act_bwd(Y[i], B[i], "sigmoid", loss_out=loss_dev), 12 * n)
    out = {}
    for name, (fn, nbytes) in cases.items():
        def rotation():
            for i in range(R):
                fn(i)
        ms = _time_ms(torch, rotation, 5, warmup=2) / R
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "gb_per_s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 3)}
    print(json.dumps({"metric": "streaming operator GB/s", "unit": "GB/s", "n_gpus": 1, "dtype": "f32",
                      "data": "synthetic",
                      "config": {"workload": f"{rows}x{cols} f32 tensors ({n * 4 >> 20} MiB each), 4 operand sets in "
                                             "rotation so no operand is L2-resident; hbm_frac is of the measured copy "
                                             "bandwidth"},
                      "peak_hbm_gbs": peaks["hbm_gbs"], "peak_kind": kind, "ops": out}),
          flush=True)


def run_gemm_sweep(args):
    """Configuration 3: square sizes and the two skinny shapes, one GPU."""
    torch, cb, L = _setup_single()
    from cleave_b200 import linalg, workloads
    peaks, kind = measured_peaks()
    shapes = [(1024,) * 3, (2048,) * 3, (4096,) * 3, (8192,) * 3, (16384,) * 3, (16384, 16384, 64), (16384, 64, 16384)]
    if args.max_size:
        shapes = [s for s in shapes if max(s) <= args.max_size]
    if args.shape:
        shapes = [tuple(int(x) for x in args.shape.split(","))]
    out = []
    for (m, n, k) in shapes:
        a = linalg.Tensor(workloads.uniform_pm1(1, m, k))
        b = linalg.Tensor(workloads.uniform_pm1(2, k, n))
        c = linalg.Tensor.empty(m, n)
        iters = 20 if m * n * k <= 8192 ** 3 else 5
        L.cleave_cuda_profile_begin()
        ms = _time_ms(torch, lambda: linalg.gemm_into(c, a, b), iters, warmup=3)
        cnt = ctypes.c_int32(0)
        kms = L.cleave_cuda_profile_end(ctypes.byref(cnt)) / max(cnt.value, 1)
        flops = 2.0 * m * n * k
        nbytes = 4.0 * (m * k + k * n + m * n)
        out.append({"m": m, "n": n, "k": k, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                    "kernel_ms": round(kms, 4), "kernel_tflops": round(flops / kms / 1e9, 1) if kms else None,
                    "min_bytes_gb_per_s": round(nbytes / ms / 1e6, 1),
                    "tensor_frac": round(flops / ms / 1e9 / (peaks["bf16_tflops"] / 6), 3),
                    "hbm_frac": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 3)})
        del a, b, c
        L.cleave_cuda_trim()
    print(json.dumps({"metric": "f32 GEMM shape sweep", "unit": "TFLOP/s", "n_gpus": 1, "dtype": "f32",
                      "data": "synthetic", "config": {"workload": "C=A*B uniform[-1,1); ms includes the operand split "
                                                                  "pre-pass; kernel_* is the tcgen05 kernel alone"},
                      "peak_tensor_tflops": peaks["bf16_tflops"] / 6, "peak_hbm_gbs": peaks["hbm_gbs"], "shapes": out}),
          flush=True)


NUMA_INFO = None   # what bind_to_gpu_numa_node did on this rank (multi-rank runs only)


def bind_to_gpu_numa_node(local: int) -> dict:
    """With several ranks on one host, run this rank's threads on the NUMA node its GPU is attached to, so that the
    pinned staging buffers it allocates afterwards (placed by first touch) and the copies from them do not cross the
    socket interconnect.  Reads sysfs only; does nothing when the node is unknown, when there is one node, or when the
    allowed CPU set leaves no CPU of that node.  Returns what it did, for the bench line."""
    info = {"node": None}
    try:
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        if len(nodes) < 2:
            info["nodes"] = len(nodes)
            return info
        import torch
        pr = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (getattr(pr, "pci_domain_id", 0), pr.pci_bus_id, pr.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info.update({"nodes": len(nodes), "gpu_pci": bus})
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        mine = cpus & allowed
        if mine and mine != allowed:
            os.sched_setaffinity(0, mine)
            info.update({"node": node, "cpus": len(mine), "of_allowed": len(allowed)})
        else:
            info.update({"node": node, "cpus": len(mine), "of_allowed": len(allowed), "bound": False})
    except Exception as e:   # noqa: BLE001 - placement is an optimisation; the run goes on unbound
        info["error"] = f"{type(e).__name__}: {e}"[:160]
    return info


def _dist_setup():
    """torch + process group (NCCL, one rank per GPU) + the library on torch's current stream; idempotent."""
    import torch
    import torch.distributed as dist

    import cleave_b200 as cb
    from cleave_b200 import dp
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    global NUMA_INFO
    if world > 1 and NUMA_INFO is None:
        NUMA_INFO = bind_to_gpu_numa_node(local)
    if world > 1 and not dist.is_initialized():
        import datetime
        # a collective that a failed rank never joins ends with an error after 5 minutes instead of hanging the job
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    L = cb.lib()
    if L.cleave_cuda_init(local) != 0:
        cb._lib.raise_last_error("init")
    if (L.cleave_cuda_get_stream() or 0) != torch.cuda.current_stream().cuda_stream or \
            torch.cuda.current_stream().cuda_stream == 0:
        dp.use_torch_stream()
    return torch, dist, cb, L, rank, world, local


def _timed_max_over_ranks(torch, dist, world, fn, steps, finish=None):
    """Average device time of fn() over `steps` calls between barriers, as the maximum over the ranks.
    `finish()` runs before the closing event (work of the last step that another stream still holds)."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if finish:
        finish()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / steps


def _device_uniform_pm1(torch, tensor, seed):
    """Fills a library tensor in place with seeded iid uniform[-1, 1) values generated on the device (torch's
    Philox generator: set-up plumbing for inputs too large to draw on the host inside a bench run)."""
    from cleave_b200 import dp
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    dp.as_torch(tensor).uniform_(-1.0, 1.0, generator=g)


def measure_batched_gemm(env, steps, warmup):
    """Configuration 4a: 64 independent 4096^3 products, batch index b on rank b mod G, no collective.
    Every problem is distinct seeded data (seed 100 + b for A, 300 + b for B), generated on the device."""
    torch, dist, cb, L, rank, world, _ = env
    from cleave_b200 import dp, linalg
    batch, sz = 64, 4096
    mine = list(dp.batch_shard(batch, rank, world))
    ta, tb = linalg.Tensor.empty(len(mine), sz, sz), linalg.Tensor.empty(len(mine), sz, sz)
    tc = linalg.Tensor.empty(len(mine), sz, sz)
    for i, b in enumerate(mine):
        for t, seed in ((ta, 100 + b), (tb, 300 + b)):
            view = linalg.Tensor.from_device_ptr(t.data_ptr + 4 * i * sz * sz, sz, sz)
            _device_uniform_pm1(torch, view, seed)

    def step():
        linalg.gemm_into(tc, ta, tb)

    for _ in range(warmup):
        step()
    l0 = L.cleave_cuda_kernel_launches()
    ms = _timed_max_over_ranks(torch, dist, world, step, steps)
    launches = L.cleave_cuda_kernel_launches() - l0
    if L.cleave_cuda_sync() != 0:
        cb._lib.raise_last_error("batched gemm")
    del ta, tb, tc
    L.cleave_cuda_trim()
    return {"workload": f"64 independent 4096^3 products (distinct seeded data), batch index b on rank b mod {world}",
            "ms_per_step": ms, "tflops": batch * 2.0 * sz ** 3 / ms / 1e9, "steps": steps, "scaling": "strong",
            "problems_per_rank": len(mine), "gpu_launches": int(launches)}


def measure_rowblock_gemm(env, steps, warmup, sz=16384):
    """Row-block sharded large GEMM: A and C split by rows over the ranks on 256-row tile boundaries, B
    replicated into every rank's own HBM by an NCCL broadcast (timed without and with that broadcast)."""
    torch, dist, cb, L, rank, world, _ = env
    from cleave_b200 import dp, linalg
    lo, hi = dp.row_block(sz, rank, world, tile=256)
    rows = hi - lo
    ta = linalg.Tensor.empty(rows, sz)
    _device_uniform_pm1(torch, ta, 500 + rank)
    tb = linalg.Tensor.empty(sz, sz)
    if rank == 0:
        _device_uniform_pm1(torch, tb, 2)
    tc = linalg.Tensor.empty(rows, sz)
    b_view = dp.as_torch(tb)

    def bcast():
        if world > 1:
            dist.broadcast(b_view, src=0)

    def product():
        linalg.gemm_into(tc, ta, tb)

    def both():
        bcast()
        product()

    bcast()
    for _ in range(warmup):
        product()
    l0 = L.cleave_cuda_kernel_launches()
    ms = _timed_max_over_ranks(torch, dist, world, product, steps)
    launches = L.cleave_cuda_kernel_launches() - l0
    ms_with = _timed_max_over_ranks(torch, dist, world, both, steps)
    chk = torch.tensor([float(b_view[:: max(1, b_view.numel() // 4096)].double().sum())], device="cuda",
                       dtype=torch.float64)
    same = True
    if world > 1:
        lo_t, hi_t = chk.clone(), chk.clone()
        dist.all_reduce(lo_t, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_t, op=dist.ReduceOp.MAX)
        same = bool(lo_t.item() == hi_t.item())
    if L.cleave_cuda_sync() != 0:
        cb._lib.raise_last_error("row-block gemm")
    del ta, tb, tc, b_view
    L.cleave_cuda_trim()
    flops = 2.0 * sz ** 3
    return {"workload": f"C = A B, M = N = K = {sz}; A and C split by rows over {world} rank(s), B replicated by an "
                        "NCCL broadcast", "ms_per_step": ms, "tflops": flops / ms / 1e9, "steps": steps,
            "scaling": "strong", "gpu_launches": int(launches),
            "with_broadcast": {"ms_per_step": ms_with, "tflops": flops / ms_with / 1e9, "broadcast_bytes": 4 * sz * sz},
            "b_identical_on_all_ranks": same}


def _make_dp_trainer(env, mode, d_in, d_hid, d_out, overlap=True):
    torch, dist, cb, L, rank, world, _ = env
    from cleave_b200 import autodiff, dp
    if mode == "nccl" or world == 1:
        net = autodiff.MLP2(d_in, d_hid, d_out)
        trainer = dp.DataParallel(dp.MLP2Replica(net), overlap=overlap)
        how = "nccl all-reduce + fused 1/G SGD pass" if world > 1 else "single rank"
    else:
        n_params = d_in * d_hid + d_hid + d_hid * d_out + d_out
        trainer = dp.FusedDataParallel(n_params, lambda p, g: autodiff.MLP2(d_in, d_hid, d_out, params=p, grads=g),
                                       multimem=mode == "fused")
        net = trainer.net
        how = "one kernel: " + ("multimem.ld_reduce in NVSwitch" if trainer.multimem else "peer loads") + \
              " + SGD + replication of the new weights"
    return trainer, net, how


def _dp_small_case_deviation(env, mode):
    """Trains a small perceptron for 5 steps through the same trainer and compares the weights with
    whole-batch SGD evaluated in float64 on the host: max |w - w64| / max |w64|."""
    torch, dist, cb, L, rank, world, _ = env
    from cleave_b200 import dp, linalg, workloads
    d_in, d_hid, d_out, per_rank, lr = 32, 64, 16, 64, 0.5
    gb = per_rank * world
    _, W1, b1, W2, b2, _ = workloads.mlp_inputs(1, d_in, d_hid, d_out)
    trainer, net, _ = _make_dp_trainer(env, mode, d_in, d_hid, d_out)
    net.load(W1, b1, W2, b2)
    Xg = workloads.normal(1000, gb, d_in)
    Tg = workloads.uniform01(2000, gb, d_out)
    lo, hi = dp.shard(gb, rank, world)
    tX, tT = linalg.Tensor(np.ascontiguousarray(Xg[lo:hi])), linalg.Tensor(np.ascontiguousarray(Tg[lo:hi]))
    loss_dev = linalg.Tensor.zero(1)
    for _ in range(5):
        trainer.step(tX, tT, lr, loss_out=loss_dev)
    if hasattr(trainer, "flush"):
        trainer.flush()
    torch.cuda.synchronize()
    got = net.params.numpy().astype(np.float64)
    w = [a.astype(np.float64) for a in (W1, b1, W2, b2)]
    X64, T64 = Xg.astype(np.float64), Tg.astype(np.float64)
    for _ in range(5):
        H = np.tanh(X64 @ w[0] + w[1])
        Y = 1.0 / (1.0 + np.exp(-(H @ w[2] + w[3])))
        dZ2 = Y * (1.0 - Y) * 2.0 * (Y - T64) / Y.size   # the mean over ranks of per-rank means is the global mean
        dZ1 = (1.0 - H * H) * (dZ2 @ w[2].T)
        g = [X64.T @ dZ1, dZ1.sum(0), H.T @ dZ2, dZ2.sum(0)]
        w = [a - lr * b for a, b in zip(w, g)]
    want = np.concatenate([a.ravel() for a in w])
    del trainer, net
    return float(np.max(np.abs(got - want)) / np.max(np.abs(want)))


def measure_dp_mlp(env, mode, steps, warmup, global_batch=32768, overlap=True, log_every=10, clocks=False):
    """Configuration 4b: the 2-layer MLP trained data-parallel, global batch split evenly over the ranks,
    SGD lr 1e-3, gradients averaged over the ranks every step."""
    torch, dist, cb, L, rank, world, local = env
    from cleave_b200 import dp, linalg, workloads
    d_in, d_hid, d_out = 1024, 4096, 1024
    _, W1, b1, W2, b2, _ = workloads.mlp_inputs(1, d_in, d_hid, d_out)
    trainer, net, how = _make_dp_trainer(env, mode, d_in, d_hid, d_out, overlap)
    net.load(W1, b1, W2, b2)
    X, T = dp.dp_batch_inputs(global_batch, rank, world, d_in, d_out)
    tX, tT = linalg.Tensor(X), linalg.Tensor(T)
    del X, T
    loss_dev = linalg.Tensor.zero(1)
    state = {"loss": None, "i": 0}

    def step():
        trainer.step(tX, tT, 1e-3, loss_out=loss_dev)
        state["i"] += 1
        if state["i"] % log_every == 0:
            state["loss"] = loss_dev[0]      # the host reads the loss back as a training loop logs it

    flush = getattr(trainer, "flush", None)
    for _ in range(warmup):
        trainer.step(tX, tT, 1e-3, loss_out=loss_dev)
    if flush:
        flush()
    l0 = L.cleave_cuda_kernel_launches()
    sampler = ClockSampler(local) if (clocks and rank == 0) else None
    ms = _timed_max_over_ranks(torch, dist, world, step, steps, finish=flush)
    clk = sampler.stop() if sampler else None
    launches = L.cleave_cuda_kernel_launches() - l0
    state["loss"] = loss_dev[0]
    psum = torch.tensor([float(dp.as_torch(net.params).double().sum())], device="cuda", dtype=torch.float64)
    pmin, pmax = psum.clone(), psum.clone()
    if world > 1:
        dist.all_reduce(pmin, op=dist.ReduceOp.MIN)
        dist.all_reduce(pmax, op=dist.ReduceOp.MAX)
    if L.cleave_cuda_sync() != 0:
        cb._lib.raise_last_error("dp_mlp")
    rec = {"workload": f"2-layer MLP 1024->4096 tanh->1024 sigmoid, MSE, SGD lr 1e-3, global batch {global_batch} over "
                       f"{world} rank(s), gradient mean every step", "exchange": how, "ms_per_step": ms,
           "samples_per_s": global_batch / (ms * 1e-3), "steps": steps, "scaling": "strong",
           "allreduce_bytes_per_step": 4 * net.n_params, "loss": state["loss"], "gpu_launches": int(launches),
           "replicas_identical": bool(pmin.item() == pmax.item()),
           "gemm_tflops_per_gpu": 5 * 2.0 * (global_batch / world) * d_hid * d_in / (ms * 1e-3) / 1e12}
    if clk:
        rec["clocks"] = clk
    del trainer, net, tX, tT
    L.cleave_cuda_trim()
    return rec


def sharded_record(env, args):
    """The three workloads that shard over GPUs, run by the ranks of this job one after the other.  At one
    rank these are the one-GPU times the N > 1 lines of the same series of runs are compared with."""
    torch, dist, cb, L, rank, world, _ = env
    out = {}
    modes = ["single"] if world == 1 else ["fused", "nccl"]
    jobs = [("batched_gemm_64x4096", lambda: measure_batched_gemm(env, steps=5, warmup=3)),
            ("rowblock_gemm_16384", lambda: measure_rowblock_gemm(env, steps=3, warmup=3))]
    for mode in modes:
        def dp_job(mode=mode):
            rec = measure_dp_mlp(env, mode, steps=20, warmup=3)
            rec["small_case_max_rel_deviation_from_f64_sgd"] = _dp_small_case_deviation(env, mode)
            return rec
        jobs.append(("dp_mlp_32768" + ("" if mode == "single" else "_" + mode), dp_job))
    for name, job in jobs:
        try:
            out[name] = job()
        except Exception as e:   # noqa: BLE001 - the headline line must still be printed
            # after a failure the ranks may no longer be in step: record it and leave the remaining workloads out
            out[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            out["aborted_after"] = name
            break
    return out


def run_batched_gemm(args):
    env = _dist_setup()
    rec = measure_batched_gemm(env, args.steps, args.warmup)
    if env[4] == 0:
        print(json.dumps({"metric": "batched f32 GEMM TFLOP/s (64 x 4096^3)", "value": rec["tflops"], "unit": "TFLOP/s",
                          "n_gpus": env[5], "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic", "config": {"workload": rec["workload"]}, **rec}),
              flush=True)
    if env[5] > 1:
        env[1].destroy_process_group()


def run_rowblock_gemm(args):
    env = _dist_setup()
    sz = args.size if args.size != 8192 else 16384
    rec = measure_rowblock_gemm(env, args.steps, args.warmup, sz)
    if env[4] == 0:
        print(json.dumps({"metric": f"row-block f32 GEMM TFLOP/s ({sz}^3)", "value": rec["tflops"], "unit": "TFLOP/s",
                          "n_gpus": env[5], "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic", "config": {"workload": rec["workload"]}, **rec}),
              flush=True)
    if env[5] > 1:
        env[1].destroy_process_group()


def run_dp_mlp(args):
    env = _dist_setup()
    mode = "single" if env[5] == 1 else args.dp_mode
    rec = measure_dp_mlp(env, mode, args.steps, args.warmup, args.global_batch, not args.no_overlap,
                         max(1, args.log_every), clocks=True)
    if env[4] == 0:
        print(json.dumps({"metric": "MLP data-parallel training samples/s", "value": rec["samples_per_s"],
                          "unit": "samples/s", "n_gpus": env[5], "warmup": args.warmup, "higher_is_better": True,
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": rec["workload"], "exchange": rec["exchange"],
                                     "overlap": not args.no_overlap}, **rec}), flush=True)
    if env[5] > 1:
        env[1].destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cleave_b200", choices=["cleave_b200", "reference"])
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded workloads that follow the headline")
    ap.add_argument("--no-mlp", action="store_true", help="skip the MLP forward+backward record")
    ap.add_argument("--workload", default="gemm", choices=["gemm", "dp_mlp", "ops", "gemm_sweep", "batched_gemm",
                                                            "rowblock_gemm"],
                    help="gemm = the headline; the others are secondary configurations")
    ap.add_argument("--ops-rows", type=int, default=4096, help="ops: rows of the 4096-column test tensors")
    ap.add_argument("--max-size", type=int, default=0, help="gemm_sweep: skip shapes with a dimension above this")
    ap.add_argument("--shape", default="", help="gemm_sweep: run only this problem, given as M,N,K")
    ap.add_argument("--global-batch", type=int, default=32768)
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--log-every", type=int, default=10, help="dp_mlp: read the loss back every this many steps")
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "fused_p2p", "nccl"],
                    help="dp_mlp: gradient exchange as one multimem kernel, one peer-load kernel, or NCCL + SGD")
    ap.add_argument("--size", type=int, default=8192,
                    help="M=N=K; anything but 8192 is a profiling case, not the headline workload")
    args = ap.parse_args()
    global M, N, K, FLOPS
    M = N = K = args.size
    FLOPS = 2.0 * M * N * K
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    if args.impl == "reference":
        run_reference(args)
        return
    # Libraries loaded below (NCCL's version banner, for one) write to stdout; keep the real
    # stdout for the single JSON line and send everything else to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w", buffering=1)
    runner = {"dp_mlp": run_dp_mlp, "ops": run_ops, "gemm_sweep": run_gemm_sweep,
              "batched_gemm": run_batched_gemm, "rowblock_gemm": run_rowblock_gemm}.get(args.workload)
    if runner:
        runner(args)
        return

    from cleave_b200 import linalg, workloads
    from cleave_b200._lib import c_f32p

    # The library runs on a torch-owned stream, made current, so torch CUDA events (which record on
    # the current stream) bracket exactly the kernels and copies the library enqueues.
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if int(os.environ.get("RANK", "0")) == 0 else None
    env = _dist_setup()
    torch, dist, cb, L, rank, world, local = env
    assert L.cleave_cuda_get_stream() == torch.cuda.current_stream().cuda_stream != 0
    peaks, peaks_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Operands: seeded per rank (independent problems), generated on the host, resident in HBM.
    a_host, b_host = workloads.gemm_inputs(M, N, K, seed_a=1 + 2 * rank, seed_b=2 + 2 * rank)
    ta, tb = linalg.Tensor(a_host), linalg.Tensor(b_host)
    tc = linalg.Tensor.empty(M, N)

    def step():
        linalg.gemm_into(tc, ta, tb, algo=linalg.GEMM_3XTF32)

    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = L.cleave_cuda_kernel_launches()
    L.cleave_cuda_profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_window0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    n_prof = ctypes.c_int32(0)
    kernel_ms_total = L.cleave_cuda_profile_end(ctypes.byref(n_prof))
    launches = L.cleave_cuda_kernel_launches() - launches0
    if L.cleave_cuda_sync() != 0:
        cb._lib.raise_last_error("timed region")
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * FLOPS / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with host buffers (pinned), copies inside the timed region.
    # Every step copies that step's A and B from pinned host memory, multiplies, and copies C back.
    # The copies run on the copy engines (cleave_cuda_upload_async_f32 / download_async_f32) and
    # two sets of device tensors alternate, so step i's product overlaps step i+1's upload and
    # step i-1's download; nothing is skipped or reused between steps.
    nbytes = M * K * 4
    pin = [L.cleave_cuda_host_alloc(nbytes) for _ in range(4)]
    if not all(pin):
        cb._lib.raise_last_error("pinned host allocation")
    ha, hb, hc0, hc1 = (np.ctypeslib.as_array(ctypes.cast(p, c_f32p), shape=(M * K,)) for p in pin)
    ha[:] = a_host.ravel()
    hb[:] = b_host.ravel()
    hcs = (hc0, hc1)
    A2 = (ta, linalg.Tensor.empty(M, K))
    B2 = (tb, linalg.Tensor.empty(K, N))
    C2 = (tc, linalg.Tensor.empty(M, N))

    def up(i):
        if L.cleave_cuda_upload_async_f32(A2[i]._h, ha.ctypes.data_as(c_f32p), ha.size) != 0 or \
                L.cleave_cuda_upload_async_f32(B2[i]._h, hb.ctypes.data_as(c_f32p), hb.size) != 0:
            cb._lib.raise_last_error("upload_async")

    def e2e_run(steps):
        up(0)
        for i in range(steps):
            cur = i & 1
            if i + 1 < steps:
                up(1 - cur)                      # next step's operands, while this step computes
            linalg.gemm_into(C2[cur], A2[cur], B2[cur], algo=linalg.GEMM_3XTF32)
            if L.cleave_cuda_download_async_f32(C2[cur]._h, hcs[cur].ctypes.data_as(c_f32p), hcs[cur].size) != 0:
                cb._lib.raise_last_error("download_async")
        # order the compute stream (where the closing event is recorded) after the last two downloads
        L.cleave_cuda_data_ptr(C2[0]._h)
        L.cleave_cuda_data_ptr(C2[1]._h)

    def copies_only(steps):
        # the same transfers on the same buffers and copy engines, no product: what the host <-> device path
        # allows at this number of ranks (all ranks copy at the same time and share the host's memory and PCIe)
        for i in range(steps):
            cur = i & 1
            up(cur)
            if L.cleave_cuda_download_async_f32(C2[cur]._h, hcs[cur].ctypes.data_as(c_f32p), hcs[cur].size) != 0:
                cb._lib.raise_last_error("download_async")
        L.cleave_cuda_data_ptr(C2[0]._h)
        L.cleave_cuda_data_ptr(C2[1]._h)
        for t in A2 + B2:
            L.cleave_cuda_data_ptr(t._h)

    def timed_region(fn, steps):
        barrier()
        e0.record()
        fn(steps)
        e1.record()
        if L.cleave_cuda_transfers_sync() != 0:
            cb._lib.raise_last_error("transfers")
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    # as many steps as the device-resident measurement (the fill of the first upload and the drain of the last
    # download are inside the timed region and amortise over the steps)
    e2e_steps = max(4, min(args.steps, 40))
    e2e_ms = copy_ms = float("nan")
    if not args.no_e2e:
        e2e_run(3)
        L.cleave_cuda_transfers_sync()
        e2e_ms = timed_region(e2e_run, e2e_steps)
        copy_ms = timed_region(copies_only, e2e_steps)
    e2e_value = world * FLOPS / (e2e_ms * 1e-3) / 1e12
    # clocks: samples stamped between the start of the timed GEMM loop and the end of the end-to-end leg (the same
    # kernels, with copies beside them); the timed loop alone is ~85 ms, too short for more than a few samples
    clocks = sampler.stop(t_window0, time.time()) if sampler else None
    if clocks is not None:
        clocks["window"] = "timed GEMM loop + end-to-end leg"
    checksum = float(hcs[(e2e_steps - 1) & 1][:4096].astype(np.float64).sum())
    # One synchronous call with host arrays (the entry point a lowering hook targets): upload, product and
    # download pipelined over row blocks inside the call.
    single_call_ms = None
    if not args.no_e2e:
        def single_call(steps):
            for _ in range(steps):
                if L.cleave_cuda_host_gemm_f32(ha.ctypes.data_as(c_f32p), ha.size, hb.ctypes.data_as(c_f32p), hb.size,
                                               hc0.ctypes.data_as(c_f32p), hc0.size, M, N, K) != hc0.size:
                    cb._lib.raise_last_error("host_gemm")
        single_call(1)
        single_call_ms = timed_region(single_call, 4)
    del A2, B2, C2
    for p in pin:
        L.cleave_cuda_host_free(p)

    # ---- second half of the metric and the sharded workloads (every rank takes part in the latter)
    del ta, tb, tc
    L.cleave_cuda_trim()
    peak_burst = peaks["bf16_tflops"] / 2.0 / 3.0
    mlp = None
    if not args.no_mlp and world == 1:
        mlp = mlp_record(cb, torch, L, peaks, peaks_kind, do_cpu=not args.no_cpu_baseline, do_e2e=not args.no_e2e)
    sharded = None
    if not args.no_sharded:
        sharded = sharded_record(env, args)

    if rank != 0:
        if world > 1:
            if sharded and "aborted_after" in sharded:
                os._exit(0)
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (tcgen05 GEMM), this rank
    kernel_ms = kernel_ms_total / max(n_prof.value, 1)
    achieved = FLOPS / (kernel_ms * 1e-3) / 1e12
    # 3xTF32-effective tensor peak: dense TF32 runs at half the bf16 rate, and the split issues
    # three MMAs per product.  The kernel is timed alone, launch by launch, so the burst bf16
    # figure is the denominator.  That figure comes from a cuBLAS run at whatever clock the measuring box
    # held under its power cap, so it is not a hard ceiling: two clock-independent bases are printed beside it.
    sm_mhz = (clocks or {}).get("sm_mhz") or 0.0
    nominal = NOMINAL_TF32_DENSE_TFLOPS / 3.0
    at_clock = nominal * sm_mhz / 1965.0 if sm_mhz else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s",
                "frac": achieved / peak_burst, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "traffic_source": NCU_TRAFFIC,
                "kernel": "gemm_3xtf32_pair_kernel", "kernel_ms": kernel_ms, "launches_timed": n_prof.value,
                "peak_basis": f"{peaks_kind} bf16_tflops (burst) / 2 (tf32) / 3 (split); "
                              f"sustained basis {peaks['bf16_tflops_sustained'] / 6.0:.1f}",
                "frac_of_nominal": achieved / nominal,
                "frac_at_sampled_clock": achieved / at_clock if at_clock else None,
                "nominal_basis": f"datasheet dense TF32 {NOMINAL_TF32_DENSE_TFLOPS:.0f} TFLOP/s at 1965 MHz / 3 = "
                                 f"{nominal:.0f}; scaled to the SM clock sampled during the timed region "
                                 f"({sm_mhz:.0f} MHz): {at_clock if at_clock else float('nan'):.0f}"}
    if roofline["frac"] > 1.0:
        roofline["note"] = ("frac > 1: the measured-peak basis (a cuBLAS bf16 run on another box and clock) is not a "
                            "ceiling for this kernel on this box; read frac_at_sampled_clock / frac_of_nominal")

    cpu = None
    if not args.no_cpu_baseline:
        v, rows, dt, cores = cpu_gemm_sample(a_host, b_host)
        v1, rows1, dt1, _ = cpu_gemm_sample(a_host, b_host, target_s=5.0, threads=1)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"rows 0..{rows} of the {M}^3 product ({dt:.1f} s), bit-identical restatement of the "
                         "reference loop, OpenMP over rows",
               "single_thread": {"value": v1, "unit": "TFLOP/s", "cores": 1,
                                 "sample": f"rows 0..{rows1} ({dt1:.1f} s); the reference itself runs on one thread "
                                           "(cleave/src/main.rs:150-152)"}}

    cfg = headline_config(world)   # identical to the reference arm's
    roofline["arithmetic"] = "3xTF32 split on tcgen05, f32 accumulate, K chunks of 256 summed in f32"
    e2e = {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": 2 * nbytes,
           "d2h_bytes_per_step": nbytes, "steps": e2e_steps, "checksum": checksum,
           "copy_ceiling_ms": copy_ms, "frac_of_copy_ceiling": copy_ms / e2e_ms if e2e_ms == e2e_ms else None,
           "single_call_ms": single_call_ms,
           "note": "copies on the copy engines, two tensor sets alternating: compute of step i overlaps the upload of "
                   "step i+1 and the download of step i-1; copy_ceiling_ms = the same copies with no product, all "
                   "ranks at once; single_call_ms = one synchronous cleave_cuda_host_gemm_f32 call per step"}
    if NUMA_INFO is not None:
        e2e["host_placement_rank0"] = NUMA_INFO   # which NUMA node rank 0's threads and pinned buffers were bound to
    line = {
        "metric": f"f32 GEMM TFLOP/s ({M}^3)", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
        "cpu_baseline": cpu,
    }
    if mlp is not None:
        # the second half of the metric, also nested where a reader of roofline / cpu_baseline / e2e looks for it
        line["mlp_fwd_bwd"] = mlp
        roofline["mlp_fwd_bwd"] = dict(mlp["roofline"], samples_per_s=mlp["value"], ms_per_step=mlp["ms_per_step"])
        if cpu is not None and "cpu_baseline" in mlp:
            cpu["mlp_fwd_bwd"] = mlp["cpu_baseline"]
        if "e2e" in mlp:
            e2e["mlp_fwd_bwd"] = mlp["e2e"]
    if sharded is not None:
        line["sharded"] = sharded
        roofline["sharded"] = {k: {kk: v[kk] for kk in ("ms_per_step", "tflops", "samples_per_s", "replicas_identical", "error")
                              if kk in v} for k, v in sharded.items() if isinstance(v, dict)}
    if not args.no_secondary and world == 1:
        line["secondary"] = secondary_configs(cb, torch, peaks)
    print(json.dumps(line), flush=True)
    if world > 1:
        if sharded and "aborted_after" in sharded:
            os._exit(0)   # a rank that failed mid-collective cannot take part in an orderly shutdown
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
