#!/usr/bin/env python
"""Benchmark of the NVFP4 projection path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the full 12-layer GPT-2-small training-step projection set (48 block linears + the tied LM head
with a 32000-entry vocabulary), forward and backward, 65536 tokens per step IN TOTAL, token-sharded over the
N GPUs (strong scaling), on seeded synthetic bf16 tensors (activations ~N(0,1), weights ~N(0,0.02), upstream
gradients ~N(0,1e-3)).  One step = weight quantization + forward + backward of every projection, plus (N > 1)
one NCCL all-reduce per layer of dW / dbias.  The step is enqueued by the C++ step driver (one host call per
step; NCCL issued from C++).  The metric is useful TFLOP/s: 6 * tokens * sum(N*K) per step, padding never
counted.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference's math (the
reference has no CPU implementation of its own and its kernels do not build here) on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL_FP4_DENSE_TFLOPS = 9000.0  # B200 dense FP4 (vendor figure; no FP4 peak is measured on this pool)
FALLBACK_HBM_GBS = 6650.0
METRIC = "NVFP4 proj fwd+bwd TFLOP/s"
TOTAL_TOKENS = 65536
# DRAM bytes moved per algorithmic byte by the GEMM kernel (operands read once + output written once), from a
# profiler capture of a small case of the same kernel (three GEMMs of the c_attn shape at 32768 tokens);
# traffic of a full launch = this ratio x the launch's algorithmic bytes (both grow with the token count).
GEMM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.08


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t_begin: float = 0.0, t_end: float = float("inf")):
        """Summary of the samples that arrived inside [t_begin, t_end] (host clock)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.lines:
            if stamp < t_begin or stamp > t_end:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# CPU leg (oracle): cpu_baseline of the GPU arm and the whole of --impl reference
# --------------------------------------------------------------------------------------------

def cpu_sample(tokens: int, steps: int, warmup: int):
    """One GPT-2-small layer (c_attn, c_proj, fc, proj), forward + backward, at `tokens` tokens,
    on the CPU oracle with every host thread OpenMP gives it.  Returns (TFLOP/s, ms/step, cores)."""
    import numpy as np

    from oracle import oracle

    # launchers such as torchrun export OMP_NUM_THREADS=1; the CPU leg is meant to use every host core
    oracle.set_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    d, h = 768, 3072
    shapes = [(d, 3 * d), (d, d), (d, h), (h, d)]
    data = []
    for i, o in shapes:
        data.append((rng.normal(0, 1, (tokens, i)).astype(np.float32), rng.normal(0, 0.02, (o, i)).astype(np.float32),
                     rng.normal(0, 0.02, o).astype(np.float32), rng.normal(0, 1e-3, (tokens, o)).astype(np.float32)))
    flops = 6.0 * tokens * sum(i * o for i, o in shapes)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for x, w, b, dy in data:
            oracle.linear_forward_backward(x, w, b, dy, 0x12345678, 0x9ABCDEF0)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    mean = sum(times) / len(times)
    return flops / mean / 1e12, mean * 1e3, oracle.max_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # bounded sample: about 4096 tokens per step for up to 16 steps, fewer tokens per step beyond that, so
    # that K steps end within a few minutes on a 16-core host
    steps = max(1, args.steps)
    tokens = max(512, min(4096, (4096 * 16 // steps) // 256 * 256))
    tflops, ms, cores = cpu_sample(tokens, steps, min(args.warmup, 1))
    sample = f"one GPT-2-small layer (c_attn, c_proj, fc, proj) fwd+bwd at {tokens} tokens per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "gpt2-small training-step projection set, fwd+bwd (CPU: bounded sample)",
                   "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's math (the reference ships no CPU path; its Rust/cuda-oxide "
                "kernels cannot be built on this box)",
    }
    emit(line)


# --------------------------------------------------------------------------------------------
# GPU arm: helpers
# --------------------------------------------------------------------------------------------

def cuda_time_us(torch, fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def graph_time_us(torch, fn, calls, replays=6):
    """Device time per call of `fn`, with `calls` consecutive calls captured into one CUDA graph and the graph
    replayed: the Python / ctypes cost of a call (about 10 us, more than these kernels take) stays out."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(calls):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(calls):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (replays * calls)


def quantize_records(pkg, torch, dev, peak_gbs):
    """The quantizer on [8192 x 768] bf16 (201 MB over 16 rotating buffers, larger than L2): rowwise scale
    with the row amax fused (what the projections call), per-tensor scale (an amax pass, then the quantizer),
    and the dequantize round trip.  GB/s on the algorithmic 2.5625 B/element."""
    q, d = pkg.Nvfp4QuantModule(), pkg.Nvfp4DecodeModule()
    rows, cols, nbuf = 8192, 768, 16
    xs = [torch.randn(rows, cols, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
    algo = rows * cols * 2.5625
    i = [0]

    def rot():
        i[0] += 1
        return i[0] % nbuf

    row_out = [q.quantize_four_six(x, rowwise=True, packed=True) for x in xs]

    def rowwise():
        k = rot()
        q.quantize_four_six(xs[k], rowwise=True, packed=True, out=row_out[k])

    amax = [q.row_amax(x) for x in xs]

    def rowwise_given_amax():
        k = rot()
        q.quantize_four_six(xs[k], amax=amax[k], rowwise=True, packed=True, out=row_out[k])

    ten_out = [q.quantize_four_six(x, rowwise=False, packed=False) for x in xs]
    ten_amax = torch.empty(1, device=dev)
    chunks = torch.empty(rows * cols // 1024, device=dev)

    def per_tensor():
        k = rot()
        q.tensor_amax(xs[k], chunks, ten_amax)
        q.quantize_four_six(xs[k], amax=ten_amax, rowwise=False, packed=False, out=ten_out[k])

    def round_trip():
        k = rot()
        q.tensor_amax(xs[k], chunks, ten_amax)
        q.quantize_four_six(xs[k], amax=ten_amax, rowwise=False, packed=False, out=ten_out[k])
        d.decode(ten_out[k])

    out = {"workload": "four-six quantize [8192x768] bf16 -> NVFP4, 16 rotating buffers (201 MB > L2)",
           "algorithmic_bytes": algo,
           "timing": "us = device time per call, 32 calls replayed from a CUDA graph; us_python_loop = the same calls "
                     "issued one by one from Python (bound by the host's per-call cost at this size)"}
    for name, fn in (("rowwise_fused_amax", rowwise), ("rowwise_amax_given", rowwise_given_amax),
                     ("per_tensor_amax_plus_quantize", per_tensor), ("per_tensor_round_trip_with_dequantize", round_trip)):
        us_loop = cuda_time_us(torch, fn, 80)
        us = graph_time_us(torch, fn, 2 * nbuf)
        gbs = algo / (us * 1e-6) / 1e9
        out[name] = {"us": us, "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak_gbs, "us_python_loop": us_loop}
    out["us"] = out["rowwise_fused_amax"]["us"]
    out["achieved_gbs"] = out["rowwise_fused_amax"]["achieved_gbs"]
    out["frac_of_hbm_peak"] = out["rowwise_fused_amax"]["frac_of_hbm_peak"]
    return out


def write_roofline(torch, dev):
    """Write-only HBM bandwidth: a plain device fill of 1 GiB (what bounds the short-K forward GEMMs)."""
    buf = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    us = cuda_time_us(torch, lambda: buf.zero_(), 10)
    del buf
    return (1 << 30) / (us * 1e-6) / 1e9


def gemm_self_check(pkg, torch, dev, tokens, shape):
    """Before anything is timed: the four GEMM kinds of the step (forward with bias, dX, dW, LM head) at this
    run's own sizes, on random NVFP4 operands, sampled 128-row blocks of the output against the CPU oracle's
    FP32-dequantized product.  Returns the largest relative Frobenius error and what was checked."""
    import numpy as np

    from oracle import oracle

    oracle.set_threads(os.cpu_count() or 1)
    gemm, pack = pkg.Nvfp4GemmModule(), pkg.Sm120ScalePackModule()
    d, v = shape.d_model, shape.vocab
    rng = np.random.default_rng(7)
    cases = [("forward c_attn", tokens, 3 * d, d, torch.bfloat16, 1), ("dX c_attn", tokens, d, 3 * d, torch.bfloat16, 0),
             ("dW c_attn", 3 * d, d, tokens, torch.float32, 0), ("lm_head logits", tokens, v, d, torch.bfloat16, 0)]
    worst, report = 0.0, []
    for name, m, n, k, dt, epi in cases:
        def rand(rows, rowwise):
            b = rng.integers(0, 256, size=rows * k // 2, dtype=np.uint8)
            s = rng.integers(0x28, 0x48, size=rows * k // 16, dtype=np.uint8)
            g = (0.5 + rng.random(rows if rowwise else 1)).astype(np.float32)
            t = pkg.Nvfp4Tensor(torch.from_numpy(b).to(dev), pack.pack(torch.from_numpy(s).to(dev), rows, k),
                                torch.from_numpy(g).to(dev), rows, k, packed=True, rowwise=rowwise)
            return (b, s, g), t

        (ab, as_, ag), A = rand(m, True)
        bh, B = rand(n, False)
        bias = rng.normal(0, 40.0, n).astype(np.float32) if epi else None
        out = gemm.gemm(A, B, bias=None if bias is None else torch.from_numpy(bias).to(dev), epilogue=epi, out_dtype=dt)
        plan = gemm.plan(A, B, bias=None if bias is None else torch.from_numpy(bias).to(dev), epilogue=epi, out=out)
        nb = (m + 127) // 128
        blocks = sorted({0, nb // 2, nb - 1})
        for blk in blocks:
            r0, r1 = blk * 128, min(m, blk * 128 + 128)
            a_s = (ab[r0 * k // 2:r1 * k // 2], as_[r0 * k // 16:r1 * k // 16], ag[r0:r1])
            want = oracle.gemm(a_s, bh, r1 - r0, k, n, 2, bias=bias, epi=epi)
            if dt == torch.bfloat16:
                want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
            got = out[r0:r1].float().cpu().numpy().astype(np.float64)
            err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
            worst = max(worst, err)
        report.append({"gemm": name, "m": m, "n": n, "k": k, "tile": plan.block_n, "k_splits": plan.k_splits,
                       "resident": plan.b_resident, "row_blocks": len(blocks)})
        del A, B, out
    torch.cuda.empty_cache()
    return {"max_rel_fro": worst, "tolerance": 1e-3, "row_blocks": 3, "checked": report,
            "device_status": pkg.read_device_status()}


def small_configs(pkg, torch, dev, peaks, write_gbs):
    """The two single-GPU configurations below the full step: one c_attn forward projection at 8192 tokens
    (per-tensor scales, bf16 out) and one GPT-2-small layer forward + backward at 8192 tokens."""
    from nanogpt_120a_b200.host_step import HostStep
    from nanogpt_120a_b200.projection_set import ModelShape, ProjectionSet

    q, gemm = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule()
    m, k, n = 8192, 768, 2304
    # rotate over enough operand sets that nothing is served from L2 (each set: 12.6 + 3.5 + 37.7 MB)
    sets = []
    for i in range(6):
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
        sets.append((x, w, q.quantize_four_six(x, rowwise=False, packed=True), q.quantize_four_six(w, rowwise=False, packed=True),
                     torch.empty(m, n, dtype=torch.bfloat16, device=dev)))
    bias = torch.randn(n, device=dev) * 0.02
    i = [0]

    def gemm_only():
        i[0] += 1
        x, w, xq, wq, y = sets[i[0] % len(sets)]
        gemm.gemm(xq, wq, bias=bias, epilogue=pkg.EPI_BIAS, out=y)

    amax, chunks = torch.empty(1, device=dev), torch.empty(m * k // 1024, device=dev)

    def quantize_and_gemm():
        i[0] += 1
        x, w, xq, wq, y = sets[i[0] % len(sets)]
        q.tensor_amax(x, chunks, amax)
        q.quantize_four_six(x, amax=amax, rowwise=False, packed=True, out=xq)
        gemm.gemm(xq, wq, bias=bias, epilogue=pkg.EPI_BIAS, out=y)

    flops = 2.0 * m * n * k
    us_g_loop = cuda_time_us(torch, gemm_only, 60)
    us_g = graph_time_us(torch, gemm_only, 2 * len(sets))   # device time: the Python cost of a call stays out
    us_qg = graph_time_us(torch, quantize_and_gemm, 2 * len(sets))
    t_compute = flops / (NOMINAL_FP4_DENSE_TFLOPS * 1e12) * 1e6
    t_write = m * n * 2 / (write_gbs * 1e9) * 1e6
    c2 = {"workload": "c_attn forward projection, X [8192x768] W [2304x768], NVFP4 x NVFP4, bias, bf16 out",
          "gemm_us": us_g, "gemm_tflops": flops / (us_g * 1e-6) / 1e12,
          "quantize_x_plus_gemm_us": us_qg, "gemm_us_python_loop": us_g_loop,
          "timing": "12 calls replayed from a CUDA graph (device time); the Python loop figure is bound by the host",
          "roofline_us": {"tensor": t_compute, "output_write": t_write, "bound": "output_write" if t_write > t_compute else "tensor"},
          "frac_of_min_roofline": max(t_compute, t_write) / us_g}
    del sets
    torch.cuda.empty_cache()
    # one layer through the step driver: a one-layer set whose head is 128 columns wide (1.4 % of the FLOPs)
    layer_shape = ModelShape("gpt2-small-one-layer", 1, 768, 3072, 128)
    ps = ProjectionSet(layer_shape, 8192, dev, seed=4321, inputs_only=True)
    host = HostStep(ps)
    us_layer = cuda_time_us(torch, lambda: host.step(), 20)
    flops_layer = 6.0 * 8192 * (768 * 2304 + 768 * 768 + 2 * 768 * 3072)
    head_flops = 6.0 * 8192 * 768 * 128
    c3 = {"workload": "one GPT-2-small layer (c_attn, c_proj, fc, proj) fwd+bwd at 8192 tokens, weight quantization "
                      "included (plus a 128-column head, 1.4 % of the FLOPs, that the step driver always carries)",
          "ms": us_layer / 1e3, "tflops": (flops_layer + head_flops) / (us_layer * 1e-6) / 1e12}
    host.close()
    del host, ps
    torch.cuda.empty_cache()
    return c2, c3


def run_small_case(args):
    """A small case of one kernel family on cuda:0, for profiler captures of single launches (a few
    hundred MB on the device, two iterations): `quantizers` = one forward quantization of
    X bf16 [32768 x 768] plus one linear backward with dY bf16 [32768 x 2304] (MS-EDEN pair, W^T and X^T
    transposers, both gradient GEMMs); `gemm` = the forward and the two backward GEMM shapes of c_attn
    at 32768 tokens.  Prints no benchmark line."""
    import torch

    import __graft_entry__ as entry

    pkg = entry.load_package()
    dev = torch.device("cuda:0")
    q, g, bwd = pkg.Nvfp4QuantModule(), pkg.Nvfp4GemmModule(), pkg.LinearBackwardModule()
    tokens, in_dim, out_dim = 32768, 768, 2304
    x = torch.randn(tokens, in_dim, device=dev).to(torch.bfloat16)
    w = (torch.randn(out_dim, in_dim, device=dev) * 0.02).to(torch.bfloat16)
    dy = (torch.randn(tokens, out_dim, device=dev) * 1e-3).to(torch.bfloat16)
    bias = torch.zeros(out_dim, device=dev)
    wq = q.quantize_four_six(w, rowwise=False, packed=True)
    scratch = pkg.LinearBackwardScratch(tokens, in_dim, out_dim, dev)
    y = torch.empty(tokens, out_dim, dtype=torch.bfloat16, device=dev)
    dx = torch.empty(tokens, in_dim, dtype=torch.bfloat16, device=dev)
    dw = torch.empty(out_dim, in_dim, dtype=torch.float32, device=dev)
    for _ in range(2):
        xq = q.quantize_four_six(x, rowwise=True, packed=True, decoded_amax=True)
        if args.small_case == "gemm":
            g.gemm(xq, wq, bias=bias, epilogue=pkg.EPI_BIAS, out=y)
        bwd.backward_ms_eden(e=dy, weight=wq, input=xq, scratch=scratch, sign_seed=1, scale_seed=2,
                             dinput=dx, dweight=dw)
    torch.cuda.synchronize()
    status = pkg.read_device_status()
    print(f"small case '{args.small_case}' done, device status {status}", flush=True)
    if status != 0:
        raise SystemExit(1)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------

def run_gpu(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.set_deterministic_reductions(bool(args.deterministic))
    from nanogpt_120a_b200.host_step import HostStep  # noqa: E402
    from nanogpt_120a_b200.projection_set import SHAPES, ProjectionSet  # noqa: E402

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product (use --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        pg = dist.group.WORLD
    if args.gpus != world and rank == 0:
        print(f"[bench] --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    peaks, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def time_steps(step, steps, warmup):
        """(ms per step on the device, max over ranks; host milliseconds to enqueue one step on an empty queue)."""
        for _ in range(warmup):
            step()
        barrier()
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        barrier()
        ms = max_over_ranks(start.elapsed_time(stop)) / steps
        # host cost of enqueueing one step, measured on an empty launch queue (inside the timed loop the host
        # runs ahead until the queue is full and then waits for the device, so its time there is the device's)
        h0 = time.perf_counter()
        step()
        host_ms = (time.perf_counter() - h0) * 1e3
        torch.cuda.synchronize()
        return ms, host_ms

    def make(shape, tokens_rank, total, with_comm=True, seed=1234):
        ps = ProjectionSet(shape, tokens_rank, dev, seed=seed, token_offset=rank * tokens_rank, total_tokens=total,
                           inputs_only=True)
        return ps, HostStep(ps, process_group=pg if with_comm else None)

    # ---- correctness of the kernel instantiations this run uses, before anything is timed -------------
    shape = SHAPES[args.model]
    if args.scaling == "strong":
        tokens_rank = args.tokens // world // 128 * 128
    else:
        tokens_rank = args.tokens
    total_tokens = tokens_rank * world
    parity = None
    if rank == 0 and not args.no_parity_check:
        parity = gemm_self_check(pkg, torch, dev, tokens_rank, shape)
        if not parity["max_rel_fro"] <= parity["tolerance"] or parity["device_status"] != 0:
            emit({"metric": METRIC, "error": "GEMM self-check failed", "parity_check": parity})
            raise SystemExit(2)
    barrier()

    # ---- the headline workload, device-resident -----------------------------------------------------------
    ps, host = make(shape, tokens_rank, total_tokens)
    flops_step_total = shape.flops_per_token() * total_tokens
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: started ahead of the warm-up steps
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        host.step()
    barrier()
    launches_before = pkg.launch_count()
    t_begin = time.time()
    ms_step, host_ms = time_steps(host.step, args.steps, 0)
    t_end = time.time()
    launches = pkg.launch_count() - launches_before
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    # ---- the dominant kernel: a second pass of K steps with every GEMM launch bracketed by a CUDA event pair on
    # its stream (the brackets cost a little, so they stay out of the region above)
    gemm_per_step = 3 * (4 * shape.n_layer + 1)
    pkg.gemm_timing_begin(gemm_per_step * args.steps)
    barrier()
    start.record()
    for _ in range(args.steps):
        host.step()
    stop.record()
    barrier()
    ms_total_bracketed = start.elapsed_time(stop)
    n_gemm, gemm_ms, gemm_flops, _, _ = pkg.gemm_timing_end(0)
    status = pkg.read_device_status()
    value = flops_step_total / (ms_step * 1e-3) / 1e12

    # ---- where the step time goes at N > 1: the same shard without the collective -------------------------------
    timeline = None
    if world > 1:
        ps_nc, host_nc = make(shape, tokens_rank, total_tokens, with_comm=False)
        ms_nc, _ = time_steps(host_nc.step, min(args.steps, 10), 3)
        host_nc.close()
        del ps_nc, host_nc
        timeline = {"step_ms": ms_step, "compute_only_ms": ms_nc, "exposed_allreduce_ms": max(0.0, ms_step - ms_nc),
                    "host_enqueue_ms_per_step": host_ms,
                    "allreduce_bytes_per_step": 4 * sum(b.numel() for b in host.buckets),
                    "note": "compute_only = the same shard stepped without a communicator; the difference is the part "
                            "of the all-reduces (and their SM use) that backward does not hide"}

    # ---- end to end: host buffers, H2D + step + D2H every step -------------------------------------------------
    # Every step's activations and output gradients start in pinned host memory.  They are copied into one of two
    # device input sets on a copy stream while the previous step computes on the other set (what a prefetching
    # loader does); each step ends with a device -> host read of the gradient digest.  All copies of all timed
    # steps lie inside the timed region.
    host_in = {}
    for name, group in (("x", ps.x), ("dy", ps.dy)):
        for w, t in group.items():
            host_in[(name, w)] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    h2d_bytes = sum(h.numel() * h.element_size() for h in host_in.values())
    digest_host = torch.empty(len(host.buckets), dtype=torch.float32, pin_memory=True)
    d2h_bytes = digest_host.numel() * 4
    input_sets = [(ps.x, ps.dy),
                  ({w: torch.empty_like(t) for w, t in ps.x.items()}, {w: torch.empty_like(t) for w, t in ps.dy.items()})]
    copy_stream = torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()

    def e2e_run(steps: int):
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        done = [torch.cuda.Event(), torch.cuda.Event()]

        def stage(step_index: int):
            which = step_index % 2
            with torch.cuda.stream(copy_stream):
                if step_index >= 2:
                    copy_stream.wait_event(done[which])  # the step that last read this set has finished
                xs, dys = input_sets[which]
                for (name, w), h in host_in.items():
                    (xs if name == "x" else dys)[w].copy_(h, non_blocking=True)
                ready[which].record(copy_stream)

        stage(0)
        for i in range(steps):
            if i + 1 < steps:
                stage(i + 1)
            which = i % 2
            main_stream.wait_event(ready[which])
            host.set_inputs(*input_sets[which])
            host.step()
            digest_host.copy_(host.result_digest(), non_blocking=True)
            done[which].record(main_stream)
        host.set_inputs(*input_sets[0])

    e2e_run(2)
    barrier()
    e2e_steps = max(2, min(args.steps, 4))
    start.record()
    e2e_run(e2e_steps)
    stop.record()
    barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(stop)) / e2e_steps
    e2e_value = flops_step_total / (e2e_ms * 1e-3) / 1e12
    del input_sets, host_in

    # ---- the same step replayed from a CUDA graph (launch-overhead-free figure, single rank) ------
    graph_info = None
    if world == 1:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                host.step()
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.steps):
                graph.replay()
            stop.record()
            torch.cuda.synchronize()
            g_ms = start.elapsed_time(stop) / args.steps
            graph_info = {"ms_per_step": g_ms, "value": flops_step_total / (g_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "device_status": pkg.read_device_status(),
                          "note": "the seeds drawn during capture are baked into the graph; the headline is the eager step"}
            del graph
        except Exception as exc:  # the eager figures above stand on their own
            graph_info = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    buckets_bytes = 4 * sum(b.numel() for b in host.buckets)
    host.close()
    del host, ps
    torch.cuda.empty_cache()

    # ---- sub-records: the other configurations the specification names --------------------------------------------------
    extra_steps = max(2, min(args.steps, 5))
    weak = None
    if world > 1 and not args.skip_extra and args.scaling == "strong":
        psw, hw = make(shape, TOTAL_TOKENS, TOTAL_TOKENS * world)
        ms_w, _ = time_steps(hw.step, extra_steps, 3)
        weak = {"scaling": "weak", "tokens_per_gpu": TOTAL_TOKENS, "ms_per_step": ms_w,
                "value": shape.flops_per_token() * TOTAL_TOKENS * world / (ms_w * 1e-3) / 1e12, "unit": "TFLOP/s"}
        hw.close()
        del psw, hw
        torch.cuda.empty_cache()
    medium = None
    if not args.skip_extra and args.model == "gpt2-small":
        med = SHAPES["gpt2-medium"]
        tok = 32768
        psm, hm = make(med, tok, tok * world, seed=99)
        ms_m, _ = time_steps(hm.step, extra_steps, 3)
        medium = {"workload": f"{med.name}: 24 layers, d_model 1024, MLP 4096, vocab 32000, fwd+bwd, {tok} tokens per GPU "
                              f"({tok * world} per step)", "scaling": "weak (32768 tokens per GPU at every N; 262144 at N = 8)",
                  "ms_per_step": ms_m, "value": med.flops_per_token() * tok * world / (ms_m * 1e-3) / 1e12,
                  "unit": "TFLOP/s", "flop_per_step": med.flops_per_token() * tok * world}
        hm.close()
        del psm, hm
        torch.cuda.empty_cache()

    quant = write_gbs = c2 = c3 = None
    if rank == 0:
        write_gbs = write_roofline(torch, dev)
        quant = quantize_records(pkg, torch, dev, peaks["hbm_gbs"])
        if world == 1 and not args.skip_extra:
            c2, c3 = small_configs(pkg, torch, dev, peaks, write_gbs)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tokens = 2048
        tflops, cms, cores = cpu_sample(tokens, 1, 0)
        cpu = {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "ms_per_sample": cms,
               "sample": f"one GPT-2-small layer (c_attn, c_proj, fc, proj) fwd+bwd at {tokens} tokens, oracle "
                         f"restatement of the reference math, all host threads"}

    if rank == 0:
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        # algorithmic bytes of the step's GEMM launches on this rank: NVFP4 operands (0.5625 B/element) read once,
        # output written once
        d, h, v, T = shape.d_model, shape.d_mlp, shape.vocab, tokens_rank
        lin = [(i, o) for _, i, o, _ in shape.linears()] * shape.n_layer + [(d, v)]
        algo = 0.0
        for i, o in lin:
            algo += (T * i + o * i) * 0.5625 + T * o * 2      # forward, bf16 out
            algo += (T * o + i * o) * 0.5625 + T * i * 2      # dX, bf16 out
            algo += (o * T + i * T) * 0.5625 + o * i * 4      # dW, f32 out
        n_launch = max(n_gemm // max(args.steps, 1), 1)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate, bf16 in/out)",
            "data": "synthetic",
            "config": {"workload": f"{shape.name}: {shape.n_layer} layers x (c_attn, c_proj, fc, proj) + LM head "
                                   f"(vocab {shape.vocab}), fwd+bwd, {total_tokens} tokens/step "
                                   f"({tokens_rank} per GPU)",
                       "parallelism": f"token-sharded dp{world}, weights replicated, per-layer NCCL all-reduce of dW "
                                      f"issued from the C++ step driver",
                       "l2": "inputs larger than L2 (every activation / gradient tensor of the step; 126 MB L2)",
                       "deterministic_reductions": bool(args.deterministic),
                       "flop_per_step": flops_step_total, "host": "C++ step driver, one host call per step"},
            "pct_of_fp4_peak": 100.0 * value / (NOMINAL_FP4_DENSE_TFLOPS * world),
            "roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_tcgen05_kernel", "achieved": achieved,
                         "peak": NOMINAL_FP4_DENSE_TFLOPS, "unit": "TFLOP/s", "frac": achieved / NOMINAL_FP4_DENSE_TFLOPS,
                         "peak_source": "nominal dense FP4 (MEASURED_PEAKS.json holds no FP4 figure; 4x its measured "
                                        f"bf16 burst would be {4 * peaks['bf16_tflops']:.0f})",
                         "frac_of_4x_measured_bf16_burst": achieved / (4 * peaks["bf16_tflops"]),
                         "launches": n_gemm, "avg_launch_ms": gemm_ms / max(n_gemm, 1),
                         "gemm_share_of_step": gemm_ms / ms_total_bracketed if ms_total_bracketed > 0 else None,
                         "bracketed_ms_per_step": ms_total_bracketed / args.steps,
                         "algorithmic_bytes_per_launch": algo / n_launch,
                         "traffic": GEMM_TRAFFIC_PER_ALGORITHMIC_BYTE * algo / n_launch,
                         "traffic_source": "DRAM read + write bytes of a small-case profiler capture of this kernel, "
                                           "as a ratio to its algorithmic bytes, times this run's algorithmic bytes",
                         "write_roofline_gbs": write_gbs, "peaks_file": peak_kind},
            "quantize": quant, "cuda_graph_replay": graph_info,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps,
                    "d2h": "digest only: one f32 per gradient bucket; the gradients themselves stay on the device "
                           f"({buckets_bytes} bytes per step), as they do in a training step",
                    "note": "bound by the host's PCIe links (shared by the ranks of a node)"},
            "gpu_launches": launches, "host_enqueue_ms_per_step": host_ms, "clocks": clocks, "device_status": status,
            "parity_check": parity,
        }
        if timeline:
            line["timeline"] = timeline
        if weak:
            line["weak"] = weak
        if medium:
            line["gpt2_medium"] = medium
        if c2:
            line["configs"] = {"c_attn_forward_8192": c2, "one_layer_8192": c3}
        if cpu is not None:
            line["cpu_baseline"] = cpu
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_STREAM = None


def _reserve_stdout() -> None:
    """Keeps the process's original stdout for the one JSON line and points file descriptor 1 at stderr for
    everything else: libraries that write to stdout on their own (NCCL prints its version banner there when
    NCCL_DEBUG is set in the environment) would otherwise put text in front of the result."""
    global _RESULT_STREAM
    if _RESULT_STREAM is None:
        sys.stdout.flush()
        _RESULT_STREAM = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _RESULT_STREAM if _RESULT_STREAM is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    _reserve_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt2-small", choices=["gpt2-small", "gpt2-medium"])
    ap.add_argument("--tokens", type=int, default=TOTAL_TOKENS,
                    help="tokens per step in total (strong scaling, the default) or per GPU (weak scaling)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity-check", action="store_true", help="skip the GEMM self-check that precedes the timing")
    ap.add_argument("--skip-extra", action="store_true",
                    help="skip the sub-records (weak scaling, GPT-2-medium, the 8192-token configurations)")
    ap.add_argument("--deterministic", action="store_true",
                    help="cap split-K at two splits (run-to-run identical dW); the default lets small dW GEMMs "
                         "take as many splits as fill the SMs")
    ap.add_argument("--small-case", default=None, choices=["quantizers", "gemm"],
                    help="run a small single-GPU case of one kernel family (for profiler captures) and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.small_case:
        run_small_case(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
