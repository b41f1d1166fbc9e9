#!/usr/bin/env python
"""Benchmark of the NVFP4 projection path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the full 12-layer GPT-2-small training-step projection set (48 block linears + the
tied LM head with a 32000-entry vocabulary), forward and backward, 65536 tokens per GPU, on
seeded synthetic bf16 tensors (activations ~N(0,1), weights ~N(0,0.02), upstream gradients
~N(0,1e-3)).  One step = weight quantization + forward + backward of every projection, plus
(N > 1) one NCCL all-reduce per layer of dW/dbias.  The metric is useful TFLOP/s:
6 * tokens * sum(N*K) per step, padding never counted.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference's math (the reference has no CPU implementation of its own and its kernels do not
build here) on a bounded sample of the same workload.
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
TOKENS_PER_GPU = 65536


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------

# dram__bytes_read.sum + dram__bytes_write.sum over the 147 GEMM launches of one step of the default
# workload (GPT-2-small projection set, 65536 tokens, 1 GPU): 17.15 GB read + 23.36 GB written.
GEMM_DRAM_BYTES_PER_STEP_65536 = 17.154715e9 + 23.360743e9
GEMM_TRAFFIC_SOURCE = ("ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum over one step's 147 GEMM launches "
                       "(profiles/gemm_tcgen05_ncu.md); algorithmic bytes of the same launches: 37.5 GB")


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
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
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
# GPU arm
# --------------------------------------------------------------------------------------------

def quantize_bandwidth(pkg, torch, dev, peak_gbs):
    """Config-1 quantizer: [8192 x 768] bf16 -> NVFP4, rotating over 16 buffers (201 MB > L2)."""
    q = pkg.Nvfp4QuantModule()
    rows, cols, nbuf = 8192, 768, 16
    xs = [torch.randn(rows, cols, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
    amax = [q.row_amax(x) for x in xs]
    outs = [q.quantize_four_six(x, amax=a, rowwise=True, packed=True) for x, a in zip(xs, amax)]
    for _ in range(3):
        for x, a, o in zip(xs, amax, outs):
            q.quantize_four_six(x, amax=a, rowwise=True, packed=True, out=o)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    start.record()
    for _ in range(reps):
        for x, a, o in zip(xs, amax, outs):
            q.quantize_four_six(x, amax=a, rowwise=True, packed=True, out=o)
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / (reps * nbuf)
    algo_bytes = rows * cols * 2.5625
    gbs = algo_bytes / (us * 1e-6) / 1e9
    return {"workload": "four-six quantize [8192x768] bf16 -> NVFP4, rowwise scale, packed scale layout "
                        "(amax precomputed), 16 rotating buffers", "us": us, "achieved_gbs": gbs,
            "algorithmic_bytes": algo_bytes, "frac_of_hbm_peak": gbs / peak_gbs}


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


def run_gpu(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.set_deterministic_reductions(bool(args.deterministic))
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

    shape = SHAPES[args.model]
    if args.scaling == "weak":
        tokens_rank = args.tokens
        total_tokens = args.tokens * world
    else:
        tokens_rank = args.tokens // world
        total_tokens = tokens_rank * world
    ps = ProjectionSet(shape, tokens_rank, dev, seed=1234, token_offset=rank * tokens_rank, process_group=pg)
    flops_step_total = shape.flops_per_token() * total_tokens
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

    # ---- device-resident timing -----------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: started ahead of the warm-up steps
    for _ in range(max(args.warmup, 3)):
        ps.step()
    barrier()
    launches_before = pkg.launch_count()
    gemm_per_step = 3 * (4 * shape.n_layer + 1)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin = time.time()
    start.record()
    for _ in range(args.steps):
        ps.step()
    stop.record()
    barrier()
    t_end = time.time()
    ms_total = max_over_ranks(start.elapsed_time(stop))
    launches = pkg.launch_count() - launches_before

    # ---- the dominant kernel: a second pass of K steps with every GEMM launch bracketed by a CUDA
    # event pair on its stream (the brackets cost a little, so they stay out of the region above)
    pkg.gemm_timing_begin(gemm_per_step * args.steps)
    barrier()
    start.record()
    for _ in range(args.steps):
        ps.step()
    stop.record()
    barrier()
    ms_total_bracketed = start.elapsed_time(stop)
    n_gemm, gemm_ms, gemm_flops, _, _ = pkg.gemm_timing_end(0)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    status = pkg.read_device_status()
    ms_step = ms_total / args.steps
    value = flops_step_total / (ms_step * 1e-3) / 1e12

    # ---- end to end: host buffers, H2D + step + D2H every step ------------------------------
    # Every step's activations and output gradients start in pinned host memory.  They are copied
    # into one of two device input sets on a copy stream while the previous step computes on the
    # other set (what a prefetching loader does); each step ends with a device -> host read of the
    # gradient digest.  All copies of all timed steps lie inside the timed region.
    host_in = {}
    for name, group in (("x", ps.x), ("dy", ps.dy)):
        for w, t in group.items():
            host_in[(name, w)] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    h2d_bytes = sum(h.numel() * h.element_size() for h in host_in.values())
    digest_host = torch.empty(len(ps.buckets), dtype=torch.float32, pin_memory=True)
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
            ps.x, ps.dy = input_sets[which]
            ps.step()
            digest_host.copy_(ps.result_digest(), non_blocking=True)
            done[which].record(main_stream)
        ps.x, ps.dy = input_sets[0]

    e2e_run(2)
    barrier()
    e2e_steps = max(2, min(args.steps, 4))
    start.record()
    e2e_run(e2e_steps)
    stop.record()
    barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(stop)) / e2e_steps
    e2e_value = flops_step_total / (e2e_ms * 1e-3) / 1e12

    quant = quantize_bandwidth(pkg, torch, dev, peaks["hbm_gbs"]) if rank == 0 else None

    # ---- the same step replayed from a CUDA graph (launch-overhead-free figure, single rank) ------
    graph_info = None
    if world == 1:
        try:
            graph = ps.capture_step()
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
                          "device_status": pkg.read_device_status()}
        except Exception as exc:  # the eager figures above stand on their own
            graph_info = {"error": f"{type(exc).__name__}: {exc}"[:200]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tokens = 2048
        tflops, cms, cores = cpu_sample(tokens, 1, 0)
        cpu = {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "ms_per_sample": cms,
               "sample": f"one GPT-2-small layer (c_attn, c_proj, fc, proj) fwd+bwd at {tokens} tokens, oracle "
                         f"restatement of the reference math, all host threads"}

    if rank == 0:
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        # DRAM bytes per GEMM launch (average over the launches of a step): profiler capture of one full
        # step of this workload at 65536 tokens per GPU; operand and output bytes grow with the tokens
        gemm_traffic = None
        if args.model == "gpt2-small" and n_gemm > 0:
            gemm_traffic = GEMM_DRAM_BYTES_PER_STEP_65536 * (tokens_rank / 65536.0) / gemm_per_step
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate, bf16 in/out)",
            "data": "synthetic",
            "config": {"workload": f"{shape.name}: {shape.n_layer} layers x (c_attn, c_proj, fc, proj) + LM head "
                                   f"(vocab {shape.vocab}), fwd+bwd, {total_tokens} tokens/step "
                                   f"({tokens_rank} per GPU)",
                       "parallelism": f"token-sharded dp{world}, weights replicated, per-layer NCCL all-reduce of dW",
                       "l2": "inputs larger than L2 (>= 100 MB per activation tensor)",
                       "deterministic_reductions": bool(args.deterministic),
                       "flop_per_step": flops_step_total},
            "pct_of_fp4_peak": 100.0 * value / (NOMINAL_FP4_DENSE_TFLOPS * world),
            "roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_tcgen05_kernel", "achieved": achieved,
                         "peak": NOMINAL_FP4_DENSE_TFLOPS, "unit": "TFLOP/s", "frac": achieved / NOMINAL_FP4_DENSE_TFLOPS,
                         "peak_source": "nominal dense FP4 (MEASURED_PEAKS.json holds no FP4 figure; 4x its measured "
                                        f"bf16 burst would be {4 * peaks['bf16_tflops']:.0f})",
                         "frac_of_4x_measured_bf16_burst": achieved / (4 * peaks["bf16_tflops"]),
                         "launches": n_gemm, "avg_launch_ms": gemm_ms / max(n_gemm, 1),
                         "gemm_share_of_step": gemm_ms / ms_total_bracketed if ms_total_bracketed > 0 else None,
                         "bracketed_ms_per_step": ms_total_bracketed / args.steps,
                         "traffic": gemm_traffic, "traffic_source": GEMM_TRAFFIC_SOURCE if gemm_traffic else None,
                         "peaks_file": peak_kind},
            "quantize": quant, "cuda_graph_replay": graph_info,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        emit(line)
    if world > 1:
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
    ap.add_argument("--tokens", type=int, default=TOKENS_PER_GPU,
                    help="tokens per GPU (weak scaling) or in total (strong scaling)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
