#!/usr/bin/env python
"""Benchmark of the binary-weight x ternary-activation (BWTA) linear forward on B200.

One JSON line on stdout (rank 0). A *step* is one pass over a pool of LAYERS independent layers of the
workload shape, each with its own prepacked weight plane, so that the weights of consecutive launches
never sit in L2 (the pool is larger than L2). Effective TOPS = 2*M*N*K*LAYERS / step time.

  value     device-resident inputs (prepacked planes, fp16 activations in HBM), the step captured in a
            CUDA graph: activation prepare + GEMM with fused per-channel scale, fp16 out.
  e2e       the same step through the `lowbit_kernel` extension calls with HOST activations: pinned
            host -> device copy of every layer's activations and device -> host copy of every output
            inside the timed region.
  roofline  the GEMM kernel alone (graph of GEMM launches only) against the int8 tensor peak.
  cpu_baseline  the reference's CPU path (dense torch fp32 matmul on sign / ternary tensors) on this
            host's cores, on a bounded sample of the same layers.

`--impl reference` times only that CPU path. Under torchrun every rank owns the row shard of a
(M * world) x K layer, i.e. the same per-GPU work (weak scaling, no data-path collective).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
for _p in (ROOT / "bgemm-cuda_b200", ROOT / "oracle"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

WORKLOADS = {
    # name: (M, K, N, op name, description)
    "c2": (4096, 4096, 128, "bwta", "BWTA GEMM: binary W[4096,4096] x ternary X[4096,128], fp16 alpha epilogue"),
    "c1": (4096, 4096, 64, "xor", "BGEMM: W[4096,4096] x X[4096,64], both {-1,+1}"),
    "c5n16": (28672, 8192, 16, "bwta", "LLM projection 28672x8192, ternary X, N=16"),
    "c5n128": (28672, 8192, 128, "bwta", "LLM projection 28672x8192, ternary X, N=128"),
    "c5n1024": (28672, 8192, 1024, "bwta", "LLM projection 28672x8192, ternary X, N=1024"),
    "c5n4096": (28672, 8192, 4096, "bwta", "LLM projection 28672x8192, ternary X, N=4096"),
}
L2_BYTES = 126 * 1024 * 1024
METRIC = "bwta_effective_tops"
UNIT = "TOPS (2*M*N*K/s)"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        busy = [s for s in sm if s > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_step(ws, xs, alphas, op_name):
    """The reference's CPU arithmetic for a list of layers: dense fp32 matmul on mapped tensors, scaled, fp16."""
    import oracle as O

    op = {"bwta": O.OP_BWTA, "xor": O.OP_XOR}[op_name]
    outs = []
    for w, x, a in zip(ws, xs, alphas):
        acc = O.map_act(x, op) @ O.map_weight(w, op).T
        outs.append((acc * a.float()).to(torch.float16))
    return outs


def make_layer_inputs(M, K, N, op_name, seed):
    import oracle as O

    g = O._gen(seed)
    w = O.rand_pm1((M, K), g)
    x = O.rand_ternary((N, K), g) if op_name == "bwta" else O.rand_pm1((N, K), g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    return w, x, alpha


def time_cpu_baseline(M, K, N, op_name, budget_s=12.0, min_layers=2, max_layers=100000):
    torch.set_num_threads(os.cpu_count() or 1)
    w, x, a = make_layer_inputs(M, K, N, op_name, 1002)
    import oracle as O

    op = {"bwta": O.OP_BWTA, "xor": O.OP_XOR}[op_name]
    wm, xm = O.map_weight(w, op), O.map_act(x, op)          # mapping once: the matmul is what the reference times
    cpu_reference_step([w], [x], [a], op_name)              # warm-up (includes mapping)
    t0 = time.perf_counter()
    n = 0
    while True:
        acc = xm @ wm.T
        _ = (acc * a.float()).to(torch.float16)
        n += 1
        dt = time.perf_counter() - t0
        if (dt > budget_s and n >= min_layers) or n >= max_layers:
            break
    return 2.0 * M * N * K * n / dt / 1e12, n, dt


def run_reference_arm(args, M, K, N, op_name, desc):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    import oracle as O

    op = {"bwta": O.OP_BWTA, "xor": O.OP_XOR}[op_name]
    sample_layers = 2 if M * K * N <= 4096 * 4096 * 128 else 1
    layers = [make_layer_inputs(M, K, N, op_name, 1002 + i) for i in range(sample_layers)]
    mapped = [(O.map_weight(w, op), O.map_act(x, op), a.float()) for w, x, a in layers]

    def step():
        for wm, xm, a in mapped:
            _ = ((xm @ wm.T) * a).to(torch.float16)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = 2.0 * M * N * K * sample_layers * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (CPU matmul on {-1,0,+1} tensors)", "data": "synthetic",
        "config": {"workload": desc, "M": M, "K": K, "N": N, "layers_per_step": sample_layers},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample_layers} layer(s) per step, {args.steps} steps, torch fp32 matmul + scale + fp16 cast"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="layers per step (0 = enough that the weight pool exceeds L2)")
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather", action="store_true", help="all-gather the row shards' outputs (multi-GPU only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    M, K, N, op_name, desc = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, M, K, N, op_name, desc)
        return

    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path for the b200 arm)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import bgemm_b200 as B
    import lowbit_kernel

    op = {"bwta": B.OP_BWTA, "xor": B.OP_XOR}[op_name]
    act_mode = B.ACT_MODE_OF_OP[op]
    plane_b = B.plane_bytes(M, K)
    layers = args.layers or max(8, -(-int(1.5 * L2_BYTES) // plane_b))
    peaks = measured_peaks()

    # ---- synthetic inputs: distinct weights per layer (packed on device), a few distinct activation sets ----
    g = torch.Generator(device=dev)
    g.manual_seed(1002 + rank)
    planes, alphas = [], []
    for _ in range(layers):
        w = (torch.randint(0, 2, (M, K), generator=g, device=dev, dtype=torch.int8) * 2 - 1)
        planes.append(B.pack_weights(w, B.WBIT_NEGATIVE)[0])
        alphas.append((0.01 + 0.09 * torch.rand(M, generator=g, device=dev)).to(torch.float16))
        del w
    n_x = min(layers, 8)
    xs_host = []
    for _ in range(n_x):
        if op_name == "bwta":
            u = torch.rand(N, K, generator=g, device=dev)
            x = torch.where(u < 0.35, -1.0, torch.where(u < 0.70, 1.0, 0.0)).to(torch.float16)
        else:
            x = (torch.randint(0, 2, (N, K), generator=g, device=dev) * 2 - 1).to(torch.float16)
        xs_host.append(x.cpu().pin_memory())
    xs_dev = [x.to(dev) for x in xs_host]
    outs = [torch.empty((N, M), dtype=torch.float16, device=dev) for _ in range(layers)]
    act_bufs = [(torch.empty((N, B.act_ld(K)), dtype=torch.int8, device=dev), torch.empty(N, dtype=torch.int32, device=dev))
                for _ in range(n_x)]
    split_k = args.split_k
    ws = B.workspace(dev, max(B.lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, 1), 1))
    stream = torch.cuda.Stream(device=dev)

    def prep(i):
        a, c = act_bufs[i % n_x]
        x = xs_dev[i % n_x]
        B.check(B.lib.bgemm_prepare_acts(stream.cuda_stream, x.data_ptr(), B.DT_F16, N, K, K, act_mode, 0, a.data_ptr(), c.data_ptr(), 1, 0), "prepare")

    def gemm(i):
        a, c = act_bufs[i % n_x]
        B.check(B.lib.bgemm_gemm(stream.cuda_stream, planes[i].data_ptr(), M, K, a.data_ptr(), c.data_ptr(), N, op, outs[i].data_ptr(),
                                 B.OUT_F16_SCALED, B.LAYOUT_NM, alphas[i].data_ptr(), split_k, ws.data_ptr(), ws.numel(), 1), "gemm")

    def full_step():
        for i in range(layers):
            prep(i)
            gemm(i)

    def gemm_only_step():
        for i in range(layers):
            gemm(i)

    # warm up outside capture (sets function attributes, fills caches), then capture both graphs
    with torch.cuda.stream(stream):
        c0 = B.launch_count()
        full_step()
        launches_per_step = B.launch_count() - c0
        stream.synchronize()
        g_full, g_gemm = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_full, stream=stream):
            full_step()
        with torch.cuda.graph(g_gemm, stream=stream):
            gemm_only_step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(graph, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                graph.replay()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_full = timed(g_full, args.steps, args.warmup)
    ms_gemm = timed(g_gemm, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None

    ops_layer = 2.0 * M * N * K
    value = ops_layer * layers * world * args.steps / (ms_full * 1e-3) / 1e12
    gemm_us = ms_gemm * 1e3 / (args.steps * layers)
    gemm_tops = ops_layer / (gemm_us * 1e-6) / 1e12
    bytes_alg = plane_b + N * B.act_ld(K) + 4 * N + 2 * M + 2 * N * M      # plane + int8 acts + colsum + alpha + fp16 out
    gemm_gbs = bytes_alg / (gemm_us * 1e-6) / 1e9
    int8_peak = 2.0 * peaks["bf16_tflops"]
    t_tensor, t_hbm = ops_layer / (int8_peak * 1e12), bytes_alg / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        roofline = {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tops / int8_peak,
                    "traffic": None, "peak_source": f"2 x bf16 GEMM peak ({peaks['source']}); int8 tcgen05 issue-rate microbenchmark on this pool: 3873",
                    "ops": "integer multiply-adds x 2"}
    else:
        roofline = {"bound": "hbm", "achieved": gemm_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gemm_gbs / peaks["hbm_gbs"],
                    "traffic": None, "peak_source": peaks["source"]}
    roofline.update({"kernel": "gemm_kernel (tcgen05 kind::i8, TMEM A operand)", "kernel_us": gemm_us, "bytes_alg_per_launch": bytes_alg,
                     "ops_per_launch": ops_layer, "kernel_gbs": gemm_gbs, "kernel_tops": gemm_tops})

    # ---- end to end through the extension with host activations -------------------------------------------------
    e2e = None
    if not args.no_e2e:
        h2d_s, d2h_s = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        x_stage = [torch.empty((N, K), dtype=torch.float16, device=dev) for _ in range(layers)]
        out_host = [torch.empty((N, M), dtype=torch.float16).pin_memory() for _ in range(min(layers, 16))]
        h2d_bytes = layers * N * K * 2
        d2h_bytes = layers * N * M * 2

        def e2e_step():
            keep = []
            for i in range(layers):
                with torch.cuda.stream(h2d_s):
                    x_stage[i].copy_(xs_host[i % n_x], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(h2d_s)
                with torch.cuda.stream(stream):
                    stream.wait_event(ev)
                    if op_name == "bwta":
                        y = lowbit_kernel.bwta_linear_forward_cuda(x_stage[i], planes[i], M, K, alphas[i], split_k)
                    else:
                        y = lowbit_kernel.bgemm_linear_forward_packed(x_stage[i], planes[i], M, K, alphas[i], split_k, 1, 2)
                    ev2 = torch.cuda.Event(); ev2.record(stream)
                with torch.cuda.stream(d2h_s):
                    d2h_s.wait_event(ev2)
                    out_host[i % len(out_host)].copy_(y, non_blocking=True)
                    y.record_stream(d2h_s)
                keep.append(y)
            return keep

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        d2h_s.synchronize(); stream.synchronize(); h2d_s.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        barrier()
        if world > 1:
            t = torch.tensor([wall_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall_ms = float(t.item())
        e2e = {"value": ops_layer * layers * world * e2e_steps / (wall_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "ms_per_step": wall_ms / e2e_steps,
               "api": "lowbit_kernel.bwta_linear_forward_cuda on pinned-host activations, outputs copied back to pinned host"}

    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        v, n, dt = time_cpu_baseline(M, K, N, op_name)
        cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{n} layer(s) of the same shape in {dt:.1f} s: torch fp32 matmul on mapped CPU tensors + scale + fp16 cast"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_full / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8 x s8 -> s32 (fp16 scaled out)", "data": "synthetic",
            "config": {"workload": desc, "M_per_gpu": M, "K": K, "N": N, "layers_per_step": layers,
                       "l2": f"weight pool {layers * plane_b / 2**20:.0f} MiB per GPU > 126 MB L2, one distinct plane per launch",
                       "split_k": split_k or B.lib.bgemm_gemm_auto_split_k(M, N, K, 1), "sharding": f"rows x{world}, no collective",
                       "timed": "CUDA graph of prepare_acts + gemm per layer"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": int(launches_per_step) * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
