#!/usr/bin/env python
"""Benchmark of the binary-weight x ternary-activation (BWTA) linear forward on B200.

One JSON line on stdout (rank 0). A *step* is one pass over a pool of LAYERS independent layers of the
workload shape, each with its own prepacked weight plane, activations and scales, so that no weight is
ever served from L2 (the pool is larger than L2). The pool is submitted through the library's batch
dimension: one activation-prepare launch and one GEMM launch per step. Effective TOPS =
2*M*N*K*LAYERS / step time.

  value     device-resident inputs (prepacked planes, fp16 activations in HBM), the step captured in a
            CUDA graph: activation prepare + GEMM with fused per-channel scale, fp16 out.
  e2e       the same step through the `lowbit_kernel` extension calls with HOST activations: pinned
            host -> device copy of every layer's activations and device -> host copy of every output
            inside the timed region.
  roofline  the GEMM kernel alone (graph of the batched GEMM launch only) against the int8 tensor peak.
  per_layer_launch  the same pool as one GEMM launch per layer (the latency-bound regime), for reference.
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
import sys
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
    "c5n1": (28672, 8192, 1, "bwta", "LLM projection 28672x8192, ternary X, N=1 (single-token decode)"),
    "c5n4": (28672, 8192, 4, "bwta", "LLM projection 28672x8192, ternary X, N=4"),
    "c5n16": (28672, 8192, 16, "bwta", "LLM projection 28672x8192, ternary X, N=16"),
    "c5n128": (28672, 8192, 128, "bwta", "LLM projection 28672x8192, ternary X, N=128"),
    "c5n1024": (28672, 8192, 1024, "bwta", "LLM projection 28672x8192, ternary X, N=1024"),
    "c5n4096": (28672, 8192, 4096, "bwta", "LLM projection 28672x8192, ternary X, N=4096"),
}
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per layer of the batched GEMM launch (gemm_persist_kernel), from the ncu
# capture summarised under profiles/ (80 layers captured; traffic grows in proportion to the layer count). Workloads
# without a capture: null.
NCU_DRAM_BYTES_PER_LAYER = {"c2": 270.15e6 / 80,     # profiles/gemm_persist_kernel_bwta_4096x4096x128_batched80.md
                            "c5n1": 29.39e6}          # profiles/gemm_skinny_kernel_bwta_28672x8192x1.md
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
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs (read-only NVML queries from a
    background thread, ~1 ms apart, so that even a few-millisecond region gets samples)."""

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []          # (time, sm MHz, throttle mask)
        self.t_begin = self.t_end = None
        self.reasons = set()
        self.max_mhz = None
        self._stop = False
        self._thread = None
        self._err = None

    def _run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu
            if vis:
                try:
                    idx = int(vis.split(",")[self.gpu])
                except (ValueError, IndexError):
                    pass
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
            self._names = names
            while not self._stop:
                self.samples.append((time.perf_counter(), float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                     nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)))
                time.sleep(0.0005)
        except Exception as e:          # NVML missing or refused: report it instead of failing the benchmark
            self._err = repr(e)

    def start(self):
        import threading

        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def begin(self):
        self.t_begin = time.perf_counter()

    def end(self):
        self.t_end = time.perf_counter()

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=5)
        win = [x for x in self.samples if self.t_begin is not None and self.t_begin <= x[0] <= (self.t_end or x[0])]
        if not win:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples: " + str(self._err)], "samples": 0}
        mask = 0
        for x in win:
            mask |= x[2]
        reasons = sorted(k for k, bit in self._names.items() if mask & bit)
        mhz = [x[1] for x in win]
        return {"sm_mhz": statistics.median(mhz), "sm_min_mhz": min(mhz), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(win), "window_ms": (self.t_end - self.t_begin) * 1e3}


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
    ap.add_argument("--steps", type=int, default=400)
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

    sampler = ClockSampler(local_rank)      # started early: NVML start-up takes longer than a short timed region
    if rank == 0:
        sampler.start()
    op = {"bwta": B.OP_BWTA, "xor": B.OP_XOR}[op_name]
    act_mode = B.ACT_MODE_OF_OP[op]
    plane_b = B.plane_bytes(M, K)
    layers = args.layers or max(8, -(-int(1.5 * L2_BYTES) // plane_b))
    peaks = measured_peaks()

    # ---- synthetic inputs: one distinct packed weight plane, activation matrix and scale vector per layer ----
    g = torch.Generator(device=dev)
    g.manual_seed(1002 + rank)
    planes = torch.empty(layers * plane_b, dtype=torch.uint8, device=dev)
    for i in range(layers):
        w = (torch.randint(0, 2, (M, K), generator=g, device=dev, dtype=torch.int8) * 2 - 1)
        B.check(B.lib.bgemm_pack_weights(None, w.data_ptr(), B.DT_I8, M, K, K, B.WBIT_NEGATIVE, planes.data_ptr() + i * plane_b,
                                         None, None, 1, 0), "pack")
        torch.cuda.synchronize()
        del w
    alphas = (0.01 + 0.09 * torch.rand(layers, M, generator=g, device=dev)).to(torch.float16)
    if op_name == "bwta":
        u = torch.rand(layers, N, K, generator=g, device=dev)
        xs_dev = torch.where(u < 0.35, -1.0, torch.where(u < 0.70, 1.0, 0.0)).to(torch.float16)
        del u
    else:
        xs_dev = (torch.randint(0, 2, (layers, N, K), generator=g, device=dev) * 2 - 1).to(torch.float16)
    xs_host = xs_dev.cpu().pin_memory()
    outs = torch.empty((layers, N, M), dtype=torch.float16, device=dev)
    acts = torch.empty((layers, N, B.act_ld(K)), dtype=torch.int8, device=dev)
    colsum = torch.empty((layers, N), dtype=torch.int32, device=dev)
    split_k = args.split_k
    ws = B.workspace(dev, max(B.lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, layers), B.lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, 1), 1))
    stream = torch.cuda.Stream(device=dev)
    act_row = N * B.act_ld(K)

    # One step = ONE batched launch of each kernel over the whole pool (the library's batch dimension).
    def prep_all():
        B.check(B.lib.bgemm_prepare_acts(stream.cuda_stream, xs_dev.data_ptr(), B.DT_F16, N, K, K, act_mode, 0, acts.data_ptr(),
                                         colsum.data_ptr(), layers, N * K), "prepare")

    def gemm_all():
        B.check(B.lib.bgemm_gemm(stream.cuda_stream, planes.data_ptr(), M, K, acts.data_ptr(), colsum.data_ptr(), N, op, outs.data_ptr(),
                                 B.OUT_F16_SCALED, B.LAYOUT_NM, alphas.data_ptr(), split_k, ws.data_ptr(), ws.numel(), layers), "gemm")

    # The same pool as one launch per layer (latency-bound regime), reported for reference only.
    def gemm_one(i):
        B.check(B.lib.bgemm_gemm(stream.cuda_stream, planes.data_ptr() + i * plane_b, M, K, acts.data_ptr() + i * act_row,
                                 colsum.data_ptr() + 4 * i * N, N, op, outs.data_ptr() + 2 * i * N * M, B.OUT_F16_SCALED, B.LAYOUT_NM,
                                 alphas.data_ptr() + 2 * i * M, split_k, ws.data_ptr(), ws.numel(), 1), "gemm")

    def full_step():
        prep_all()
        gemm_all()

    def per_layer_step():
        for i in range(layers):
            gemm_one(i)

    # warm up outside capture (sets function attributes, fills caches), then capture the graphs
    with torch.cuda.stream(stream):
        c0 = B.launch_count()
        full_step()
        launches_per_step = B.launch_count() - c0
        per_layer_step()
        stream.synchronize()
        g_full, g_gemm, g_layers = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_full, stream=stream):
            full_step()
        with torch.cuda.graph(g_gemm, stream=stream):
            gemm_all()
        with torch.cuda.graph(g_layers, stream=stream):
            per_layer_step()
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

    if rank == 0:
        sampler.begin()
    ms_full = timed(g_full, args.steps, args.warmup)
    ms_gemm = timed(g_gemm, args.steps, args.warmup)
    if rank == 0:
        sampler.end()
    clocks = sampler.stop() if rank == 0 else None
    ms_layers = timed(g_layers, max(3, args.steps // 5), 3)
    status = B.lib.bgemm_device_status(1)
    assert status == 0, f"a bounded wait inside a kernel ran out (device status {status}): results invalid"

    ops_layer = 2.0 * M * N * K
    value = ops_layer * layers * world * args.steps / (ms_full * 1e-3) / 1e12
    launch_us = ms_gemm * 1e3 / args.steps                                   # one batched GEMM launch
    gemm_tops = ops_layer * layers / (launch_us * 1e-6) / 1e12
    bytes_layer = plane_b + N * B.act_ld(K) + 4 * N + 2 * M + 2 * N * M      # plane + int8 acts + colsum + alpha + fp16 out
    gemm_gbs = bytes_layer * layers / (launch_us * 1e-6) / 1e9
    int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    t_tensor, t_hbm = ops_layer / (int8_peak * 1e12), bytes_layer / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        roofline = {"bound": "tensor", "achieved": gemm_tops, "peak": int8_peak, "unit": "TFLOP/s", "frac": gemm_tops / int8_peak,
                    "traffic": (NCU_DRAM_BYTES_PER_LAYER[args.workload] * layers if args.workload in NCU_DRAM_BYTES_PER_LAYER else None),
                    "peak_source": f"2 x sustained bf16 GEMM peak ({peaks['source']}; the int8 pipe runs at twice the bf16 rate); burst "
                                   f"2 x {peaks['bf16_tflops']}; tcgen05 kind::i8 issue-rate microbenchmark on this pool: 3873",
                    "ops": "integer multiply-adds x 2"}
    else:
        roofline = {"bound": "hbm", "achieved": gemm_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gemm_gbs / peaks["hbm_gbs"],
                    "traffic": (NCU_DRAM_BYTES_PER_LAYER[args.workload] * layers if args.workload in NCU_DRAM_BYTES_PER_LAYER else None), "peak_source": peaks["source"]}
    roofline.update({"kernel": "gemm_skinny_kernel (CUDA cores, weight streaming) for N <= 4; gemm_persist_kernel for pools with one tile across N, else gemm_kernel (tcgen05 kind::i8, A operand unpacked into tensor memory)", "launch_us": launch_us,
                     "layers_per_launch": layers, "bytes_alg_per_launch": bytes_layer * layers, "ops_per_launch": ops_layer * layers,
                     "kernel_gbs": gemm_gbs, "kernel_tops": gemm_tops})
    lsteps = max(3, args.steps // 5)
    per_layer = {"us_per_layer": ms_layers * 1e3 / (lsteps * layers),
                 "tops": ops_layer * layers * lsteps / (ms_layers * 1e-3) / 1e12,
                 "what": "same pool, one GEMM launch per layer in a CUDA graph (latency-bound regime)",
                 "split_k": split_k or B.lib.bgemm_gemm_auto_split_k(M, N, K, 1)}

    # ---- end to end through the extension with host activations -------------------------------------------------
    e2e = None
    if not args.no_e2e:
        # The pool goes through the `lowbit_kernel` calls in groups on three streams, so that the host -> device
        # copies of a group's activations and the device -> host copies of its outputs overlap other groups' GEMMs.
        groups = max(1, min(8, layers // 8))
        bounds = [layers * j // groups for j in range(groups + 1)]
        h2d_s, d2h_s = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        x_stage = torch.empty((layers, N, K), dtype=torch.float16, device=dev)
        out_host = torch.empty((layers, N, M), dtype=torch.float16).pin_memory()
        h2d_bytes = layers * N * K * 2
        d2h_bytes = layers * N * M * 2
        plane_groups = [planes[bounds[j] * plane_b: bounds[j + 1] * plane_b] for j in range(groups)]
        alpha_groups = [alphas[bounds[j]: bounds[j + 1]].contiguous() for j in range(groups)]

        def e2e_step():
            keep = []
            for j in range(groups):
                lo, hi = bounds[j], bounds[j + 1]
                with torch.cuda.stream(h2d_s):
                    x_stage[lo:hi].copy_(xs_host[lo:hi], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(h2d_s)
                with torch.cuda.stream(stream):
                    stream.wait_event(ev)
                    a, c = lowbit_kernel.prepare_acts(x_stage[lo:hi], act_mode, False)
                    y = lowbit_kernel.gemm_prepared(plane_groups[j], M, K, a, c, op, B.OUT_F16_SCALED, B.LAYOUT_NM, alpha_groups[j], split_k)
                    ev2 = torch.cuda.Event(); ev2.record(stream)
                with torch.cuda.stream(d2h_s):
                    d2h_s.wait_event(ev2)
                    out_host[lo:hi].copy_(y, non_blocking=True)
                    y.record_stream(d2h_s)
                keep.append((a, c, y))
            return keep

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
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
               "api": f"lowbit_kernel.prepare_acts + gemm_prepared (batched, {groups} groups on 3 streams): fp16 activations from pinned host "
                      "memory, fp16 outputs copied back to pinned host memory, weights resident (prepacked)"}

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
                       "l2": f"weight pool {layers * plane_b / 2**20:.0f} MiB per GPU > 126 MB L2, every layer has its own plane",
                       "split_k": split_k or B.lib.bgemm_gemm_auto_split_k(M, N, K, layers), "sharding": f"rows x{world}, no collective",
                       "timed": "CUDA graph of one batched prepare_acts launch + one batched gemm launch over the pool"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "per_layer_launch": per_layer,
            "gpu_launches": int(launches_per_step) * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
