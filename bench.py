#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path: decode dequant-matvec HBM GB/s (headline), with the
prefill dequant-GEMM TFLOP/s reported beside it.

    python bench.py --gpus N --steps K --warmup W            # this library (one process per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores

Workload (N = 1): the 4-bit group-64 matvec of the bit-width x group sweep, W out=11008 x in=4096, M = 1,
fp16 activations, fp32 output.  One step = one pass over LAYERS distinct weight sets (LAYERS x 25.4 MB =
406 MB, larger than the 126 MB L2, so every launch streams its weights from HBM), i.e. LAYERS launches.
value = algorithmic bytes (packed codes + scales + biases + x + y) per second.

N > 1 (weak scaling): every rank holds its own 11008-row shard of a (N x 11008)-row projection; a step
is the same pass, each launch followed by the all-gather of the fp32 output slices over NVLink.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

O_ROWS, K_COLS, BITS, GS = 11008, 4096, 4, 64
LAYERS = 16          # distinct weight sets per step; --layers overrides it (profiling runs use fewer)
NCU_DRAM_BYTES_PER_LAUNCH = 25442048     # ncu capture of the decode kernel at this shape, see profiles/
METRIC = "decode_qmv_hbm_gbs"
UNIT = "GB/s"


def alg_bytes(O, K, bits, gs, M, s_size=2, x_size=2, y_size=4):
    """Algorithmic bytes of one call: packed codes + scales + biases + activations + outputs."""
    return O * K * bits // 8 + 2 * O * (K // gs) * s_size + M * K * x_size + M * O * y_size


def workload_name(layers):
    per_launch = alg_bytes(O_ROWS, K_COLS, BITS, GS, 1)
    return (f"decode matvec {O_ROWS}x{K_COLS} b{BITS} g{GS} M=1, fp16 x, fp32 y; "
            f"{layers} distinct weight sets per step ({layers * per_launch / 1e6:.0f} MB > L2)")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained":
                d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (a read-only query) every few milliseconds while
    the timed regions run."""

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.stop_flag, self.thread, self.err = gpu_index, [], False, None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu
            if vis:
                ent = vis.split(",")[self.gpu].strip()
                if ent.isdigit():
                    idx = int(ent)
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:      # no NVML: report that instead of a number
            self.err = str(e)[:100]
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.rows.append((time.perf_counter(), float(mhz), int(reasons)))
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self, windows=None):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + str(self.err)]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        nv = self.nv
        rows = self.rows
        if windows:
            inside = [r for r in rows if any(a <= r[0] <= b for a, b in windows)]
            rows = inside or rows
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        seen = sorted(n for n, bit in names.items() if any(r[2] & bit for r in rows))
        sm = [r[1] for r in rows]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": seen,
                "samples": len(sm)}


def cpu_sample(seconds_target: float = 12.0):
    """The oracle's restatement of the reference's CPU path (unpack + fp32 dequant + fp32 dot, OpenMP over
    output rows) timed on the host cores, on one 11008 x 4096 layer of the same workload."""
    from oracle import oracle
    synth = importlib.import_module("mlx-runner_b200.synth")
    lay = synth.make_layer(O_ROWS, K_COLS, BITS, GS, synth.F16, seed=0, keep_codes=False)
    _, x = synth.make_activations(1, K_COLS, synth.F16, seed=1)
    cores = len(os.sched_getaffinity(0))
    packed8 = lay.packed.view(np.uint8)
    call = lambda: oracle.qmatmul(packed8, lay.scales_raw, lay.biases_raw, lay.scale_dtype, x, K_COLS, BITS, GS,
                                  accumulate_double=False, threads=cores)
    call()
    t0 = time.perf_counter()
    call()
    one = time.perf_counter() - t0
    reps = max(3, min(200, int(seconds_target / max(one, 1e-4))))
    best = one
    for _ in range(reps):
        t0 = time.perf_counter()
        call()
        best = min(best, time.perf_counter() - t0)
    gbs = alg_bytes(O_ROWS, K_COLS, BITS, GS, 1) / best / 1e9
    return {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one {O_ROWS}x{K_COLS} 4-bit g64 layer, M=1, best of {reps + 1} calls, fp32 accumulate",
            "ms_per_call": best * 1e3}


def run_sweep(args):
    """--sweep: the decode matvec over bit widths, group sizes, batch sizes and the two projection shapes of the
    reference's sweep configuration, as a markdown table on stdout (not the benchmark's JSON line).  Every case
    runs eight distinct weight sets per step, replayed as a CUDA graph, timed with CUDA events."""
    import torch
    mlxq = importlib.import_module("mlx-runner_b200")
    synth = importlib.import_module("mlx-runner_b200.synth")
    dev = torch.device("cuda", 0)

    def one(O, K, bits, gs, M, L=8, reps=10):
        layers, keep = [], []
        for i in range(L):
            lay = synth.make_layer(O, K, bits, gs, synth.F16, seed=i, keep_codes=False)
            w = torch.from_numpy(lay.packed.view(np.int32)).to(dev)
            sc = torch.from_numpy(lay.scales_raw.view(np.int16)).to(dev).view(torch.float16)
            bi = torch.from_numpy(lay.biases_raw.view(np.int16)).to(dev).view(torch.float16)
            keep.append((w, sc, bi))
            layers.append(mlxq.Linear(w, sc, bi, None, inDim=K))
        x = torch.randn((M, K), device=dev, dtype=torch.float16)
        y = torch.empty((L, M, O), device=dev, dtype=torch.float32)

        def step():
            st = torch.cuda.current_stream()
            for i, lin in enumerate(layers):
                lin.encode(st, x, K, y[i], O, M)
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        mlxq.streamStatus(None, 0)
        us = e0.elapsed_time(e1) * 1e3 / (reps * L)
        return us, alg_bytes(O, K, bits, gs, M) / us / 1e3

    print("| shape (out x in) | bits | group | M | us per launch | GB/s |")
    print("|---|---|---|---|---|---|")
    cases = [(11008, 4096, b, 64, m) for b in (2, 3, 4, 5, 6, 8) for m in (1, 8)]
    cases += [(4096, 11008, 4, 64, m) for m in (1, 8)] + [(11008, 4096, 4, gs, m) for gs in (32, 128) for m in (1, 4)]
    for O, K, bits, gs, M in cases:
        us, gbs = one(O, K, bits, gs, M)
        print(f"| {O} x {K} | {bits} | {gs} | {M} | {us:.1f} | {gbs:.0f} |", flush=True)


def run_reference(args):
    """--impl reference: the reference's CPU algorithm (oracle port; the Swift sources cannot be built on
    Linux) on all host cores.  A step is one matvec over one layer of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    synth = importlib.import_module("mlx-runner_b200.synth")
    lay = synth.make_layer(O_ROWS, K_COLS, BITS, GS, synth.F16, seed=0, keep_codes=False)
    _, x = synth.make_activations(1, K_COLS, synth.F16, seed=1)
    cores = len(os.sched_getaffinity(0))
    packed8 = lay.packed.view(np.uint8)
    call = lambda: oracle.qmatmul(packed8, lay.scales_raw, lay.biases_raw, lay.scale_dtype, x, K_COLS, BITS, GS,
                                  accumulate_double=False, threads=cores)
    for _ in range(max(args.warmup, 1)):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    dt = time.perf_counter() - t0
    gbs = args.steps * alg_bytes(O_ROWS, K_COLS, BITS, GS, 1) / dt / 1e9
    sample = f"one {O_ROWS}x{K_COLS} 4-bit g64 layer per step, M=1, fp32 accumulate, OpenMP over rows"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(LAYERS), "rows_per_gpu": O_ROWS, "in_dim": K_COLS, "bits": BITS,
                   "group_size": GS, "batch": 1, "launches_per_step": 1,
                   "sample": "each CPU step is one of the workload's weight sets (a step of the GPU arm is 16 of them)"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def prefill_probe(mlxq, torch, device, peaks):
    """The prefill dequant-GEMM beside the headline: 14336 x 4096, 4-bit g64, bf16 in/out, M = 2048."""
    synth = importlib.import_module("mlx-runner_b200.synth")
    O, K, M = 14336, 4096, 2048
    try:
        lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=3, keep_codes=False)
        w = torch.from_numpy(lay.packed.view(np.int32)).to(device)
        s = torch.from_numpy(lay.scales_raw.view(np.int16)).to(device).view(torch.bfloat16)
        b = torch.from_numpy(lay.biases_raw.view(np.int16)).to(device).view(torch.bfloat16)
        lin = mlxq.Linear(w, s, b, None, inDim=K, name="prefill")
        if lin.kernelFor(M, mlxq.BF16, mlxq.BF16) != "qgemm":
            return {"available": False}
        x = torch.randn((M, K), device=device, dtype=torch.bfloat16)
        ys = [torch.empty((M, O), device=device, dtype=torch.bfloat16) for _ in range(2)]
        for i in range(3):
            lin.encode(None, x, K, ys[i % 2], O, M)
        torch.cuda.synchronize()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            lin.encode(None, x, K, ys[i % 2], O, M)
        e1.record()
        torch.cuda.synchronize()
        mlxq.streamStatus(None, device.index or 0)
        ms = e0.elapsed_time(e1) / reps
        tf = 2.0 * M * O * K / (ms * 1e-3) / 1e12
        return {"available": True, "workload": f"prefill GEMM {O}x{K} b4 g64 M={M} bf16", "tflops": tf, "ms": ms,
                "frac_of_burst_peak": tf / peaks["bf16_tflops"], "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"]}
    except Exception as e:      # the probe must never take the headline down
        return {"available": False, "error": str(e)[:200]}


def run_ours(args):
    LAYERS = args.layers
    import torch
    import torch.distributed as dist
    mlxq = importlib.import_module("mlx-runner_b200")
    synth = importlib.import_module("mlx-runner_b200.synth")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the layer has no CPU path")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="nccl", device_id=device)
        idt = torch.zeros(128, dtype=torch.uint8, device=device)
        if rank == 0:
            idt.copy_(torch.tensor(list(mlxq.Comm.uniqueId()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        comm = mlxq.Comm(rank, world, local, bytes(idt.cpu().tolist()))
    peaks = measured_peaks()

    # LAYERS distinct weight sets on this rank (its shard of each layer when world > 1).
    layers, keep = [], []
    for i in range(LAYERS):
        lay = synth.make_layer(O_ROWS, K_COLS, BITS, GS, synth.F16, seed=1000 * rank + i, keep_codes=False)
        w = torch.from_numpy(lay.packed.view(np.int32)).to(device)
        s = torch.from_numpy(lay.scales_raw.view(np.int16)).to(device).view(torch.float16)
        b = torch.from_numpy(lay.biases_raw.view(np.int16)).to(device).view(torch.float16)
        keep.append((w, s, b))
        if world > 1:
            layers.append(mlxq.Linear.shard(w, s, b, None, inDim=K_COLS, rank=rank, nranks=world, full=False,
                                            name=f"layer{i}", device=local))
        else:
            layers.append(mlxq.Linear(w, s, b, None, inDim=K_COLS, name=f"layer{i}", device=local))
    total_rows = O_ROWS * world
    x_raw, _ = synth.make_activations(1, K_COLS, synth.F16, seed=7)
    x_host = torch.from_numpy(x_raw.view(np.int16)).view(torch.float16).pin_memory()
    x_dev = x_host.to(device)
    y_dev = torch.zeros((LAYERS, total_rows), dtype=torch.float32, device=device)
    y_host = torch.empty((LAYERS, total_rows), dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()

    fused = comm is not None and args.gather == "fused"
    if fused:
        comm.window(((total_rows * 4 + 255) // 256) * 256)      # collective: the peer-mapped gather windows

    def step(keep_outputs=False):
        stream = torch.cuda.current_stream()        # the capture stream while the step is being recorded into a graph
        for i, lin in enumerate(layers):
            if fused:
                # the decode kernel stores its rows into every rank's window itself; no collective kernel
                # (each call waits for the peers' rows of the one before it, the explicit wait covers the last)
                out = comm.forwardGatherFused(lin, stream, x_dev, K_COLS, 1, wait=keep_outputs)
                if keep_outputs:
                    y_dev[i].copy_(out[0], non_blocking=True)
            elif comm is not None:
                comm.forwardGather(lin, stream, x_dev, K_COLS, y_dev[i], total_rows, 1)
            else:
                lin.encode(stream, x_dev, K_COLS, y_dev[i], O_ROWS, 1)
        if fused and not keep_outputs:
            comm.wait(stream)

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        step(keep_outputs=True)
        y_host.copy_(y_dev, non_blocking=True)
        stream.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    # One GPU: the step's launches are recorded once into a CUDA graph and replayed, so that the figure is the
    # kernels' and not the Python loop's (per-call host cost is 5-15 us here, the kernel takes ~10 us).  The
    # end-to-end leg below keeps calling the public API.  Sharded runs are not graphed: every fused-gather call
    # carries a fresh epoch.
    timed_step, launch_mode = step, "one API call per launch"
    if world == 1 and not args.no_graph:
        try:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            mlxq.streamStatus(stream, local)
            timed_step, launch_mode = graph.replay, "CUDA graph of the step's launches, replayed"
        except Exception as e:  # noqa: BLE001
            launch_mode = f"one API call per launch (graph capture failed: {type(e).__name__})"
    windows = []
    t_a = time.perf_counter()
    ms = timed(timed_step, args.steps)
    windows.append((t_a, time.perf_counter()))
    for _ in range(2):
        step_e2e()
    t_a = time.perf_counter()
    ms_e2e = timed(step_e2e, args.steps)
    windows.append((t_a, time.perf_counter()))
    clocks = sampler.stop(windows) if rank == 0 else None
    mlxq.streamStatus(stream, local)

    per_launch = alg_bytes(O_ROWS, K_COLS, BITS, GS, 1)
    launches = args.steps * LAYERS
    value = world * launches * per_launch / (ms * 1e-3) / 1e9
    e2e_value = world * launches * per_launch / (ms_e2e * 1e-3) / 1e9
    # Roofline of the dominant kernel (the matvec): per-launch algorithmic bytes over the mean launch time
    # of the timed region (at N > 1 that time includes the gather, so the N = 1 line is the kernel's figure).
    achieved = per_launch / (ms * 1e-3 / launches) / 1e9
    out = None
    if rank == 0:
        probe = prefill_probe(mlxq, torch, device, peaks) if world == 1 and not args.no_prefill else {"available": False}
        cpu = cpu_sample(args.cpu_seconds) if world == 1 and args.cpu_seconds > 0 else None
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(LAYERS),
                       "rows_per_gpu": O_ROWS, "in_dim": K_COLS, "bits": BITS, "group_size": GS, "batch": 1,
                       "launches_per_step": LAYERS, "l2": "inputs larger than L2", "launch": launch_mode,
                       "parallelism": (f"row-shard x{world} + " + ("peer-store gather fused into the kernel" if fused else
                                                                   "ncclAllGather")) if world > 1 else "single GPU"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel() * 2),
                    "d2h_bytes_per_step": int(y_host.numel() * 4), "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "frac_of_nominal_8000": achieved / 8000.0, "bytes_per_launch": per_launch},
            "prefill": probe,
        }
        if cpu:
            out["cpu_baseline"] = cpu
        # DRAM bytes one launch of the decode kernel moved under ncu (dram__bytes_read.sum + dram__bytes_write.sum,
        # from the capture summarised under profiles/); the capture is of this workload's kernel at this shape.
        out["roofline"]["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH      # every rank runs this shape (weak scaling)
        print(json.dumps(out), flush=True)
    if comm is not None:
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline sample length (0 = skip)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM probe")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: rows stored into the peers' windows by the decode kernel (fused) or ncclAllGather after it")
    ap.add_argument("--sweep", action="store_true", help="print the decode sweep table (bits x group x M) instead of the JSON line")
    ap.add_argument("--no-graph", action="store_true", help="time plain API calls instead of a replayed CUDA graph")
    ap.add_argument("--layers", type=int, default=LAYERS, help="distinct weight sets per step (default 16)")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
