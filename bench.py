#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path: decode dequant-matvec HBM GB/s (headline), with the
prefill dequant-GEMM TFLOP/s reported beside it.

    python bench.py --gpus N --steps K --warmup W            # this library (one process per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores
    python bench.py --config c5 [--bits 6|8] [--batch B]     # vocabulary-sized head, rows split over the ranks
    python bench.py --config c4 [--batch B]                  # projection walk of a 36-layer transformer, rows split

Default workload (N = 1): the 4-bit group-64 matvec of the bit-width x group sweep, W out=11008 x in=4096, M = 1,
fp16 activations, fp32 output.  One step = PASSES passes over LAYERS distinct weight sets (LAYERS x 25.4 MB =
406 MB, larger than the 126 MB L2, so every launch streams its weights from HBM), i.e. PASSES x LAYERS launches
and at least 5 ms of device time.  value = algorithmic bytes (packed codes + scales + biases + x + y) per second.
N > 1 (weak scaling): every rank holds its own 11008-row shard of a (N x 11008)-row projection; a step is the
same, each launch followed by the gather of the fp32 output slices over NVLink.

--config c4 / c5 are strong scaling: the fixed layers are split by output rows over the N ranks and every call
ends with the gather; the JSON line then also carries the kernel-only time of the same step.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

O_ROWS, K_COLS, BITS, GS = 11008, 4096, 4, 64
LAYERS = 16          # distinct weight sets per pass; --layers overrides it (profiling runs use fewer)
PASSES = 48          # passes per step: 768 launches, ~6 ms of device time
# DRAM bytes one launch of the decode kernel moved in an ncu capture of this workload's kernel at this shape
# (dram__bytes_read.sum + dram__bytes_write.sum); reported as roofline.traffic for that shape on one GPU only.
NCU_DRAM_BYTES_PER_LAUNCH = 25403904
NCU_TRAFFIC_SOURCE = "ncu capture summarised in profiles/qmv_pipe_b4g64_m1.md (not measured in this run)"
METRIC = "decode_qmv_hbm_gbs"
UNIT = "GB/s"


def alg_bytes(O, K, bits, gs, M, s_size=2, x_size=2, y_size=4):
    """Algorithmic bytes of one call: packed codes + scales + biases + activations + outputs."""
    return O * K * bits // 8 + 2 * O * (K // gs) * s_size + M * K * x_size + M * O * y_size


def load_synth():
    """The synthetic-layer generators, loaded from their file so that the CPU arm does not import the product
    package (whose import loads the CUDA library)."""
    spec = importlib.util.spec_from_file_location("mlxq_synth", os.path.join(ROOT, "mlx-runner_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mlxq_synth"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained":
                d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- the workloads: name, per-call shapes, what both arms put into `config` ------------------------------------
C4_PROJ = [("q|k|v", 6144, 4096), ("o", 4096, 4096), ("gate|up", 24576, 4096), ("down", 4096, 12288)]
C4_LAYERS = 36
C5_ROWS, C5_K = 151936, 4096


def workload(args):
    """Description shared by both arms: config dict, algorithmic bytes of one step on the whole job."""
    if args.config == "c5":
        per_call = alg_bytes(C5_ROWS, C5_K, args.bits, 64, args.batch)
        calls = args.calls or 64
        return {"workload": f"vocabulary head {C5_ROWS}x{C5_K} b{args.bits} g64, batch {args.batch}, fp16 x, fp32 logits; "
                            f"{calls} calls per step ({per_call / 1e6:.0f} MB per call > L2)",
                "rows": C5_ROWS, "in_dim": C5_K, "bits": args.bits, "group_size": 64, "batch": args.batch,
                "launches_per_step": calls, "l2": "inputs larger than L2"}, per_call * calls
    if args.config == "c4":
        per_walk = C4_LAYERS * sum(alg_bytes(o, k, 4, 64, args.batch) for _, o, k in C4_PROJ)
        walks = args.calls or 6
        return {"workload": f"projection walk of a {C4_LAYERS}-layer transformer (hidden 4096, q|k|v 6144, gate|up 24576, down from 12288), "
                            f"b4 g64, batch {args.batch}, fp16 x, fp32 y; {walks} walks per step ({per_walk / 1e9:.2f} GB per walk > L2)",
                "layers": C4_LAYERS, "bits": 4, "group_size": 64, "batch": args.batch,
                "launches_per_step": walks * C4_LAYERS * len(C4_PROJ), "l2": "inputs larger than L2"}, per_walk * walks
    per_launch = alg_bytes(O_ROWS, K_COLS, BITS, GS, args.batch)
    launches = args.layers * args.passes
    return {"workload": f"decode matvec {O_ROWS}x{K_COLS} b{BITS} g{GS} M={args.batch}, fp16 x, fp32 y; {args.passes} passes over "
                        f"{args.layers} distinct weight sets per step ({args.layers * per_launch / 1e6:.0f} MB > L2)",
            "rows_per_gpu": O_ROWS, "in_dim": K_COLS, "bits": BITS, "group_size": GS, "batch": args.batch,
            "launches_per_step": launches, "l2": "inputs larger than L2"}, per_launch * launches


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


# ---- CPU arm ----------------------------------------------------------------------------------------------------
def cpu_layer(args, synth):
    """(layer, activations, note) of the CPU sample: one layer of the workload."""
    if args.config == "c5":
        lay = synth.make_layer_fast(C5_ROWS, C5_K, args.bits, 64, synth.F16, seed=0)
        _, x = synth.make_activations(args.batch, C5_K, synth.F16, seed=1)
        return [(lay, x, C5_K)], f"one {C5_ROWS}x{C5_K} {args.bits}-bit g64 head call, batch {args.batch}"
    if args.config == "c4":
        out = []
        for i, (_, o, k) in enumerate(C4_PROJ):
            lay = synth.make_layer_fast(o, k, 4, 64, synth.F16, seed=i)
            _, x = synth.make_activations(args.batch, k, synth.F16, seed=10 + i)
            out.append((lay, x, k))
        return out, f"the four projections of one layer of the walk, batch {args.batch}"
    lay = synth.make_layer(O_ROWS, K_COLS, BITS, GS, synth.F16, seed=0, keep_codes=False)
    _, x = synth.make_activations(1, K_COLS, synth.F16, seed=1)
    return [(lay, x, K_COLS)], f"one {O_ROWS}x{K_COLS} 4-bit g64 layer, M=1"


def cpu_call(oracle, items, cores, double=False):
    for lay, x, K in items:
        oracle.qmatmul(lay.packed.view(np.uint8), lay.scales_raw, lay.biases_raw, lay.scale_dtype, x, K, lay.bits, lay.gs,
                       accumulate_double=double, threads=cores)


def cpu_bytes(items):
    return sum(alg_bytes(l.packed.shape[0], K, l.bits, l.gs, x.shape[0]) for l, x, K in items)


def cpu_sample(args, seconds_target: float = 12.0):
    """The oracle's restatement of the reference's CPU path (unpack + fp32 dequant + fp32 dot, OpenMP over
    output rows) timed on the host cores on one layer of the workload; beside it the same with a double
    accumulator (the reference's test oracle) and the reference's other CPU route, dequantise to fp32 then BLAS."""
    from oracle import oracle
    synth = load_synth()
    items, what = cpu_layer(args, synth)
    cores = len(os.sched_getaffinity(0))
    nbytes = cpu_bytes(items)

    def best_of(fn, budget):
        fn()
        t0 = time.perf_counter()
        fn()
        one = time.perf_counter() - t0
        reps = max(2, min(200, int(budget / max(one, 1e-4))))
        best = one
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        return best, reps + 1

    best, reps = best_of(lambda: cpu_call(oracle, items, cores), seconds_target * 0.6)
    best_d, _ = best_of(lambda: cpu_call(oracle, items, cores, double=True), seconds_target * 0.2)
    out = {"value": nbytes / best / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
           "sample": f"{what}, best of {reps} calls, fp32 accumulate, OpenMP over rows", "ms_per_call": best * 1e3,
           "double_accumulate_gbs": nbytes / best_d / 1e9}
    try:        # dequantise-then-BLAS (SieveImport.swift:90-112, 346): the dense fp32 matrix is built once, the product timed
        lay, x, K = items[0]
        dense = oracle.dequantize(lay.packed[:4096], lay.scales_raw[:4096], lay.biases_raw[:4096], lay.scale_dtype, K, lay.bits, lay.gs)
        xt = np.ascontiguousarray(x.T)
        b2, _ = best_of(lambda: dense @ xt, seconds_target * 0.1)
        out["numpy_blas_dense_gbs"] = dense.nbytes / b2 / 1e9
        out["numpy_blas_note"] = "x @ W_deq.T on 4096 dequantised fp32 rows (dense bytes / time; the dequantisation itself is not timed)"
    except Exception as e:      # noqa: BLE001
        out["numpy_blas_note"] = f"unavailable: {type(e).__name__}"
    return out


def run_reference(args):
    """--impl reference: the reference's CPU algorithm (oracle port; the Swift sources cannot be built on
    Linux) on all host cores.  A step is one layer of the workload (a bounded sample of the GPU arm's step)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    synth = load_synth()
    cfg, _ = workload(args)
    items, what = cpu_layer(args, synth)
    cores = len(os.sched_getaffinity(0))
    for _ in range(max(args.warmup, 1)):
        cpu_call(oracle, items, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_call(oracle, items, cores)
    dt = time.perf_counter() - t0
    gbs = args.steps * cpu_bytes(items) / dt / 1e9
    sample = f"each CPU step is {what} (a bounded sample of the GPU arm's step), fp32 accumulate, OpenMP over rows"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.config == "default" else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg, "sample": sample,
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------------------------------
def prefill_probe(mlxq, torch, device, peaks, quick=False):
    """The prefill dequant-GEMM beside the headline: 14336 x 4096 and 4096 x 14336, 4-bit g64, bf16 in / bf16 out,
    M = 128, 512, 2048, 8192; the pre-pass that rewrites the activations is inside the timed call."""
    synth = importlib.import_module("mlx-runner_b200.synth")
    rows = []
    try:
        for (O, K) in ((14336, 4096), (4096, 14336)):
            lay = synth.make_layer(O, K, 4, 64, synth.BF16, seed=3, keep_codes=False)
            w = torch.from_numpy(lay.packed.view(np.int32)).to(device)
            s = torch.from_numpy(lay.scales_raw.view(np.int16)).to(device).view(torch.bfloat16)
            b = torch.from_numpy(lay.biases_raw.view(np.int16)).to(device).view(torch.bfloat16)
            lin = mlxq.Linear(w, s, b, None, inDim=K, name="prefill")
            for M in ((2048,) if quick else (128, 512, 2048, 8192)):
                if lin.kernelFor(M, mlxq.BF16, mlxq.BF16) != "qgemm":
                    rows.append({"shape": f"{O}x{K}", "M": M, "available": False})
                    continue
                x = torch.randn((M, K), device=device, dtype=torch.bfloat16)
                ys = [torch.empty((M, O), device=device, dtype=torch.bfloat16) for _ in range(2)]
                for i in range(3):
                    lin.encode(None, x, K, ys[i % 2], O, M)
                torch.cuda.synchronize()
                reps = 10 if M <= 2048 else 5
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(reps):
                    lin.encode(None, x, K, ys[i % 2], O, M)
                e1.record()
                torch.cuda.synchronize()
                mlxq.streamStatus(None, device.index or 0)
                ms = e0.elapsed_time(e1) / reps
                tf = 2.0 * M * O * K / (ms * 1e-3) / 1e12
                rows.append({"shape": f"{O}x{K}", "M": M, "tflops": tf, "ms": ms, "frac_of_burst_peak": tf / peaks["bf16_tflops"],
                             "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"]})
            del lin, w, s, b
        head = next((r for r in rows if r["shape"] == "14336x4096" and r["M"] == 2048 and "tflops" in r), None)
        out = {"available": head is not None, "workload": "prefill GEMM b4 g64 bf16 in/out, 14336x4096 and 4096x14336", "cases": rows}
        if head:
            out.update({"tflops": head["tflops"], "ms": head["ms"], "frac_of_burst_peak": head["frac_of_burst_peak"],
                        "frac_of_sustained_peak": head["frac_of_sustained_peak"], "headline_case": "14336x4096 M=2048"})
        return out
    except Exception as e:      # the probe must never take the headline down
        return {"available": False, "error": str(e)[:200], "cases": rows}


def device_layer(torch, device, O, K, bits, gs, seed):
    """A synthetic layer drawn on the device (uniform packed bits = uniform codes; scales and biases as the CPU
    generator draws them) for the layers that are too large to build on the host in reasonable time."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randint(-(1 << 31), (1 << 31) - 1, (O, K * bits // 32), dtype=torch.int32, device=device, generator=g)
    s32 = torch.randn((O, K // gs), device=device, generator=g).abs() * 0.002 + 1e-4
    s = s32.to(torch.float16)
    b = (-(1 << (bits - 1)) * s.float()).to(torch.float16)
    return w, s, b


def oracle_rows(torch, w, s, b, rows, x_np, K, bits, gs):
    """The oracle's outputs for a few rows of a device-resident layer."""
    from oracle import oracle
    idx = torch.as_tensor(rows, device=w.device)
    wp = w[idx].cpu().numpy().view(np.uint32)
    sp = s[idx].cpu().view(torch.int16).numpy().view(np.uint16)
    bp = b[idx].cpu().view(torch.int16).numpy().view(np.uint16)
    return oracle.qmatmul(wp, sp, bp, 1, x_np, K, bits, gs)


def run_ours(args):
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
    cfg, step_bytes = workload(args)
    fused = comm is not None and args.gather == "fused"
    strong = args.config != "default"
    batch = args.batch

    # ---- the step's calls: (layer, activations, rows of the whole layer) in order ---------------------------------
    calls, keep = [], []
    if args.config == "default":
        for i in range(args.layers):
            lay = synth.make_layer(O_ROWS, K_COLS, BITS, GS, synth.F16, seed=1000 * rank + i, keep_codes=False)
            w = torch.from_numpy(lay.packed.view(np.int32)).to(device)
            s = torch.from_numpy(lay.scales_raw.view(np.int16)).to(device).view(torch.float16)
            b = torch.from_numpy(lay.biases_raw.view(np.int16)).to(device).view(torch.float16)
            keep.append((w, s, b))
            if world > 1:
                lin = mlxq.Linear.shard(w, s, b, None, inDim=K_COLS, rank=rank, nranks=world, full=False, name=f"layer{i}", device=local)
            else:
                lin = mlxq.Linear(w, s, b, None, inDim=K_COLS, name=f"layer{i}", device=local)
            calls.append((lin, K_COLS, O_ROWS * world))
        calls = calls * args.passes
    else:
        shapes = [(C5_ROWS, C5_K, args.bits)] if args.config == "c5" else [(o, k, 4) for _ in range(C4_LAYERS) for _, o, k in C4_PROJ]
        distinct = {}
        for i, (O, K, bits) in enumerate(shapes):
            # every rank draws the whole layer's rows it owns: the same seed gives the same full layer on every rank
            rows = O // world
            w, s, b = device_layer(torch, device, O, K, bits, 64, seed=7 + i)
            r0 = rank * rows
            w, s, b = w[r0:r0 + rows].contiguous(), s[r0:r0 + rows].contiguous(), b[r0:r0 + rows].contiguous()
            keep.append((w, s, b))
            if world > 1:
                lin = mlxq.Linear.shard(w, s, b, None, inDim=K, rank=rank, nranks=world, full=False, name=f"call{i}", device=local)
            else:
                lin = mlxq.Linear(w, s, b, None, inDim=K, name=f"call{i}", device=local)
            distinct[i] = (lin, K, O)
        n_rep = args.calls or (64 if args.config == "c5" else 6)
        calls = [distinct[i] for _ in range(n_rep) for i in range(len(shapes))]
    ks = sorted({k for _, k, _ in calls})
    x_host = {k: torch.from_numpy(synth.make_activations(batch, k, synth.F16, seed=7 + k)[0].view(np.int16)).view(torch.float16).pin_memory() for k in ks}
    x_dev = {k: x_host[k].to(device) for k in ks}
    max_rows = max(o for _, _, o in calls)
    last = calls[-1]
    y_dev = torch.zeros((batch, max_rows), dtype=torch.float32, device=device)          # non-fused paths write here
    y_keep = torch.zeros((batch, last[2]), dtype=torch.float32, device=device)          # the step's result (last call)
    y_host = torch.empty((batch, last[2]), dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()
    if fused:
        comm.window(((batch * max_rows * 4 + 255) // 256) * 256)      # collective: the peer-mapped gather windows

    def step(keep_output=False, gather=True):
        st = torch.cuda.current_stream()        # the capture stream while the step is being recorded into a graph
        out = None
        for lin, K, total in calls:
            if comm is not None and gather:
                if fused:
                    # the decode kernel stores its rows into every rank's window itself; no collective kernel
                    # (each call waits for the peers' rows of the one before it, the explicit wait covers the last)
                    out = comm.forwardGatherFused(lin, st, x_dev[K], K, batch, wait=False)
                else:
                    comm.forwardGather(lin, st, x_dev[K], K, y_dev, total, batch)
                    out = y_dev[:, :total]
            else:
                lin.encode(st, x_dev[K], K, y_dev[:, lin.rowOffset:], max_rows, batch)
                out = y_dev[:, :total]
        if fused and gather:
            comm.wait(st)
        if keep_output:
            y_keep.copy_(out[:, :last[2]], non_blocking=True)

    e2e_launch = {"fn": lambda: step(keep_output=True), "mode": "one API call per launch"}

    def step_e2e():
        # a user's step from host buffers: activations in from pinned memory, the step's calls (through the C ABI,
        # recorded once into a graph where the timed step is one), the result out to pinned memory, then wait
        for k in ks:
            x_dev[k].copy_(x_host[k], non_blocking=True)
        e2e_launch["fn"]()
        y_host.copy_(y_keep, non_blocking=True)
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
    # kernels' and not the Python loop's (per-call host cost is 5-15 us here, a launch takes ~8 us).  The same
    # step with one API call per launch is timed beside it ("api_calls").  Sharded runs with the fused gather are
    # captured the same way (the gather's call number lives on the device); the NCCL variant is not.
    timed_step, launch_mode = step, "one API call per launch"
    graphable = world == 1 or (fused and len(calls) % 2 == 0)      # a replayed sequence keeps the two window buffers alternating
    if graphable and not args.no_graph:
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
    ms_api = timed(step, max(3, args.steps // 4)) / max(3, args.steps // 4) if timed_step is not step else ms / args.steps
    ms_kernel_only = None
    if world > 1:
        # the step without its gathers, launched the same way as the timed step (a replayed graph when that was one)
        n = max(3, args.steps // 4)
        plain = lambda: step(gather=False)      # noqa: E731
        if timed_step is not step:
            try:
                torch.cuda.synchronize()
                graph_k = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph_k):
                    step(gather=False)
                graph_k.replay()
                torch.cuda.synchronize()
                plain = graph_k.replay
            except Exception:       # noqa: BLE001
                pass
        ms_kernel_only = timed(plain, n) / n
    if timed_step is not step:
        try:
            torch.cuda.synchronize()
            graph_e = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_e):
                step(keep_output=True)
            graph_e.replay()
            torch.cuda.synchronize()
            e2e_launch["fn"], e2e_launch["mode"] = graph_e.replay, launch_mode
        except Exception:       # noqa: BLE001
            pass
    for _ in range(2):
        step_e2e()
    t_a = time.perf_counter()
    ms_e2e = timed(step_e2e, args.steps)
    windows.append((t_a, time.perf_counter()))
    clocks = sampler.stop(windows) if rank == 0 else None
    mlxq.streamStatus(stream, local)

    # ---- correctness of what was timed: the last call's output on this rank against the oracle, a sample of rows ----
    lin, K, total = last
    step(keep_output=True)
    torch.cuda.synchronize()
    got = y_keep.cpu().numpy()
    check = "ok"
    try:
        from oracle import oracle
        g = np.random.default_rng(rank)
        if args.config == "default":
            w, s, b = keep[(len(calls) - 1) % args.layers]
            bits_l, rows_l = BITS, O_ROWS
        else:
            w, s, b = keep[-1]
            bits_l, rows_l = lin.bits, w.shape[0]
        sample = np.sort(g.choice(rows_l, size=64, replace=False))
        xv = x_host[K].float().numpy()
        ref = oracle_rows(torch, w, s, b, sample, xv, K, bits_l, 64)
        err = oracle.max_rel_err(got[:, lin.rowOffset + sample], ref)
        ok = err < 1e-3
        if world > 1:
            # the rows the other ranks computed: compare with what they hold
            mine = torch.from_numpy(got).to(device)
            ref_all = mine.clone()
            dist.broadcast(ref_all, 0)
            same = bool(torch.equal(mine, ref_all)) if fused or args.gather == "nccl" else True
            flag = torch.tensor([1 if (ok and same) else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        if not ok:
            check = f"FAILED (max relative error {err:.3g} on rank {rank})"
    except Exception as e:      # noqa: BLE001
        check = f"not run: {type(e).__name__}: {str(e)[:80]}"

    launches = args.steps * len(calls)
    scale = world if args.config == "default" else 1          # weak scaling: every rank does a full step's bytes
    value = scale * args.steps * step_bytes / (ms * 1e-3) / 1e9
    e2e_value = scale * args.steps * step_bytes / (ms_e2e * 1e-3) / 1e9
    # Roofline of the dominant kernel (the matvec): this rank's algorithmic bytes of a step over the step's time
    # (at N > 1 that time includes the gather, so the N = 1 line is the kernel's figure).
    per_rank_bytes = step_bytes / (1 if args.config == "default" else world)
    achieved = per_rank_bytes * args.steps / (ms * 1e-3) / 1e9
    select = None
    if args.config == "c5":
        try:
            select = select_probe(mlxq, torch, dist if world > 1 else None, comm, last[0], x_dev[last[1]], last[1], batch, last[2], world, rank,
                                  local, fused, y_dev, keep[-1], x_host[last[1]].float().numpy())
        except Exception as e:      # noqa: BLE001
            select = {"error": f"{type(e).__name__}: {str(e)[:120]}"}
    glu = None
    if args.config == "c4" and world == 1 and batch <= 8:
        try:
            downs = [lin for (lin, k, o) in distinct.values() if k == 12288]
            glu = glu_probe(mlxq, torch, downs, 12288, batch, local)
        except Exception as e:      # noqa: BLE001
            glu = {"error": f"{type(e).__name__}: {str(e)[:120]}"}
    if rank == 0:
        probe = prefill_probe(mlxq, torch, device, peaks) if world == 1 and not args.no_prefill and args.config == "default" else {"available": False}
        cpu = cpu_sample(args, args.cpu_seconds) if world == 1 and args.cpu_seconds > 0 else None
        cfg = dict(cfg)
        cfg["launch"] = launch_mode
        cfg["parallelism"] = (f"row-shard x{world} + " + ("peer-store gather fused into the kernel" if fused else "ncclAllGather")) if world > 1 else "single GPU"
        captured_shape = args.config == "default" and world == 1 and args.layers == LAYERS and args.batch == 1
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": cfg,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(sum(x_host[k].numel() for k in ks) * 2),
                    "d2h_bytes_per_step": int(y_host.numel() * 4), "ms_per_step": ms_e2e / args.steps, "launch": e2e_launch["mode"]},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH if captured_shape else None,
                         "traffic_source": NCU_TRAFFIC_SOURCE if captured_shape else None, "peak_source": peaks["source"],
                         "frac_of_nominal_8000": achieved / 8000.0, "bytes_per_step_per_gpu": per_rank_bytes},
            "api_calls": {"ms_per_step": ms_api, "value": scale * step_bytes / (ms_api * 1e-3) / 1e9,
                          "note": "the same step with one API call per launch"},
            "output_check": check,
            "prefill": probe,
        }
        if world > 1:
            out["gather_check"] = check
            out["split"] = {"kernel_ms_per_step": ms_kernel_only, "gather_ms_per_step": ms / args.steps - ms_kernel_only,
                            "note": "the step without its gathers (shard matvecs only), then the difference"}
        if cpu:
            out["cpu_baseline"] = cpu
        if select is not None:
            out["select"] = select
        if glu is not None:
            out["glu"] = glu
        print(json.dumps(out), flush=True)
        if check.startswith("FAILED"):
            raise SystemExit(f"bench.py: {check}")
    if comm is not None:
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
        dist.destroy_process_group()


def select_probe(mlxq, torch, dist, comm, lin, x, K, batch, total, world, rank, local, fused, y_dev, keep, x_np):
    """Config 5 with greedy selection after the head: the full logits gathered and then scanned (block maxima over
    the whole vocabulary, then the greedy pass), against the head whose shard kernel is followed by the block maxima
    of the shard alone, so that only maxima are gathered.  Device time per token step from CUDA events around 32
    steps enqueued back to back (one API call per launch: at 8 ranks the host's pace shows).  The tokens of the two
    paths must agree on every rank, and the winner's logit is checked against the oracle."""
    device = torch.device("cuda", local)
    st = torch.cuda.current_stream()
    rows = total // world
    nb_full = (total + mlxq.SELECT_BLOCK - 1) // mlxq.SELECT_BLOCK
    nb = (rows + mlxq.SELECT_BLOCK - 1) // mlxq.SELECT_BLOCK
    y_local = torch.zeros((batch, rows), dtype=torch.float32, device=device)
    pairs_full = torch.zeros((2, batch, nb_full), dtype=torch.int32, device=device)
    pairs = torch.zeros((world, 2, batch, nb), dtype=torch.int32, device=device)
    tok_a = torch.zeros(batch, dtype=torch.int32, device=device)
    tok_b = torch.zeros(batch, dtype=torch.int32, device=device)
    val_b = torch.zeros(batch, dtype=torch.float32, device=device)

    def path_logits():
        if comm is not None:
            if fused:
                out = comm.forwardGatherFused(lin, st, x, K, batch, wait=True)
            else:
                comm.forwardGather(lin, st, x, K, y_dev, total, batch)
                out = y_dev[:, :total]
        else:
            lin.encode(st, x, K, y_dev, total, batch)
            out = y_dev[:, :total]
        mlxq.blockMax(st, out, total, batch, out.stride(0), pairs_full, device=local)
        mlxq.blockArgmax(st, pairs_full, 1, batch, nb_full, tok_a, None, device=local)

    def path_block_max():
        if comm is not None:
            comm.forwardBlockMaxGather(lin, st, x, K, batch, y_local, pairs)
        else:
            lin.encode(st, x, K, y_local, rows, batch)
            mlxq.blockMax(st, y_local, rows, batch, rows, pairs, device=local)
        mlxq.blockArgmax(st, pairs, world, batch, nb, tok_b, val_b, device=local)

    def timed_us(fn, n=32):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e3 / n

    us_a = timed_us(path_logits)
    us_b = timed_us(path_block_max)
    mlxq.streamStatus(st, local)
    agree = bool(torch.equal(tok_a, tok_b))
    winner_ok = True
    try:
        from oracle import oracle
        w, s, b = keep
        toks = tok_b.cpu().numpy()
        mine = [(t, int(r) - lin.rowOffset) for t, r in enumerate(toks) if lin.rowOffset <= int(r) < lin.rowOffset + rows]
        if mine:
            ref = oracle_rows(torch, w, s, b, np.array(sorted({r for _, r in mine})), x_np, K, lin.bits, 64)
            order = {r: i for i, r in enumerate(sorted({r for _, r in mine}))}
            got = val_b.cpu().numpy()
            winner_ok = all(abs(got[t] - ref[t, order[r]]) <= 1e-3 * max(1.0, abs(ref[t, order[r]])) for t, r in mine)
    except Exception:       # noqa: BLE001
        winner_ok = False
    if world > 1:
        flag = torch.tensor([1 if (agree and winner_ok) else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        agree = winner_ok = bool(flag.item())
    return {"greedy_tokens_agree": agree, "winner_matches_oracle": winner_ok,
            "logits_then_select_us_per_step": us_a, "block_max_gather_us_per_step": us_b,
            "gathered_bytes_per_step": {"logits": int(total * 4 * batch) if world > 1 else 0,
                                        "block_maxima": int(world * 2 * nb * 4 * batch) if world > 1 else 0},
            "note": "head call + selection per token step; one API call per launch, CUDA events around 32 steps"}


def glu_probe(mlxq, torch, downs, K, batch, device_index):
    """Config 4's MLP tail: the activation product as a kernel of its own followed by the down projection (the
    reference's sequence, Transformer.swift:1528-1536) against the down projection that reads the [gate | up] buffer
    itself.  Every down projection of the walk once per graph (distinct weights), fp32 activations, CUDA events
    around ten replays."""
    dev = torch.device("cuda", device_index)
    O = downs[0].outDim
    gu = torch.randn((batch, 2 * K), device=dev, dtype=torch.float32)
    xbuf = torch.empty((batch, K), device=dev, dtype=torch.float32)
    y = torch.empty((batch, O), device=dev, dtype=torch.float32)
    y2 = torch.empty((batch, O), device=dev, dtype=torch.float32)

    def separate():
        st = torch.cuda.current_stream()
        for lin in downs:
            mlxq.actMul(st, gu, 2 * K, K, batch, 0, xbuf, device=device_index)
            lin.encode(st, xbuf, K, y, O, batch)

    def folded():
        st = torch.cuda.current_stream()
        for lin in downs:
            lin.encodeGLU(st, gu, 2 * K, 0, y2, O, batch)

    def timed_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (10 * len(downs))
    us_sep, us_fold = timed_us(separate), timed_us(folded)
    mlxq.streamStatus(None, device_index)
    same = float((y - y2).abs().max()) <= 1e-4 * max(1.0, float(y.abs().max()))
    return {"act_mul_then_down_us": us_sep, "down_with_gated_input_us": us_fold, "outputs_agree": bool(same),
            "note": f"down projection {O}x{K} b4 g64, batch {batch}, fp32 activations; per layer, {len(downs)} layers per graph"}


def run_sweep(args):
    """--sweep: the decode matvec over bit widths, group sizes, batch sizes and the two projection shapes of the
    reference's sweep configuration, as a markdown table on stdout (not the benchmark's JSON line).  Every case
    runs eight distinct weight sets per step, replayed as a CUDA graph, timed with CUDA events."""
    import torch
    mlxq = importlib.import_module("mlx-runner_b200")
    synth = importlib.import_module("mlx-runner_b200.synth")
    dev = torch.device("cuda", 0)
    peak = measured_peaks()["hbm_gbs"]

    def one(O, K, bits, gs, M, L=8, reps=10):
        if O * K * bits // 8 > 200e6:
            L = 2                                       # (two sets of a vocabulary-sized layer already exceed L2 several times)
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

    print("| shape (out x in) | bits | group | M | us per launch | GB/s | of measured peak |")
    print("|---|---|---|---|---|---|---|")
    cases = [(11008, 4096, b, 64, m) for b in (2, 3, 4, 5, 6, 8) for m in (1, 8)]
    cases += [(11008, 4096, 4, 64, m) for m in (2, 4, 16)]
    cases += [(4096, 11008, 4, 64, m) for m in (1, 8)] + [(11008, 4096, 4, gs, m) for gs in (32, 128) for m in (1, 4)]
    cases += [(24576, 4096, 4, 64, 1), (6144, 4096, 4, 64, 1), (4096, 12288, 4, 64, 1), (4096, 4096, 4, 64, 1)]
    cases += [(151936, 4096, b, 64, m) for b in (6, 8) for m in (1, 4, 16)]
    for O, K, bits, gs, M in cases:
        us, gbs = one(O, K, bits, gs, M)
        print(f"| {O} x {K} | {bits} | {gs} | {M} | {us:.1f} | {gbs:.0f} | {gbs / peak:.2f} |", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="default", choices=["default", "c4", "c5"],
                    help="default: the 11008x4096 sweep shape (weak scaling); c4: projection walk; c5: vocabulary head (strong scaling)")
    ap.add_argument("--bits", type=int, default=8, choices=[6, 8], help="c5: bit width of the head")
    ap.add_argument("--batch", type=int, default=1, help="tokens per call (the headline is 1)")
    ap.add_argument("--calls", type=int, default=0, help="c4: walks per step, c5: calls per step (0 = default)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline sample length (0 = skip)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM probe")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: rows stored into the peers' windows by the decode kernel (fused) or ncclAllGather after it")
    ap.add_argument("--sweep", action="store_true", help="print the decode sweep table (bits x group x M) instead of the JSON line")
    ap.add_argument("--no-graph", action="store_true", help="time plain API calls instead of a replayed CUDA graph")
    ap.add_argument("--layers", type=int, default=LAYERS, help="distinct weight sets per pass (default 16)")
    ap.add_argument("--passes", type=int, default=PASSES, help="passes over the weight sets per step (default 48)")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
