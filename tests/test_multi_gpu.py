"""Row-sharded decode on 2 GPUs (one process per GPU): the NCCL all-gather path and the fused path whose
kernel stores its rows into every rank's window, against the oracle's full-layer result.

Skipped on machines with fewer than two GPUs.  The ranks are child processes; failures on the host side come
back through the exit code, nothing here faults a GPU."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, os.path.dirname(HERE))
        sys.path.insert(0, HERE)
        import torch.distributed as dist
        mlxq = importlib.import_module("mlx-runner_b200")
        from oracle import oracle
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        ids = [mlxq.Comm.uniqueId() if rank == 0 else None]
        dist.broadcast_object_list(ids, 0)
        comm = mlxq.Comm(rank, world, rank, ids[0])
        O, K, bits, gs = 64 * world * 3, 1024, 4, 64
        fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=gs, seed=11)          # same layer on every rank
        dev = f"cuda:{rank}"
        w = torch.from_numpy(fx.packed.view(np.int32).reshape(O, -1)).to(dev)
        s = torch.from_numpy(fx.scales_raw.view(np.int16)).to(dev).view(torch.float16)
        b = torch.from_numpy(fx.biases_raw.view(np.int16)).to(dev).view(torch.float16)
        lin = mlxq.Linear.shard(w, s, b, None, inDim=K, rank=rank, nranks=world, full=True, name="shard", device=rank)
        assert lin.totalOut == O and lin.outDim == O // world and lin.rowOffset == rank * (O // world)
        comm.window(64 * O * 4)
        for it in range(6):                                                 # alternates the two window buffers
            T = 1 if it % 2 == 0 else 4
            x = oracle.RNG(50 + it).floats(T * K).reshape(T, K).astype(np.float32)
            ref = fx.reference(x)
            x_dev = torch.from_numpy(x).to(dev)
            y = torch.full((T, O), float("nan"), dtype=torch.float32, device=dev)
            comm.forwardGather(lin, None, x_dev, K, y, O, T)
            out = comm.forwardGatherFused(lin, None, x_dev, K, T)
            torch.cuda.synchronize()
            mlxq.streamStatus(None, rank)
            got_nccl, got_fused = y.cpu().numpy(), out.cpu().numpy().copy()
            assert oracle.max_rel_err(got_nccl, ref) < 1e-3, f"rank {rank} call {it}: NCCL gather"
            assert oracle.max_rel_err(got_fused, ref) < 1e-3, f"rank {rank} call {it}: fused gather"
            # the sharded head with the selection's first pass folded in: only block maxima are gathered, and the greedy
            # token over them is the argmax of the gathered logits (same kernel, same rows: bit-identical values)
            rows = O // world
            nb = (rows + mlxq.SELECT_BLOCK - 1) // mlxq.SELECT_BLOCK
            y_local = torch.zeros((T, rows), dtype=torch.float32, device=dev)
            pairs = torch.zeros((world, 2, T, nb), dtype=torch.int32, device=dev)
            token = torch.zeros(T, dtype=torch.int32, device=dev)
            value = torch.zeros(T, dtype=torch.float32, device=dev)
            comm.forwardBlockMaxGather(lin, None, x_dev, K, T, y_local, pairs)
            mlxq.blockArgmax(None, pairs, world, T, nb, token, value, device=rank)
            torch.cuda.synchronize()
            assert np.array_equal(token.cpu().numpy(), got_nccl.argmax(axis=1).astype(np.int32)), f"rank {rank} call {it}: greedy token"
            assert np.array_equal(value.cpu().numpy(), got_nccl.max(axis=1)), f"rank {rank} call {it}: greedy value"
            assert np.array_equal(got_nccl.view(np.uint32), got_fused.view(np.uint32)), "the two gathers disagree"
            dist.barrier()
        # a batch the decode kernel does not take is refused and leaves the communicator usable
        xb = torch.zeros((64, K), dtype=torch.bfloat16, device=dev)
        with pytest.raises(mlxq.Unsupported):
            comm.forwardGatherFused(lin, None, xb, K, 64)
        x = oracle.RNG(99).floats(K).reshape(1, K).astype(np.float32)
        out = comm.forwardGatherFused(lin, None, torch.from_numpy(x).to(dev), K, 1)
        torch.cuda.synchronize()
        assert oracle.max_rel_err(out.cpu().numpy(), fx.reference(x)) < 1e-3
        dist.barrier()
        # A chain: the gathered rows of one fused call are the activations of the next, with no wait between them
        # (the second call itself waits for the peers' rows before it reads them), then two more links.
        K2 = O                                                              # 384 rows gathered -> 384 inputs
        fx2 = oracle.QuantFixture(O=O, K=K2, bits=bits, gs=gs, seed=12)
        w2 = torch.from_numpy(fx2.packed.view(np.int32).reshape(O, -1)).to(dev)
        s2 = torch.from_numpy(fx2.scales_raw.view(np.int16)).to(dev).view(torch.float16)
        b2 = torch.from_numpy(fx2.biases_raw.view(np.int16)).to(dev).view(torch.float16)
        lin2 = mlxq.Linear.shard(w2, s2, b2, None, inDim=K2, rank=rank, nranks=world, full=True, name="shard2", device=rank)
        x = oracle.RNG(123).floats(K).reshape(1, K).astype(np.float32)
        h = comm.forwardGatherFused(lin, None, torch.from_numpy(x).to(dev), K, 1, wait=False)
        ref = fx.reference(x)
        for _ in range(3):
            h = comm.forwardGatherFused(lin2, None, h, K2, 1, wait=False)
            ref = fx2.reference(ref)
        comm.wait(None)
        torch.cuda.synchronize()
        mlxq.streamStatus(None, rank)
        assert oracle.max_rel_err(h.cpu().numpy(), ref) < 1e-3, f"rank {rank}: chained fused calls"
        dist.barrier()
        # The same two calls captured into a CUDA graph and replayed with new activations: the call numbers come from
        # the device, so every replay waits for its own peers' rows.
        x_buf = torch.zeros((1, K), dtype=torch.float32, device=dev)
        keep = torch.zeros((1, O), dtype=torch.float32, device=dev)
        x_buf.copy_(torch.from_numpy(x).to(dev))
        for _ in range(2):                                                   # warm-up outside the capture (even count)
            comm.forwardGatherFused(lin, None, x_buf, K, 1, wait=False)
        comm.wait(None)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            st = torch.cuda.current_stream()
            h1 = comm.forwardGatherFused(lin, st, x_buf, K, 1, wait=False)
            h2 = comm.forwardGatherFused(lin2, st, h1, K2, 1, wait=False)
            comm.wait(st)
            keep.copy_(h2)
        for rep in range(3):
            xr = oracle.RNG(200 + rep).floats(K).reshape(1, K).astype(np.float32)
            x_buf.copy_(torch.from_numpy(xr).to(dev))
            g.replay()
            torch.cuda.synchronize()
            mlxq.streamStatus(None, rank)
            want = fx2.reference(fx.reference(xr))
            assert oracle.max_rel_err(keep.cpu().numpy(), want) < 1e-3, f"rank {rank}: graph replay {rep}"
            dist.barrier()
        del g
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "".join(traceback.format_exception(type(e), e, e.__traceback__))))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_decode_nccl_and_fused_gather_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in procs:
        rank, msg = q.get(timeout=300)
        results[rank] = msg
    for p in procs:
        p.join(timeout=60)
    assert all(v == "ok" for v in results.values()), "\n".join(f"rank {k}: {v}" for k, v in results.items())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_layers_on_two_devices():
    # the kernels' shared-memory opt-in is per device: a process that holds layers on two GPUs must be able to run both
    mlxq = importlib.import_module("mlx-runner_b200")
    from oracle import oracle
    fx = oracle.QuantFixture(O=256, K=1024, bits=4, gs=64, seed=5)
    x = oracle.RNG(6).floats(2 * 1024).reshape(2, 1024).astype(np.float32)
    ref = fx.reference(x)
    for d in (0, 1, 0):
        dev = f"cuda:{d}"
        w = torch.from_numpy(fx.packed.view(np.int32).reshape(256, -1)).to(dev)
        s = torch.from_numpy(fx.scales_raw.view(np.int16)).to(dev).view(torch.float16)
        b = torch.from_numpy(fx.biases_raw.view(np.int16)).to(dev).view(torch.float16)
        lin = mlxq.Linear(w, s, b, None, inDim=1024, name=f"dev{d}", device=d)
        for T in (1, 2):
            y = torch.full((T, 256), float("nan"), dtype=torch.float32, device=dev)
            with torch.cuda.device(d):
                lin.encode(None, torch.from_numpy(x[:T]).to(dev), 1024, y, 256, T)
                torch.cuda.synchronize()
            mlxq.streamStatus(None, d)
            assert oracle.max_rel_err(y.cpu().numpy(), ref[:T]) < 1e-3, f"device {d} T={T}"
