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
