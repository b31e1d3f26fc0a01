"""Output-row sharding without a GPU: the partitioning arithmetic of the shard constructor, and a
world-size-2 gloo run of the host-side exchange (rendezvous bytes broadcast, slice placement, gather) with
the oracle standing in for the device matvec.  The NCCL path itself runs on the GPU box (test_sharding_gpu)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, O, K, bits, gs, out):
    import importlib
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import oracle
    mlxq = importlib.import_module("mlx-runner_b200")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # rank 0 draws the rendezvous bytes, everybody receives them (the channel the NCCL unique id takes)
    token = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        token = torch.arange(128, dtype=torch.uint8)
    dist.broadcast(token, 0)
    assert token.tolist() == list(range(128))
    # every rank builds the same full layer, then its shard through the C ABI (fake device addresses: no compute)
    fx = oracle.QuantFixture(O=O, K=K, bits=bits, gs=gs, seed=3)
    tv = mlxq.TensorView
    shard = mlxq.Linear.shard(tv(0x100000, "u32", (O, K * bits // 32)), tv(0x800000, "f16", (O, K // gs)),
                              tv(0xA00000, "f16", (O, K // gs)), None, inDim=K, rank=rank, nranks=world)
    rows, off = shard.outDim, shard.rowOffset
    assert rows == O // world and off == rank * rows
    # the shard's slice of the matvec (oracle), placed at its offset, then gathered in place like ncclAllGather
    x = oracle.RNG(5).floats(2 * K).reshape(2, K)
    y = torch.zeros((2, O), dtype=torch.float32)
    mine = oracle.qmatmul(fx.packed[off:off + rows], fx.scales_raw[off:off + rows], fx.biases_raw[off:off + rows],
                          fx.scale_type, x, K, bits, gs)
    y[:, off:off + rows] = torch.from_numpy(mine)
    for t in range(2):                     # one gather per token row, as mlxq_linear_forward_gather issues them
        parts = [torch.zeros(rows) for _ in range(world)]
        dist.all_gather(parts, y[t, off:off + rows].contiguous())
        y[t] = torch.cat(parts)
    full = oracle.qmatmul(fx.packed, fx.scales_raw, fx.biases_raw, fx.scale_type, x, K, bits, gs)
    ok = np.array_equal(y.numpy(), full)
    out.put((rank, bool(ok)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_row_shards_gather_to_the_full_output(world, oracle, mlxq):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 64, 256, 4, 64, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert res == [(r, True) for r in range(world)]


def test_comm_of_one_rank_needs_no_collective(mlxq):
    c = mlxq.Comm(0, 1, 0)
    assert (c.rank, c.size) == (0, 1)
    c.close()
    with pytest.raises(mlxq.InvalidArgument):
        mlxq.Comm(0, 2, 0, unique_id=b"short")


def test_shard_and_comm_must_agree(mlxq):
    tv = mlxq.TensorView
    sh = mlxq.Linear.shard(tv(0x100000, "u32", (64, 32)), tv(0x800000, "f16", (64, 4)), tv(0xA00000, "f16", (64, 4)), None,
                           inDim=256, rank=1, nranks=2)
    c = mlxq.Comm(0, 1, 0)
    y = tv(0x900000, "f32", (64,))
    with pytest.raises(mlxq.InvalidArgument, match="shard 1 of 2"):
        c.forwardGather(sh, 0, tv(0x700000, "f16", (256,)), 256, y, 64, 1)
    c.close()
