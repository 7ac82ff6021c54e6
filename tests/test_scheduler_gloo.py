"""Host-side multi-rank logic on CPU: two gloo ranks shard the heads, each runs the (oracle)
operator on its slice, and rank 0 reassembles exactly the single-rank result."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from piper_kernels_b200.scheduler import gather_outputs, shard_heads, sharded_attention


def test_shard_heads_partitions_exactly():
    for total in (1, 5, 8, 40, 48):
        for world in (1, 2, 3, 4, 8):
            chunks = [shard_heads(total, world, r) for r in range(world)]
            assert [i for c in chunks for i in c] == list(range(total))
            assert max(len(c) for c in chunks) - min(len(c) for c in chunks) <= 1
    with pytest.raises(ValueError):
        shard_heads(4, 2, 2)


def _oracle_op(q, k, v, **kw):
    out = oracle.piper_attention_oracle(q.float().numpy(), k.float().numpy(), v.float().numpy(), 64**-0.5, False,
                                        center_value=True, qk_quantization="per_warp", out_dtype="f16")
    return torch.from_numpy(out).to(torch.float16)


def _worker(rank, world, port, q, k, v, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local, mine = sharded_attention(_oracle_op, q, k, v, world=world, rank=rank)
        full = gather_outputs(local, mine, q.shape[0] * q.shape[1], q.shape)
        # timing contract of the benchmark: max over ranks
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret["full"] = full.float().numpy()
            ret["tmax"] = float(t.item())
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_rank_result():
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(1, 3, 70, 64, generator=gen).to(torch.float16)
    k = torch.randn(1, 3, 90, 64, generator=gen).to(torch.float16)
    v = torch.randn(1, 3, 90, 64, generator=gen).to(torch.float16)
    want = _oracle_op(q, k, v).float().numpy()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, q, k, v, ret), nprocs=2, join=True)
        assert np.array_equal(ret["full"], want)
        assert ret["tmax"] == 2.0
