"""Sequence-block sharding with the halo exchange, on CPU ranks (gloo).

Each rank owns a contiguous block of the sequence, fetches the w1-1 / w2-1 key
rows that precede it from the previous rank, runs the attention on its block
(the CPU oracle stands in for the CUDA operator) and sends the halo rows of the
key/value gradients back.  The result must equal the monolithic computation.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, w1, w2, hq, hk, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from simplicial_attention_b200 import shard
        torch.set_num_threads(1)
        q, k1, k2, v1, v2, do = O.make_inputs(2, n, hq, hk, 32, seed=77, dtype=torch.float64)
        ref = O.two_simplicial_fwd_bwd(q, k1, k2, v1, v2, do, w1, w2, dtype=torch.float64)
        blk = n // world
        sl = slice(rank * blk, (rank + 1) * blk)
        loc = [t[:, sl].clone().requires_grad_() for t in (q, k1, k2, v1, v2)]
        out = shard.sequence_parallel_attn(loc[0], (loc[1], loc[2]), (loc[3], loc[4]), w1=w1, w2=w2, attend=O.attend)
        out.backward(do[:, sl])
        errs = [(out.detach() - ref["out"][:, sl]).abs().max().item()]
        for t, k in zip(loc, ("dq", "dk1", "dk2", "dv1", "dv2")):
            errs.append((t.grad - ref[k][:, sl]).abs().max().item())
        result[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,w1,w2,hq,hk", [(2, 96, 20, 6, 2, 2), (3, 96, 30, 9, 4, 2), (2, 64, 33, 1, 2, 1)])
def test_sequence_blocks_equal_monolithic(world, n, w1, w2, hq, hk):
    port = _free_port()
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, port, n, w1, w2, hq, hk, result), nprocs=world, join=True)
        assert len(result) == world
        assert max(result.values()) < 1e-10, dict(result)


def test_batch_head_slices_are_views():
    from simplicial_attention_b200 import shard
    t = torch.arange(2 * 4 * 8 * 3).reshape(2, 4, 8, 3)
    s = shard.shard_batch_heads(t, rank=1, world=2, dim=2)
    assert s.shape == (2, 4, 4, 3) and s.data_ptr() == t[:, :, 4:].data_ptr()
    with pytest.raises(AssertionError):
        shard.shard_batch_heads(t, 0, 3, dim=0)
