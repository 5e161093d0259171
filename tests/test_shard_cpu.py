"""Sequence-block sharding with the halo exchange, on CPU ranks (gloo).

Each rank owns a contiguous block of the sequence, fetches the w1-1 / w2-1 key
rows that precede it from the previous rank in one batched exchange, runs the
interior rows while the exchange is in flight and the first rows after it (the
CPU oracle stands in for the CUDA kernels, behind the same engine interface),
and sends the halo rows of the key/value gradients back.  The result must equal
the monolithic computation.  A second test makes a rank leave between two
steps: the survivor must get a HaloExchangeError within the time limit instead
of blocking.
"""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O

NAMES = ("dq", "dk1", "dk2", "dv1", "dv2")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def oracle_forward(q, k1, k2, v1, v2, w1, w2, out=None):
    o, lse = O.two_simplicial_fwd(q, k1, k2, v1, v2, w1, w2, dtype=q.dtype)
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse


def oracle_backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, grads=None):
    with torch.enable_grad():       # the oracle differentiates its forward; autograd is off inside a backward
        r = O.two_simplicial_fwd_bwd(q, k1, k2, v1, v2, dout, w1, w2, dtype=q.dtype)
    res = [r[k] for k in NAMES]
    if grads is not None:
        for g, t in zip(grads, res):
            g.copy_(t)
        res = list(grads)
    return res


ENGINE = (oracle_forward, oracle_backward)


def _worker(rank, world, port, n, w1, w2, hq, hk, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from simplicial_attention_b200 import shard
        torch.set_num_threads(1)
        shard.TILE = 16          # small tiles, so that short test blocks still have interior rows
        q, k1, k2, v1, v2, do = O.make_inputs(2, n, hq, hk, 32, seed=77, dtype=torch.float64)
        ref = O.two_simplicial_fwd_bwd(q, k1, k2, v1, v2, do, w1, w2, dtype=torch.float64)
        blk = n // world
        sl = slice(rank * blk, (rank + 1) * blk)
        loc = [t[:, sl].clone().requires_grad_() for t in (q, k1, k2, v1, v2)]
        out = shard.sequence_parallel_attn(loc[0], (loc[1], loc[2]), (loc[3], loc[4]), w1=w1, w2=w2, engine=ENGINE, timeout=30)
        out.backward(do[:, sl])
        errs = [(out.detach() - ref["out"][:, sl]).abs().max().item()]
        for t, k in zip(loc, NAMES):
            errs.append((t.grad - ref[k][:, sl]).abs().max().item())
        result[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,w1,w2,hq,hk", [(2, 96, 20, 6, 2, 2), (3, 96, 30, 9, 4, 2), (2, 64, 33, 1, 2, 1),
                                                  (2, 96, 40, 48, 2, 2)])
def test_sequence_blocks_equal_monolithic(world, n, w1, w2, hq, hk):
    port = _free_port()
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, port, n, w1, w2, hq, hk, result), nprocs=world, join=True)
        assert len(result) == world
        assert max(result.values()) < 1e-10, dict(result)


def _leaver(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from simplicial_attention_b200 import shard
    torch.set_num_threads(1)
    shard.TILE = 16
    n, w1, w2 = 48, 20, 6
    ins = O.make_inputs(1, n, 2, 2, 32, seed=5, dtype=torch.float64)

    def step():
        loc = [t.clone().requires_grad_() for t in ins[:5]]
        out = shard.sequence_parallel_attn(loc[0], (loc[1], loc[2]), (loc[3], loc[4]), w1=w1, w2=w2, engine=ENGINE, timeout=3)
        out.backward(ins[5])

    step()                       # both ranks take part in the first step
    if rank == 1:
        # rank 1 leaves between two steps, with none of its requests in flight
        result["left"] = True
        dist.destroy_process_group()
        return
    t0 = time.time()
    try:
        step()
        result["error"] = None
    except shard.HaloExchangeError as e:
        result["error"] = (e.status, e.rank, e.direction)
    result["seconds"] = time.time() - t0
    # no destroy_process_group: the peer is gone and a collective shutdown could block


def test_survivor_gets_an_error_when_a_rank_leaves():
    port = _free_port()
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_leaver, args=(2, port, result), nprocs=2, join=True)
        assert result.get("left") is True
        assert result["error"] is not None, "rank 0 finished a step without its neighbour"
        status, rank, direction = result["error"]
        assert status in ("timeout", "peer") and rank == 0
        assert result["seconds"] < 20


def test_batch_head_slices_are_views():
    from simplicial_attention_b200 import shard
    t = torch.arange(2 * 4 * 8 * 3).reshape(2, 4, 8, 3)
    s = shard.shard_batch_heads(t, rank=1, world=2, dim=2)
    assert s.shape == (2, 4, 4, 3) and s.data_ptr() == t[:, :, 4:].data_ptr()
    with pytest.raises(AssertionError):
        shard.shard_batch_heads(t, 0, 3, dim=0)
