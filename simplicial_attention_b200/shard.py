"""Multi-GPU sharding of the sliding-window 2-simplicial attention operator.

The reference is single-GPU; the operator shards in two ways:

* by (batch, head): every rank runs the operator on its own slice with no
  communication on the data path (``shard_batch_heads``);
* by sequence blocks for long sequences: rank r owns rows [s_r, e_r) and needs,
  because the windows are causal, only the LAST ``w1 - 1`` rows of k1/v1 and
  ``w2 - 1`` rows of k2/v2 of rank r-1 (the "halo").  ``halo_exchange`` fetches
  them with one point-to-point send/recv per neighbour pair (NCCL on GPUs, gloo
  on CPU) and prepends them; the kernels take the extended tensors directly
  (their ``off1/off2`` arguments).  In the backward pass the gradient rows that
  belong to the halo travel the other way and are added to the owner's tail
  rows, which autograd does through ``HaloExchange.backward``.

No collective (all-reduce, all-gather) is needed for the operator itself.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function

from .attention import sliding_two_simplicial_attn


def shard_batch_heads(t: Tensor, rank: int, world: int, dim: int = 0) -> Tensor:
    """Slice of ``t`` (batch dim 0 or head dim 2) owned by ``rank``; a strided view, no copy."""
    size = t.shape[dim]
    assert size % world == 0, "the sharded dimension must divide by the number of ranks"
    step = size // world
    return t.narrow(dim, rank * step, step)


def _via_host(send, recv, group, fn) -> bool:
    """gloo moves host memory only: stage device tensors through the host (tests on one GPU)."""
    tensors = (send or []) + (recv or [])
    if dist.get_backend(group) != "gloo" or not any(t.is_cuda for t in tensors):
        return False
    send_h = [t.cpu() for t in send] if send is not None else None
    recv_h = [torch.empty(t.shape, dtype=t.dtype) for t in recv] if recv is not None else None
    fn(send_h, recv_h, group)
    if recv is not None:
        for d, h in zip(recv, recv_h):
            d.copy_(h)
    return True


def _exchange(send_right: list[Tensor] | None, recv_left: list[Tensor] | None, group) -> None:
    """One step of the chain: post every send to rank+1 and every recv from rank-1, then wait."""
    if _via_host(send_right, recv_left, group, _exchange):
        return
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ops = []
    if recv_left is not None and rank > 0:
        src = dist.get_global_rank(group, rank - 1) if group is not None else rank - 1
        ops += [dist.P2POp(dist.irecv, t, src, group) for t in recv_left]
    if send_right is not None and rank < world - 1:
        dst = dist.get_global_rank(group, rank + 1) if group is not None else rank + 1
        ops += [dist.P2POp(dist.isend, t, dst, group) for t in send_right]
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


def _exchange_back(send_left: list[Tensor] | None, recv_right: list[Tensor] | None, group) -> None:
    """The mirror step: sends go to rank-1, receives come from rank+1."""
    if _via_host(send_left, recv_right, group, _exchange_back):
        return
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ops = []
    if recv_right is not None and rank < world - 1:
        src = dist.get_global_rank(group, rank + 1) if group is not None else rank + 1
        ops += [dist.P2POp(dist.irecv, t, src, group) for t in recv_right]
    if send_left is not None and rank > 0:
        dst = dist.get_global_rank(group, rank - 1) if group is not None else rank - 1
        ops += [dist.P2POp(dist.isend, t, dst, group) for t in send_left]
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


class HaloExchange(Function):
    """``apply(t, rows, group)``: returns ``cat(last `rows` rows of rank-1's t, t)`` along
    the sequence dim (1).  Rank 0 has no left neighbour and returns ``t`` itself.
    Backward: the gradient of the halo rows is sent to rank-1, which adds it to the
    gradient of its last ``rows`` rows."""

    @staticmethod
    def forward(ctx, t: Tensor, rows: int, group=None):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx.rows, ctx.group, ctx.rank, ctx.world = rows, group, rank, world
        if rows <= 0 or world == 1:
            ctx.rows = 0
            return t.view_as(t)
        assert t.shape[1] >= rows, "a sequence block must be at least as long as the halo (w - 1 rows)"
        tail = t[:, -rows:].contiguous()
        halo = torch.empty_like(tail)
        _exchange([tail], [halo], group)
        return torch.cat([halo, t], dim=1) if rank > 0 else t.view_as(t)

    @staticmethod
    def backward(ctx, grad: Tensor):
        rows, group, rank, world = ctx.rows, ctx.group, ctx.rank, ctx.world
        if rows == 0:
            return grad, None, None
        if rank > 0:
            g_halo, g_own = grad[:, :rows].contiguous(), grad[:, rows:]
        else:
            g_halo, g_own = None, grad
        g_from_right = torch.empty_like(g_own[:, -rows:]).contiguous() if rank < world - 1 else None
        _exchange_back([g_halo] if g_halo is not None else None,
                       [g_from_right] if g_from_right is not None else None, group)
        if g_from_right is not None:
            g_own = g_own.clone()
            g_own[:, -rows:] += g_from_right
        return g_own, None, None


def halo_exchange(t: Tensor, rows: int, group=None) -> Tensor:
    return HaloExchange.apply(t, rows, group)


def sequence_parallel_attn(q: Tensor, keys, values, w1=512, w2=32, group=None, attend=None, **kw):
    """Sliding-window 2-simplicial attention over a sequence split into contiguous
    blocks, one per rank of ``group`` in rank order.  Inputs and the result are the
    local block ``(b, n_local, h, d)``.  ``attend`` defaults to the CUDA operator; the
    CPU tests pass an oracle with the same signature."""
    attend = sliding_two_simplicial_attn if attend is None else attend
    k1, k2 = keys
    v1, v2 = values
    k1e, v1e = halo_exchange(k1, w1 - 1, group), halo_exchange(v1, w1 - 1, group)
    k2e, v2e = halo_exchange(k2, w2 - 1, group), halo_exchange(v2, w2 - 1, group)
    return attend(q, (k1e, k2e), (v1e, v2e), w1=w1, w2=w2, causal=True, **kw)
