"""Multi-GPU sharding of the sliding-window 2-simplicial attention operator.

The reference is single-GPU; the operator shards in two ways:

* by (batch, head): every rank runs the operator on its own slice with no
  communication on the data path (``shard_batch_heads``);
* by sequence blocks for long sequences (``sequence_parallel_attn``): rank r
  owns rows [s_r, e_r) and needs, because the windows are causal, only the LAST
  ``w1 - 1`` rows of k1/v1 and ``w2 - 1`` rows of k2/v2 of rank r-1 (the
  "halo").  All four halos travel in ONE batched point-to-point exchange per
  direction (NCCL on GPUs, gloo on CPU), and the exchange overlaps the work that
  does not need it:

  forward   post the exchange; run the interior query rows (local row >= r0,
            r0 = the halo length rounded up to the 128-row tile - they see local
            keys only); wait; run the first r0 rows against [halo | first r0
            local key rows].
  backward  run the backward of the first r0 rows (it yields the gradient rows
            that belong to the halo); post the exchange of those rows; run the
            interior backward; wait; add the rows received from rank r+1 to the
            tail of the local key/value gradients.

  The kernels take the extended key tensors directly (their ``off1/off2``
  arguments) and write their results into views of the result tensors, so no
  full-size tensor is copied or concatenated.  On CUDA the exchange and the
  launches over the first r0 rows run on a side stream next to the interior
  launches (they fill a fraction of one wave of CTAs; back to back on one stream
  each of them would still cost a whole CTA's run time).

No collective (all-reduce, all-gather) is needed for the operator itself.

Failure handling: the exchange has a time limit.  With a host-driven backend
(gloo) every request is waited for with that limit; with NCCL the requests are
ordered on the stream (no host block) unless ``blocking=True``.  A limit that
runs out, or a peer that has gone away, raises ``HaloExchangeError`` - the
caller learns of it on the host and no kernel waits for a peer.
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function

from .attention import sa2_backward, sa2_forward

TILE = 128      # query rows per CTA of the kernels: the interior launch starts on a tile boundary


class HaloExchangeError(RuntimeError):
    """The halo exchange with a neighbouring rank failed or ran out of time.  ``status`` is
    ``"timeout"`` or ``"peer"``; ``rank`` the local rank; ``direction`` ``"forward"`` (keys/values
    from rank-1) or ``"backward"`` (gradient rows from rank+1)."""

    def __init__(self, status: str, rank: int, direction: str, detail: str = ""):
        self.status, self.rank, self.direction = status, rank, direction
        super().__init__(f"halo exchange ({direction}) failed on rank {rank}: {status}" + (f" ({detail})" if detail else ""))


def shard_batch_heads(t: Tensor, rank: int, world: int, dim: int = 0) -> Tensor:
    """Slice of ``t`` (batch dim 0 or head dim 2) owned by ``rank``; a strided view, no copy."""
    size = t.shape[dim]
    assert size % world == 0, "the sharded dimension must divide by the number of ranks"
    step = size // world
    return t.narrow(dim, rank * step, step)


class _Exchange:
    """One batched exchange in flight: ``send`` tensors go to rank ``dst``, ``recv`` tensors are filled
    from rank ``src`` (either side may be absent).  gloo moves host memory only, so device tensors are
    staged through the host there (tests that run several ranks on one GPU)."""

    def __init__(self, send, dst, recv, src, group, direction):
        self.group, self.direction = group, direction
        self.rank = dist.get_rank(group)
        self.recv, self.staged = recv, None
        backend = dist.get_backend(group)
        self.host_driven = backend != "nccl"
        if backend == "gloo" and any(t.is_cuda for t in (send or []) + (recv or [])):
            send = [t.cpu() for t in send] if send else send
            self.staged = [torch.empty(t.shape, dtype=t.dtype) for t in recv] if recv else None
            recv = self.staged
        ops = []
        if recv:
            peer = dist.get_global_rank(group, src) if group is not None else src
            ops += [dist.P2POp(dist.irecv, t, peer, group) for t in recv]
        if send:
            peer = dist.get_global_rank(group, dst) if group is not None else dst
            ops += [dist.P2POp(dist.isend, t, peer, group) for t in send]
        self.keep = (send, recv)
        try:
            self.reqs = dist.batch_isend_irecv(ops) if ops else []
        except RuntimeError as e:
            raise HaloExchangeError("peer", self.rank, direction, str(e)) from e

    def wait(self, timeout: float | None, blocking: bool = False):
        """Order the received data before whatever the caller launches next.  Host-driven backends (and
        ``blocking``) wait on the host for at most ``timeout`` seconds."""
        limit = datetime.timedelta(seconds=timeout) if timeout is not None else None
        for req in self.reqs:
            try:
                if (self.host_driven or blocking) and limit is not None:
                    ok = req.wait(limit)
                else:
                    ok = req.wait()
            except RuntimeError as e:
                msg = str(e).lower()
                status = "timeout" if ("timed out" in msg or "timeout" in msg) else "peer"
                raise HaloExchangeError(status, self.rank, self.direction, str(e).splitlines()[0]) from e
            if ok is False:
                raise HaloExchangeError("timeout", self.rank, self.direction)
        if self.staged is not None:
            for d_, h_ in zip(self.recv, self.staged):
                d_.copy_(h_)
        self.reqs = []


_side_streams = {}


class _Side:
    """``with side:`` runs on a per-device side stream that starts after everything queued on the
    current stream so far; ``side.join(*tensors)`` makes the current stream wait for it and tells the
    allocator that the tensors made on the side stream are used on the current one.  A no-op for CPU
    tensors."""

    def __init__(self, ref: Tensor):
        self.on = ref.is_cuda
        if self.on:
            dev = ref.device
            if dev not in _side_streams:
                _side_streams[dev] = torch.cuda.Stream(dev)
            self.main, self.side = torch.cuda.current_stream(dev), _side_streams[dev]
            self.side.wait_stream(self.main)
            self.ctx = None

    def __enter__(self):
        if self.on:
            self.ctx = torch.cuda.stream(self.side)
            self.ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.on:
            self.ctx.__exit__(*exc)
        return False

    def join(self, *tensors):
        if self.on:
            self.main.wait_stream(self.side)
            for t in tensors:
                if t is not None and t.is_cuda:
                    t.record_stream(self.main)


def _cuda_forward(q, k1, k2, v1, v2, w1, w2, out=None, **kw):
    return sa2_forward(q, k1, k2, v1, v2, w1, w2, out=out, **kw)


def _cuda_backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, grads=None, **kw):
    return sa2_backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, grads=grads, **kw)


class SequenceParallelAttention(Function):
    """Autograd function behind ``sequence_parallel_attn``: the schedule described in the module
    docstring.  ``engine = (forward, backward)`` are the block-local operators
    ``forward(q, k1, k2, v1, v2, w1, w2, out=view) -> (out, lse)`` and
    ``backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, grads=views) -> 5 gradients``; keys / values may
    carry leading halo rows.  The default engine is the CUDA library."""

    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, w1, w2, group, engine, timeout, blocking, kw):
        fwd, _ = engine
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        n = q.shape[1]
        h1, h2 = min(w1 - 1, n), min(w2 - 1, n)
        assert world == 1 or n >= max(w1, w2) - 1, "a sequence block must be at least as long as the halo (w - 1 rows)"
        if world == 1:
            h1 = h2 = 0
        # rows [r0, n) see local keys only
        r0 = min(n, -(-max(h1, h2) // TILE) * TILE) if rank > 0 else 0
        ex = None
        halos = None
        out = torch.empty_like(q)
        lse_i = lse_b = None
        send = recv = None
        if world > 1:
            send = [k1[:, n - h1:].contiguous(), v1[:, n - h1:].contiguous(),
                    k2[:, n - h2:].contiguous(), v2[:, n - h2:].contiguous()] if rank < world - 1 else None
            halos = [torch.empty_like(k1[:, :h1]), torch.empty_like(v1[:, :h1]),
                     torch.empty_like(k2[:, :h2]), torch.empty_like(v2[:, :h2])] if rank > 0 else None
        side = _Side(q)
        with side:
            if world > 1:
                ex = _Exchange(send, rank + 1, halos, rank - 1, group, "forward")
        if r0 < n:      # interior rows (all rows on rank 0): no halo needed
            _, lse_i = fwd(q[:, r0:], k1[:, r0 - h1 if rank > 0 else 0:], k2[:, r0 - h2 if rank > 0 else 0:],
                           v1[:, r0 - h1 if rank > 0 else 0:], v2[:, r0 - h2 if rank > 0 else 0:], w1, w2, out=out[:, r0:], **kw)
        ext = []
        with side:
            if ex is not None:
                ex.wait(timeout, blocking)
            if rank > 0:    # the first r0 rows against [halo | first r0 local rows]
                ext = [torch.cat((h_, t[:, :r0]), dim=1) for h_, t in zip(halos, (k1, v1, k2, v2))]
                _, lse_b = fwd(q[:, :r0], ext[0], ext[2], ext[1], ext[3], w1, w2, out=out[:, :r0], **kw)
        side.join(lse_b, *ext)
        ctx.save_for_backward(q, k1, k2, v1, v2, out, lse_i, lse_b, *(halos or []))
        ctx.cfg = (w1, w2, group, engine, timeout, blocking, kw, rank, world, n, h1, h2, r0)
        return out

    @staticmethod
    def backward(ctx, dout):
        w1, w2, group, engine, timeout, blocking, kw, rank, world, n, h1, h2, r0 = ctx.cfg
        _, bwd = engine
        q, k1, k2, v1, v2, out, lse_i, lse_b, *halos = ctx.saved_tensors
        dout = dout.contiguous() if dout.stride(-1) != 1 else dout
        grads = [torch.empty_like(t) for t in (q, k1, k2, v1, v2)]
        dq, dk1, dk2, dv1, dv2 = grads
        ex = None
        bnd = None
        ext, send = [], None
        recv = [torch.empty_like(k1[:, :h1]), torch.empty_like(v1[:, :h1]),
                torch.empty_like(k2[:, :h2]), torch.empty_like(v2[:, :h2])] if world > 1 and rank < world - 1 else None
        side = _Side(q)
        with side:
            if rank > 0:
                # the first r0 rows first: their backward yields the gradient rows of the halo
                ext = [torch.cat((h_, t[:, :r0]), dim=1) for h_, t in zip(halos, (k1, v1, k2, v2))]
                bnd = bwd(q[:, :r0], ext[0], ext[2], ext[1], ext[3], out[:, :r0], lse_b, dout[:, :r0], w1, w2, **kw)
            if world > 1:
                send = [bnd[1][:, :h1].contiguous(), bnd[3][:, :h1].contiguous(),
                        bnd[2][:, :h2].contiguous(), bnd[4][:, :h2].contiguous()] if rank > 0 else None
                ex = _Exchange(send, rank - 1, recv, rank + 1, group, "backward")
        if r0 < n:
            # interior rows: written straight into the rows [r0 - halo, n) of the local gradients
            a1, a2 = (r0 - h1, r0 - h2) if rank > 0 else (0, 0)
            bwd(q[:, r0:], k1[:, a1:], k2[:, a2:], v1[:, a1:], v2[:, a2:], out[:, r0:], lse_i, dout[:, r0:], w1, w2,
                grads=(dq[:, r0:], dk1[:, a1:], dk2[:, a2:], dv1[:, a1:], dv2[:, a2:]), **kw)
        with side:
            if ex is not None:
                ex.wait(timeout, blocking)
        side.join(*ext, *(bnd or []), *(send or []))
        if rank > 0:
            # local rows [0, r0) of the first launch: rows below the interior's range are its alone, the
            # overlap [r0 - halo, r0) has a contribution from both launches
            dq[:, :r0] = bnd[0]
            for g_, b_, h_ in ((dk1, bnd[1], h1), (dk2, bnd[2], h2), (dv1, bnd[3], h1), (dv2, bnd[4], h2)):
                loc = b_[:, h_:]                     # rows [0, r0) of the local tensor
                lo = r0 - h_ if r0 < n else r0       # first local row the interior launch has written
                g_[:, :lo] = loc[:, :lo]
                if lo < r0:
                    g_[:, lo:r0] += loc[:, lo:r0]
        if ex is not None and rank < world - 1:
            for g_, r_, h_ in zip((dk1, dv1, dk2, dv2), ex.recv, (h1, h1, h2, h2)):
                g_[:, n - h_:] += r_
        return (dq, dk1, dk2, dv1, dv2) + (None,) * 7


def sequence_parallel_attn(q: Tensor, keys, values, w1=512, w2=32, group=None, engine=None, timeout: float | None = 60.0,
                           blocking: bool = False, **kw):
    """Sliding-window 2-simplicial attention over a sequence split into contiguous
    blocks, one per rank of ``group`` in rank order.  Inputs and the result are the
    local block ``(b, n_local, h, d)``.  ``engine`` defaults to the CUDA library; the
    CPU tests pass an oracle pair.  ``timeout`` (seconds) bounds every wait of a
    host-driven exchange; see the module docstring."""
    engine = (_cuda_forward, _cuda_backward) if engine is None else engine
    k1, k2 = keys
    v1, v2 = values
    if q.is_cuda and torch.is_autocast_enabled():
        dt = torch.get_autocast_dtype("cuda")
        q, k1, k2, v1, v2 = (t.to(dt) for t in (q, k1, k2, v1, v2))
    return SequenceParallelAttention.apply(q, k1, k2, v1, v2, int(w1), int(w2), group, engine, timeout, blocking, kw)
