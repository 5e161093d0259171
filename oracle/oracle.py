"""CPU oracle for sliding-window causal 2-simplicial attention.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file;
only the tests, the smoke check and the CPU-baseline leg of the benchmark do.

It restates, on the CPU with plain PyTorch, the arithmetic of the reference
(lucidrains/simplicial-attention):

* scale, joint softmax over the (j, k) rectangle and the aggregation
  follow ``naive_two_simplicial_attend``
  (simplicial_attention/simplicial_attention.py:78-127): ``scale = d**-0.5``
  (:102-104), logits ``sum_c q_ic k_jc k'_kc`` (:109), softmax over the
  flattened (j, k) axis (:119-123), ``out = sum_jk P_ijk v_j * v'_k`` (:125);
* the window mask ``0 <= i-j < w1`` and ``0 <= i-k < w2`` follows the forward
  kernel (simplicial_attention/triton_two_simplicial_attention.py:191-193)
  and the reference's own test oracle (tests/test_triton.py:33-47);
* the ``(b, n, h, d)`` layout and the grouped-query mapping (kv head ``g``
  serves q heads ``g*groups .. g*groups+groups-1``) follow
  triton_two_simplicial_attention.py:1029-1034 and
  simplicial_attention.py:97-98;
* the saved statistic is the natural-log logsumexp per row
  (triton_two_simplicial_attention.py:225-228).

Parity pinning: the reference holds no golden vectors for this path, so the
oracle is pinned against outputs of the reference's own
``naive_two_simplicial_attend(causal=True)`` generated in a container that has
the reference (``tests/golden/make_golden.py``); with ``w1, w2 >= n`` the two
must agree.  The windowed cases have no CPU implementation in the reference
and are covered by the closed-form known answers in the tests.

The dense logits are O(n * w1 * w2) per head, so queries are processed in
chunks and each chunk only sees the keys inside its window.
"""
from __future__ import annotations

import math

import torch


def valid_pairs(n: int, w1: int, w2: int) -> int:
    """Number of unmasked (i, j, k) triples for one (batch, head)."""
    return sum(min(i + 1, w1) * min(i + 1, w2) for i in range(n))


def flops(b: int, h: int, n: int, d: int, w1: int, w2: int) -> dict:
    """Algorithmic flop counts: 2 GEMM-equivalents forward, 5 backward."""
    p = valid_pairs(n, w1, w2) * b * h
    return {"fwd": 4 * d * p, "bwd": 10 * d * p, "fwd_bwd": 14 * d * p}


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and return in the original dtype (what a bf16 kernel sees)."""
    return t.to(torch.bfloat16).to(t.dtype)


def _forward_chunked(q, k1, k2, v1, v2, w1, w2, scale, chunk):
    b, n, hq, d = q.shape
    hk = k1.shape[2]
    assert hq % hk == 0
    g = hq // hk
    dv = v1.shape[-1]
    # keys may carry extra leading rows (the halo of the previous sequence block):
    # query row i then sits at key row i + off
    off1, off2 = k1.shape[1] - n, k2.shape[1] - n

    # (b, hk, g, n, d) queries; (b, hk, n, d) keys / values
    qh = q.permute(0, 2, 1, 3).reshape(b, hk, g, n, d) * scale
    k1h, k2h, v1h, v2h = (t.permute(0, 2, 1, 3) for t in (k1, k2, v1, v2))

    outs, lses = [], []
    for i0 in range(0, n, chunk):
        i1 = min(n, i0 + chunk)
        j0 = max(0, i0 + off1 - w1 + 1)
        m0 = max(0, i0 + off2 - w2 + 1)
        qi = qh[:, :, :, i0:i1]
        kj, vj = k1h[:, :, j0:i1 + off1], v1h[:, :, j0:i1 + off1]
        km, vm = k2h[:, :, m0:i1 + off2], v2h[:, :, m0:i1 + off2]

        sim = torch.einsum("bhgid,bhjd,bhkd->bhgijk", qi, kj, km)

        ii = torch.arange(i0, i1)[:, None]
        dj = ii + off1 - torch.arange(j0, i1 + off1)[None, :]
        dk = ii + off2 - torch.arange(m0, i1 + off2)[None, :]
        ok = ((dj >= 0) & (dj < w1))[:, :, None] & ((dk >= 0) & (dk < w2))[:, None, :]
        sim = sim.masked_fill(~ok, float("-inf"))

        flat = sim.flatten(-2)
        lse = torch.logsumexp(flat, dim=-1)
        attn = torch.exp(flat - lse[..., None]).view_as(sim)
        out = torch.einsum("bhgijk,bhjd,bhkd->bhgid", attn, vj, vm)
        outs.append(out)
        lses.append(lse)

    out = torch.cat(outs, dim=3).reshape(b, hq, n, dv).permute(0, 2, 1, 3)
    lse = torch.cat(lses, dim=3).reshape(b, hq, n)
    return out.contiguous(), lse.contiguous()


def two_simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale=None, chunk=32,
                       dtype=torch.float32):
    """Forward.  q (b,n,hq,d); k1,k2,v1,v2 (b,n,hk,d).  Returns out (b,n,hq,d)
    and the natural-log logsumexp (b,hq,n), both in ``dtype``."""
    q, k1, k2, v1, v2 = (t.detach().to("cpu", dtype) for t in (q, k1, k2, v1, v2))
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    with torch.no_grad():
        return _forward_chunked(q, k1, k2, v1, v2, w1, w2, scale, chunk)


def two_simplicial_fwd_bwd(q, k1, k2, v1, v2, dout, w1, w2, scale=None, chunk=32,
                           dtype=torch.float32):
    """Forward and gradients (autograd over the chunked forward).

    Returns a dict with out, lse, dq, dk1, dk2, dv1, dv2 in ``dtype``; the key
    and value gradients are summed over each kv head's query group, as
    autograd does through the reference's ``repeat``
    (triton_two_simplicial_attention.py:1033-1034).
    """
    ins = [t.detach().to("cpu", dtype).clone().requires_grad_() for t in (q, k1, k2, v1, v2)]
    scale = ins[0].shape[-1] ** -0.5 if scale is None else scale
    out, lse = _forward_chunked(*ins, w1, w2, scale, chunk)
    grads = torch.autograd.grad(out, ins, dout.detach().to("cpu", dtype))
    names = ("dq", "dk1", "dk2", "dv1", "dv2")
    res = {"out": out.detach(), "lse": lse.detach()}
    res.update({k: g for k, g in zip(names, grads)})
    return res


def two_simplicial_bwd_explicit(q, k1, k2, v1, v2, dout, w1, w2, scale=None,
                                dtype=torch.float64):
    """Gradients from the closed-form expressions, one query row at a time
    (small cases only).  With D_i = sum_c O_ic dO_ic, dP_ijk = sum_c dO_ic
    v_jc v'_kc and dS = P (dP - D):  dq_i = scale sum_jk dS k_j k'_k,
    dk_j = scale sum_ik dS q_i k'_k, dk'_k = scale sum_ij dS q_i k_j,
    dv_j = sum_ik P dO_i v'_k, dv'_k = sum_ij P dO_i v_j.
    Independent of autograd; used to cross-check ``two_simplicial_fwd_bwd``.
    """
    q, k1, k2, v1, v2, dout = (t.detach().to("cpu", dtype) for t in (q, k1, k2, v1, v2, dout))
    b, n, hq, d = q.shape
    hk = k1.shape[2]
    g = hq // hk
    scale = d ** -0.5 if scale is None else scale
    out = torch.zeros_like(q)
    lse = torch.zeros(b, hq, n, dtype=dtype)
    dq = torch.zeros_like(q)
    dk1, dk2, dv1, dv2 = (torch.zeros_like(t) for t in (k1, k2, v1, v2))
    for bi in range(b):
        for h in range(hq):
            hh = h // g
            for i in range(n):
                j0, m0 = max(0, i - w1 + 1), max(0, i - w2 + 1)
                kj, km = k1[bi, j0:i + 1, hh], k2[bi, m0:i + 1, hh]
                vj, vm = v1[bi, j0:i + 1, hh], v2[bi, m0:i + 1, hh]
                qi, do = q[bi, i, h], dout[bi, i, h]
                s = scale * torch.einsum("c,jc,kc->jk", qi, kj, km)
                l = torch.logsumexp(s.flatten(), 0)
                p = torch.exp(s - l)
                o = torch.einsum("jk,jc,kc->c", p, vj, vm)
                out[bi, i, h], lse[bi, h, i] = o, l
                dp = torch.einsum("c,jc,kc->jk", do, vj, vm)
                ds = p * (dp - (o * do).sum())
                dq[bi, i, h] = scale * torch.einsum("jk,jc,kc->c", ds, kj, km)
                dk1[bi, j0:i + 1, hh] += scale * torch.einsum("jk,c,kc->jc", ds, qi, km)
                dk2[bi, m0:i + 1, hh] += scale * torch.einsum("jk,c,jc->kc", ds, qi, kj)
                dv1[bi, j0:i + 1, hh] += torch.einsum("jk,c,kc->jc", p, do, vm)
                dv2[bi, m0:i + 1, hh] += torch.einsum("jk,c,jc->kc", p, do, vj)
    return {"out": out, "lse": lse, "dq": dq, "dk1": dk1, "dk2": dk2, "dv1": dv1, "dv2": dv2}


def make_inputs(b, n, hq, hk, d, seed, dtype=torch.float32, with_dout=True):
    """Seeded N(0,1) inputs drawn in fp32 in the fixed order q, k, k', v, v',
    dO on the CPU generator, then cast to ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    shapes = [(b, n, hq, d)] + [(b, n, hk, d)] * 4 + ([(b, n, hq, d)] if with_dout else [])
    return [torch.randn(s, generator=gen, dtype=torch.float32).to(dtype) for s in shapes]


def lse_row0(q, k1, k2, scale=None):
    """Known answer: row 0 sees only (j,k)=(0,0)."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    g = q.shape[2] // k1.shape[2]
    k1e = k1[:, 0].repeat_interleave(g, dim=1)
    k2e = k2[:, 0].repeat_interleave(g, dim=1)
    return scale * (q[:, 0] * k1e * k2e).sum(-1)


def attend(q, keys, values, w1=512, w2=32, causal=True, **_):
    """Differentiable CPU stand-in with the signature of ``sliding_two_simplicial_attn``."""
    assert causal
    out, _ = _forward_chunked(q, keys[0], keys[1], values[0], values[1], w1, w2, q.shape[-1] ** -0.5, 32)
    return out


__all__ = [
    "valid_pairs", "flops", "bf16_round", "two_simplicial_fwd", "two_simplicial_fwd_bwd",
    "two_simplicial_bwd_explicit", "make_inputs", "lse_row0",
]
