"""Host side of the sliding-window causal 2-simplicial attention operator.

Mirrors the reference's functional interface
(simplicial_attention/triton_two_simplicial_attention.py):

* ``SlidingTwoSimplicialAttention.apply(q, k1, k2, v1, v2, w1, w2, causal)``
  - the autograd function (:718-1008);
* ``sliding_two_simplicial_attn(q, keys, values, w1, w2, causal,
  pad_to_multiple_of)`` - the functional wrapper (:1020-1056).

Tensors are ``(batch, seq, heads, dim_head)``.  Everything is computed by the
CUDA library behind the C ABI in ``include/sa2.h``; this file only turns
tensors into pointers, sizes and strides.  CPU tensors are rejected, as in the
reference (:729).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor
from torch.autograd import Function

from . import _lib

_DTYPES = {torch.float32: _lib.SA2_F32, torch.bfloat16: _lib.SA2_BF16}


def exists(v):
    return v is not None


def divisible_by(num, den):
    return (num % den) == 0


def _usable(t: Tensor) -> Tensor:
    """Return ``t`` if the kernels can address it in place, else a contiguous copy
    (the reference copies whenever the last dim is not contiguous, :731)."""
    ok = t.stride(-1) == 1 and all(s % 4 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def _strides(t: Tensor) -> _lib.Strides:
    return _lib.Strides(t.stride(0), t.stride(1), t.stride(2))


def _shape(q, k1, k2, w1, w2, scale, kernel) -> _lib.Shape:
    b, n, hq, d = q.shape
    hk = k1.shape[2]
    off1, off2 = k1.shape[1] - n, k2.shape[1] - n
    return _lib.Shape(b, n, hq, hk, d, int(w1), int(w2), off1, off2, _DTYPES[q.dtype],
                      _lib.KERNELS[kernel], float(scale))


def _check_inputs(q, k1, k2, v1, v2):
    assert all(t.is_cuda for t in (q, k1, k2, v1, v2)), "sliding 2-simplicial attention needs CUDA tensors"
    if q.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {q.dtype}: use float32 or bfloat16")
    if any(t.dtype != q.dtype for t in (k1, k2, v1, v2)):
        raise ValueError("q, keys and values must share one dtype")
    if any(t.dim() != 4 for t in (q, k1, k2, v1, v2)):
        raise ValueError("expected (batch, seq, heads, dim_head) tensors")
    b, n, hq, d = q.shape
    assert divisible_by(hq, k1.shape[2]), "query heads must be a multiple of key/value heads"
    if d not in (32, 64, 128):
        raise ValueError(f"dim_head {d} is not supported (32, 64 or 128)")
    if k1.shape != v1.shape or k2.shape != v2.shape:
        raise ValueError("each key must have the shape of its value")
    for t in (k1, k2):
        if t.shape[0] != b or t.shape[2] != k1.shape[2] or t.shape[3] != d or t.shape[1] < n:
            raise ValueError("key/value shape does not match the queries")


def _check_result_buffer(t, shape, dtype, what):
    if tuple(t.shape) != tuple(shape) or t.dtype != dtype or not t.is_cuda:
        raise ValueError(f"{what}: expected a CUDA tensor of shape {tuple(shape)} and dtype {dtype}")
    if _usable(t) is not t:
        raise ValueError(f"{what}: the kernels cannot write this view in place (last stride 1, other strides "
                         "multiples of 4 elements, 16-byte aligned base)")


def sa2_forward(q, k1, k2, v1, v2, w1, w2, scale=None, kernel="auto", out=None):
    """Raw forward: returns ``(out, lse)``; ``lse`` is ``(b, hq, n)`` fp32, natural log.

    ``k1``/``v1`` may carry ``k1.shape[1] - n`` extra leading rows (and likewise
    ``k2``/``v2``): the halo of the previous sequence block.  ``out`` may be a
    preallocated tensor or strided view to write the result into.
    """
    _check_inputs(q, k1, k2, v1, v2)
    q, k1, k2, v1, v2 = (_usable(t) for t in (q, k1, k2, v1, v2))
    b, n, hq, d = q.shape
    scale = d ** -0.5 if scale is None else scale
    if out is None:
        out = torch.empty((b, n, hq, d), dtype=q.dtype, device=q.device)
    else:
        _check_result_buffer(out, (b, n, hq, d), q.dtype, "out")
    lse = torch.empty((b, hq, n), dtype=torch.float32, device=q.device)
    args = _lib.FwdArgs(
        _shape(q, k1, k2, w1, w2, scale, kernel),
        q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
        out.data_ptr(), lse.data_ptr(),
        _strides(q), _strides(k1), _strides(k2), _strides(v1), _strides(v2), _strides(out),
        torch.cuda.current_stream(q.device).cuda_stream,
    )
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().sa2_fwd(C.byref(args)), "sa2_fwd")
    return out, lse


class BackwardCall:
    """A prepared ``sa2_bwd`` call: gradients and workspace are allocated once, ``launch(phases)``
    issues the kernels.  ``phases`` is 0 for the whole backward or an OR of ``_lib.BWD_ROWSUM``,
    ``_lib.BWD_K1`` (dK1, dV1), ``_lib.BWD_Q`` (dQ, dK2, dV2); the row sums must have been launched
    (same stream, or otherwise ordered) before either of the other two."""

    def __init__(self, q, k1, k2, v1, v2, out, lse, dout, w1, w2, scale=None, kernel="auto", grad_dtype=None,
                 grads=None):
        _check_inputs(q, k1, k2, v1, v2)
        q, k1, k2, v1, v2, out, dout = (_usable(t) for t in (q, k1, k2, v1, v2, out, dout))
        if dout.dtype != q.dtype:
            dout = dout.to(q.dtype)
        lse = lse.contiguous()
        d = q.shape[-1]
        scale = d ** -0.5 if scale is None else scale
        if grads is None:
            grad_dtype = q.dtype if grad_dtype is None else grad_dtype
            grads = tuple(torch.empty(t.shape, dtype=grad_dtype, device=q.device) for t in (q, k1, k2, v1, v2))
        else:
            grad_dtype = grads[0].dtype
            for g_, t, name in zip(grads, (q, k1, k2, v1, v2), ("dq", "dk1", "dk2", "dv1", "dv2")):
                _check_result_buffer(g_, t.shape, grad_dtype, name)
        dq, dk1, dk2, dv1, dv2 = grads
        shape = _shape(q, k1, k2, w1, w2, scale, kernel)
        self.lib = _lib.lib()
        ws_bytes = self.lib.sa2_bwd_workspace_bytes(C.byref(shape))
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=q.device)
        self.device = q.device
        self.grads = grads
        self.keep = (q, k1, k2, v1, v2, out, lse, dout, ws)       # referenced by the argument block
        self.args = _lib.BwdArgs(
            shape,
            q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
            out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk1.data_ptr(), dv1.data_ptr(), dk2.data_ptr(), dv2.data_ptr(),
            _strides(q), _strides(k1), _strides(k2), _strides(v1), _strides(v2),
            _strides(out), _strides(dout), _strides(dq),
            _strides(dk1), _strides(dk2), _strides(dv1), _strides(dv2),
            _DTYPES[grad_dtype], 0,
            ws.data_ptr(), ws.numel(),
            0,
        )

    def launch(self, phases=0):
        self.args.phases = int(phases)
        self.args.stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _lib.check(self.lib.sa2_bwd(C.byref(self.args)), "sa2_bwd")
        return self.grads


def sa2_backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, scale=None, kernel="auto", grad_dtype=None, grads=None):
    """Raw backward: returns ``(dq, dk1, dk2, dv1, dv2)`` in ``grad_dtype``
    (default: the input dtype).  Key/value gradients are already summed over
    each kv head's query group and cover the halo rows too.  ``grads`` may be
    five preallocated tensors or strided views to write the results into."""
    return BackwardCall(q, k1, k2, v1, v2, out, lse, dout, w1, w2, scale, kernel, grad_dtype, grads).launch(0)


class SlidingTwoSimplicialAttention(Function):
    """``apply(q, k1, k2, v1, v2, w1, w2, causal)`` -> out, as in the reference
    (:721-726).  Optional trailing arguments ``scale, kernel, return_lse``
    extend it; with ``return_lse`` the result is ``(out, lse)``."""

    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, w1=512, w2=32, causal=True, scale=None, kernel="auto", return_lse=False):
        assert causal, "only the causal sliding-window form is implemented (the reference's module always passes causal=True)"
        out, lse = sa2_forward(q, k1, k2, v1, v2, w1, w2, scale, kernel)
        ctx.save_for_backward(q, k1, k2, v1, v2, out, lse)
        ctx.cfg = (w1, w2, scale, kernel)
        if return_lse:
            ctx.mark_non_differentiable(lse)
            return out, lse
        return out

    @staticmethod
    def backward(ctx, dout, *_):
        q, k1, k2, v1, v2, out, lse = ctx.saved_tensors
        w1, w2, scale, kernel = ctx.cfg
        grads = sa2_backward(q, k1, k2, v1, v2, out, lse, dout, w1, w2, scale, kernel)
        return (*grads, None, None, None, None, None, None)


def sliding_two_simplicial_attn(
    q: Tensor,                      # (b n hq d)
    keys: tuple[Tensor, Tensor],    # (b n h d) * 2
    values: tuple[Tensor, Tensor],  # (b n h d) * 2
    w1=512,
    w2=32,
    causal=True,
    pad_to_multiple_of=64,
    *,
    kernel="auto",
    return_lse=False,
    k2_bias=0.0,
    v2_bias=0.0,
):
    """Drop-in for the reference's ``sliding_two_simplicial_attn`` (:1020-1056).

    Grouped-query heads are read in place (no ``repeat``) and ragged sequence
    lengths are masked inside the kernels, so ``pad_to_multiple_of`` is
    accepted for compatibility and has no effect.

    ``k2_bias`` / ``v2_bias`` are the reference kernels' ``K2_BIAS`` / ``V2_BIAS``
    constants (:105-106,175-176: added to every element of the second keys /
    values).  The reference passes 0 at all its call sites (:795-796,929-930,
    1000-1001); a non-zero value is applied here as one elementwise add in front
    of the kernels, whose gradient is the identity.
    """
    q_heads, k_heads = q.shape[-2], keys[0].shape[-2]
    assert divisible_by(q_heads, k_heads)
    assert len(keys) == len(values) == 2
    k1, k2 = keys
    v1, v2 = values
    if k2_bias:
        k2 = k2 + k2_bias
    if v2_bias:
        v2 = v2 + v2_bias
    if q.is_cuda and torch.is_autocast_enabled():
        # under autocast the norms in front of the attention hand over fp32: run in the autocast dtype
        dt = torch.get_autocast_dtype("cuda")
        if dt in _DTYPES:
            q, k1, k2, v1, v2 = (t.to(dt) for t in (q, k1, k2, v1, v2))
    return SlidingTwoSimplicialAttention.apply(q, k1, k2, v1, v2, w1, w2, causal, None, kernel, return_lse)


def sliding_two_simplicial_attn_with_lse(q, keys, values, w1=512, w2=32, causal=True, kernel="auto"):
    """Same operator, returning ``(out, lse)``; the reference keeps the
    logsumexp private to its autograd function (:740,802)."""
    return sliding_two_simplicial_attn(q, keys, values, w1, w2, causal, kernel=kernel, return_lse=True)


def check_device(reset: bool = True) -> None:
    """Synchronise and raise ``Sa2Error(SA2_ERR_DEVICE)`` if a kernel gave up on a bounded wait since the
    last reset (the rows that kernel owned were written as NaN)."""
    _lib.check(_lib.lib().sa2_check_device(1 if reset else 0), "sa2_check_device")


def device_status(reset: bool = True) -> int:
    """Synchronise and return the library's device status word (0 = every kernel
    ran to completion; non-zero = a kernel gave up on a bounded wait)."""
    return int(_lib.lib().sa2_device_status(1 if reset else 0))
