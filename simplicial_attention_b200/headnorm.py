"""Per-head RMSNorm of a packed projection in one kernel (forward and backward).

The reference normalises q, k, k', v, v' with five ``RMSNorm(dim_head)`` modules
after splitting its fused projection (simplicial_attention/simplicial_mha.py:69-73,
124-127).  ``head_rmsnorm`` does the same arithmetic on the projection as a whole:
``x`` is ``(..., channels)``, every ``d`` consecutive channels are one head and
``weight`` holds one gain per channel.  The CUDA kernels sit behind the C ABI
(``sa2_headnorm_fwd`` / ``sa2_headnorm_bwd`` in ``include/sa2.h``).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch.autograd import Function

from . import _lib

_DTYPES = {torch.float32: _lib.SA2_F32, torch.bfloat16: _lib.SA2_BF16}


class HeadRMSNorm(Function):
    @staticmethod
    def forward(ctx, x, weight, d, eps, out_dtype):
        assert x.is_cuda and x.dtype in _DTYPES and out_dtype in _DTYPES
        channels = x.shape[-1]
        x2 = x.reshape(-1, channels)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        w = weight.detach().to(torch.float32).contiguous()
        y = torch.empty((rows, channels), dtype=out_dtype, device=x.device)
        rstd = torch.empty((rows, channels // d), dtype=torch.float32, device=x.device)
        args = _lib.HeadnormArgs(
            x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), rstd.data_ptr(), None, None, 0,
            rows, x2.stride(0), y.stride(0), 0, channels, d, _DTYPES[x.dtype], _DTYPES[out_dtype],
            float(eps), torch.cuda.current_stream(x.device).cuda_stream)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().sa2_headnorm_fwd(C.byref(args)), "sa2_headnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.cfg = (d, eps, x.shape, weight.dtype)
        return y.view(*x.shape[:-1], channels)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        d, eps, shape, wdtype = ctx.cfg
        rows, channels = x2.shape
        dy2 = dy.reshape(rows, channels)
        if dy2.stride(1) != 1 or dy2.dtype not in _DTYPES:
            dy2 = dy2.contiguous().to(dy.dtype if dy.dtype in _DTYPES else torch.float32)
        dx = torch.empty((rows, channels), dtype=x2.dtype, device=x2.device)
        dw = torch.empty(channels, dtype=torch.float32, device=x2.device)
        lib = _lib.lib()
        nbytes = lib.sa2_headnorm_partial_bytes(rows, channels)
        partial = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x2.device)
        args = _lib.HeadnormArgs(
            x2.data_ptr(), dy2.data_ptr(), w.data_ptr(), dx.data_ptr(), rstd.data_ptr(), dw.data_ptr(),
            partial.data_ptr(), partial.numel(),
            rows, x2.stride(0), dx.stride(0), dy2.stride(0), channels, d, _DTYPES[x2.dtype], _DTYPES[dy2.dtype],
            float(eps), torch.cuda.current_stream(x2.device).cuda_stream)
        with torch.cuda.device(x2.device):
            _lib.check(lib.sa2_headnorm_bwd(C.byref(args)), "sa2_headnorm_bwd")
        return dx.view(shape), dw.to(wdtype), None, None, None


def head_rmsnorm(x, weight, d, eps, out_dtype=None):
    """``y[..., c] = x[..., c] * rsqrt(mean over c's head of x^2 + eps) * weight[c]``; ``weight`` has one
    entry per channel.  ``out_dtype`` defaults to ``x.dtype``."""
    return HeadRMSNorm.apply(x, weight, int(d), float(eps), x.dtype if out_dtype is None else out_dtype)


class RMSNorm(torch.nn.Module):
    """``torch.nn.RMSNorm(dim)`` with the same parameter (``weight``) and arithmetic, run by the fused kernel
    on CUDA when ``dim`` is 32 ... 512 (a power of two times 32); under autocast the result is produced in
    the autocast dtype directly - its consumers here are linear layers, which would round it anyway."""

    def __init__(self, dim, eps=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = torch.nn.Parameter(torch.ones(dim))

    def forward(self, x):
        fused = x.is_cuda and self.dim in (32, 64, 128, 256, 512) and x.dtype in _DTYPES
        if not fused:
            return torch.nn.functional.rms_norm(x, (self.dim,), self.weight, self.eps)
        autocast = torch.is_autocast_enabled()
        eps = self.eps if self.eps is not None else torch.finfo(torch.float32 if autocast else x.dtype).eps
        out_dtype = torch.get_autocast_dtype("cuda") if autocast else x.dtype
        if out_dtype not in _DTYPES:
            out_dtype = x.dtype
        return head_rmsnorm(x, self.weight, self.dim, eps, out_dtype)
