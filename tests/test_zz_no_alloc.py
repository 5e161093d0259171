"""sa2_bwd_static_scratch: the backward for hosts that cannot give the library a
workspace (all device memory already handed to their own pools, or allocator
calls forbidden where the kernel is launched).  Its scratch is an array built
into the library, so the call itself allocates nothing.

The test drives the entry point through the C ABI exactly as such a host would
(raw pointers, no workspace) and compares every gradient with the regular
entry point, sa2_bwd, on two calls in a row that share the built-in array.
This file sorts last so that a run stopping at the first failure has already
executed every other test.
"""
import ctypes as C

import pytest
import torch

import simplicial_attention_b200 as sa
from simplicial_attention_b200 import _lib
from simplicial_attention_b200.attention import _DTYPES, _shape, _strides
from oracle import oracle as O
from util import rel_err

pytestmark = pytest.mark.gpu

FP32_REL = 1e-4     # the fp32 tolerance used by the other GPU tests
GRADS = ("dq", "dk1", "dk2", "dv1", "dv2")


def backward_static(q, k1, k2, v1, v2, out, lse, dout, w1, w2, grad_dtype=torch.float32, grads=None):
    """Call sa2_bwd_static_scratch with caller-owned inputs and outputs and no workspace."""
    if grads is None:
        grads = [torch.empty(t.shape, dtype=grad_dtype, device=q.device) for t in (q, k1, k2, v1, v2)]
    dq, dk1, dk2, dv1, dv2 = grads
    args = _lib.BwdArgs(
        _shape(q, k1, k2, w1, w2, q.shape[-1] ** -0.5, "simt"),
        q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
        out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), dk1.data_ptr(), dv1.data_ptr(), dk2.data_ptr(), dv2.data_ptr(),
        _strides(q), _strides(k1), _strides(k2), _strides(v1), _strides(v2),
        _strides(out), _strides(dout), _strides(dq),
        _strides(dk1), _strides(dk2), _strides(dv1), _strides(dv2),
        _DTYPES[grad_dtype], 0,
        None, 0,                                   # no workspace: the point of this entry point
        torch.cuda.current_stream(q.device).cuda_stream,
    )
    status = _lib.lib().sa2_bwd_static_scratch(C.byref(args))
    return status, grads


def _case(b, n, hq, hk, d, w1, w2, seed, dtype, oracle=False):
    cpu = O.make_inputs(b, n, hq, hk, d, seed=seed, dtype=dtype)
    ins = [t.cuda() for t in cpu]
    q, k1, k2, v1, v2, do = ins
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel="simt")
    expect = sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel="simt", grad_dtype=torch.float32)
    # the caller owns the outputs too: they exist before the call, which must then take no device memory at all
    got = [torch.empty(t.shape, dtype=torch.float32, device=q.device) for t in (q, k1, k2, v1, v2)]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status, got = backward_static(q, k1, k2, v1, v2, out, lse, do, w1, w2, grads=got)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert status == 0, _lib.lib().sa2_strerror(status)
    assert free_after == free_before, "the call changed the amount of free device memory"
    for name, g, e in zip(GRADS, got, expect):
        assert rel_err(g, e) <= FP32_REL, (name, rel_err(g, e))
    if oracle:
        # and against the CPU oracle itself (fp32 tensors: nothing but fp32 rounding in between)
        ref = O.two_simplicial_fwd_bwd(*cpu, w1, w2)
        for name, g in zip(GRADS, got):
            assert rel_err(g, ref[name]) <= FP32_REL, (name, rel_err(g, ref[name]))


def test_two_calls_in_a_row_match_the_regular_entry_point():
    # the larger problem first, so that the second call finds stale row sums beyond its own size
    _case(2, 200, 4, 2, 64, 70, 9, seed=41, dtype=torch.float32, oracle=True)
    _case(1, 96, 2, 2, 32, 40, 6, seed=42, dtype=torch.bfloat16)


def test_rejects_sizes_beyond_the_built_in_array():
    rows = _lib.STATIC_SCRATCH_ROWS
    n = rows // 8 + 1                                  # b * hq * n = rows + 8 > limit
    q = torch.zeros(1, n, 8, 32, device="cuda")
    lse = torch.zeros(1, 8, n, device="cuda")
    status, _ = backward_static(q, q, q, q, q, q, lse, q, 4, 2)
    assert status == 6
    assert b"SA2_STATIC_SCRATCH_ROWS" in _lib.lib().sa2_strerror(status)


def test_tensor_core_request_is_refused():
    q = torch.zeros(1, 64, 2, 64, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(1, 2, 64, device="cuda")
    grads = [torch.empty_like(q) for _ in range(5)]
    args = _lib.BwdArgs(
        _shape(q, q, q, 16, 4, 0.125, "tcgen05"),
        *[q.data_ptr()] * 7, lse.data_ptr(), *[g.data_ptr() for g in grads],
        *[_strides(q)] * 12, _lib.SA2_BF16, 0, None, 0, torch.cuda.current_stream().cuda_stream)
    assert _lib.lib().sa2_bwd_static_scratch(C.byref(args)) == 2
