"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU
oracle and the committed golden vectors.

Tolerances (stated by the task for this operator):
  * fp32 path: ||x - ref||_inf / ||ref||_inf <= 1e-4 on out, lse and all five gradients;
  * bf16 path: max-abs <= 2e-2 against the fp32 oracle fed the same bf16-rounded inputs.
"""
import pytest
import torch

import simplicial_attention_b200 as sa
from oracle import oracle as O
from util import NAMES, golden_files, load_golden, max_abs, rel_err

pytestmark = pytest.mark.gpu

FP32_REL = 1e-4
BF16_ABS = 2e-2
GRADS = ("dq", "dk1", "dk2", "dv1", "dv2")


def _dev(ts):
    return [t.cuda() for t in ts]


def run_ours(q, k1, k2, v1, v2, do, w1, w2, kernel="simt", grad_dtype=torch.float32, scale=None):
    q, k1, k2, v1, v2, do = _dev((q, k1, k2, v1, v2, do))
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, scale=scale, kernel=kernel)
    grads = sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, scale=scale, kernel=kernel, grad_dtype=grad_dtype)
    torch.cuda.synchronize()
    res = {"out": out, "lse": lse}
    res.update(dict(zip(GRADS, grads)))
    return res


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1])
def test_fp32_matches_golden(path):
    t, w1, w2 = load_golden(path)
    r = run_ours(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["do"], w1, w2)
    for k in NAMES:
        assert rel_err(r[k], t[k]) <= FP32_REL, (k, rel_err(r[k], t[k]))


CASES = [
    # b, n, hq, hk, d, w1, w2
    (1, 1, 1, 1, 32, 4, 2),          # single row
    (1, 63, 2, 2, 32, 16, 8),        # shorter than a tile
    (2, 130, 4, 2, 64, 70, 9),       # ragged length, grouped-query heads
    (1, 200, 2, 1, 128, 512, 32),    # windows longer than the sequence
    (1, 257, 2, 2, 64, 1, 1),        # degenerate windows
    (1, 300, 3, 3, 32, 100, 1),
    (1, 300, 2, 2, 64, 1, 40),       # w2 > w1, w2 above the reference's 32 limit
    (2, 384, 2, 2, 64, 128, 32),
    (1, 192, 2, 2, 128, 96, 16),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_n%d_hq%d_hk%d_d%d_w%d_%d" % c)
def test_fp32_matches_oracle(case):
    b, n, hq, hk, d, w1, w2 = case
    ins = O.make_inputs(b, n, hq, hk, d, seed=100 + n)
    ref = O.two_simplicial_fwd_bwd(*ins, w1, w2, dtype=torch.float64)
    r = run_ours(*ins, w1, w2)
    # gradients that are analytically zero (single-key windows) are judged on the scale of the other gradients
    floor = 0.05 * max(ref[k].abs().max().item() for k in GRADS)
    for k in NAMES + ("lse",):
        assert rel_err(r[k], ref[k], floor) <= FP32_REL, (k, rel_err(r[k], ref[k], floor))


def test_bf16_inputs_fp32_math():
    """bf16 tensors through the SIMT kernels: only the inputs and the output are rounded."""
    b, n, hq, hk, d, w1, w2 = 2, 200, 4, 2, 64, 64, 16
    ins = O.make_inputs(b, n, hq, hk, d, seed=11, dtype=torch.bfloat16)
    ref = O.two_simplicial_fwd_bwd(*[t.float() for t in ins], w1, w2, dtype=torch.float64)
    r = run_ours(*ins, w1, w2)
    for k in NAMES + ("lse",):
        assert max_abs(r[k], ref[k]) <= BF16_ABS, (k, max_abs(r[k], ref[k]))


def test_known_answers_on_device():
    b, n, h, d, w1, w2 = 2, 333, 2, 64, 50, 7
    q, k1, k2, v1, v2, do = O.make_inputs(b, n, h, h, d, seed=21)
    r = run_ours(q, k1, k2, v1, v2, do, w1, w2)
    # row 0 sees only (j, k) = (0, 0)
    assert rel_err(r["out"][:, 0], (v1 * v2)[:, 0]) < 1e-5
    assert rel_err(r["lse"][:, :, 0], O.lse_row0(q, k1, k2)) < 1e-5
    # v = v' = 1  =>  out = 1, dq = dk = dk' = 0
    one = torch.ones_like(v1)
    r = run_ours(q, k1, k2, one, one, do, w1, w2)
    assert max_abs(r["out"], torch.ones_like(q)) < 1e-5
    for k in ("dq", "dk1", "dk2"):
        assert r[k].abs().max().item() < 1e-4
    # w1 = w2 = 1  =>  out_i = v_i * v'_i
    r = run_ours(q, k1, k2, v1, v2, do, 1, 1)
    assert rel_err(r["out"], v1 * v2) < 1e-6
    assert rel_err(r["dv1"], do * v2) < 1e-6 and rel_err(r["dv2"], do * v1) < 1e-6


def test_bitwise_reproducible():
    ins = O.make_inputs(2, 260, 4, 2, 64, seed=5)
    a = run_ours(*ins, 100, 12)
    b = run_ours(*ins, 100, 12)
    for k in NAMES + ("lse",):
        assert torch.equal(a[k], b[k]), k


def test_halo_blocks_equal_monolithic():
    """Splitting the sequence into blocks that carry the previous block's last
    w1-1 / w2-1 key rows as a halo reproduces the monolithic result; the halo
    rows of dK/dV are the partial sums owed to the previous block."""
    b, n, hq, hk, d, w1, w2 = 1, 320, 2, 1, 64, 48, 9
    q, k1, k2, v1, v2, do = _dev(O.make_inputs(b, n, hq, hk, d, seed=9))
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel="simt")
    full = sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel="simt", grad_dtype=torch.float32)
    acc = [torch.zeros_like(t, dtype=torch.float32) for t in (q, k1, k2, v1, v2)]
    outs = []
    for s, e in ((0, 100), (100, 230), (230, 320)):
        o1, o2 = min(w1 - 1, s), min(w2 - 1, s)
        qb, dob = q[:, s:e], do[:, s:e]
        k1b, v1b = k1[:, s - o1:e], v1[:, s - o1:e]
        k2b, v2b = k2[:, s - o2:e], v2[:, s - o2:e]
        ob, lb = sa.sa2_forward(qb, k1b, k2b, v1b, v2b, w1, w2, kernel="simt")
        g = sa.sa2_backward(qb, k1b, k2b, v1b, v2b, ob, lb, dob, w1, w2, kernel="simt", grad_dtype=torch.float32)
        outs.append(ob)
        acc[0][:, s:e] += g[0]
        acc[1][:, s - o1:e] += g[1]
        acc[2][:, s - o2:e] += g[2]
        acc[3][:, s - o1:e] += g[3]
        acc[4][:, s - o2:e] += g[4]
    assert rel_err(torch.cat(outs, 1), out) < 1e-5   # forward rows do not depend on the split
    for a, f in zip(acc, full):
        assert rel_err(a, f) < 1e-5


def test_strided_views_and_autograd():
    """Inputs that are views into one fused projection (as in the module with
    qk_rmsnorm=False) are read in place; autograd returns input-dtype grads."""
    b, n, h, d, w1, w2 = 2, 96, 2, 32, 40, 6
    torch.manual_seed(0)
    fused = torch.randn(b, n, h, 5 * d, device="cuda", requires_grad=True)
    q, k1, k2, v1, v2 = fused.split(d, dim=-1)
    out = sa.sliding_two_simplicial_attn(q, (k1, k2), (v1, v2), w1=w1, w2=w2, kernel="simt")
    do = torch.randn_like(out)
    out.backward(do)
    parts = [t.detach().cpu() for t in (q, k1, k2, v1, v2)]
    ref = O.two_simplicial_fwd_bwd(*parts, do.cpu(), w1, w2, dtype=torch.float64)
    gref = torch.cat([ref[k] for k in GRADS], dim=-1)
    assert rel_err(out, ref["out"]) <= FP32_REL
    assert rel_err(fused.grad, gref) <= FP32_REL


def test_reference_test_design():
    """Shapes and tolerances of the reference's own GPU test (tests/test_triton.py:68-115):
    b2 n128 h4 d64, w1=64, w2=32, out atol 3e-2, grads atol 5e-2 after out.sum().backward()."""
    torch.manual_seed(1)
    ts = [torch.randn(2, 128, 4, 64, device="cuda", requires_grad=True) for _ in range(5)]
    out = sa.sliding_two_simplicial_attn(ts[0], (ts[1], ts[2]), (ts[3], ts[4]), w1=64, w2=32, causal=True)
    out.sum().backward()
    cpu = [t.detach().cpu() for t in ts]
    ref = O.two_simplicial_fwd_bwd(*cpu, torch.ones(2, 128, 4, 64), 64, 32)
    assert torch.allclose(out.detach().cpu(), ref["out"], atol=3e-2)
    for t, k in zip(ts, GRADS):
        assert torch.allclose(t.grad.cpu(), ref[k], atol=5e-2), k


def test_module_forward_backward():
    torch.manual_seed(2)
    m = sa.SlidingWindowTwoSimplicialMHA(dim=128, heads=4, key_value_heads=2, dim_head=32, w1=24, w2=6).cuda()
    x = torch.randn(2, 70, 128, device="cuda", requires_grad=True)
    y = m(x)
    assert y.shape == x.shape
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())

    # same weights, attention swapped for the oracle: module outputs agree
    def oracle_attend(queries, keys, values, causal=True):
        o, _ = O.two_simplicial_fwd(queries, *keys, *values, 24, 6)
        return o.to(queries.device)

    m2 = sa.HigherOrderAttention(dim=128, heads=4, key_value_heads=2, dim_head=32, attend=oracle_attend,
                                 head_first_dim=False).cuda()
    m2.load_state_dict(m.state_dict())
    with torch.no_grad():
        assert rel_err(m(x), m2(x)) < 1e-4


def test_errors_raise():
    q = torch.randn(1, 8, 2, 48, device="cuda")
    with pytest.raises(ValueError):
        sa.sliding_two_simplicial_attn(q, (q, q), (q, q))
    q = torch.randn(1, 8, 2, 32, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError):
        sa.sliding_two_simplicial_attn(q, (q, q), (q, q))
    q = torch.randn(1, 8, 2, 32, device="cuda")
    with pytest.raises(AssertionError):
        sa.sliding_two_simplicial_attn(q, (q, q), (q, q), causal=False)
    with pytest.raises(sa._lib.Sa2Error):          # fp32 tensors cannot take the bf16 tensor-core path
        sa.sa2_forward(q, q, q, q, q, 4, 2, kernel="tcgen05")


def test_wide_projection_uses_the_module_norms():
    """32 heads x 128 channels with 8 kv heads is an 8192-channel projection: beyond what the fused per-head
    norm keeps in shared memory in its backward, so the module must run the five RMSNorm modules, as the
    reference does - forward and backward, with the same result as the fused path on a narrower slice."""
    torch.manual_seed(0)
    m = sa.SlidingWindowTwoSimplicialMHA(dim=64, heads=32, key_value_heads=8, dim_head=128, w1=16, w2=4).cuda()
    assert sum(m.split_dims) == 8192 > m.fused_head_norm_max_channels
    x = torch.randn(1, 32, 64, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x)
    y.float().sum().backward()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad).all()
    assert sa.device_status() == 0


def test_second_key_value_bias():
    """K2_BIAS / V2_BIAS of the reference kernels (triton_two_simplicial_attention.py:105-106,175-176):
    a constant added to every element of the second keys / values."""
    ins = O.make_inputs(1, 96, 2, 2, 32, seed=12)
    q, k1, k2, v1, v2 = (t.cuda().requires_grad_() for t in ins[:5])
    out = sa.sliding_two_simplicial_attn(q, (k1, k2), (v1, v2), w1=40, w2=6, k2_bias=0.25, v2_bias=-0.5)
    out.backward(ins[5].cuda())
    ref = O.two_simplicial_fwd_bwd(ins[0], ins[1], ins[2] + 0.25, ins[3], ins[4] - 0.5, ins[5], 40, 6)
    assert rel_err(out, ref["out"]) <= 1e-4
    for t, k in zip((q, k1, k2, v1, v2), ("dq", "dk1", "dk2", "dv1", "dv2")):
        assert rel_err(t.grad, ref[k]) <= 1e-4, k
