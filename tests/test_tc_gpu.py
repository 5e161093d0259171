"""GPU parity tests of the tcgen05 tensor-core path (bf16 operands, fp32 accumulation).

Bar: max-abs <= 2e-2 against the fp32 oracle fed the same bf16-rounded inputs."""
import pytest
import torch

import simplicial_attention_b200 as sa
from oracle import oracle as O
from util import max_abs, rel_err

pytestmark = pytest.mark.gpu

BF16_ABS = 2e-2


def bf16_err(x, ref):
    """max-abs error after discounting the rounding of a bf16 result itself (half an ulp,
    2^-9 relative, taken as 2^-8 |ref|): outputs such as v * v' exceed 4 in magnitude, where
    one bf16 ulp alone is larger than the 2e-2 bar."""
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    return ((x - ref).abs() - ref.abs() / 256).clamp_min(0).max().item()


def _fwd(ins, w1, w2, kernel):
    q, k1, k2, v1, v2 = (t.cuda() for t in ins[:5])
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=kernel)
    torch.cuda.synchronize()
    assert sa.device_status() == 0
    return out, lse


FWD_CASES = [
    # b, n, hq, hk, w1, w2
    (1, 128, 1, 1, 128, 1),
    (1, 128, 1, 1, 128, 4),
    (1, 256, 2, 2, 64, 8),
    (2, 300, 4, 2, 100, 5),       # ragged length, grouped-query heads, odd windows
    (1, 77, 2, 1, 512, 32),       # shorter than one tile, windows longer than the sequence
    (1, 1024, 2, 2, 512, 32),     # the forward-only configuration's sequence and windows
    (1, 640, 1, 1, 513, 40),      # largest resident window, w2 above the reference's 32 limit
    (1, 400, 2, 2, 1, 1),
]


@pytest.mark.parametrize("case", FWD_CASES, ids=lambda c: "b%d_n%d_hq%d_hk%d_w%d_%d" % c)
def test_tc_forward_matches_oracle(case):
    b, n, hq, hk, w1, w2 = case
    ins = O.make_inputs(b, n, hq, hk, 64, seed=300 + n + w2, dtype=torch.bfloat16)
    ref_out, ref_lse = O.two_simplicial_fwd(*[t.float() for t in ins[:5]], w1, w2)
    out, lse = _fwd(ins, w1, w2, "tcgen05")
    assert bf16_err(out, ref_out) <= BF16_ABS, bf16_err(out, ref_out)
    assert max_abs(lse, ref_lse) <= BF16_ABS, max_abs(lse, ref_lse)
    if min(w1, w2) >= 4:
        assert max_abs(out, ref_out) <= BF16_ABS, max_abs(out, ref_out)


def test_tc_forward_c2_full_config():
    """The forward-only configuration: b2 h8 n1024 d64 w1=512 w2=32, bf16; out and lse checked."""
    ins = O.make_inputs(2, 1024, 8, 8, 64, seed=2024, dtype=torch.bfloat16)
    ref_out, ref_lse = O.two_simplicial_fwd(*[t.float() for t in ins[:5]], 512, 32)
    out, lse = _fwd(ins, 512, 32, "auto")
    assert max_abs(out, ref_out) <= BF16_ABS, max_abs(out, ref_out)
    assert max_abs(lse, ref_lse) <= BF16_ABS, max_abs(lse, ref_lse)


def test_tc_forward_halo_blocks():
    b, n, hq, hk, w1, w2 = 1, 700, 2, 1, 200, 9
    ins = [t.cuda() for t in O.make_inputs(b, n, hq, hk, 64, seed=9, dtype=torch.bfloat16)]
    q, k1, k2, v1, v2 = ins[:5]
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel="tcgen05")
    for s, e in ((0, 250), (250, 700)):
        o1, o2 = min(w1 - 1, s), min(w2 - 1, s)
        ob, lb = sa.sa2_forward(q[:, s:e], k1[:, s - o1:e], k2[:, s - o2:e], v1[:, s - o1:e], v2[:, s - o2:e],
                                w1, w2, kernel="tcgen05")
        assert max_abs(ob, out[:, s:e]) <= 1e-2
        assert max_abs(lb, lse[:, :, s:e]) <= 1e-3
    assert sa.device_status() == 0


def test_tc_forward_large_logits_take_the_rescale_path():
    """Keys whose logits jump by far more than 2^64 between tiles force the in-TMEM rescale."""
    b, n, h, w1, w2 = 1, 512, 1, 512, 4
    q, k1, k2, v1, v2, _ = O.make_inputs(b, n, h, h, 64, seed=17, dtype=torch.bfloat16)
    # second keys of +-1 keep q * k' exact in bf16, so the huge logits are not blurred by operand rounding
    k2 = torch.sign(k2.float()).to(torch.bfloat16)
    k1 = k1.float()
    k1[:, 300:310] *= 64.0          # a burst of huge logits in the middle of the window
    k1[:, 5] *= 32.0
    k1 = k1.to(torch.bfloat16)
    ins = (q, k1, k2, v1, v2)
    ref_out, ref_lse = O.two_simplicial_fwd(*[t.float() for t in ins], w1, w2, dtype=torch.float64)
    assert (ref_lse[0, 0, 300:] > 90).any()          # far beyond 2^64 above the early rows' reference
    out, lse = _fwd(ins, w1, w2, "tcgen05")
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert bf16_err(out, ref_out) <= BF16_ABS, bf16_err(out, ref_out)
    assert rel_err(lse, ref_lse) <= 1e-4


def test_tc_forward_bitwise_reproducible():
    ins = O.make_inputs(2, 384, 2, 2, 64, seed=5, dtype=torch.bfloat16)
    a = _fwd(ins, 200, 16, "tcgen05")
    b = _fwd(ins, 200, 16, "tcgen05")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_auto_picks_tensor_cores_for_bf16_d64():
    ins = O.make_inputs(1, 256, 2, 2, 64, seed=6, dtype=torch.bfloat16)
    a = _fwd(ins, 128, 8, "auto")
    t = _fwd(ins, 128, 8, "tcgen05")
    assert torch.equal(a[0], t[0])
