"""CPU tests of the oracle: golden vectors of the reference, an independent
closed-form backward, and known answers that need no reference."""
import math

import pytest
import torch

from oracle import oracle as O
from util import NAMES, golden_files, load_golden, rel_err


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1])
def test_oracle_matches_golden(path):
    """naive_*: outputs of the reference's naive_two_simplicial_attend(causal=True);
    outer_*: masked attention over the outer-product keys (the reference's test design)."""
    t, w1, w2 = load_golden(path)
    r = O.two_simplicial_fwd_bwd(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["do"], w1, w2, dtype=torch.float64)
    for k in NAMES:
        assert rel_err(r[k], t[k]) < 2e-6, k


def test_autograd_matches_closed_form():
    q, k1, k2, v1, v2, do = O.make_inputs(2, 37, 4, 2, 32, seed=3, dtype=torch.float64)
    a = O.two_simplicial_fwd_bwd(q, k1, k2, v1, v2, do, 9, 4, dtype=torch.float64, chunk=16)
    e = O.two_simplicial_bwd_explicit(q, k1, k2, v1, v2, do, 9, 4)
    for k in NAMES + ("lse",):
        assert rel_err(a[k], e[k]) < 1e-12, k


def test_chunk_size_does_not_matter():
    q, k1, k2, v1, v2, _ = O.make_inputs(1, 100, 2, 2, 32, seed=4)
    a, la = O.two_simplicial_fwd(q, k1, k2, v1, v2, 33, 7, chunk=8)
    b, lb = O.two_simplicial_fwd(q, k1, k2, v1, v2, 33, 7, chunk=100)
    assert rel_err(a, b) < 1e-5 and rel_err(la, lb) < 1e-5


def test_known_answers():
    b, n, h, d = 1, 50, 2, 32
    q, k1, k2, v1, v2, do = O.make_inputs(b, n, h, h, d, seed=8, dtype=torch.float64)
    w1, w2 = 12, 5
    # row 0 sees only (0, 0)
    out, lse = O.two_simplicial_fwd(q, k1, k2, v1, v2, w1, w2, dtype=torch.float64)
    assert torch.allclose(out[:, 0], v1[:, 0] * v2[:, 0], atol=1e-12)
    assert torch.allclose(lse[:, :, 0], O.lse_row0(q, k1, k2), atol=1e-12)
    # q = 0: uniform probabilities
    out, lse = O.two_simplicial_fwd(torch.zeros_like(q), k1, k2, v1, v2, w1, w2, dtype=torch.float64)
    for i in (0, 3, 20, 49):
        m1 = v1[:, max(0, i - w1 + 1):i + 1].mean(1)
        m2 = v2[:, max(0, i - w2 + 1):i + 1].mean(1)
        assert torch.allclose(out[:, i], m1 * m2, atol=1e-12)
        assert abs(lse[0, 0, i].item() - math.log(min(i + 1, w1) * min(i + 1, w2))) < 1e-12
    # v = v' = 1: out = 1 and dq = dk = dk' = 0
    one = torch.ones_like(v1)
    r = O.two_simplicial_fwd_bwd(q, k1, k2, one, one, do, w1, w2, dtype=torch.float64)
    assert torch.allclose(r["out"], torch.ones_like(q), atol=1e-12)
    for k in ("dq", "dk1", "dk2"):
        assert r[k].abs().max() < 1e-12
    # w1 = w2 = 1: out_i = v_i * v'_i
    r = O.two_simplicial_fwd_bwd(q, k1, k2, v1, v2, do, 1, 1, dtype=torch.float64)
    assert torch.allclose(r["out"], v1 * v2, atol=1e-12)
    assert torch.allclose(r["dv1"], do * v2, atol=1e-12)
    assert torch.allclose(r["dv2"], do * v1, atol=1e-12)
    assert r["dq"].abs().max() < 1e-12


def test_valid_pairs_formula():
    assert O.valid_pairs(128, 128, 128) == 707264
    assert O.valid_pairs(1024, 512, 32) == 12585648
    assert O.flops(2, 8, 1024, 64, 512, 32)["fwd"] == 4 * 64 * 16 * 12585648
