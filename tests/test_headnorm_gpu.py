"""Fused per-head RMSNorm against torch's RMSNorm modules (forward and backward), and the module with
and without it."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,d,tol", [(torch.float32, 64, 1e-5), (torch.bfloat16, 64, 2e-2), (torch.float32, 32, 1e-5),
                                         (torch.float32, 128, 1e-5)])
def test_head_rmsnorm_matches_torch(dtype, d, tol):
    from simplicial_attention_b200.headnorm import head_rmsnorm

    torch.manual_seed(0)
    heads, rows = 6, 1000
    x = torch.randn(3, rows, heads * d, device="cuda", dtype=dtype).requires_grad_()
    gain = (1 + 0.1 * torch.randn(heads * d, device="cuda")).requires_grad_()
    dy = torch.randn(3, rows, heads * d, device="cuda", dtype=dtype)
    eps = 1e-6

    y = head_rmsnorm(x, gain, d, eps)
    y.backward(dy)
    got = (y.detach().float(), x.grad.float(), gain.grad.float())
    x.grad = None
    gain.grad = None

    xf = x.detach().double().requires_grad_()
    gf = gain.detach().double().requires_grad_()
    xh = xf.view(3, rows, heads, d)
    ref = (xh * torch.rsqrt(xh.pow(2).mean(-1, keepdim=True) + eps)).view(3, rows, -1) * gf
    ref.backward(dy.double())
    want = (ref.detach().float(), xf.grad.float(), gf.grad.float())
    for g, w in zip(got, want):
        assert (g - w).abs().max().item() <= tol * max(1.0, w.abs().max().item())


def test_module_with_and_without_the_fused_norm():
    from simplicial_attention_b200 import SlidingWindowTwoSimplicialMHA

    torch.manual_seed(1)
    m = SlidingWindowTwoSimplicialMHA(dim=128, dim_head=32, heads=4, key_value_heads=2, w1=16, w2=4, prenorm=True).cuda()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    x = torch.randn(2, 50, 128, device="cuda")
    outs, grads = [], []
    for fused in (True, False):
        m.fused_head_norm = fused
        m.zero_grad()
        xi = x.clone().requires_grad_()
        out = m(xi)
        out.square().sum().backward()
        outs.append(out.detach())
        grads.append([xi.grad] + [p.grad.clone() for p in m.parameters()])
    assert (outs[0] - outs[1]).abs().max().item() <= 1e-4 * outs[1].abs().max().item()
    for a, b in zip(*grads):
        assert (a - b).abs().max().item() <= 1e-3 * max(1e-6, b.abs().max().item())


def test_bitwise_repeatable():
    from simplicial_attention_b200.headnorm import head_rmsnorm

    x = torch.randn(4096, 1536, device="cuda", dtype=torch.bfloat16).requires_grad_()
    gain = torch.ones(1536, device="cuda").requires_grad_()
    dy = torch.randn_like(x)
    res = []
    for _ in range(2):
        x.grad = None
        gain.grad = None
        head_rmsnorm(x, gain, 64, 1e-6).backward(dy)
        res.append((x.grad.clone(), gain.grad.clone()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])


@pytest.mark.parametrize("dim", [256, 512])
def test_row_rmsnorm_module_matches_torch(dim):
    from simplicial_attention_b200.headnorm import RMSNorm

    torch.manual_seed(2)
    ours, ref = RMSNorm(dim).cuda(), torch.nn.RMSNorm(dim).cuda()
    with torch.no_grad():
        ours.weight.add_(0.1 * torch.randn(dim, device="cuda"))
        ref.weight.copy_(ours.weight)
    x = torch.randn(4, 333, dim, device="cuda")
    dy = torch.randn_like(x)
    res = []
    for m in (ours, ref):
        xi = x.clone().requires_grad_()
        m(xi).backward(dy)
        res.append((m(xi).detach(), xi.grad, m.weight.grad.clone()))
        m.weight.grad = None
    for a, b in zip(*res):
        assert (a - b).abs().max().item() <= 1e-5 * max(1.0, b.abs().max().item())
    # under autocast: bf16 out, fp32 gradients for the fp32 input
    xi = x.clone().requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = ours(xi)
    assert y.dtype == torch.bfloat16
    y.backward(dy.to(torch.bfloat16))
    assert xi.grad.dtype == torch.float32
    assert (y.float() - res[1][0]).abs().max().item() <= 2e-2 * res[1][0].abs().max().item()
