"""Generate the golden fixtures in this directory.

Run where the reference project is checked out; ``SA2_REFERENCE`` (or the first
argument) names its directory:

    python tests/golden/make_golden.py <path to the reference checkout>

Two families of fixtures are written:

``naive_*.npz``  outputs and gradients of the reference's own
    ``naive_two_simplicial_attend(causal=True)``
    (simplicial_attention/simplicial_attention.py:78-127) on seeded inputs.
    The reference imports ``opt_einsum.contract``, which is not installed
    here; a stub that forwards to ``torch.einsum`` is registered *after*
    ``import torch`` (the equations are plain einsum strings).
``outer_*.npz``  windowed cases.  The reference has no CPU implementation of
    the window, only a test design (tests/test_triton.py:33-64): ordinary
    masked attention of q against the n*n outer-product keys ``k_j * k'_k``
    and values ``v_j * v'_k`` with mask ``0<=i-j<w1 and 0<=i-k<w2``.  That
    design is rebuilt here on ``torch.nn.functional.scaled_dot_product_attention``
    (CPU, fp64), which shares no code with the oracle.

``stack_*.npz``  the reference's own decoder stack, ``TwoSimplicialTransformer``
    with its ``Attention`` and ``FeedForward`` layers
    (simplicial_attention/two_simplicial_transformer.py:25-141), run on CPU: the
    sliding-window layers' ``attend`` (a Triton kernel) is swapped for the
    reference's naive attend with windows that cover the sequence, where the two
    are the same function.  Stored: the input activations, every parameter
    (``param.<name>``) and the output.

Each file stores the inputs as well as the outputs so that the tests do not
depend on the random generator of the installed torch.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = (sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SA2_REFERENCE")) or ""


def _import_reference():
    if not os.path.isdir(os.path.join(REF, "simplicial_attention")):
        sys.exit("make_golden.py: pass the directory of the reference checkout (argument or SA2_REFERENCE)")
    stub = types.ModuleType("opt_einsum")
    stub.contract = lambda eq, *ops: torch.einsum(eq, *ops)
    sys.modules["opt_einsum"] = stub
    sys.path.insert(0, REF)
    from simplicial_attention.simplicial_attention import naive_two_simplicial_attend
    return naive_two_simplicial_attend


def _inputs(b, n, hq, hk, d, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    shapes = [(b, n, hq, d)] + [(b, n, hk, d)] * 4 + [(b, n, hq, d)]
    return [torch.randn(s, generator=gen, dtype=torch.float32).to(dtype) for s in shapes]


def naive_case(name, b, n, hq, hk, d, seed, dtype=torch.float32):
    naive = _import_reference()
    q, k1, k2, v1, v2, do = _inputs(b, n, hq, hk, d, seed, dtype)
    ins = [t.clone().requires_grad_() for t in (q, k1, k2, v1, v2)]
    # the reference's naive path is head-first (b, h, n, d)
    hf = [t.permute(0, 2, 1, 3) for t in ins]
    out = naive(hf[0], (hf[1], hf[2]), (hf[3], hf[4]), causal=True).permute(0, 2, 1, 3)
    grads = torch.autograd.grad(out, ins, do)
    arrays = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do, out=out.detach(),
                  dq=grads[0], dk1=grads[1], dk2=grads[2], dv1=grads[3], dv2=grads[4])
    arrays = {k: v.numpy() for k, v in arrays.items()}
    np.savez(os.path.join(HERE, f"naive_{name}.npz"), w1=n, w2=n, seed=seed, **arrays)
    print("wrote", name, {k: v.shape for k, v in arrays.items() if k in ("q", "k1")})


def outer_case(name, b, n, hq, hk, d, w1, w2, seed):
    import torch.nn.functional as F
    dtype = torch.float64
    q, k1, k2, v1, v2, do = _inputs(b, n, hq, hk, d, seed, dtype)
    ins = [t.clone().requires_grad_() for t in (q, k1, k2, v1, v2)]
    g = hq // hk
    qh = ins[0].permute(0, 2, 1, 3)
    k1h, k2h, v1h, v2h = (t.permute(0, 2, 1, 3).repeat_interleave(g, dim=1) for t in ins[1:])
    kk = torch.einsum("bhid,bhjd->bhijd", k1h, k2h).reshape(b, hq, n * n, d)
    vv = torch.einsum("bhid,bhjd->bhijd", v1h, v2h).reshape(b, hq, n * n, d)
    qi = torch.arange(n)[:, None]
    kv = torch.arange(n * n)[None, :]
    d1, d2 = qi - kv // n, qi - kv % n
    mask = (d1 < w1) & (d2 < w2) & (d1 >= 0) & (d2 >= 0)
    out = F.scaled_dot_product_attention(qh, kk, vv, attn_mask=mask).permute(0, 2, 1, 3)
    grads = torch.autograd.grad(out, ins, do)
    arrays = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do, out=out.detach(),
                  dq=grads[0], dk1=grads[1], dk2=grads[2], dv1=grads[3], dv2=grads[4])
    arrays = {k: v.to(torch.float32).numpy() for k, v in arrays.items()}
    np.savez(os.path.join(HERE, f"outer_{name}.npz"), w1=w1, w2=w2, seed=seed, **arrays)
    print("wrote", name)


def stack_case(name, b, n, dim, depth, heads, kv_heads, dim_head, every, seed):
    naive = _import_reference()
    from simplicial_attention.two_simplicial_transformer import TwoSimplicialTransformer
    torch.manual_seed(seed)
    net = TwoSimplicialTransformer(dim, depth=depth, heads=heads, key_value_heads=kv_heads, dim_head=dim_head,
                                   two_simplicial_attn_every=every,
                                   two_simplicial_attn_kwargs=dict(w1=n, w2=n, qk_rmsnorm=True))

    def attend(q, keys, values, **_):          # (b, n, h, d) in and out, as the sliding-window module calls it
        hf = [t.permute(0, 2, 1, 3) for t in (q, *keys, *values)]
        return naive(hf[0], (hf[1], hf[2]), (hf[3], hf[4]), causal=True).permute(0, 2, 1, 3)

    swapped = 0
    for attn, _ in net.layers:
        if type(attn).__name__ == "SlidingWindowTwoSimplicialMHA":
            attn.attend = attend
            swapped += 1
    assert swapped == depth // every
    # norm gains away from one, so that a wrong gain-to-channel mapping cannot hide
    with torch.no_grad():
        for k, p_ in net.named_parameters():
            if k.endswith("norm.weight") or "norms." in k or k.endswith("prenorm.weight"):
                p_.mul_(1 + 0.2 * torch.randn_like(p_))
    x = torch.randn(b, n, dim)
    with torch.no_grad():
        y = net(x)
    arrays = {"x": x.numpy(), "y": y.numpy()}
    arrays.update({"param." + k: v.detach().numpy() for k, v in net.state_dict().items()})
    np.savez_compressed(os.path.join(HERE, f"stack_{name}.npz"), n=n, dim=dim, depth=depth, heads=heads, kv_heads=kv_heads,
                        dim_head=dim_head, every=every, seed=seed, **arrays)
    print("wrote", name, y.shape, len(arrays) - 2, "parameters")


if __name__ == "__main__":
    torch.manual_seed(0)
    # the reference's CPU-runnable configuration: b1 h2 n128 d32, full causal, fp32
    naive_case("c1_b1h2n128d32", 1, 128, 2, 2, 32, seed=1234)
    # grouped-query heads (4 q heads on 2 kv heads), d = 64
    naive_case("gqa_b2h4k2n40d64", 2, 40, 4, 2, 64, seed=77)
    # windowed, same window ratio as the reference's GPU test (w1 = 2*w2)
    outer_case("b1h2n48d32_w16_8", 1, 48, 2, 2, 32, 16, 8, seed=5)
    outer_case("gqa_b1h4k2n40d64_w24_5", 1, 40, 4, 2, 64, 24, 5, seed=6)
    # the reference decoder stack: 2 layers (standard, then sliding-window 2-simplicial), grouped-query heads
    stack_case("b2n24dim32_depth2", 2, 24, 32, 2, 2, 1, 32, 2, seed=11)
