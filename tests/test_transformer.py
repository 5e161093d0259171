"""Decoder stack / LM wrapper (the training-step harness)."""
import pytest
import torch

from simplicial_attention_b200.transformer import TwoSimplicialLM, TwoSimplicialTransformer, training_step


def _lm(**kw):
    return TwoSimplicialLM(num_tokens=256, dim=128, depth=4, max_seq_len=64, dim_head=32, heads=4,
                           two_simplicial_attn_every=2,
                           transformer_kwargs=dict(key_value_heads=2, two_simplicial_attn_kwargs=dict(w1=16, w2=4)), **kw)


def test_parameter_names_follow_the_reference():
    keys = set(_lm().state_dict())
    # standard layer 0, simplicial layer 1 (every 2nd), feed-forward, embeddings, head
    for k in ("token_emb.weight", "pos_emb.weight", "to_logits.weight", "transformer.norm.weight",
              "transformer.layers.0.0.prenorm.weight", "transformer.layers.0.0.to_q.weight",
              "transformer.layers.0.0.to_kv.weight", "transformer.layers.0.0.to_out.weight",
              "transformer.layers.0.1.0.weight", "transformer.layers.0.1.1.weight", "transformer.layers.0.1.3.bias",
              "transformer.layers.1.0.prenorm.weight", "transformer.layers.1.0.to_qkv.weight",
              "transformer.layers.1.0.q_norm.weight", "transformer.layers.1.0.k_norms.1.weight",
              "transformer.layers.1.0.v_norms.0.weight", "transformer.layers.1.0.combine_heads.weight"):
        assert k in keys, k
    assert "transformer.layers.0.0.to_qkv.weight" not in keys and "transformer.layers.1.0.to_kv.weight" not in keys


def test_layer_pattern():
    t = TwoSimplicialTransformer(64, depth=8, heads=2, key_value_heads=2, dim_head=32, two_simplicial_attn_every=2)
    kinds = [type(a).__name__ for a, _ in t.layers]
    assert kinds == ["Attention", "SlidingWindowTwoSimplicialMHA"] * 4


@pytest.mark.gpu
def test_training_steps_reduce_the_loss():
    torch.manual_seed(0)
    model = _lm().cuda()
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    tokens = torch.randint(0, 256, (4, 65), device="cuda")
    losses = []
    for _ in range(12):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            losses.append(training_step(model, opt, tokens).item())
    assert all(l == l for l in losses)                  # finite
    assert losses[-1] < losses[0] - 0.3, losses         # memorises the fixed batch


def test_standard_attention_cache_matches_full_pass():
    from simplicial_attention_b200.transformer import Attention

    torch.manual_seed(1)
    layer = Attention(dim=64, dim_head=16, heads=4, key_value_heads=2)
    x = torch.randn(2, 9, 64)
    full = layer(x)
    out, cache = layer(x[:, :6], return_cache=True)
    steps = [out]
    for t in range(6, 9):
        o, cache = layer(x[:, t:t + 1], cache=cache, return_cache=True)
        steps.append(o)
    assert torch.allclose(torch.cat(steps, dim=1), full, atol=1e-5)


@pytest.mark.gpu
def test_cached_decoding_matches_full_prefix():
    # fp32 weights and activations: the simplicial layers run the fp32 kernels, so the cached path
    # (window rows carried as a halo) must agree with re-running the whole prefix
    torch.manual_seed(2)
    model = _lm().cuda().eval()
    tokens = torch.randint(0, 256, (2, 40), device="cuda")      # longer than both windows (16, 4)
    with torch.no_grad():
        full = model(tokens)
        logits, cache = model(tokens[:, :21], return_cache=True)
        got = [logits]
        for t in range(21, 40):
            step, cache = model(tokens[:, t:t + 1], cache=cache, return_cache=True)
            got.append(step)
    got = torch.cat(got, dim=1)
    assert (got - full).abs().max().item() <= 1e-3 * full.abs().max().item()
    # the simplicial layers keep windows, not the prefix
    k1_rows = cache["layers"][1][0][0].shape[1]
    k2_rows = cache["layers"][1][0][1].shape[1]
    assert (k1_rows, k2_rows) == (15, 3)


@pytest.mark.gpu
def test_sample_with_and_without_cache():
    torch.manual_seed(3)
    model = _lm().cuda().eval()
    prompt = torch.randint(0, 256, (2, 10), device="cuda")
    torch.manual_seed(7)
    a = model.sample(prompt, 30, temperature=1e-6, filter_thres=0.99, use_cache=True)
    torch.manual_seed(7)
    b = model.sample(prompt, 30, temperature=1e-6, filter_thres=0.99, use_cache=False)
    assert a.shape == (2, 20) and torch.equal(a, b)              # greedy: identical continuations


@pytest.mark.gpu
def test_stack_matches_the_reference_stack_with_shared_weights():
    """The decoder stack against the reference's own ``TwoSimplicialTransformer`` (golden written by
    tests/golden/make_golden.py: the reference's modules on CPU, its sliding-window layers' Triton attend
    swapped for its naive attend with windows that cover the sequence).  Same parameters, same input; here
    the sliding-window layers run the CUDA kernels (fp32) and the fused per-head norm."""
    import os

    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "stack_b2n24dim32_depth2.npz"))
    n = int(z["n"])
    net = TwoSimplicialTransformer(int(z["dim"]), depth=int(z["depth"]), heads=int(z["heads"]), key_value_heads=int(z["kv_heads"]),
                                   dim_head=int(z["dim_head"]), two_simplicial_attn_every=int(z["every"]),
                                   two_simplicial_attn_kwargs=dict(w1=n, w2=n, qk_rmsnorm=True))
    state = {k[len("param."):]: torch.from_numpy(z[k]) for k in z.files if k.startswith("param.")}
    assert set(state) == set(net.state_dict()), set(state) ^ set(net.state_dict())
    net.load_state_dict(state)
    net = net.cuda()
    x, want = torch.from_numpy(z["x"]).cuda(), torch.from_numpy(z["y"])
    for fused in (True, False):         # one kernel for the five per-head norms, or the separate modules
        for attn, _ in net.layers:
            if hasattr(attn, "fused_head_norm"):
                attn.fused_head_norm = fused
        with torch.no_grad():
            got = net(x).cpu()
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err <= 1e-4, (fused, err)
