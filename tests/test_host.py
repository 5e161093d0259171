"""Host-side mirror of the reference interface (CPU; no kernels run)."""
import pytest
import torch

import simplicial_attention_b200 as sa


def test_module_state_dict_keys_match_reference():
    m = sa.SlidingWindowTwoSimplicialMHA(dim=512, heads=8, key_value_heads=4, dim_head=64)
    sd = m.state_dict()
    assert sorted(sd) == sorted([
        "q_norm.weight", "k_norms.0.weight", "k_norms.1.weight", "v_norms.0.weight", "v_norms.1.weight",
        "to_qkv.weight", "combine_heads.weight"])
    assert sd["to_qkv.weight"].shape == (8 * 64 + 2 * 4 * 64 + 2 * 4 * 64, 512)
    assert sd["combine_heads.weight"].shape == (512, 512)
    m = sa.SlidingWindowTwoSimplicialMHA(dim=64, heads=2, dim_head=32, prenorm=True, postnorm=True, qk_rmsnorm=False)
    assert sorted(m.state_dict()) == ["combine_heads.weight", "postnorm.weight", "prenorm.weight", "to_qkv.weight"]


def test_module_rejects_reserved_kwargs():
    with pytest.raises(AssertionError):
        sa.SlidingWindowTwoSimplicialMHA(dim=64, number_key_value_sets=3)
    with pytest.raises(AssertionError):
        sa.SlidingWindowTwoSimplicialMHA(dim=64, head_first_dim=True)


def test_cpu_tensors_are_rejected_not_computed():
    q = torch.randn(1, 8, 2, 32)
    with pytest.raises(AssertionError):
        sa.sliding_two_simplicial_attn(q, (q, q), (q, q), w1=4, w2=2)


def test_bad_heads_and_dims():
    q = torch.randn(1, 8, 3, 32)
    k = torch.randn(1, 8, 2, 32)
    with pytest.raises(AssertionError):
        sa.sliding_two_simplicial_attn(q, (k, k), (k, k))


def test_plugin_slot_receives_split_heads():
    seen = {}

    def attend(queries, keys, values, causal=False):
        seen["q"], seen["k"], seen["v"], seen["causal"] = queries.shape, [k.shape for k in keys], len(values), causal
        return queries

    m = sa.HigherOrderAttention(dim=64, heads=4, key_value_heads=2, dim_head=32, attend=attend,
                                head_first_dim=False, causal=True)
    out = m(torch.randn(2, 10, 64))
    assert out.shape == (2, 10, 64)
    assert seen["q"] == (2, 10, 4, 32) and seen["k"] == [(2, 10, 2, 32)] * 2 and seen["v"] == 2 and seen["causal"]


def test_distinct_value_head_dim_is_rejected_at_construction():
    """The kernels aggregate values over the key head dim; the module says so up front instead of failing at
    the first forward (the reference accepts dim_head_values, simplicial_mha.py:34, and then fails in its kernels)."""
    import pytest
    with pytest.raises(ValueError):
        sa.SlidingWindowTwoSimplicialMHA(dim=64, heads=2, dim_head=32, dim_head_values=16)
    sa.SlidingWindowTwoSimplicialMHA(dim=64, heads=2, dim_head=32, dim_head_values=32)      # equal is fine


def test_cpu_binding_is_a_no_op_without_a_gpu():
    """bind_to_device_cpus only narrows the affinity mask when NVML names CPUs local to the GPU; without
    a device it must leave the process alone and say so."""
    import os
    from simplicial_attention_b200.host import bind_to_device_cpus
    before = os.sched_getaffinity(0)
    if not torch.cuda.is_available():
        assert bind_to_device_cpus("cuda:0") is None
        assert os.sched_getaffinity(0) == before


def test_wait_accounting_tool_names_every_kernel():
    """The diagnostic front end knows the three tensor-core kernels and builds beside the normal library."""
    from simplicial_attention_b200 import waitprof, build
    assert sorted(waitprof.SLOTS) == ["dk1_dv1", "dq_dk2_dv2", "fwd"]
    assert waitprof.PROF_LIB != build.LIB and waitprof.PROF_LIB.endswith("libsa2_prof.so")
