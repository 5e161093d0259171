"""Multi-head module around the sliding-window 2-simplicial attention operator.

``SlidingWindowTwoSimplicialMHA`` keeps the constructor, forward signature and
``state_dict`` keys of the reference module
(simplicial_attention/triton_two_simplicial_attention.py:1062-1081, built on
``HigherOrderAttention``, simplicial_attention/simplicial_mha.py:28-138), so
checkpoints of the reference load unchanged:
``q_norm.weight, k_norms.{0,1}.weight, v_norms.{0,1}.weight, to_qkv.weight,
combine_heads.weight`` (+ ``prenorm.weight`` / ``postnorm.weight`` when on).

The projections and norms are plain PyTorch; only ``attend`` is ours.
"""
from __future__ import annotations

from functools import partial
from typing import Callable

import torch
from torch.nn import Identity, Linear, Module, ModuleList, RMSNorm

from .attention import divisible_by, exists, sliding_two_simplicial_attn
from .headnorm import RMSNorm as RowRMSNorm


def default(v, d):
    return v if exists(v) else d


class HigherOrderAttention(Module):
    """Projection / head-split / norm shell with a pluggable ``attend``
    callable ``attend(queries, keys, values[, causal=True]) -> out``
    (simplicial_mha.py:41,97-103,131)."""

    def __init__(
        self,
        dim,
        causal=False,
        dim_head=64,
        dim_head_values=None,
        heads=8,
        key_value_heads=None,
        number_key_value_sets=2,
        qk_rmsnorm=True,
        prenorm=False,
        postnorm=False,
        attend: Callable | None = None,
        head_first_dim=True,
    ):
        super().__init__()
        if not exists(attend):
            raise ValueError("pass attend=..., or use SlidingWindowTwoSimplicialMHA: this package ships only "
                             "the sliding-window 2-simplicial attend")
        self.causal = causal
        self.scale = dim_head ** -0.5
        self.heads = heads
        self.key_value_heads = default(key_value_heads, heads)
        assert divisible_by(heads, self.key_value_heads)
        self.query_head_groups = heads // self.key_value_heads
        self.dim_head = dim_head
        self.dim_head_values = default(dim_head_values, dim_head)
        self.kv_sets = number_key_value_sets
        self.head_first_dim = head_first_dim

        # same parameter as torch.nn.RMSNorm; one fused kernel on CUDA
        self.prenorm = RowRMSNorm(dim) if prenorm else Identity()
        self.postnorm = RowRMSNorm(dim) if postnorm else Identity()

        self.qk_rmsnorm = qk_rmsnorm
        if qk_rmsnorm:
            self.q_norm = RMSNorm(dim_head)
            self.k_norms = ModuleList([RMSNorm(dim_head) for _ in range(self.kv_sets)])
            self.v_norms = ModuleList([RMSNorm(dim_head) for _ in range(self.kv_sets)])

        self.split_dims = (
            heads * dim_head,
            self.kv_sets * self.key_value_heads * dim_head,
            self.kv_sets * self.key_value_heads * self.dim_head_values,
        )
        self.to_qkv = Linear(dim, sum(self.split_dims), bias=False)

        if causal:
            attend = partial(attend, causal=causal)
        self.attend = attend

        self.combine_heads = Linear(heads * self.dim_head_values, dim, bias=False)

    def _split(self, t, heads):
        b, n, _ = t.shape
        t = t.view(b, n, heads, -1)
        return t.transpose(1, 2) if self.head_first_dim else t

    # One kernel normalises the whole fused projection instead of five RMSNorm modules plus casts
    # (CUDA tensors only; set to False to run the norms as separate torch modules, as the reference does).
    fused_head_norm = True
    # The backward of that kernel keeps one fp32 partial row of the gain gradient per warp in shared
    # memory (8 warps x channels x 4 bytes <= 200 KB); wider projections use the separate modules.
    fused_head_norm_max_channels = 6400

    def _fused_norm(self, proj):
        """Per-head RMSNorm of the packed projection with the gains of q_norm / k_norms / v_norms tiled to
        one entry per channel; same arithmetic as the modules, applied before the split."""
        import torch

        from .headnorm import head_rmsnorm
        kw = torch.cat([n.weight for n in self.k_norms]).repeat(self.key_value_heads)
        vw = torch.cat([n.weight for n in self.v_norms]).repeat(self.key_value_heads)
        weight = torch.cat((self.q_norm.weight.repeat(self.heads), kw, vw))
        autocast = torch.is_autocast_enabled()
        # the modules leave eps unset: the machine epsilon of the dtype they compute in (fp32 under autocast)
        eps = self.q_norm.eps if self.q_norm.eps is not None else \
            torch.finfo(torch.float32 if autocast else proj.dtype).eps
        out_dtype = torch.get_autocast_dtype("cuda") if autocast else proj.dtype
        return head_rmsnorm(proj, weight, self.dim_head, eps, out_dtype)

    def _project(self, tokens):
        """tokens -> (queries, keys, values) after the head split and the per-head norms."""
        tokens = self.prenorm(tokens)
        proj = self.to_qkv(tokens)
        fused = (self.fused_head_norm and self.qk_rmsnorm and proj.is_cuda and not self.head_first_dim
                 and self.dim_head_values == self.dim_head and self.dim_head in (32, 64, 128)
                 and proj.shape[-1] <= self.fused_head_norm_max_channels
                 and proj.dtype in (torch.float32, torch.bfloat16))
        if fused:
            q, k, v = self._fused_norm(proj).split(self.split_dims, dim=-1)
            queries = self._split(q, self.heads)
            keys = self._split(k, self.key_value_heads).chunk(self.kv_sets, dim=-1)
            values = self._split(v, self.key_value_heads).chunk(self.kv_sets, dim=-1)
            return queries, keys, values
        q, k, v = proj.split(self.split_dims, dim=-1)

        queries = self._split(q, self.heads)
        # each kv head's slice holds its key sets side by side: [k1 | k2]
        keys = self._split(k, self.key_value_heads).chunk(self.kv_sets, dim=-1)
        values = self._split(v, self.key_value_heads).chunk(self.kv_sets, dim=-1)

        if self.qk_rmsnorm:
            queries = self.q_norm(queries)
            keys = tuple(norm(t) for norm, t in zip(self.k_norms, keys))
            values = tuple(norm(t) for norm, t in zip(self.v_norms, values))
        return queries, keys, values

    def _merge(self, out):
        if self.head_first_dim:
            out = out.transpose(1, 2)
        out = out.reshape(out.shape[0], out.shape[1], -1)
        return self.postnorm(self.combine_heads(out))

    def forward(self, tokens):
        queries, keys, values = self._project(tokens)
        return self._merge(self.attend(queries, keys, values))


class SlidingWindowTwoSimplicialMHA(HigherOrderAttention):
    def __init__(self, *args, w1=512, w2=32, **kwargs):
        assert "number_key_value_sets" not in kwargs
        assert "head_first_dim" not in kwargs
        # the kernels contract q, k, k' and aggregate v, v' over one head dimension; say so at construction
        # instead of failing at the first forward (the reference accepts the argument, simplicial_mha.py:34,
        # and then fails inside its kernels, which read values with the key head dim)
        dim_head = kwargs.get("dim_head", args[2] if len(args) > 2 else 64)
        dim_head_values = kwargs.get("dim_head_values", args[3] if len(args) > 3 else None)
        if dim_head_values is not None and dim_head_values != dim_head:
            raise ValueError(f"dim_head_values ({dim_head_values}) must equal dim_head ({dim_head}) for the "
                             "sliding-window 2-simplicial kernels")
        attend = partial(sliding_two_simplicial_attn, w1=w1, w2=w2, causal=True)
        super().__init__(*args, number_key_value_sets=2, head_first_dim=False, attend=attend, **kwargs)
        self.w1, self.w2 = w1, w2

    def forward(self, tokens, cache=None, return_cache=False):
        """``cache`` (from an earlier call with ``return_cache=True``) holds the last ``w1 - 1`` rows of the
        first key/value set and the last ``w2 - 1`` rows of the second: all a later token can still see.
        With a cache, ``tokens`` are only the new positions; the cached rows ride in front of the new keys
        as the halo the kernels already understand, so decoding a token costs one window, not the prefix
        (the reference's sampling loop re-runs the whole prefix for every token, train.py:103-104)."""
        queries, keys, values = self._project(tokens)
        if cache is not None:
            keys = tuple(torch.cat((c, t), dim=1) for c, t in zip(cache[0], keys))
            values = tuple(torch.cat((c, t), dim=1) for c, t in zip(cache[1], values))
        out = self._merge(self.attend(queries, keys, values))
        if not return_cache:
            return out
        keep = (self.w1 - 1, self.w2 - 1)
        new_cache = (tuple(t[:, t.shape[1] - min(k, t.shape[1]):].detach() for t, k in zip(keys, keep)),
                     tuple(t[:, t.shape[1] - min(k, t.shape[1]):].detach() for t, k in zip(values, keep)))
        return out, new_cache
