"""Decoder stack and language-model wrapper around the sliding-window
2-simplicial attention module: the harness for the training-step configuration
(8 layers, dim 512, every 2nd layer simplicial, byte vocabulary).

Restates, in plain PyTorch, ``TwoSimplicialTransformer`` / ``Attention`` /
``FeedForward`` (simplicial_attention/two_simplicial_transformer.py:25-141) and
the ``TwoSimplicialLM`` wrapper of the reference's example script
(train.py:64-135; the script itself runs its training loop at import and needs
a dataset blob that is not shipped).  Parameter names match the reference, so
its checkpoints load.  Only the simplicial layers run our kernels; the standard
layers use torch's scaled-dot-product attention, as in the reference; the RMSNorm modules are
``headnorm.RMSNorm`` (same parameter, fused CUDA kernel).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import Module, ModuleList

from .attention import divisible_by
from .headnorm import RMSNorm
from .mha import SlidingWindowTwoSimplicialMHA


class Attention(Module):
    """Pre-norm causal grouped-query attention (two_simplicial_transformer.py:25-65)."""

    def __init__(self, dim, dim_head=64, heads=8, key_value_heads=8):
        super().__init__()
        assert divisible_by(heads, key_value_heads)
        self.heads, self.key_value_heads, self.dim_head = heads, key_value_heads, dim_head
        self.prenorm = RMSNorm(dim)
        self.to_q = nn.Linear(dim, heads * dim_head, bias=False)
        self.to_kv = nn.Linear(dim, key_value_heads * dim_head * 2, bias=False)
        self.to_out = nn.Linear(heads * dim_head, dim, bias=False)

    def forward(self, x, cache=None, return_cache=False):
        """``cache`` = (keys, values) of every earlier position; with a cache ``x`` is one new position."""
        b, n, _ = x.shape
        x = self.prenorm(x)
        q = self.to_q(x).view(b, n, self.heads, self.dim_head).transpose(1, 2)
        # the fused projection is laid out (kv, h, d), as in the reference's rearrange
        kv = self.to_kv(x).view(b, n, 2, self.key_value_heads, self.dim_head)
        k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
        if cache is not None:
            assert n == 1, "with a cache, feed one new position at a time"
            k, v = torch.cat((cache[0], k), dim=2), torch.cat((cache[1], v), dim=2)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=cache is None, enable_gqa=self.heads != self.key_value_heads)
        out = self.to_out(out.transpose(1, 2).reshape(b, n, -1))
        return (out, (k.detach(), v.detach())) if return_cache else out


def FeedForward(dim, expansion=4.0):
    inner = int(dim * expansion)
    return nn.Sequential(RMSNorm(dim), nn.Linear(dim, inner), nn.GELU(), nn.Linear(inner, dim))


class TwoSimplicialTransformer(Module):
    def __init__(self, dim, *, depth, heads=8, key_value_heads=4, dim_head=64, ff_expansion=4.0,
                 two_simplicial_attn_every=4, attn_kwargs: dict = dict(),
                 two_simplicial_attn_kwargs: dict = dict(w1=512, w2=32, qk_rmsnorm=True), final_norm=True):
        super().__init__()
        layers = []
        for index in range(depth):
            if divisible_by(index + 1, two_simplicial_attn_every):
                attn = SlidingWindowTwoSimplicialMHA(dim=dim, heads=heads, key_value_heads=key_value_heads,
                                                     dim_head=dim_head, prenorm=True, **two_simplicial_attn_kwargs)
            else:
                attn = Attention(dim=dim, heads=heads, key_value_heads=key_value_heads, dim_head=dim_head, **attn_kwargs)
            layers.append(ModuleList([attn, FeedForward(dim=dim, expansion=ff_expansion)]))
        self.layers = ModuleList(layers)
        self.norm = RMSNorm(dim) if final_norm else nn.Identity()

    def forward(self, x, cache=None, return_cache=False):
        """``cache``: one entry per layer, as returned by an earlier call with ``return_cache=True``."""
        if cache is None and not return_cache:
            for attn, ff in self.layers:
                x = attn(x) + x
                x = ff(x) + x
            return self.norm(x)
        new_cache = []
        for index, (attn, ff) in enumerate(self.layers):
            a, c = attn(x, cache=None if cache is None else cache[index], return_cache=True)
            new_cache.append(c)
            x = a + x
            x = ff(x) + x
        return self.norm(x), new_cache


class TwoSimplicialLM(Module):
    """Token + learned absolute position embedding, the decoder stack, a linear head
    (train.py:64-135).  ``forward(x, return_loss=True)`` takes ``(b, n + 1)`` token ids and
    returns the next-token cross entropy."""

    def __init__(self, *, num_tokens, dim, depth, max_seq_len=1024, dim_head=64, heads=8,
                 two_simplicial_attn_every=4, transformer_kwargs=dict()):
        super().__init__()
        self.token_emb = nn.Embedding(num_tokens, dim)
        self.pos_emb = nn.Embedding(max_seq_len, dim)
        self.transformer = TwoSimplicialTransformer(dim=dim, depth=depth, dim_head=dim_head, heads=heads,
                                                    two_simplicial_attn_every=two_simplicial_attn_every,
                                                    **transformer_kwargs)
        self.to_logits = nn.Linear(dim, num_tokens, bias=False)

    def forward(self, x, return_loss=False, cache=None, return_cache=False):
        if return_loss:
            x, target = x[:, :-1], x[:, 1:]
        n = x.shape[-1]
        start = 0 if cache is None else cache["length"]
        tokens = self.token_emb(x) + self.pos_emb(torch.arange(start, start + n, device=x.device))
        if cache is None and not return_cache:
            logits = self.to_logits(self.transformer(tokens))
        else:
            embed, layers = self.transformer(tokens, cache=None if cache is None else cache["layers"], return_cache=True)
            logits = self.to_logits(embed)
            return logits, {"length": start + n, "layers": layers}
        if not return_loss:
            return logits
        return F.cross_entropy(logits.transpose(1, 2), target)

    @torch.no_grad()
    def sample(self, prompt: torch.Tensor, seq_len: int, temperature=1.0, filter_thres=0.9, use_cache=True):
        """Same contract as the reference's ``sample`` (train.py:92-111): top-k filtered Gumbel sampling
        until ``seq_len`` tokens, returning only the generated part.  With ``use_cache`` the prompt is run
        once and every further token costs one position: the standard layers keep their keys and values,
        the simplicial layers only their ``w1 - 1`` / ``w2 - 1`` row windows."""
        out = prompt.clone()
        steps = max(0, seq_len - prompt.shape[-1])
        cache = None
        for step in range(steps):
            if not use_cache:
                logits = self.forward(out)
            elif cache is None:
                logits, cache = self.forward(out, return_cache=True)
            else:
                logits, cache = self.forward(out[:, -1:], cache=cache, return_cache=True)
            logits = logits[:, -1].float()
            k = max(1, math.ceil((1 - filter_thres) * logits.shape[-1]))
            val, ind = torch.topk(logits, k)
            kept = torch.full_like(logits, float("-inf")).scatter_(-1, ind, val)
            noise = -torch.log(-torch.log(torch.rand_like(kept).clamp_min(1e-20)).clamp_min(1e-20))
            nxt = (kept / max(temperature, 1e-10) + noise).argmax(dim=-1, keepdim=True)
            out = torch.cat((out, nxt), dim=-1)
        return out[..., prompt.shape[-1]:]


def training_step(model: Module, optimizer: torch.optim.Optimizer, tokens: torch.Tensor, max_grad_norm=0.5) -> torch.Tensor:
    """One step of the reference's loop (train.py:179-194, without gradient accumulation):
    loss, backward, clip to 0.5, Adam step.  Returns the loss tensor (no host sync)."""
    loss = model(tokens, return_loss=True)
    loss.backward()
    torch.nn.utils.clip_grad_norm_(model.parameters(), max_grad_norm)
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return loss
