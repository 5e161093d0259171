"""Decoder stack and language-model wrapper around the sliding-window
2-simplicial attention module: the harness for the training-step configuration
(8 layers, dim 512, every 2nd layer simplicial, byte vocabulary).

Restates, in plain PyTorch, ``TwoSimplicialTransformer`` / ``Attention`` /
``FeedForward`` (simplicial_attention/two_simplicial_transformer.py:25-141) and
the ``TwoSimplicialLM`` wrapper of the reference's example script
(train.py:64-135; the script itself runs its training loop at import and needs
a dataset blob that is not shipped).  Parameter names match the reference, so
its checkpoints load.  Only the simplicial layers run our kernels; the standard
layers use torch's scaled-dot-product attention, as in the reference.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import Module, ModuleList

from .attention import divisible_by
from .mha import SlidingWindowTwoSimplicialMHA


class Attention(Module):
    """Pre-norm causal grouped-query attention (two_simplicial_transformer.py:25-65)."""

    def __init__(self, dim, dim_head=64, heads=8, key_value_heads=8):
        super().__init__()
        assert divisible_by(heads, key_value_heads)
        self.heads, self.key_value_heads, self.dim_head = heads, key_value_heads, dim_head
        self.prenorm = nn.RMSNorm(dim)
        self.to_q = nn.Linear(dim, heads * dim_head, bias=False)
        self.to_kv = nn.Linear(dim, key_value_heads * dim_head * 2, bias=False)
        self.to_out = nn.Linear(heads * dim_head, dim, bias=False)

    def forward(self, x):
        b, n, _ = x.shape
        x = self.prenorm(x)
        q = self.to_q(x).view(b, n, self.heads, self.dim_head).transpose(1, 2)
        # the fused projection is laid out (kv, h, d), as in the reference's rearrange
        kv = self.to_kv(x).view(b, n, 2, self.key_value_heads, self.dim_head)
        k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.heads != self.key_value_heads)
        return self.to_out(out.transpose(1, 2).reshape(b, n, -1))


def FeedForward(dim, expansion=4.0):
    inner = int(dim * expansion)
    return nn.Sequential(nn.RMSNorm(dim), nn.Linear(dim, inner), nn.GELU(), nn.Linear(inner, dim))


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
        self.norm = nn.RMSNorm(dim) if final_norm else nn.Identity()

    def forward(self, x):
        for attn, ff in self.layers:
            x = attn(x) + x
            x = ff(x) + x
        return self.norm(x)


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

    def forward(self, x, return_loss=False):
        if return_loss:
            x, target = x[:, :-1], x[:, 1:]
        n = x.shape[-1]
        tokens = self.token_emb(x) + self.pos_emb(torch.arange(n, device=x.device))
        logits = self.to_logits(self.transformer(tokens))
        if not return_loss:
            return logits
        return F.cross_entropy(logits.transpose(1, 2), target)


def training_step(model: Module, optimizer: torch.optim.Optimizer, tokens: torch.Tensor, max_grad_norm=0.5) -> torch.Tensor:
    """One step of the reference's loop (train.py:179-194, without gradient accumulation):
    loss, backward, clip to 0.5, Adam step.  Returns the loss tensor (no host sync)."""
    loss = model(tokens, return_loss=True)
    loss.backward()
    torch.nn.utils.clip_grad_norm_(model.parameters(), max_grad_norm)
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return loss
