"""B200-native sliding-window causal 2-simplicial attention (forward + backward).

Drop-in for the sliding path of lucidrains/simplicial-attention:
``SlidingWindowTwoSimplicialMHA``, ``sliding_two_simplicial_attn`` and
``SlidingTwoSimplicialAttention`` keep the reference's signatures and run on
hand-written sm_100a CUDA kernels behind the C ABI of ``include/sa2.h``.
"""
from .attention import (
    BackwardCall,
    SlidingTwoSimplicialAttention,
    check_device,
    device_status,
    sa2_backward,
    sa2_forward,
    sliding_two_simplicial_attn,
    sliding_two_simplicial_attn_with_lse,
)
from .host import HostPipeline
from .mha import HigherOrderAttention, SlidingWindowTwoSimplicialMHA

__all__ = [
    "SlidingTwoSimplicialAttention",
    "sliding_two_simplicial_attn",
    "sliding_two_simplicial_attn_with_lse",
    "sa2_forward",
    "sa2_backward",
    "device_status",
    "check_device",
    "BackwardCall",
    "HostPipeline",
    "HigherOrderAttention",
    "SlidingWindowTwoSimplicialMHA",
]
