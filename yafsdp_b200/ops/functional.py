"""Autograd-level ops of the Llama training step.

Every op has two implementations selected by the device of its inputs: the hand-written sm_100a
kernels (:mod:`yafsdp_b200.ops.kernels`) for CUDA tensors and plain PyTorch math for CPU tensors
(used by the gloo plumbing tests).  On a CUDA device the native path is the only one: there is no
fallback to library kernels.
"""

from __future__ import annotations

import torch


def rope_table(seq_len: int, head_dim: int, theta: float, device: torch.device | str) -> torch.Tensor:
    """``[seq_len, head_dim/2, 2]`` fp32 table of (cos, sin) for the rotate-half RoPE convention."""
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim))
    ang = torch.arange(seq_len, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()
