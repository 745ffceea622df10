"""Pieces shared by the two served architectures: RoPE tables, the fused
projection + RoPE + K/V scatter step, and the block-level kernels."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


def build_rope_table(length: int, head_dim: int, theta: float, dtype: torch.dtype, device) -> tuple[torch.Tensor, torch.Tensor]:
    """``(cos, sin)`` tables ``[length, head_dim]`` in the half-split layout
    ``cat(freqs, freqs)`` (reference: nano-vdllm/model/modeling_llada.py:392-402).
    Built once on the host in fp32 so that every device holds identical bits."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(length, dtype=torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype).to(device), emb.sin().to(dtype).to(device)


class RopeCache:
    """Grows on demand (reference: nano-vdllm/model/modeling_llada.py:373-402)."""

    def __init__(self, head_dim: int, theta: float, table_dtype: torch.dtype):
        self.head_dim, self.theta, self.table_dtype = head_dim, theta, table_dtype
        self.cos = self.sin = None

    def get(self, length: int, device):
        if self.cos is None or self.cos.shape[0] < length or self.cos.device != torch.device(device):
            n = max(int(length), 1)
            n = 1 << (n - 1).bit_length()  # power of two: few rebuilds
            self.cos, self.sin = build_rope_table(n, self.head_dim, self.theta, self.table_dtype, device)
        return self.cos, self.sin


class RMSNorm(nn.Module):
    def __init__(self, size: int, eps: float, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x, delta=None):
        """``delta`` (optional): a residual update that is added to ``x`` IN PLACE before the
        normalisation (one fused kernel)."""
        if delta is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        if x.shape[-1] % (16 // x.element_size()) != 0 or x.shape[-1] > 1024 * (16 // x.element_size()):
            x.add_(delta)  # row shapes the fused kernel does not take
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps)
