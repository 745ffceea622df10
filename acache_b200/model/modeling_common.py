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


# The projection of q/k/v, the rotary embedding and the K/V scatter can run as one tcgen05 GEMM
# with a fused epilogue (16-bit, head_dim 128).  Measured on B200 it is slower than the library
# GEMM followed by the RoPE + scatter kernel (84 us against 54 us for 512 x 4096 x 12288: with
# 128 x 128 tiles it is bound by L2 -> SM traffic), so it is off unless switched on here.
FUSED_QKV = False


def project_qkv(h, w_qkv, b_qkv, n_heads, n_kv_heads, head_dim, position_ids, cos, sin, attn, ctx):
    """Returns ``(q, k, v)`` views for the attention call; with the fused path ``k``/``v`` are
    ``None`` because they only exist in the paged cache."""
    import torch.nn.functional as F

    n = h.shape[0]
    D, nh, hkv = head_dim, n_heads, n_kv_heads
    caching = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None
    if (FUSED_QKV and caching and D == 128 and h.dtype in (torch.bfloat16, torch.float16) and h.shape[1] % 64 == 0
            and h.stride(0) % 8 == 0):
        q = ops.qkv_rope_scatter(h, w_qkv, b_qkv, nh, hkv, D, position_ids, cos, sin, attn.k_cache, attn.v_cache,
                                 ctx.slot_mapping)
        attn.kv_already_stored = True
        return q, None, None
    qkv = F.linear(h, w_qkv, b_qkv)
    q, k, v = qkv[:, : nh * D], qkv[:, nh * D: (nh + hkv) * D], qkv[:, (nh + hkv) * D:]
    q, k, v = q.view(n, nh, D), k.view(n, hkv, D), v.view(n, hkv, D)
    if caching:
        ops.rope_store(q, k, v, position_ids, cos, sin, attn.k_cache, attn.v_cache, ctx.slot_mapping)
        attn.kv_already_stored = True
    else:
        ops.rope_store(q, k, None, position_ids, cos, sin)
        attn.kv_already_stored = False
    return q, k, v


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
