"""K/V scatter and the attention module the model layers call.

reference: nano-vdllm/model/attention.py:34-41 (store_kvcache), :44-123 (Attention).
The module reads the step metadata from the process-global Context, writes this
step's K/V rows into the paged cache and attends through the slot map (affix
reuse) or the block tables (baseline).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _lib, ops
from .._lib import check, dtype_code, ptr, stream_ptr
from ..utils import get_context
from .acache_attention import acache_attention, baseline_decode_attention, baseline_ragged_attention


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor):
    """Scatter ``key/value [N, Hkv, D]`` rows into the flat paged cache at
    ``slot_mapping[i]`` (``-1`` skips the row)."""
    N, num_heads, head_dim = key.shape
    D = num_heads * head_dim
    assert key.is_cuda and value.is_cuda and k_cache.is_cuda and v_cache.is_cuda and slot_mapping.is_cuda
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == D and v_cache.stride(1) == D
    assert slot_mapping.numel() == N and slot_mapping.dtype == torch.int32
    assert key.dtype == k_cache.dtype and value.dtype == v_cache.dtype
    num_slots = k_cache.numel() // D
    flag = _lib.err_flag(key.device)
    check(_lib.load().acache_store_kvcache(
        ptr(key), key.stride(0), ptr(value), value.stride(0), ptr(k_cache), ptr(v_cache), ptr(slot_mapping), N, D,
        num_slots, dtype_code(key.dtype), ptr(flag), stream_ptr()), "store_kvcache")


class Attention(nn.Module):
    def __init__(self, num_heads, head_dim, num_kv_heads, scale=None):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.num_kv_heads = num_kv_heads
        self.scale = scale
        self.use_reference_attention = False  # accepted for interface parity; there is one attention path
        self.shared_prefix_len = 0
        self.relocation_rope_cos = self.relocation_rope_sin = torch.tensor([])
        self.k_cache = self.v_cache = torch.tensor([])
        # set by the model block: K/V of this step were already scattered by the fused RoPE+store kernel
        self.kv_already_stored = False
        # set by the engine during the anchor-selection probe: one entry per request of the batch
        self.probe = None
        # the same probes in the form of the batched score kernel (None: one request, or no mask rows)
        self.probe_batch = None

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        ctx = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        assert k_cache.numel() and v_cache.numel()
        batched = q.dim() == 4
        if batched:
            bs, seqlen = q.shape[:2]
            q = q.reshape(bs * seqlen, self.num_heads, self.head_dim)
            if k is not None:  # None: this step's K/V already sit in the cache (fused projection)
                k = k.reshape(bs * seqlen, self.num_kv_heads, self.head_dim)
                v = v.reshape(bs * seqlen, self.num_kv_heads, self.head_dim)
        if self.probe:
            # anchor-selection probe: add this layer's influence score of every affix token
            # (reference: nano-vdllm/model_runner.py:730-773)
            scale = self.scale if self.scale is not None else self.head_dim ** -0.5
            flat_k = k_cache.view(-1, self.num_kv_heads, self.head_dim)
            pb = self.probe_batch
            if pb is not None and pb.usable:   # all requests in one launch
                pb.usable = ops.anchor_importance_batched(q, pb.q_rows, pb.offsets, pb.max_q_rows, flat_k[: pb.affix_len],
                                                          pb.shifts, pb.rope_cos, pb.rope_sin, scale, pb.importance)
            if pb is None or not pb.usable:
                for p in self.probe:
                    ops.anchor_importance(q, p.q_rows, flat_k[: p.affix_len], p.affix_shift, p.rope_cos, p.rope_sin,
                                          scale, p.importance)
        if not self.kv_already_stored:
            store_kvcache(k, v, k_cache, v_cache, ctx.slot_mapping)
        if ctx.use_acache:
            relocating = self.shared_prefix_len > 0
            o = acache_attention(
                q, k_cache, v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.read_slot_mapping, self.scale,
                self.shared_prefix_len, ctx.shared_kv_lens, ctx.affix_shifts,
                self.relocation_rope_cos if relocating else None, self.relocation_rope_sin if relocating else None,
                max_seqlen_q=ctx.max_seqlen_q or None, max_seqlen_k=ctx.max_seqlen_k or None,
                group_shared_span=ctx.group_shared_span)
        elif ctx.is_caching:
            o = baseline_ragged_attention(q, k_cache, v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.block_tables,
                                          self.scale, max_seqlen_q=ctx.max_seqlen_q or None)
        else:
            o = baseline_decode_attention(q.view(bs, seqlen, self.num_heads, self.head_dim), k_cache, v_cache,
                                          ctx.seqlens, ctx.block_tables, self.scale)
            return o
        if batched:
            o = o.view(bs, seqlen, self.num_heads, self.head_dim)
        return o
