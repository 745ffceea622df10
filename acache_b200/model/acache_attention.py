"""Attention and relocation operators over the paged KV cache.

Same callables, argument order and tensor conventions as the reference operator
module (reference: nano-vdllm/model/acache_attention.py:88-128 materialise,
:525-582 ragged, :585-640 decode, :643-738 slot-map attention), executed by the
sm_100a kernels behind the C ABI.  Metadata tensors are int32 on the device.

Differences a caller can see:
* ``max_seqlen_q`` may be passed to avoid the device synchronisation the
  reference does to find it; when omitted it is computed the same way.
* ``relocate_affix_batched`` is the batched form of ``materialize_relocated_affix``
  (all layers and all requests in one launch, per-request destination block tables
  and shifts); the single form is that call with one request.
"""
from __future__ import annotations

import torch

from .. import _lib
from .._lib import check, dtype_code, ptr, stream_ptr


# Set by the engine before a forward so that the optional device timers can attribute an
# attention launch to its phase and to its algorithmic work (bytes for decode, FLOPs for
# refresh).  They do not influence the computation.
ATTENTION_PHASE = "refresh"
ATTENTION_WORK = 0.0


def _require_cuda(*tensors):
    for t in tensors:
        assert t is None or t.is_cuda, "operator inputs must live on the GPU"


def _rope_args(rope_cos, rope_sin):
    if rope_cos is None:
        return None, None, 0, 0, _lib.F32
    assert rope_cos.dim() == 2 and rope_sin.shape == rope_cos.shape
    assert rope_cos.stride(1) == 1 and rope_sin.stride(1) == 1 and rope_sin.stride(0) == rope_cos.stride(0)
    assert rope_sin.dtype == rope_cos.dtype
    return ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0], dtype_code(rope_cos.dtype)


def materialize_relocated_affix(k_cache, v_cache, rope_cos, rope_sin, dst_slot: int, affix_len: int, affix_shift: int):
    """k_cache/v_cache ``[L, slots, Hkv, D]``; in place (reference: acache_attention.py:88-128)."""
    dev = k_cache.device
    shifts = torch.tensor([int(affix_shift)], dtype=torch.int32, device=dev)
    dst = torch.tensor([int(dst_slot)], dtype=torch.int32, device=dev)
    relocate_affix_batched(k_cache, v_cache, rope_cos, rope_sin, affix_len, shifts, dst_slots=dst)


def relocate_affix_batched(k_cache, v_cache, rope_cos, rope_sin, affix_len: int, shifts, *, dst_slots=None,
                           dst_block_tables=None, block_size: int = 0):
    """Relocate the shared affix (slots ``0..affix_len-1`` of every layer) for
    ``len(shifts)`` requests in one launch.  ``dst_slots`` int32 ``[R]`` gives one
    contiguous destination per request, or ``dst_block_tables`` int32 ``[R, nb]``
    (+ ``block_size``) scatters token t to ``table[t // block_size] * block_size +
    t % block_size``."""
    assert k_cache.dim() == 4 and v_cache.shape == k_cache.shape
    _require_cuda(k_cache, v_cache, rope_cos, rope_sin, shifts, dst_slots, dst_block_tables)
    assert k_cache.stride(-1) == 1 and k_cache.stride(2) == k_cache.shape[3]
    assert k_cache.stride(1) == k_cache.shape[2] * k_cache.shape[3]
    assert v_cache.stride() == k_cache.stride()
    L, slots, hkv, D = k_cache.shape
    rc, rs, rstride, rrows, rdt = _rope_args(rope_cos, rope_sin)
    assert shifts.dtype == torch.int32 and shifts.is_contiguous()
    table_stride = 0
    if dst_block_tables is not None:
        assert dst_block_tables.dtype == torch.int32 and dst_block_tables.dim() == 2
        assert dst_block_tables.stride(1) == 1 and block_size > 0
        table_stride = dst_block_tables.stride(0)
    else:
        assert dst_slots is not None and dst_slots.dtype == torch.int32 and dst_slots.is_contiguous()
    flag = _lib.err_flag(k_cache.device)
    check(_lib.load().acache_relocate_affix(
        ptr(k_cache), ptr(v_cache), k_cache.stride(0), L, slots, hkv, D, dtype_code(k_cache.dtype), rc, rs, rstride,
        rrows, rdt, int(affix_len), shifts.numel(), ptr(shifts), ptr(dst_slots), ptr(dst_block_tables), table_stride,
        int(block_size), ptr(flag), stream_ptr()), "relocate_affix")


def _attention_call(q, out, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, max_q, max_k, softmax_scale, *,
                    read_slot_mapping=None, block_tables=None, shared_prefix_len=0, shared_kv_lens=None,
                    affix_shifts=None, rope_cos=None, rope_sin=None, group_shared_span=False):
    total_q, nh, D = q.shape
    hkv = k_cache.shape[-2]
    num_slots = k_cache.numel() // (hkv * D)
    batch = cu_seqlens_q.numel() - 1
    flag = _lib.err_flag(q.device)
    lib = _lib.load()
    if read_slot_mapping is not None:
        rc, rs, rstride, rrows, rdt = _rope_args(rope_cos, rope_sin)
        with _lib.timed("attention_decode" if ATTENTION_PHASE == "decode" else "attention_refresh", ATTENTION_WORK):
            if group_shared_span and shared_kv_lens is not None:
                status = lib.acache_attention_grouped(
                    ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_cache), ptr(v_cache), num_slots, nh, hkv, D,
                    dtype_code(q.dtype), ptr(cu_seqlens_q), ptr(cu_seqlens_k), batch, total_q, int(max_q),
                    ptr(read_slot_mapping), float(softmax_scale), int(shared_prefix_len), ptr(shared_kv_lens),
                    ptr(affix_shifts), rc, rs, rstride, rrows, rdt, None, 0, ptr(flag), stream_ptr())
                if status != _lib.ACACHE_EUNSUPPORTED:
                    check(status, "acache_attention_grouped")
                    return
            check(lib.acache_attention(
                ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_cache), ptr(v_cache), num_slots, nh, hkv, D,
                dtype_code(q.dtype), ptr(cu_seqlens_q), ptr(cu_seqlens_k), batch, int(max_q), int(max_k),
                ptr(read_slot_mapping), float(softmax_scale), int(shared_prefix_len), ptr(shared_kv_lens),
                ptr(affix_shifts), rc, rs, rstride, rrows, rdt, ptr(flag), stream_ptr()), "acache_attention")
    else:
        check(lib.acache_paged_attention(
            ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_cache), ptr(v_cache), num_slots, nh, hkv, D,
            dtype_code(q.dtype), ptr(cu_seqlens_q), ptr(cu_seqlens_k), batch, int(max_q), int(max_k),
            ptr(block_tables), block_tables.stride(0), k_cache.shape[1], float(softmax_scale), ptr(flag),
            stream_ptr()), "paged_attention")


def reset_grouped_scratch():
    """Kept for callers of the earlier two-part kernel, which held tickets in a scratch buffer;
    the grouped kernel keeps nothing between calls, so there is nothing to reset."""


def _check_qkv(q, k_cache, v_cache):
    assert q.dim() == 3
    _require_cuda(q, k_cache, v_cache)
    assert q.stride(-1) == 1 and q.stride(1) == q.shape[2]
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.dtype == q.dtype and v_cache.dtype == q.dtype


def _max_len(cu):
    return int((cu[1:] - cu[:-1]).max().item())


def acache_attention(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, read_slot_mapping, softmax_scale=None,
                     shared_prefix_len: int = 0, shared_kv_lens=None, affix_shifts=None, rope_cos=None, rope_sin=None,
                     *, max_seqlen_q: int | None = None, max_seqlen_k: int | None = None,
                     group_shared_span: bool = False):
    """Bidirectional varlen attention through a flat slot map (reference:
    acache_attention.py:643-738).  An entry of -1 in ``read_slot_mapping`` is a key that takes
    no part; ``shared_kv_lens`` without relocation only splits the keys into two runs.
    ``group_shared_span``: the caller guarantees that the first ``shared_kv_lens[b]`` entries of
    all requests name the same slots up to holes; block decode then serves four requests per CTA
    and stages that span once for the four (falls back to the plain kernel for shapes the grouped
    one declines)."""
    _check_qkv(q, k_cache, v_cache)
    _require_cuda(cu_seqlens_q, cu_seqlens_k, read_slot_mapping)
    batch = cu_seqlens_q.numel() - 1
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    apply_relocation = shared_prefix_len > 0 and affix_shifts is not None
    if apply_relocation and (rope_cos is None or rope_sin is None):
        raise ValueError("Post-RoPE affix relocation requires shifts and RoPE tables.")
    if (rope_cos is None) != (rope_sin is None):
        raise ValueError("rope_cos and rope_sin must be provided together.")
    if max_seqlen_q is None:
        max_seqlen_q = _max_len(cu_seqlens_q)
    if apply_relocation:
        assert affix_shifts.is_cuda and affix_shifts.numel() == batch and affix_shifts.dtype == torch.int32
        assert rope_cos.shape[1] == q.shape[-1]
        if max_seqlen_k is None:
            max_seqlen_k = _max_len(cu_seqlens_k)
        assert rope_cos.shape[0] >= max_seqlen_k
        if shared_kv_lens is not None:
            assert shared_kv_lens.is_cuda and shared_kv_lens.numel() == batch
    else:
        # shared_kv_lens alone stays: it only splits the keys into two separately tiled runs
        shared_prefix_len, affix_shifts, rope_cos, rope_sin = 0, None, None, None
    out = torch.empty_like(q)
    _attention_call(q, out, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k or 0,
                    softmax_scale, read_slot_mapping=read_slot_mapping, shared_prefix_len=shared_prefix_len,
                    shared_kv_lens=shared_kv_lens, affix_shifts=affix_shifts, rope_cos=rope_cos, rope_sin=rope_sin,
                    group_shared_span=group_shared_span)
    return out


def baseline_ragged_attention(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, softmax_scale=None, *,
                              max_seqlen_q: int | None = None):
    """Ragged queries, K/V through per-request block tables (reference: acache_attention.py:525-582)."""
    _check_qkv(q, k_cache, v_cache)
    assert block_tables is not None and block_tables.is_cuda and block_tables.dtype == torch.int32
    assert block_tables.stride(1) == 1
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    if max_seqlen_q is None:
        max_seqlen_q = _max_len(cu_seqlens_q)
    out = torch.empty_like(q)
    _attention_call(q, out, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, 0, softmax_scale,
                    block_tables=block_tables)
    return out


def baseline_decode_attention(q, k_cache, v_cache, seqlens, block_tables, softmax_scale=None):
    """Batched ``[B, T, nh, D]`` queries against paged K/V (reference: acache_attention.py:585-640)."""
    assert q.dim() == 4
    B, T, nh, D = q.shape
    q3 = q.reshape(B * T, nh, D)
    cu_q = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q.device)
    cu_k = torch.zeros(B + 1, dtype=torch.int32, device=q.device)
    cu_k[1:] = torch.cumsum(seqlens.to(torch.int32), 0)
    out = baseline_ragged_attention(q3, k_cache, v_cache, cu_q, cu_k, block_tables, softmax_scale, max_seqlen_q=T)
    return out.view(B, T, nh, D)
