"""Paged-cache scatter and affix relocation.

store_kvcache: reference nano-vdllm/model/attention.py:11-41.
materialize_relocated_affix: reference nano-vdllm/model/acache_attention.py:7-128
(K' = K*cos[s] + rotate_half(K)*sin[s], V' = V, source slots 0..A-1).
"""
import torch

from .rope import apply_rope


def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """key/value [N, Hkv, D]; caches [num_blocks, Bk, Hkv, D] addressed flat;
    slot -1 is skipped.  In place."""
    flat_k = k_cache.view(-1, *k_cache.shape[-2:])
    flat_v = v_cache.view(-1, *v_cache.shape[-2:])
    slots = slot_mapping.long()
    keep = slots >= 0
    flat_k[slots[keep]] = key[keep]
    flat_v[slots[keep]] = value[keep]


def materialize_relocated_affix(k_cache, v_cache, rope_cos, rope_sin, dst_slot, affix_len, affix_shift):
    """k_cache/v_cache [L, slots, Hkv, D].  In place; the source span is read
    completely before anything is written, like a kernel whose source and
    destination do not overlap."""
    L = k_cache.shape[0]
    src_k = k_cache[:, :affix_len].clone()
    src_v = v_cache[:, :affix_len].clone()
    cos = rope_cos[affix_shift].expand(L * affix_len, -1)
    sin = rope_sin[affix_shift].expand(L * affix_len, -1)
    new_k = apply_rope(src_k.reshape(L * affix_len, *k_cache.shape[-2:]), cos, sin).view_as(src_k)
    k_cache[:, dst_slot : dst_slot + affix_len] = new_k
    v_cache[:, dst_slot : dst_slot + affix_len] = src_v


def relocate_affix_batched(k_cache, v_cache, rope_cos, rope_sin, dst_block_tables, shifts, affix_len, block_size):
    """Batched form: request r gets the affix relocated by shifts[r] into the
    blocks dst_block_tables[r] (token t -> slot table[t // Bk] * Bk + t % Bk).
    Same arithmetic as the single form, once per request."""
    L = k_cache.shape[0]
    src_k = k_cache[:, :affix_len].clone()
    src_v = v_cache[:, :affix_len].clone()
    t = torch.arange(affix_len)
    for table, shift in zip(dst_block_tables, shifts):
        table = torch.as_tensor(table, dtype=torch.long)
        dst = table[t // block_size] * block_size + t % block_size
        cos = rope_cos[int(shift)].expand(L * affix_len, -1)
        sin = rope_sin[int(shift)].expand(L * affix_len, -1)
        new_k = apply_rope(src_k.reshape(L * affix_len, *k_cache.shape[-2:]), cos, sin).view_as(src_k)
        k_cache[:, dst] = new_k
        v_cache[:, dst] = src_v
