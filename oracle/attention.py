"""Dense reference for bidirectional varlen attention over a slot-mapped cache.

reference: nano-vdllm/tests/test_attention_kernels.py:88-109 (dense fp32 softmax
attention with GQA by head // group) and :262-289 (gather of K/V rows through the
flat slot map); relocation variants restate nano-vdllm/model/acache_attention.py:
399-419,428-448 (query side) and :480-497 (key side).
"""
import torch

from .rope import apply_rope, apply_rope_inverse


def dense_attention(q, k, v, num_heads, num_kv_heads, scale=None):
    """q [nq, nh, D], k/v [nk, Hkv, D] -> [nq, nh, D] in q.dtype; fp32 math."""
    g = num_heads // num_kv_heads
    qf, kf, vf = q.float(), k.float(), v.float()
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    out = torch.empty_like(qf)
    for h in range(num_heads):
        s = (qf[:, h] @ kf[:, h // g].T) * scale
        out[:, h] = torch.softmax(s, dim=-1) @ vf[:, h // g]
    return out.to(q.dtype)


def acache_attention(
    q,
    k_cache,
    v_cache,
    cu_seqlens_q,
    cu_seqlens_k,
    read_slot_mapping,
    softmax_scale=None,
    shared_prefix_len=0,
    shared_kv_lens=None,
    affix_shifts=None,
    rope_cos=None,
    rope_sin=None,
):
    """Same signature as the reference operator (acache_attention.py:643-656).
    k_cache/v_cache [num_blocks, Bk, Hkv, D], addressed flat by slot."""
    nh, D = q.shape[1], q.shape[2]
    Hkv = k_cache.shape[-2]
    g = nh // Hkv
    flat_k = k_cache.reshape(-1, Hkv, D)
    flat_v = v_cache.reshape(-1, Hkv, D)
    scale = D ** -0.5 if softmax_scale is None else softmax_scale
    relocate = shared_prefix_len > 0 and affix_shifts is not None
    query_side = relocate and shared_kv_lens is not None
    out = torch.empty_like(q)
    B = cu_seqlens_q.numel() - 1
    for b in range(B):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        k0, k1 = int(cu_seqlens_k[b]), int(cu_seqlens_k[b + 1])
        if q1 == q0:
            continue
        if k1 <= k0:
            out[q0:q1] = 0
            continue
        slots = read_slot_mapping[k0:k1].long()
        # extension over the reference: an entry of -1 is a hole, a key that takes no part
        # (used to read the shared span as one contiguous run with the anchors punched out)
        live = slots >= 0
        slots = slots.clamp(min=0)
        k = flat_k[slots]
        v = flat_v[slots]
        qb = q[q0:q1]
        if relocate and not query_side:
            # key side: keys living in the shared span are rotated by (logical index - slot)
            idx = torch.arange(k1 - k0)
            delta = idx - slots
            shared = slots < shared_prefix_len
            # only shared keys look the table up (the reference masks the load)
            row = torch.where(shared, delta.abs(), torch.zeros_like(delta))
            cos = rope_cos[row]
            sin = rope_sin[row]
            sin = torch.where((delta < 0).unsqueeze(-1), -sin, sin)
            rotated = apply_rope(k, cos, sin)
            k = torch.where(shared.view(-1, 1, 1), rotated, k)
            sf = (qb.float().permute(1, 0, 2) @ k.float().permute(1, 2, 0).repeat_interleave(g, dim=0)) * scale
        elif query_side:
            n_sh = int(shared_kv_lens[b])
            s = int(affix_shifts[b])
            A_ = qb.shape[0]
            q_sh = apply_rope_inverse(qb, rope_cos[s].expand(A_, -1), rope_sin[s].expand(A_, -1))
            kf = k.float().permute(1, 2, 0).repeat_interleave(g, dim=0)
            s_sh = q_sh.float().permute(1, 0, 2) @ kf[:, :, :n_sh]
            s_pr = qb.float().permute(1, 0, 2) @ kf[:, :, n_sh:]
            sf = torch.cat((s_sh, s_pr), dim=-1) * scale
        else:
            sf = (qb.float().permute(1, 0, 2) @ k.float().permute(1, 2, 0).repeat_interleave(g, dim=0)) * scale
        sf = sf.masked_fill(~live.view(1, 1, -1), float("-inf"))
        w = torch.nan_to_num(torch.softmax(sf, dim=-1), nan=0.0)  # no live key: zeros
        o = w @ v.float().permute(1, 0, 2).repeat_interleave(g, dim=0)
        out[q0:q1] = o.permute(1, 0, 2).to(q.dtype)
    return out


def block_table_slots(block_table_row, length, block_size):
    pos = torch.arange(length)
    return block_table_row.long()[pos // block_size] * block_size + pos % block_size


def baseline_ragged_attention(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, softmax_scale=None):
    """reference: nano-vdllm/model/acache_attention.py:132-233,525-582."""
    Bk = k_cache.shape[1]
    maps = []
    for b in range(cu_seqlens_q.numel() - 1):
        n = int(cu_seqlens_k[b + 1]) - int(cu_seqlens_k[b])
        maps.append(block_table_slots(block_tables[b], n, Bk))
    rsm = torch.cat(maps).to(torch.int32)
    return acache_attention(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, rsm, softmax_scale)


def baseline_decode_attention(q, k_cache, v_cache, seqlens, block_tables, softmax_scale=None):
    """q [B, T, nh, D]; reference: nano-vdllm/model/acache_attention.py:237-334,585-640."""
    B, T = q.shape[:2]
    cu_q = torch.arange(0, (B + 1) * T, T, dtype=torch.int32)
    cu_k = torch.zeros(B + 1, dtype=torch.int32)
    cu_k[1:] = torch.cumsum(seqlens.to(torch.int32), 0)
    out = baseline_ragged_attention(q.reshape(B * T, *q.shape[2:]), k_cache, v_cache, cu_q, cu_k, block_tables, softmax_scale)
    return out.view_as(q)
