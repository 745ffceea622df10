"""Per-affix-token influence score of one layer.

reference: nano-vdllm/model_runner.py:730-773 (nano engine) and
llada/generate_ACache.py:139-183 (HF path): re-rotate the cached post-RoPE affix
keys by R(affix_start), repeat KV heads for GQA, scores = Q_mask K^T * scale,
softmax over the affix only, sum over mask queries then heads, accumulate in fp32.
"""
import torch

from .rope import apply_rope


def relocate_keys(cached_affix_k, rope_cos, rope_sin, affix_start):
    """cached_affix_k [A, Hkv, D] rotated by the single angle row affix_start."""
    A = cached_affix_k.shape[0]
    return apply_rope(cached_affix_k, rope_cos[affix_start].expand(A, -1), rope_sin[affix_start].expand(A, -1))


def layer_importance(q_mask, affix_k, scale, exact=False):
    """q_mask [n_q, nh, D] (rows of mask tokens only, post-RoPE);
    affix_k [A, Hkv, D] (already relocated).  Returns fp32 [A].

    exact=False follows the reference's dtype flow (matmul, scale, softmax and
    the two sums all produce the activation dtype, then .float()).
    exact=True computes everything in fp64 and returns fp32: the value a fused
    kernel with fp32 accumulation approximates."""
    nh = q_mask.shape[1]
    groups = nh // affix_k.shape[1]
    k = affix_k.permute(1, 0, 2)
    if groups > 1:
        k = k.repeat_interleave(groups, dim=0)
    q = q_mask.permute(1, 0, 2)
    if exact:
        q, k = q.double(), k.double()
    s = torch.matmul(q, k.transpose(-2, -1)) * scale
    w = torch.softmax(s, dim=-1)
    return w.sum(dim=-2).sum(dim=-2).float()
