"""Anchor top-k with a defined tie rule.

reference: nano-vdllm/model_runner.py:833-843 and llada/generate_ACache.py:225-262
(topk over the per-affix-token score, largest unless selection_mode == 'bottom',
then the chosen indices sorted ascending).  torch.topk leaves the order among
equal scores unspecified; the contract here is stricter: among equal scores the
lowest index wins.  NaN never occurs in a softmax sum; it is ordered like
torch.topk does (NaN counts as the largest value).
"""
import numpy as np
import torch


def anchor_topk(scores: torch.Tensor, k: int, largest: bool = True) -> torch.Tensor:
    """scores [B, A] fp32 -> int64 [B, k], ascending indices."""
    s = scores.detach().cpu().numpy().astype(np.float32)
    B, A = s.shape
    k = min(int(k), A)
    out = np.empty((B, k), dtype=np.int64)
    for b in range(B):
        key = s[b].copy()
        if largest:
            key = np.where(np.isnan(key), np.float32(np.inf), key)
            order = np.argsort(-key, kind="stable")
        else:
            key = np.where(np.isnan(key), np.float32(np.inf), key)
            order = np.argsort(key, kind="stable")
        out[b] = np.sort(order[:k])
    return torch.from_numpy(out)
