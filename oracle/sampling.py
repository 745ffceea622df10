"""Confidence-threshold unmasking.

reference: nano-vdllm/model_runner.py:2279-2314: x0 = argmax(logits); confidence
= exp(logit[x0] - logsumexp(float32(logits))); non-mask positions keep their
token and get confidence -inf; commit where confidence >= threshold; a row that
still has masks but committed nothing commits its most confident position.
"""
import torch


def get_transfer_index(logits, mask_index, x, threshold=0.9):
    """logits [B, T, V]; mask_index bool [B, T]; x int64 [B, T].  Temperature 0,
    'low_confidence' remasking.  Returns (x0 [B,T], transfer_index bool [B,T])."""
    x0 = torch.argmax(logits, dim=-1)
    lf = logits.float()
    chosen = torch.gather(lf, -1, x0.unsqueeze(-1)).squeeze(-1)
    p = torch.exp(chosen - torch.logsumexp(lf, dim=-1))
    x0 = torch.where(mask_index, x0, x)
    conf = torch.where(mask_index, p, torch.full_like(p, float("-inf")))
    transfer = (conf >= threshold) & mask_index
    needs = mask_index.any(dim=1) & ~transfer.any(dim=1)
    best = torch.argmax(conf, dim=1)
    rows = torch.where(needs)[0]
    transfer[rows, best[rows]] = True
    return x0, transfer
