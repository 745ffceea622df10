"""RoPE tables and rotation, half-split layout.

reference: nano-vdllm/model/modeling_llada.py:372-410 (table = cat(freqs, freqs),
rotate_half = cat(-x2, x1)); nano-vdllm/model/modeling_dream.py:159-170 (same
table, cast to the activation dtype); nano-vdllm/tests/test_attention_kernels.py:112-124.
"""
import torch


def rope_table(length: int, head_dim: int, theta: float, dtype=torch.float32):
    """Returns (cos, sin), each [length, head_dim]; computed in fp32, then cast."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(length, dtype=torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., heads, D]; cos/sin [..., D] (one row per token, broadcast over
    heads).  Arithmetic happens in promote(x.dtype, cos.dtype) with eager
    per-op rounding, and the result is cast back to x.dtype
    (reference: tests/test_attention_kernels.py:112-115)."""
    c = cos.unsqueeze(-2)
    s = sin.unsqueeze(-2)
    return (x * c + rotate_half(x) * s).to(x.dtype)


def apply_rope_inverse(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotation by the negative angle, as used for query-side relocation
    (reference: nano-vdllm/model/acache_attention.py:399-419)."""
    c = cos.unsqueeze(-2)
    s = sin.unsqueeze(-2)
    return (x * c - rotate_half(x) * s).to(x.dtype)


def llada_rope_qk(q, k, positions, theta, full_precision=True):
    """reference: nano-vdllm/model/modeling_llada.py:412-453 (fp32 math, cast back)."""
    D = q.shape[-1]
    n = int(positions.max().item()) + 1
    cos, sin = rope_table(n, D, theta, torch.float32)
    q_, k_ = (q.float(), k.float()) if full_precision else (q, k)
    c, s = cos[positions].unsqueeze(-2), sin[positions].unsqueeze(-2)
    q_rot = q_ * c + rotate_half(q_) * s
    k_rot = k_ * c + rotate_half(k_) * s
    return q_rot.type_as(q), k_rot.type_as(k)


def dream_rope_qk(q, k, positions, theta):
    """reference: nano-vdllm/model/modeling_dream.py:159-170,472-476 (table cast
    to the activation dtype first, arithmetic in that dtype)."""
    D = q.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    freqs = torch.outer(positions.float(), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    c = emb.cos().to(q.dtype).unsqueeze(-2)
    s = emb.sin().to(q.dtype).unsqueeze(-2)
    return q * c + rotate_half(q) * s, k * c + rotate_half(k) * s
