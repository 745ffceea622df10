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


# Which projections of the model blocks run on this package's CTA-pair tcgen05 GEMMs
# (``ops.linear*``) instead of the library GEMM, for 16-bit models whose shapes the kernels take:
#   OWN_QKV      q/k/v projection with bias, RoPE and the cache scatter in its epilogue
#   OWN_GATE_UP  gate and up projections as one GEMM with the gated activation in its epilogue
#   OWN_DENSE    the plain projections (attention output, feed-forward output): "sliced" = where
#                the K range is cut into slices (few rows: block decode), True = always
#   OWN_HEAD     the output head; for greedy unmasking it returns arg-max and confidence and
#                never writes the logits
# Without a TMA multicast of operand tiles every SM pulls its own tiles from L2, which bounds a
# CTA-pair GEMM at 55-70 GB/s of operand bytes per SM: 0.82-0.93 of the library GEMM at these
# shapes.  With the work fused into their epilogues the QKV, gate/up and output-head projections
# come out level with or ahead of the library GEMM plus the separate kernels, so they are on.  The
# two plain projections have 4096 output columns: at block-decode row counts that is 16-32 whole
# tiles for 74 CTA pairs, so there the K range can be cut into slices that run as tiles of their
# own, and the normalisation kernel that follows adds the fp32 slices (``dense_pending``).  A
# sliced launch costs 6-9 us more than the library GEMM whatever K, so the launch plan
# (``ops.linear_partials_splits``) only slices long K ranges: the feed-forward output projection
# (K = 12288: 46 against 41 us) runs here, the attention output projection (K = 4096: 22 against
# 15 us) stays with the library.
OWN_QKV = True
OWN_GATE_UP = True
OWN_DENSE = "sliced"
OWN_HEAD = True

# The older single-CTA form of the fused QKV projection (128 x 128 tiles); kept for comparison,
# slower than both the CTA-pair kernel and the library GEMM + RoPE/scatter kernel.
FUSED_QKV = False


def set_own_gemm(on: bool):
    """Switches every projection to this package's kernels (True) or to the library GEMM (False)."""
    global OWN_QKV, OWN_GATE_UP, OWN_DENSE, OWN_HEAD
    OWN_QKV = OWN_GATE_UP = OWN_DENSE = OWN_HEAD = bool(on)


def dense(x, weight, bias=None):
    """An ``nn.Linear`` of the model blocks on 2-D activations."""
    if OWN_DENSE is True and ops._gemm_ok(x, weight):
        return ops.linear(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


def dense_pending(x, weight, bias=None):
    """A projection whose output is only ever added to the residual stream by the next
    ``RMSNorm.forward(x, delta)``: returns either the output itself or, where slicing the K range
    pays (``ops.linear_partials_splits``), its float32 slices ``[n_splits, n, out]``."""
    if OWN_DENSE and bias is None and ops._gemm_ok(x, weight):
        if ops.linear_partials_splits(x.shape[0], x.shape[1], weight.shape[0]) > 1:
            return ops.linear_partials(x, weight)
        if OWN_DENSE is True:
            return ops.linear(x, weight)
        return torch.nn.functional.linear(x, weight)
    if OWN_DENSE is True and ops._gemm_ok(x, weight):
        return ops.linear(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


def select_pending(delta, rows):
    """``delta`` restricted to the given rows, for either form ``dense_pending`` returns."""
    if delta is None:
        return None
    return delta.index_select(1 if delta.dim() == 3 else 0, rows)


class FusedProjections:
    """Weights of one block in the layouts the fused projection kernels read: q/k/v rows
    interleaved inside every head (``ops.interleave_heads``), gate and up rows interleaved with
    each other (``ops.interleave_rows``).  These are copies (the parameters keep their natural
    layout for state dicts), made on first use by the kernel that needs them; ``stale()`` tells
    when the parameters were replaced since."""

    def __init__(self):
        self.qkv_w = self.qkv_b = self.gate_up_w = None
        self._stamp = None

    @staticmethod
    def _stamp_of(params):
        return tuple((p.data_ptr(), p._version) for p in params if p is not None)

    def stale(self, params):
        return self._stamp != self._stamp_of(params)

    def reset(self, params):
        self.qkv_w = self.qkv_b = self.gate_up_w = None
        self._stamp = self._stamp_of(params)

    def qkv(self, w_qkv, b_qkv, head_dim):
        if self.qkv_w is None and head_dim == 128 and w_qkv.is_cuda and w_qkv.dtype in (torch.bfloat16, torch.float16):
            self.qkv_w = ops.interleave_heads(w_qkv)
            self.qkv_b = ops.interleave_heads(b_qkv) if b_qkv is not None else None
        return self.qkv_w, self.qkv_b

    def gate_up(self, gate, up):
        if (self.gate_up_w is None and gate.shape[0] % 8 == 0 and gate.is_cuda
                and gate.dtype in (torch.bfloat16, torch.float16)):
            self.gate_up_w = ops.interleave_rows(gate, up)
        return self.gate_up_w


def concat_gate_up(gate_proj, up_proj):
    """One buffer ``[2F, in]`` holding the gate rows then the up rows; the two parameters become
    views of it (state-dict names and values unchanged), so one library GEMM computes both."""
    w = torch.cat([gate_proj.weight.data, up_proj.weight.data], dim=0)
    f = gate_proj.out_features
    gate_proj.weight.data, up_proj.weight.data = w[:f], w[f:]
    return w


def gated_mlp_input(h, fused: FusedProjections, gate_proj, up_proj, act: str, gate_up_cat=None):
    """``act(gate_proj(h)) * up_proj(h)``: one GEMM of this package with the activation in its
    epilogue (``OWN_GATE_UP``), else one library GEMM over the concatenated weights followed by the
    activation kernel on its two halves, else two projections and the activation kernel."""
    if OWN_GATE_UP and gate_proj.bias is None and h.dtype in (torch.bfloat16, torch.float16) and h.is_cuda:
        w = fused.gate_up(gate_proj.weight.data, up_proj.weight.data)
        if w is not None and ops._gemm_ok(h, w):
            return ops.linear_swiglu(h, w, act)
    if (gate_up_cat is not None and gate_proj.bias is None
            and gate_up_cat.data_ptr() == gate_proj.weight.data_ptr() and h.shape[1] % 8 == 0):
        return ops.act_mul_halves(dense(h, gate_up_cat), act)
    return ops.act_mul(dense(h, gate_proj.weight, gate_proj.bias), dense(h, up_proj.weight, up_proj.bias), act)


def project_qkv(h, w_qkv, b_qkv, n_heads, n_kv_heads, head_dim, position_ids, cos, sin, attn, ctx, fused=None):
    """Returns ``(q, k, v)`` views for the attention call; with the fused path ``k``/``v`` are
    ``None`` because they only exist in the paged cache."""
    n = h.shape[0]
    D, nh, hkv = head_dim, n_heads, n_kv_heads
    caching = attn.k_cache.numel() > 0 and ctx.slot_mapping is not None
    if OWN_QKV and caching and fused is not None and cos.stride(0) * cos.element_size() % 16 == 0:
        wi, bi = fused.qkv(w_qkv, b_qkv, D)
        if wi is not None and ops._gemm_ok(h, wi):
            q = ops.linear_qkv_rope_scatter(h, wi, bi, nh, hkv, D, position_ids, cos, sin, attn.k_cache, attn.v_cache,
                                            ctx.slot_mapping)
            attn.kv_already_stored = True
            return q, None, None
    if (FUSED_QKV and caching and D == 128 and h.dtype in (torch.bfloat16, torch.float16) and h.shape[1] % 64 == 0
            and h.stride(0) % 8 == 0):
        q = ops.qkv_rope_scatter(h, w_qkv, b_qkv, nh, hkv, D, position_ids, cos, sin, attn.k_cache, attn.v_cache,
                                 ctx.slot_mapping)
        attn.kv_already_stored = True
        return q, None, None
    qkv = dense(h, w_qkv, b_qkv)
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
        normalisation (one fused kernel); either form that ``dense_pending`` returns."""
        if delta is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        if x.shape[-1] % (16 // x.element_size()) != 0 or x.shape[-1] > 1024 * (16 // x.element_size()):
            if delta.dim() == 3:    # float32 slices of the projection (``dense_pending``)
                delta = delta.sum(0).to(x.dtype)
            x.add_(delta)  # row shapes the fused kernel does not take
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps)
