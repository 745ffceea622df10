"""Operators that replace eager PyTorch sequences of the reference engine:
anchor scoring and top-k, RoPE + K/V scatter, RMSNorm, gated activation and
threshold unmasking.  Thin wrappers over the C ABI."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, dtype_code, ptr, stream_ptr

_ACT = {"silu": 0, "relu": 1, "gelu": 2}


def anchor_topk(scores: torch.Tensor, k: int, largest: bool = True, offsets: torch.Tensor | None = None):
    """``scores`` fp32 ``[B, A]`` -> int64 ``[B, k]`` ascending indices (+ ``offsets[b]``).
    Replaces topk + sort + add (reference: nano-vdllm/model_runner.py:833-843); among
    equal scores the lowest index is selected."""
    assert scores.is_cuda and scores.dtype == torch.float32 and scores.dim() == 2 and scores.stride(1) == 1
    B, A = scores.shape
    k = min(int(k), A)
    out = torch.empty(B, k, dtype=torch.int64, device=scores.device)
    if offsets is not None:
        assert offsets.dtype == torch.int32 and offsets.numel() == B and offsets.is_cuda
    check(_lib.load().acache_anchor_topk(ptr(scores), B, A, scores.stride(0), k, int(bool(largest)), ptr(offsets),
                                         ptr(out), stream_ptr()), "anchor_topk")
    return out


_scratch: dict[int, torch.Tensor] = {}


def _scratch_for(device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _scratch.get(idx)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[idx] = buf
    return buf


def anchor_importance(q, q_rows, affix_k, affix_shift: int, rope_cos, rope_sin, scale: float, importance):
    """Accumulates one layer's influence score of every affix token into
    ``importance`` fp32 ``[A]`` (reference: nano-vdllm/model_runner.py:730-773).
    ``q`` ``[n, nh, D]`` post-RoPE; ``q_rows`` int32 indices of the mask-token rows;
    ``affix_k`` ``[A, Hkv, D]`` = the layer's cached affix keys (slots ``0..A-1``)."""
    assert q.is_cuda and q.dim() == 3 and q.stride(2) == 1 and q.stride(1) == q.shape[2]
    assert q_rows.dtype == torch.int32 and q_rows.is_cuda
    assert affix_k.dim() == 3 and affix_k.stride(2) == 1 and affix_k.stride(1) == affix_k.shape[2]
    assert importance.dtype == torch.float32 and importance.is_contiguous()
    n_q, (nh, D) = q_rows.numel(), q.shape[1:]
    A, hkv = affix_k.shape[:2]
    if n_q == 0 or A == 0:
        return
    lib = _lib.load()
    nbytes = lib.acache_anchor_importance_scratch_bytes(n_q, nh, A)
    scratch = _scratch_for(q.device, nbytes)
    if affix_shift != 0:
        rc, rs, rstride, rrows, rdt = ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0], dtype_code(rope_cos.dtype)
    else:
        rc, rs, rstride, rrows, rdt = None, None, 0, 0, _lib.F32
    check(lib.acache_anchor_importance(
        ptr(q), q.stride(0), ptr(q_rows), n_q, nh, hkv, D, dtype_code(q.dtype), ptr(affix_k), affix_k.stride(0), A,
        int(affix_shift), rc, rs, rstride, rrows, rdt, float(scale), ptr(importance), ptr(scratch), scratch.numel(),
        ptr(_lib.err_flag(q.device)), stream_ptr()), "anchor_importance", 2)


def anchor_importance_batched(q, q_rows, q_row_offsets, max_q_rows: int, affix_k, affix_shifts, rope_cos, rope_sin,
                              scale: float, importance) -> bool:
    """``anchor_importance`` for all requests of a probe batch in one launch: request ``r`` owns the
    mask rows ``q_rows[q_row_offsets[r]:q_row_offsets[r + 1]]`` (both int32 on the device, at most
    ``max_q_rows`` rows per request), the rotation row ``affix_shifts[r]`` (int32 on the device, or
    None) and the scores ``importance[r]`` (fp32 ``[n_requests, A]``, accumulated in place with the
    bits of the per-request call).  Returns False, with nothing launched, for shapes only the
    per-request call takes (fp32, head sizes other than 64 / 128, affixes beyond 2048 tokens)."""
    assert q.is_cuda and q.dim() == 3 and q.stride(2) == 1 and q.stride(1) == q.shape[2]
    assert q_rows.dtype == torch.int32 and q_rows.is_cuda and q_row_offsets.dtype == torch.int32 and q_row_offsets.is_cuda
    assert affix_shifts is None or (affix_shifts.dtype == torch.int32 and affix_shifts.is_cuda)
    assert affix_k.dim() == 3 and affix_k.stride(2) == 1 and affix_k.stride(1) == affix_k.shape[2]
    assert importance.dtype == torch.float32 and importance.dim() == 2 and importance.stride(1) == 1
    n_req, (nh, D) = q_row_offsets.numel() - 1, q.shape[1:]
    A, hkv = affix_k.shape[:2]
    assert importance.shape[0] == n_req and importance.shape[1] == A
    if n_req <= 0 or max_q_rows <= 0 or A == 0:
        return True
    lib = _lib.load()
    nbytes = lib.acache_anchor_importance_batched_scratch_bytes(n_req, int(max_q_rows), nh, A)
    scratch = _scratch_for(q.device, nbytes)
    if affix_shifts is not None:
        rc, rs, rstride, rrows, rdt = ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0], dtype_code(rope_cos.dtype)
    else:
        rc, rs, rstride, rrows, rdt = None, None, 0, 0, _lib.F32
    status = lib.acache_anchor_importance_batched(
        ptr(q), q.stride(0), ptr(q_rows), ptr(q_row_offsets), n_req, int(max_q_rows), nh, hkv, D, dtype_code(q.dtype),
        ptr(affix_k), affix_k.stride(0), A, ptr(affix_shifts), rc, rs, rstride, rrows, rdt, float(scale),
        ptr(importance), importance.stride(0), ptr(scratch), scratch.numel(), ptr(_lib.err_flag(q.device)), stream_ptr())
    if status == -2:
        return False
    check(status, "anchor_importance_batched", 2)
    return True


def anchor_importance_noalloc(q, q_rows, affix_k, affix_shift: int, rope_cos, rope_sin, scale: float, importance):
    """``anchor_importance`` for callers that may not allocate device memory (a host that owns
    the whole GPU through its own arena, a plugin that only gets input and output buffers, a
    loop that cannot take the stall of an allocation).  The per-CTA partial sums go to a fixed
    8 MiB array inside the library instead of a caller-provided or torch-allocated buffer, and
    this wrapper itself creates no tensor.  Raises ``OverflowError`` when
    ``ceil(n_q / 32) * n_heads * affix_len`` floats do not fit that array.  Calls share the
    array: do not let two of them overlap on different streams.  The first call on a device
    resolves the array's address and must be made before any stream capture (inside one it raises
    ``NotImplementedError``).  A kernel-side failure is reported through the device's error flag
    only if an earlier operator call has already created that flag."""
    assert q.is_cuda and q.dim() == 3 and q.stride(2) == 1 and q.stride(1) == q.shape[2]
    assert q_rows.dtype == torch.int32 and q_rows.is_cuda
    assert affix_k.dim() == 3 and affix_k.stride(2) == 1 and affix_k.stride(1) == affix_k.shape[2]
    assert importance.dtype == torch.float32 and importance.is_contiguous()
    n_q, (nh, D) = q_rows.numel(), q.shape[1:]
    A, hkv = affix_k.shape[:2]
    if n_q == 0 or A == 0:
        return
    if affix_shift != 0:
        rc, rs, rstride, rrows, rdt = ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0], dtype_code(rope_cos.dtype)
    else:
        rc, rs, rstride, rrows, rdt = None, None, 0, 0, _lib.F32
    check(_lib.load().acache_anchor_importance_static(
        ptr(q), q.stride(0), ptr(q_rows), n_q, nh, hkv, D, dtype_code(q.dtype), ptr(affix_k), affix_k.stride(0), A,
        int(affix_shift), rc, rs, rstride, rrows, rdt, float(scale), ptr(importance),
        ptr(_lib.existing_err_flag(q.device)), stream_ptr()), "anchor_importance_static", 2)


def rope_store(q, k, v, positions, rope_cos, rope_sin, k_cache=None, v_cache=None, slot_mapping=None):
    """Rotates ``q [n, nh, D]`` and ``k [n, Hkv, D]`` in place by table rows
    ``positions`` and scatters the rotated ``k`` and ``v`` to ``slot_mapping``
    (reference: nano-vdllm/model/modeling_llada.py:412-453 + model/attention.py:34-41)."""
    n, nh, D = q.shape
    hkv = k.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D
    assert positions.dtype == torch.int64 and positions.numel() == n
    num_slots = 0
    if slot_mapping is not None:
        assert v is not None and v.stride(2) == 1 and v.stride(1) == D
        assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() == n
        num_slots = k_cache.numel() // (hkv * D)
    flag = _lib.err_flag(q.device)
    check(_lib.load().acache_rope_store(
        ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0) if v is not None else 0, n, nh, hkv, D,
        dtype_code(q.dtype), ptr(positions), ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0],
        dtype_code(rope_cos.dtype), ptr(k_cache), ptr(v_cache), ptr(slot_mapping), num_slots, ptr(flag),
        stream_ptr()), "rope_store")


def qkv_rope_scatter(x, w_qkv, bias, n_heads, n_kv_heads, head_dim, positions, rope_cos, rope_sin, k_cache, v_cache,
                     slot_mapping):
    """Fused QKV projection + RoPE + K/V scatter of ``x [n, hidden]`` (one tcgen05 GEMM with a
    fused epilogue, replacing three ``nn.Linear`` calls, the rotary embedding and ``store_kvcache``
    of the reference block).  Returns the rotated queries ``[n, n_heads, head_dim]``; the rotated
    keys and the values only exist in the paged cache.  Raises ``NotImplementedError`` for shapes
    the kernel does not take (the caller then uses the library GEMM + ``rope_store``)."""
    n, hidden = x.shape
    assert x.stride(1) == 1 and w_qkv.is_contiguous() and w_qkv.shape == ((n_heads + 2 * n_kv_heads) * head_dim, hidden)
    assert positions.dtype == torch.int64 and positions.numel() == n
    assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() == n
    q = torch.empty(n, n_heads, head_dim, dtype=x.dtype, device=x.device)
    num_slots = k_cache.numel() // (n_kv_heads * head_dim)
    flag = _lib.err_flag(x.device)
    check(_lib.load().acache_qkv_rope_scatter(
        ptr(x), x.stride(0), n, hidden, ptr(w_qkv), ptr(bias), n_heads, n_kv_heads, head_dim, dtype_code(x.dtype),
        ptr(positions), ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0), rope_cos.shape[0], dtype_code(rope_cos.dtype),
        ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache), ptr(slot_mapping), num_slots, ptr(flag), stream_ptr()),
        "qkv_rope_scatter")
    return q


# ---- dense projections on CTA-pair tcgen05 GEMMs ---------------------------------------------
# tile override for experiments: (row blocks per pair, columns per tile); (0, 0) = chosen per launch
GEMM_TILE = (0, 0)


def interleave_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Rows of ``a`` and ``b`` (same shape) interleaved in groups of 8: the weight layout of
    ``linear_swiglu`` (``a`` = gate projection, ``b`` = up projection)."""
    assert a.shape == b.shape and a.shape[0] % 8 == 0
    n = a.shape[0] // 8
    return torch.stack((a.reshape(n, 8, *a.shape[1:]), b.reshape(n, 8, *b.shape[1:])), dim=1).reshape(2 * a.shape[0], *a.shape[1:])


def interleave_heads(w: torch.Tensor, head_dim: int = 128) -> torch.Tensor:
    """Rows (or entries) of a fused q/k/v weight (bias) interleaved inside every head in groups of
    8, low half against high half: the layout of ``linear_qkv_rope_scatter``."""
    assert head_dim == 128 and w.shape[0] % head_dim == 0
    h = w.shape[0] // head_dim
    v = w.reshape(h, 2, 8, 8, *w.shape[1:])            # head, half, group, lane
    return v.transpose(1, 2).reshape(w.shape).contiguous()


def _gemm_ok(x, w):
    return (x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype
            and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1] and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.shape[0] % 16 == 0)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x [n, in] @ weight[out, in]^T (+ bias)`` (an ``nn.Linear`` of the reference model blocks)."""
    assert _gemm_ok(x, weight), "shape or dtype the projection kernel does not take"
    n, N = x.shape[0], weight.shape[0]
    out = torch.empty(n, N, dtype=x.dtype, device=x.device)
    if n:
        check(_lib.load().acache_linear(ptr(x), x.stride(0), n, x.shape[1], ptr(weight), N, ptr(bias), dtype_code(x.dtype),
                                        ptr(out), out.stride(0), GEMM_TILE[0], GEMM_TILE[1], ptr(_lib.err_flag(x.device)),
                                        stream_ptr()), "linear")
    return out


def linear_partials_splits(n_rows: int, in_features: int, out_features: int) -> int:
    """Slices of the ``in_features`` range that ``linear_partials`` would use for this shape; 1 means
    the projection has enough output tiles to fill the GPU whole (use ``linear``)."""
    return int(_lib.load().acache_linear_partials_splits(int(n_rows), int(in_features), int(out_features)))


def linear_partials(x: torch.Tensor, weight: torch.Tensor, n_splits: int = 0, tile=(0, 0)) -> torch.Tensor:
    """``x [n, in] @ weight[out, in]^T`` left as fp32 sums over ``n_splits`` slices of the ``in`` range:
    returns ``[n_splits, n, out]`` float32, to be summed by ``add_rmsnorm`` (which takes it as its
    update).  For projections with too few output tiles to occupy every SM with whole tiles."""
    assert _gemm_ok(x, weight), "shape or dtype the projection kernel does not take"
    n, N = x.shape[0], weight.shape[0]
    s = int(n_splits) or linear_partials_splits(n, x.shape[1], N)
    out = torch.empty(s, n, N, dtype=torch.float32, device=x.device)
    if n:
        check(_lib.load().acache_linear_partials(ptr(x), x.stride(0), n, x.shape[1], ptr(weight), N, dtype_code(x.dtype),
                                                 ptr(out), s, tile[0], tile[1], ptr(_lib.err_flag(x.device)),
                                                 stream_ptr()), "linear_partials")
    return out


def linear_swiglu(x: torch.Tensor, weight_gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(x @ Wg^T) * (x @ Wu^T)`` with the two weights interleaved by ``interleave_rows``."""
    assert _gemm_ok(x, weight_gate_up)
    n, F = x.shape[0], weight_gate_up.shape[0] // 2
    out = torch.empty(n, F, dtype=x.dtype, device=x.device)
    if n:
        check(_lib.load().acache_linear_swiglu(ptr(x), x.stride(0), n, x.shape[1], ptr(weight_gate_up), F, _ACT[act],
                                               dtype_code(x.dtype), ptr(out), out.stride(0), GEMM_TILE[0], GEMM_TILE[1],
                                               ptr(_lib.err_flag(x.device)), stream_ptr()), "linear_swiglu")
    return out


def linear_qkv_rope_scatter(x, w_qkv_interleaved, bias_interleaved, n_heads, n_kv_heads, head_dim, positions, rope_cos,
                            rope_sin, k_cache, v_cache, slot_mapping):
    """``qkv_rope_scatter`` on CTA pairs; the weight (and bias) rows are in the ``interleave_heads``
    layout.  Returns the rotated queries ``[n, n_heads, head_dim]``."""
    assert _gemm_ok(x, w_qkv_interleaved) and w_qkv_interleaved.shape[0] == (n_heads + 2 * n_kv_heads) * head_dim
    n = x.shape[0]
    assert positions.dtype == torch.int64 and positions.numel() == n
    assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() == n
    q = torch.empty(n, n_heads, head_dim, dtype=x.dtype, device=x.device)
    num_slots = k_cache.numel() // (n_kv_heads * head_dim)
    if n:
        check(_lib.load().acache_linear_qkv_rope_scatter(
            ptr(x), x.stride(0), n, x.shape[1], ptr(w_qkv_interleaved), ptr(bias_interleaved), n_heads, n_kv_heads,
            head_dim, dtype_code(x.dtype), ptr(positions), ptr(rope_cos), ptr(rope_sin), rope_cos.stride(0),
            rope_cos.shape[0], dtype_code(rope_cos.dtype), ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache),
            ptr(slot_mapping), num_slots, GEMM_TILE[0], GEMM_TILE[1], ptr(_lib.err_flag(x.device)), stream_ptr()),
            "linear_qkv_rope_scatter")
    return q


def linear_argmax(x: torch.Tensor, weight: torch.Tensor):
    """Output head + greedy statistics: ``(argmax over the vocabulary int64 [n], confidence fp32
    [n])`` of ``x @ weight^T`` without materialising the logits."""
    assert _gemm_ok(x, weight)
    n, N = x.shape[0], weight.shape[0]
    x0 = torch.empty(n, dtype=torch.int64, device=x.device)
    conf = torch.empty(n, dtype=torch.float32, device=x.device)
    if n:
        lib = _lib.load()
        nbytes = lib.acache_linear_argmax_scratch_bytes(n, N)
        # a tensor of this call's own (not the shared growing buffer): inside a CUDA-graph capture it
        # then belongs to the graph's pool and stays valid for every replay
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        check(lib.acache_linear_argmax(ptr(x), x.stride(0), n, x.shape[1], ptr(weight), N, dtype_code(x.dtype), ptr(x0),
                                       ptr(conf), ptr(scratch), scratch.numel(), GEMM_TILE[0], GEMM_TILE[1],
                                       ptr(_lib.err_flag(x.device)), stream_ptr()), "linear_argmax", 2)
    return x0, conf


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * cast(x * rsqrt(mean(x^2) + eps))`` with the mean in fp32
    (reference: nano-vdllm/model/modeling_llada.py:308-323)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    assert x2.stride(1) == 1
    y = torch.empty_like(x2)
    check(_lib.load().acache_rmsnorm(ptr(x2), x2.stride(0), ptr(weight), ptr(y), y.stride(0), x2.shape[0], x2.shape[1],
                                     float(eps), dtype_code(x.dtype), stream_ptr()), "rmsnorm")
    return y.view(shape)


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x += delta`` (in place, rounded to x.dtype) and returns ``rmsnorm(x)``: the residual add of
    the previous sub-layer fused into the normalisation that follows it.  ``delta`` may also be the
    float32 slices ``[n_splits, rows, cols]`` that ``linear_partials`` returns; they are summed in
    order and rounded to x.dtype first."""
    shape = x.shape
    if delta.dtype == torch.float32 and x.dtype != torch.float32:
        # fp32 slices of a projection's K range (``linear_partials``): [n_splits, rows, cols]
        x2 = x.view(-1, shape[-1])
        assert delta.dim() == 3 and delta.shape[1:] == x2.shape and delta.stride(2) == 1 and x2.stride(1) == 1
        y = torch.empty_like(x2)
        check(_lib.load().acache_add_rmsnorm_partials(ptr(x2), x2.stride(0), ptr(delta), delta.shape[0], delta.stride(0),
                                                      delta.stride(1), ptr(weight), ptr(y), y.stride(0), x2.shape[0],
                                                      x2.shape[1], float(eps), dtype_code(x.dtype), stream_ptr()),
              "add_rmsnorm_partials")
        return y.view(shape)
    x2, d2 = x.view(-1, shape[-1]), delta.reshape(-1, shape[-1])
    assert x2.stride(1) == 1 and d2.stride(1) == 1 and x2.shape == d2.shape
    y = torch.empty_like(x2)
    check(_lib.load().acache_add_rmsnorm(ptr(x2), x2.stride(0), ptr(d2), d2.stride(0), ptr(weight), ptr(y), y.stride(0),
                                         x2.shape[0], x2.shape[1], float(eps), dtype_code(x.dtype), stream_ptr()),
          "add_rmsnorm")
    return y.view(shape)


def act_mul(gate: torch.Tensor, up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` (reference: nano-vdllm/model/modeling_llada.py:757-763)."""
    assert gate.shape == up.shape and gate.is_contiguous() and up.is_contiguous()
    y = torch.empty_like(gate)
    check(_lib.load().acache_act_mul(ptr(gate), ptr(up), ptr(y), gate.numel(), _ACT[act], dtype_code(gate.dtype),
                                     stream_ptr()), "act_mul")
    return y


def act_mul_halves(x: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(x[:, :F]) * x[:, F:]`` for ``x [n, 2F]``: the gate and up projections computed by one
    GEMM over the concatenated weights."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 2 == 0
    n, F = x.shape[0], x.shape[1] // 2
    y = torch.empty(n, F, dtype=x.dtype, device=x.device)
    check(_lib.load().acache_act_mul_halves(ptr(x), x.stride(0), ptr(y), y.stride(0), n, F, _ACT[act],
                                            dtype_code(x.dtype), stream_ptr()), "act_mul_halves")
    return y


def transfer_tokens(logits: torch.Tensor, blocks: torch.Tensor, mask_id: int, threshold: float):
    """Threshold unmasking at temperature 0 applied in place to ``blocks`` int64
    ``[R, T]`` from ``logits [R*T, V]`` (reference: nano-vdllm/model_runner.py:2279-2314).
    Returns ``(x0, confidence)`` of every position."""
    R, T = blocks.shape
    logits = logits.reshape(R * T, -1)
    assert logits.stride(1) == 1 and blocks.is_contiguous() and blocks.dtype == torch.int64
    x0 = torch.empty(R, T, dtype=torch.int64, device=blocks.device)
    conf = torch.empty(R, T, dtype=torch.float32, device=blocks.device)
    check(_lib.load().acache_transfer_tokens(ptr(logits), logits.stride(0), logits.shape[1], dtype_code(logits.dtype),
                                             ptr(blocks), R, T, int(mask_id), float(threshold), ptr(x0), ptr(conf),
                                             stream_ptr()), "transfer_tokens", 2)
    return x0, conf


def apply_transfer(x0: torch.Tensor, conf: torch.Tensor, blocks: torch.Tensor, mask_id: int, threshold: float):
    """The commit rule of ``transfer_tokens`` from statistics that already exist (``linear_argmax``):
    edits ``blocks`` int64 ``[R, T]`` in place from ``x0`` int64 / ``conf`` fp32 of ``R * T`` entries."""
    R, T = blocks.shape
    assert blocks.is_contiguous() and blocks.dtype == torch.int64
    assert x0.is_contiguous() and x0.dtype == torch.int64 and x0.numel() == R * T
    assert conf.is_contiguous() and conf.dtype == torch.float32 and conf.numel() == R * T
    check(_lib.load().acache_apply_transfer(ptr(blocks), ptr(x0), ptr(conf), R, T, int(mask_id), float(threshold),
                                            stream_ptr()), "apply_transfer")
