"""Serving configuration (field names and defaults follow the reference
dataclass, reference: nano-vdllm/config.py:5-29)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class Config:
    hf_config: Any = None
    mask_id: int = 126336
    recompute_batch_size: int = 4
    max_num_seqs: int = 0
    gen_length: int = 1024
    block_length: int = 1024
    remasking: str = "low_confidence"  # 'low_confidence', 'random', 'none'
    threshold: float = 0.9
    cache_block_size: int = 256
    max_num_batched_tokens: int = 16384
    gpu_memory_utilization: float = 0.9
    num_kvcache_blocks: int = -1
    temperature: float = 0.0
    enable_acache: bool = False
    enable_dkv_cache: bool = False
    dkv_steps: int = 0
    dkv_cache_interval: int = 8
    anchor_ratio: float = 0.05
    selection_mode: str = "top"
    use_reference_attention: bool = False
    acache_memory_reserve_gb: float = 4.0
    profile_timing: bool = False
    model_type: str = "llada"
    # --- additions of this implementation (all default to reference behaviour) ---
    # dtype of the paged KV cache; the reference hard-codes bfloat16
    kv_cache_dtype: str = "bfloat16"
    # replay the block-decode forward (all layers and the output head) from a CUDA graph with the
    # step metadata in fixed buffers; the same kernels with the same arguments, without the host
    # cost of about 330 launches per step
    use_cuda_graphs: bool = True
    # block decode: hand attention every request's shared span as the same run of slots (with -1
    # where an anchor's private copy replaces the shared row) and let one CTA serve two requests
    # of a KV head, staging the span once for both (same result as the logical order up to the
    # order of the floating-point sums).  On B200: 69 against 78 us per launch at 800 shared / 560
    # other keys (16 requests, 32 heads), level with the per-request kernel over a long span (1.52
    # ms at 8192 / 3700)
    group_shared_span: bool = True
    # anchor selection: probe the newly admitted requests in ragged batches of at most
    # ``max_num_batched_tokens`` query rows (the reference runs one forward per request) and then
    # replay the reference's per-request allocate / free sequence on the host, so the free list,
    # and with it every block table, ends up exactly as after one probe per request
    batch_anchor_selection: bool = True
    # eos id and block size aliases read by the block scheduler
    eos: int = -1

    @property
    def kvcache_block_size(self) -> int:
        return self.cache_block_size
