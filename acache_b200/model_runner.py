"""Serving engine for block-wise diffusion-LLM decoding with affix-KV reuse.

Interface of the reference engine (reference: nano-vdllm/model_runner.py:13-2314):
``ModelRunner(model, config)``, ``generate_with_acache(list[Sequence]) -> (tokens, nfe)``,
``generate_with_dual_cache``, ``kv_cache``, ``block_manager``, ``last_timing`` and the
``prepare_*`` / ``_compute_anchor_positions*`` helpers its tests drive.  What is
different underneath:

* every device operator is one of this package's sm_100a kernels (see
  ``include/acache_b200.h``); GEMMs are library calls;
* step metadata is assembled with numpy into ONE pinned buffer and shipped with one
  host-to-device copy per step, instead of one copy per tensor;
* the output head runs only on the rows whose logits are consumed, and unmasking is a
  fused kernel that edits the working blocks in place (no logits gather, no ``where``);
* timing sections are CUDA-event pairs resolved once at the end of a call.

The allocator call sequence (shared-affix reservation, the probe's temporary
allocation, the relocation workspace) is kept exactly, because it decides the block
tables, and those are part of the parity contract.
"""
from __future__ import annotations

import gc
import time
from contextlib import contextmanager
from itertools import islice

import numpy as np
import torch

from . import _lib, ops
from .block_manager import BlockManager
from .model import acache_attention as aa
from .model.acache_attention import materialize_relocated_affix
from .model.modeling_common import build_rope_table
from .scheduler import admissible_prefix
from .sequence import Sequence
from .dkv import DkvMixin
from .utils import add_gumbel_noise, get_context, reset_context, set_context

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def attention_read_layout(seq, use_query_relocation: bool, shared_prefix_len: int):
    """Order in which attention reads a request's K/V slots (reference:
    nano-vdllm/model_runner.py:275-282).  With query-side relocation the slots that
    still point into the shared span come first (``shared_kv_len`` of them), so one
    inverse-rotated copy of the queries serves that whole partition."""
    slots = list(seq.read_slot_map)
    if not use_query_relocation or seq.affix_start == 0:
        return slots, 0
    lo = seq.shared_slot_offset
    hi = lo + shared_prefix_len
    shared = [s for s in slots if lo <= s < hi]
    private = [s for s in slots if not (lo <= s < hi)]
    return shared + private, len(shared)


def attention_read_runs(seq):
    """Read order in which every request names the shared span the same way: the affix span
    as the consecutive slots it occupies, with -1 (a key that takes no part) where a private
    copy replaces the shared row, then those private copies, then the request's other tokens.
    Attention does not depend on the order of the keys, so the result equals the logical
    order of ``seq.read_slot_map`` up to the order of the floating-point sums; block decode
    can then stage the span once for several requests.
    Returns ``(slots, affix_len, first slot of the span)``."""
    cached = getattr(seq, "_read_runs", None)
    if cached is not None and cached[0] is seq.read_slot_map:
        return cached[1:]
    slots = np.asarray(seq.read_slot_map, dtype=np.int32)
    a0, a1 = seq.affix_start, seq.affix_end
    if not getattr(seq, "acache_enabled", False) or a1 <= a0:
        out = (slots, 0, -1)
    else:
        span = slots[a0:a1].copy()
        start = span - np.arange(a1 - a0, dtype=np.int32)      # slot the run would start at
        values, counts = np.unique(start, return_counts=True)
        first = int(values[np.argmax(counts)])
        moved = start != first
        private = span[moved]
        span[moved] = -1
        out = (np.concatenate([span, private, slots[:a0], slots[a1:]]), a1 - a0, first)
    seq._read_runs = (seq.read_slot_map,) + out
    return out


class _Staging:
    """Packs the integer arrays of one step into a single pinned buffer and moves it to
    the device with one copy; returns typed device views."""

    def __init__(self, device):
        self.device = device
        self.pinned = device.type == "cuda"
        self.h2d_bytes = 0

    def ship(self, **arrays):
        order = sorted(arrays, key=lambda k: -np.dtype(arrays[k].dtype).itemsize)  # int64 first: alignment
        offsets, total = {}, 0
        for k in order:
            a = arrays[k]
            total = -(-total // 16) * 16
            offsets[k] = total
            total += a.nbytes
        host = torch.empty(max(total, 16), dtype=torch.uint8, pin_memory=self.pinned)
        hv = host.numpy()
        for k in order:
            a = np.ascontiguousarray(arrays[k])
            hv[offsets[k]: offsets[k] + a.nbytes] = a.view(np.uint8).reshape(-1)
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += total
        out = {}
        for k in order:
            a = arrays[k]
            tdt = torch.int64 if a.dtype == np.int64 else torch.int32
            out[k] = dev[offsets[k]: offsets[k] + a.nbytes].view(tdt).view(a.shape)
        return out


class _StaticStaging:
    """Same interface as ``_Staging`` but with a fixed layout: every named array has a fixed
    capacity and always lands at the same device address, so kernels captured in a CUDA graph
    keep reading the step metadata from where they were captured.  One pinned host buffer, one
    device buffer, one copy per ``ship``."""

    def __init__(self, device, capacities: dict, counter: _Staging | None = None):
        self.device = device
        self.counter = counter
        self.offsets, total = {}, 0
        for name, (dtype, n) in sorted(capacities.items(), key=lambda kv: -np.dtype(kv[1][0]).itemsize):
            total = -(-total // 16) * 16
            self.offsets[name] = (total, np.dtype(dtype), int(n))
            total += np.dtype(dtype).itemsize * int(n)
        self.nbytes = max(total, 16)
        self.host = torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=device.type == "cuda")
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        self.copied = None   # event after the last copy: the pinned buffer is rewritten only after it

    def fits(self, **arrays) -> bool:
        return set(arrays) == set(self.offsets) and all(
            np.dtype(a.dtype) == self.offsets[k][1] and a.size <= self.offsets[k][2] for k, a in arrays.items())

    def ship(self, **arrays):
        assert self.fits(**arrays), "step metadata does not fit the captured layout"
        if self.copied is not None:
            self.copied.synchronize()
        hv = self.host.numpy()
        out, moved = {}, 0
        for k, a in arrays.items():
            off, dt, _ = self.offsets[k]
            a = np.ascontiguousarray(a)
            hv[off: off + a.nbytes] = a.view(np.uint8).reshape(-1)
            moved += a.nbytes
            tdt = torch.int64 if dt == np.int64 else torch.int32
            out[k] = self.dev[off: off + a.nbytes].view(tdt).view(a.shape)
        self.dev.copy_(self.host, non_blocking=True)
        if self.device.type == "cuda":
            self.copied = torch.cuda.Event()
            self.copied.record()
        if self.counter is not None:
            self.counter.h2d_bytes += moved
        return out


class _DecodeGraph:
    """One block-decode forward (all layers and the output head) of ``n_rows`` requests captured
    in a CUDA graph.  Inputs live at fixed addresses: the block's tokens, and the step metadata
    in a ``_StaticStaging``; the logits come back in a tensor of the graph's memory pool.  The
    graph is replayed for every decode step with this many rows, whatever the requests are.
    ``logits`` holds what the forward returns: ``(logits, None)`` or ``(None, (x0, confidence))``."""

    def __init__(self, runner, n_rows: int, names_and_dtypes: dict, read_capacity: int, max_pos: int):
        T = runner.config.block_length
        caps = {}
        for name, dtype in names_and_dtypes.items():
            n = {"positions": n_rows * T, "cu_q": n_rows + 1, "cu_k": n_rows + 1, "slots": n_rows * T,
                 "read": read_capacity}.get(name, n_rows)
            caps[name] = (dtype, n)
        self.staging = _StaticStaging(runner.device, caps, runner._staging)
        self.tokens = torch.zeros(n_rows, T, dtype=torch.int64, device=runner.device)
        self.max_pos = max_pos
        self.graph = None
        self.logits = None
        self.events: list = []
        self.with_timers = False
        self.launches = 0
        self.pending_work = None   # work units of a replay whose event times were not read yet
        self.stamp = None
        self.eager = False         # set when a capture failed: this object then only forwards eagerly

    def run(self, runner, block_tokens, positions):
        self.tokens.copy_(block_tokens)
        timers = _lib.kernel_timers_enabled()
        for rope in runner._rope_caches:      # the table the capture will see (and later eager forwards keep)
            rope.get(self.max_pos, runner.device)
        if not self.eager and (self.graph is None or (timers and not self.with_timers)
                               or self.stamp != runner._graph_stamp()):
            try:
                self._capture(runner, positions, timers)
            except RuntimeError as exc:
                # a capture that the installed stack refuses: keep serving, eagerly, and say so once
                import warnings

                warnings.warn(f"CUDA-graph capture of the decode forward failed ({exc}); continuing without graphs")
                self.graph, self.eager = None, True
                runner.config.use_cuda_graphs = False
        if self.eager:
            return runner._decode_forward(self.tokens, positions, self.max_pos)
        runner.harvest_graph_timers()
        self.graph.replay()
        _lib.LAUNCHES += self.launches
        if self.events:
            self.pending_work = aa.ATTENTION_WORK
            runner._graph_with_pending_timers = self
        return self.logits

    def _capture(self, runner, positions, timers: bool):
        def forward():
            return runner._decode_forward(self.tokens, positions, self.max_pos)

        forward()   # eager once: tables, workspaces and library handles exist before the capture
        torch.cuda.synchronize()
        self.graph, self.logits = None, None
        graph = torch.cuda.CUDAGraph()
        self.events = _lib.begin_graph_capture()
        launches0 = _lib.LAUNCHES
        if runner._graph_pool is None:
            # one memory pool for all decode graphs: they never run at the same time and the
            # logits of one replay are consumed before the next replay
            runner._graph_pool = torch.cuda.graph_pool_handle()
        try:
            with torch.cuda.graph(graph, pool=runner._graph_pool):
                self.logits = forward()
        finally:
            _lib.end_graph_capture()
        self.launches = _lib.LAUNCHES - launches0
        _lib.LAUNCHES = launches0   # nothing ran during the capture
        self.graph, self.with_timers, self.stamp = graph, timers, runner._graph_stamp()


class _Probe:
    """State of one anchor-selection probe, read by the attention layers."""

    __slots__ = ("q_rows", "affix_len", "affix_shift", "importance", "rope_cos", "rope_sin")


class _ProbeBatch:
    """The probes of one ragged forward in the form ``ops.anchor_importance_batched`` takes: all
    mask rows behind one another, per-request offsets into them, rotation rows (None when no
    request needs one) and the ``[requests, affix_len]`` score matrix.  ``usable`` is cleared by
    the first layer whose call is declined, so the other layers loop over the requests at once."""

    __slots__ = ("q_rows", "offsets", "max_q_rows", "shifts", "importance", "affix_len", "rope_cos", "rope_sin",
                 "usable")


class ModelRunner(DkvMixin):
    def __init__(self, model, config):
        self.config = config
        self.model = model
        self.base_model = model.module if hasattr(model, "module") else model
        self.device = model.device
        self.kv_cache = None
        self.kv_cache_block_bytes = 0
        self.block_manager = None
        self.shared_prefix_len = 0
        self.shared_prefix_blocks = 0
        self.acache_ready = False
        self.shared_prefix_token_ids: tuple[int, ...] = ()
        self._affix_relocation_enabled = False
        self._affix_relocation_max_position = 0
        self._relocated_affix_slot_offset = None
        self.profile_timing = bool(getattr(config, "profile_timing", False))
        self.last_timing = {}
        self._active_timing = None
        self._pending_events = []
        self._staging = _Staging(self.device)
        self.d2h_bytes = 0
        self._attn_layers = [m for m in self.model.modules() if hasattr(m, "k_cache") and hasattr(m, "v_cache")]
        # captured block-decode forwards, by (rows, layout of the step metadata)
        self._decode_graphs: dict = {}
        self._graph_pool = None
        self._decode_graph = None
        self._graph_with_pending_timers = None
        self._rope_caches = [m.rope for m in self.model.modules() if hasattr(m, "rope") and hasattr(m.rope, "get")]
        self.allocate_kv_cache()

    # ------------------------------------------------------------------ model access
    def _is_dream_model(self):
        return str(getattr(self.config, "model_type", "")).lower() == "dream"

    def _uses_decoder_layers(self):
        return self._is_dream_model()

    def _arch(self):
        hf = self.config.hf_config
        nh = getattr(hf, "n_heads", getattr(hf, "num_attention_heads", None))
        if nh is None:
            raise AttributeError("HF config must define n_heads or num_attention_heads.")
        hkv = getattr(hf, "effective_n_kv_heads", None) or getattr(hf, "n_kv_heads", None) \
            or getattr(hf, "num_key_value_heads", None) or nh
        hidden = getattr(hf, "d_model", getattr(hf, "hidden_size", None))
        if hidden is None:
            raise AttributeError("HF config must define d_model or hidden_size.")
        layers = getattr(hf, "n_layers", getattr(hf, "num_hidden_layers", None))
        if layers is None:
            raise AttributeError("HF config must define n_layers or num_hidden_layers.")
        return nh, hkv, hidden // nh, layers

    def _rope_spec(self):
        hf = self.config.hf_config
        theta = float(getattr(hf, "rope_theta", 10000.0))
        # LLaDA rotates in fp32; Dream casts the table to the cache dtype first
        # (reference: model_runner.py:258-271)
        table_dtype = self.kv_cache.dtype if self._is_dream_model() else torch.float32
        return theta, table_dtype

    def _forward_model(self, input_ids, position_ids=None, compute_logits=True, logits_keep_indices=None, max_pos=None,
                       greedy_stats=False):
        return self.base_model(input_ids=input_ids, position_ids=position_ids, compute_logits=compute_logits,
                               logits_keep_indices=logits_keep_indices, max_pos=max_pos, greedy_stats=greedy_stats)

    def _greedy(self):
        """Unmasking only needs each position's arg-max and confidence (temperature 0, confidence
        remasking): the output head may then return those instead of the logits."""
        return self.config.temperature == 0 and self.config.remasking == "low_confidence"

    def _decode_forward(self, block_tokens, positions, max_pos):
        """Block-decode forward as unmasking sees it: ``(logits [B, T, V], None)`` or
        ``(None, (x0 [B, T], confidence [B, T]))``, Dream's shift by one position applied."""
        out = self._forward_model(block_tokens, positions, max_pos=max_pos, greedy_stats=self._greedy())
        if out.stats is None:
            return self._dream_decode_logits(out.logits), None
        x0, conf = (t.view(block_tokens.shape) for t in out.stats)
        if self._is_dream_model():
            x0 = torch.cat([x0[:, :1], x0[:, :-1]], dim=1).contiguous()
            conf = torch.cat([conf[:, :1], conf[:, :-1]], dim=1).contiguous()
        return None, (x0, conf)

    def _dream_decode_logits(self, logits):
        """Dream predicts token j from position j-1: shift right inside the block
        (reference: model_runner.py:56-61)."""
        if not self._is_dream_model() or logits.dim() != 3:
            return logits
        return torch.cat([logits[:, :1], logits[:, :-1]], dim=1)

    def _dream_shift_keep_indices(self, keep_indices, row_starts):
        row_starts = row_starts.to(device=keep_indices.device, dtype=keep_indices.dtype)
        return torch.maximum(keep_indices, row_starts.unsqueeze(1) + 1) - 1

    # ------------------------------------------------------------------ timing
    def _new_timing(self, mode: str, num_prompts: int):
        if not self.profile_timing:
            return None
        return {"mode": mode, "num_prompts": int(num_prompts)}

    def _start_timing(self):
        """Opens a timed section.  A no-op (returns None) unless profiling is on."""
        if not self.profile_timing:
            return None
        if self.device.type != "cuda":
            return time.perf_counter()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def _finish_timing(self, timing, key, start):
        if start is None or timing is None:
            return
        if self.device.type != "cuda":
            timing[key] = timing.get(key, 0.0) + (time.perf_counter() - start)
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self._pending_events.append((timing, key, start, end))

    def _resolve_timing(self):
        if not self._pending_events:
            return
        torch.cuda.synchronize(self.device)
        for timing, key, start, end in self._pending_events:
            timing[key] = timing.get(key, 0.0) + start.elapsed_time(end) / 1e3
        self._pending_events = []

    def _add_timing_count(self, timing, key, value=1):
        if timing is None:
            return
        timing[key] = timing.get(key, 0) + int(value)

    def _record_kv_cache_usage(self, timing):
        if timing is None or self.block_manager is None:
            return
        bs = int(self.config.cache_block_size)
        used = len(self.block_manager.used_block_ids)
        cap = len(self.block_manager.blocks)
        timing["kv_cache_block_size"] = bs
        timing["kv_cache_block_bytes"] = int(self.kv_cache_block_bytes)
        timing["kv_cache_slot_bytes"] = int(self.kv_cache_block_bytes // bs)
        for name, val in (("used_blocks", used), ("used_slots", used * bs), ("used_bytes", used * self.kv_cache_block_bytes),
                          ("capacity_blocks", cap), ("capacity_slots", cap * bs),
                          ("capacity_bytes", cap * self.kv_cache_block_bytes)):
            key = f"kv_cache_peak_{name}"
            timing[key] = max(timing.get(key, 0), val)
        timing["kv_cache_peak_used_gb"] = timing["kv_cache_peak_used_bytes"] / (1024 ** 3)
        timing["kv_cache_peak_capacity_gb"] = timing["kv_cache_peak_capacity_bytes"] / (1024 ** 3)

    # ------------------------------------------------------------------ KV cache
    def _reset_acache_state(self):
        self.shared_prefix_len = 0
        self.shared_prefix_blocks = 0
        self.acache_ready = False
        self.shared_prefix_token_ids = ()
        self._affix_relocation_enabled = False
        self._affix_relocation_max_position = 0
        self._relocated_affix_slot_offset = None

    def _release_kv_cache(self):
        self._decode_graphs.clear()   # they read the cache that goes away (and hold memory of their own)
        self._decode_graph = self._graph_with_pending_timers = None
        for m in self._attn_layers:
            m.k_cache = m.v_cache = torch.tensor([])
        self.kv_cache = None
        self.block_manager = None
        self._reset_acache_state()
        if self.device.type == "cuda":
            gc.collect()
            torch.cuda.empty_cache()

    def allocate_kv_cache(self, num_blocks: int | None = None):
        """One tensor ``[2 (K|V), layers, blocks, block_size, kv_heads, head_dim]``; layer l
        binds ``kv_cache[0, l]`` / ``kv_cache[1, l]`` (reference: model_runner.py:165-218)."""
        config = self.config
        nh, hkv, D, layers = self._arch()
        bs = config.cache_block_size
        dtype = _TORCH_DTYPES[getattr(config, "kv_cache_dtype", "bfloat16")]
        self.kv_cache_block_bytes = 2 * layers * bs * hkv * D * torch.empty((), dtype=dtype).element_size()
        if num_blocks is None and config.num_kvcache_blocks < 0:
            free, total = torch.cuda.mem_get_info()
            stats = torch.cuda.memory_stats()
            peak, current = stats["allocated_bytes.all.peak"], stats["allocated_bytes.all.current"]
            reserve = int(max(float(config.acache_memory_reserve_gb), 0.0) * (1024 ** 3)) if config.enable_acache else 0
            available = total * config.gpu_memory_utilization - (total - free) - peak + current - reserve
            num_blocks = int(available // self.kv_cache_block_bytes)
        elif num_blocks is None:
            num_blocks = config.num_kvcache_blocks
        config.num_kvcache_blocks = int(num_blocks)
        assert config.num_kvcache_blocks >= 1, "Not enough GPU memory."
        if self.kv_cache is not None:
            self._release_kv_cache()
        self.kv_cache = torch.empty(2, layers, config.num_kvcache_blocks, bs, hkv, D, dtype=dtype, device=self.device)
        self._reset_acache_state()
        for layer_id, m in enumerate(self._attn_layers):
            m.k_cache = self.kv_cache[0, layer_id]
            m.v_cache = self.kv_cache[1, layer_id]
            m.use_reference_attention = config.use_reference_attention
            m.shared_prefix_len = 0
            m.probe = m.probe_batch = None
        self.block_manager = BlockManager(config.num_kvcache_blocks, bs)

    def _flat_kv(self):
        """K and V as ``[layers, slots, kv_heads, head_dim]`` views."""
        _, layers, nb, bs, hkv, D = self.kv_cache.shape
        k = self.kv_cache[0].view(layers, nb * bs, hkv, D)
        return k, self.kv_cache[1].view_as(k)

    def _shared_affix_k(self, layer_idx: int):
        return self._flat_kv()[0][layer_idx, : self.shared_prefix_len]

    # ------------------------------------------------------------------ relocation
    def _configure_affix_relocation(self, seqs):
        """Builds the relocation RoPE tables when some request places the affix at a
        non-zero offset, and tells the attention layers how long the shared span is
        (reference: model_runner.py:231-273)."""
        uses_rope = bool(getattr(self.config.hf_config, "rope", True))
        required = uses_rope and any(seq.affix_start != 0 for seq in seqs)
        max_position = max((len(seq) for seq in seqs), default=0)
        if not required and not self._affix_relocation_enabled:
            return
        if required and self._affix_relocation_enabled and self._affix_relocation_max_position >= max_position:
            return
        cos = sin = None
        for m in self._attn_layers:
            m.shared_prefix_len = self.shared_prefix_len if required else 0
            if not required:
                continue
            if m.relocation_rope_cos.shape[0] >= max_position:
                continue
            if cos is None:
                theta, tdt = self._rope_spec()
                n = 1 << max(max_position - 1, 1).bit_length()
                cos, sin = build_rope_table(n, m.head_dim, theta, tdt, self.device)
            m.relocation_rope_cos, m.relocation_rope_sin = cos, sin
        self._affix_relocation_enabled = required
        self._affix_relocation_max_position = max_position if required else 0

    def _attention_read_layout(self, seq, use_query_relocation: bool):
        return attention_read_layout(seq, use_query_relocation, self.shared_prefix_len)

    def _group_shared_span(self, seqs, relocation_materialized: bool, use_query_relocation: bool) -> bool:
        """Whether block decode hands attention the run layout (``attention_read_runs``) and lets it
        stage the shared span once per group of requests.  Needs: every request reads the same
        span (same first slot, same length); at most 32 (query, head-in-group) rows per request;
        no key-side relocation, which rotates a key by (its index - its slot) and so needs the
        logical order."""
        if not getattr(self.config, "group_shared_span", False) or len(seqs) < 2:
            return False
        if self._affix_relocation_enabled and not relocation_materialized and not use_query_relocation:
            return False
        n_heads, n_kv, _, _ = self._arch()
        if self.config.block_length * (n_heads // n_kv) > 32 or self.kv_cache.dtype == torch.float32:
            return False
        spans = {attention_read_runs(s)[1:] for s in seqs}
        if len(spans) != 1 or next(iter(spans))[0] <= 0:
            return False
        return True

    def _use_query_side_affix_relocation(self, relocation_materialized: bool):
        return self._affix_relocation_enabled and not relocation_materialized and self.config.max_num_seqs != 1

    def _reserve_single_sequence_relocation_workspace(self, seq, *, force: bool = False):
        """Pins the blocks right behind the shared affix as the destination of a
        materialised relocation (reference: model_runner.py:291-312)."""
        bm = self.block_manager
        if (self.config.max_num_seqs != 1 and not force) or seq.affix_start == 0:
            return False
        if self._relocated_affix_slot_offset is not None:
            if bm.can_allocate(seq):
                return True
            bm.release_prefix_tail(self.shared_prefix_blocks)
            self._relocated_affix_slot_offset = None
            return False
        need = self.shared_prefix_blocks
        if len(bm.free_block_ids) < need + seq.num_cache_blocks:
            return False
        end = self.shared_prefix_blocks + need
        if any(not bm.blocks[b].is_free for b in range(self.shared_prefix_blocks, end)):
            return False
        bm.reserve_prefix(end)
        self._relocated_affix_slot_offset = self.shared_prefix_blocks * self.config.cache_block_size
        self._record_kv_cache_usage(self._active_timing)
        return True

    def _materialize_single_sequence_affix(self, seq):
        """Relocated copy of the affix in the workspace + re-pointing of the request's
        shared read slots (reference: model_runner.py:314-341)."""
        if self._relocated_affix_slot_offset is None or seq.affix_start == 0:
            seq.relocated_affix_materialized = False
            return
        self._configure_affix_relocation([seq])
        t0 = self._start_timing()
        k, v = self._flat_kv()
        a = self._attn_layers[0]
        materialize_relocated_affix(k, v, a.relocation_rope_cos, a.relocation_rope_sin,
                                    self._relocated_affix_slot_offset, seq.affix_len, seq.affix_start)
        lo = seq.shared_slot_offset
        hi = lo + seq.affix_len
        base = self._relocated_affix_slot_offset
        rsm = seq.read_slot_map
        for local, pos in enumerate(range(seq.affix_start, seq.affix_end)):
            if lo <= rsm[pos] < hi:
                rsm[pos] = base + local
        seq._read_runs = None   # the map was edited in place: the cached run layout is stale
        seq.relocated_affix_materialized = True
        self._finish_timing(self._active_timing, "affix_materialize", t0)

    # ------------------------------------------------------------------ shared affix
    def _resolve_declared_prefix_tokens(self, seqs) -> tuple[int, ...]:
        if not seqs or seqs[0].prompt_affix_len <= 0:
            return ()
        n = seqs[0].prompt_affix_len
        toks = tuple(seqs[0].prompt_affix_token_ids)
        for seq in seqs[1:]:
            if seq.prompt_affix_len != n:
                raise ValueError("ACache requires the same explicit affix length for every sequence in the batch.")
            if tuple(seq.prompt_affix_token_ids) != toks:
                raise ValueError("ACache requires identical explicit affix tokens for every sequence in the batch.")
        return toks

    def _precompute_shared_prefix(self, prefix_tokens):
        """Forward of the affix alone at positions ``0..A-1``; K (post-RoPE) and V land in
        slots ``0..A-1`` of blocks ``0..ceil(A/Bk)-1`` (reference: model_runner.py:492-541)."""
        n = len(prefix_tokens)
        if n == 0:
            return
        toks = tuple(prefix_tokens)
        if self.acache_ready and self.shared_prefix_token_ids == toks:
            return
        bs = self.config.cache_block_size
        shared_blocks = -(-n // bs)
        self.block_manager.reserve_prefix(shared_blocks)
        self._record_kv_cache_usage(self._active_timing)
        timing = self._active_timing
        t0 = self._start_timing()
        dev = self._staging.ship(
            input_ids=np.asarray(prefix_tokens, dtype=np.int64), cu=np.asarray([0, n], dtype=np.int32),
            slots=np.arange(n, dtype=np.int32), table=np.arange(shared_blocks, dtype=np.int32)[None, :],
            positions=np.arange(n, dtype=np.int64))
        self._finish_timing(timing, "shared_prefix_prepare", t0)
        set_context(True, dev["cu"], dev["cu"], None, n, n, dev["slots"], dev["table"])
        try:
            t0 = self._start_timing()
            self._forward_model(dev["input_ids"], dev["positions"], compute_logits=False, max_pos=n)
            self._finish_timing(timing, "shared_prefix_forward", t0)
            self._add_timing_count(timing, "shared_prefix_forward_calls", 1)
        finally:
            reset_context()
        self.shared_prefix_len = n
        self.shared_prefix_blocks = shared_blocks
        self.shared_prefix_token_ids = toks
        self.acache_ready = True

    def load_shared_prefix_kv(self, prefix_tokens, packed_kv: torch.Tensor):
        """Installs affix K/V computed elsewhere (another replica) instead of running
        the affix forward: ``packed_kv [2, layers, A, kv_heads, head_dim]``."""
        n = len(prefix_tokens)
        bs = self.config.cache_block_size
        shared_blocks = -(-n // bs)
        self.block_manager.reserve_prefix(shared_blocks)
        k, v = self._flat_kv()
        k[:, :n].copy_(packed_kv[0])
        v[:, :n].copy_(packed_kv[1])
        self.shared_prefix_len, self.shared_prefix_blocks = n, shared_blocks
        self.shared_prefix_token_ids = tuple(prefix_tokens)
        self.acache_ready = True

    def export_shared_prefix_kv(self) -> torch.Tensor:
        """Contiguous ``[2, layers, A, kv_heads, head_dim]`` copy of the shared affix K/V (the
        packing a collective needs: in the cache a layer's affix rows are ``blocks * block_size``
        slots apart)."""
        k, v = self._flat_kv()
        n = self.shared_prefix_len
        return torch.stack((k[:, :n], v[:, :n]))

    def _minimum_kv_cache_blocks_for_acache(self, seqs, prefix_len):
        shared = -(-prefix_len // self.config.cache_block_size)
        if not seqs:
            return max(shared, 1)
        return max(shared + max(seq.num_cache_blocks for seq in seqs), 1)

    _selection_kv_cache_blocks = _minimum_kv_cache_blocks_for_acache  # selection is per request

    def _shrink_kv_cache_for_acache(self, seqs, prefix_len, minimum_blocks=None):
        """Out-of-memory recovery: give 4 blocks back and retry (reference: model_runner.py:592-616)."""
        if self.device.type != "cuda" or self.kv_cache_block_bytes <= 0:
            return False
        current = int(self.config.num_kvcache_blocks)
        if minimum_blocks is None:
            minimum_blocks = self._minimum_kv_cache_blocks_for_acache(seqs, prefix_len)
        if current <= minimum_blocks:
            return False
        new_blocks = max(minimum_blocks, current - min(4, current - minimum_blocks))
        if new_blocks >= current:
            return False
        print(f"[acache] anchor selection OOM, shrinking KV cache blocks from {current} to {new_blocks} and retrying.")
        self.allocate_kv_cache(num_blocks=new_blocks)
        return True

    def _ensure_shared_prefix(self, prefix_token_ids, seqs, minimum_blocks=None):
        while True:
            try:
                self._precompute_shared_prefix(list(prefix_token_ids))
                return
            except torch.OutOfMemoryError as oom:
                err = torch.OutOfMemoryError(str(oom))
            gc.collect()
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
            if not self._shrink_kv_cache_for_acache(seqs, len(prefix_token_ids), minimum_blocks=minimum_blocks):
                raise err

    # ------------------------------------------------------------------ anchor selection
    def _compute_anchor_positions(self, seq):
        return self._compute_anchor_positions_batch([seq])[0]

    def _finalize_anchor_selection_probe_layout(self, seq, shared_slot_offset: int = 0):
        """Probe layout: anchor slots stay reserved but unused; the queries are the
        request's own tokens, the keys the whole shared affix plus those tokens
        (reference: model_runner.py:546-569)."""
        own = seq.private_slots()
        dynamic = own[seq.num_anchor_tokens:]
        outside = np.asarray(seq.non_affix_positions, dtype=np.int64)
        assert dynamic.shape[0] == outside.shape[0]
        read = np.full(seq.num_tokens, -1, dtype=np.int64)
        read[seq.affix_start: seq.affix_end] = shared_slot_offset + np.arange(seq.affix_len)
        read[outside] = dynamic
        seq.shared_slot_offset = shared_slot_offset
        seq.recompute_positions = outside.tolist()
        seq.recompute_slot_mapping = dynamic.tolist()
        seq.read_slot_map = read.tolist()

    def anchor_importance_scores(self, seqs):
        """Runs the anchor-selection probe and returns the fp32 influence scores
        ``[len(seqs), affix_len]`` (device tensor).  One full-depth forward over each
        request's own tokens; every layer adds softmax-over-affix attention mass of the
        mask-token queries (reference: model_runner.py:640-832).  Temporarily allocates
        blocks for requests that have none, exactly as the reference does."""
        affix_len = seqs[0].affix_len
        for seq in seqs[1:]:
            if seq.affix_len != affix_len:
                raise ValueError("Batched Anchor Selection requires a consistent explicit prefix affix length.")
        timing = self._active_timing
        t_prep = self._start_timing()
        importance = torch.zeros(len(seqs), affix_len, device=self.device, dtype=torch.float32)
        saved, temporarily_allocated, workspace = [], [], False
        try:
            for seq in seqs:
                saved.append((seq, list(seq.block_table), list(seq.anchor_positions), list(seq.recompute_positions),
                              list(seq.recompute_slot_mapping), list(seq.read_slot_map), seq.shared_slot_offset,
                              seq.relocated_affix_materialized))
                if not seq.block_table:
                    if len(seqs) == 1:
                        workspace = self._reserve_single_sequence_relocation_workspace(seq, force=True)
                    if not self.block_manager.can_allocate(seq):
                        raise torch.OutOfMemoryError("Not enough KV cache blocks for anchor-selection probe.")
                    self.block_manager.allocate(seq)
                    self._record_kv_cache_usage(timing)
                    temporarily_allocated.append(seq)
                seq.anchor_positions = []
                self._finalize_anchor_selection_probe_layout(seq)
                if workspace:
                    self._materialize_single_sequence_affix(seq)
            input_ids, position_ids, _ = self.prepare_caching_acache(seqs, use_query_relocation=False)
            cu = self._last_cu_q_host
            self._add_timing_count(timing, "anchor_selection_query_tokens", int(input_ids.numel()))
            self._add_timing_count(timing, "anchor_selection_kv_tokens", sum(len(s) for s in seqs))
            # rows of mask tokens, per request, as indices into the ragged query batch
            probes = []
            a0 = self._attn_layers[0]
            for b, seq in enumerate(seqs):
                toks = np.asarray(seq.token_ids, dtype=np.int64)[np.asarray(seq.recompute_positions, dtype=np.int64)]
                rows = (np.nonzero(toks == self.config.mask_id)[0] + cu[b]).astype(np.int32)
                p = _Probe()
                p.q_rows = rows
                p.affix_len = affix_len
                p.affix_shift = int(seq.affix_start)
                p.importance = importance[b]
                p.rope_cos, p.rope_sin = a0.relocation_rope_cos, a0.relocation_rope_sin
                probes.append(p)
            batch = None
            if any(p.q_rows.size for p in probes):
                host = {f"r{i}": p.q_rows for i, p in enumerate(probes)}
                if len(probes) > 1:   # the same rows once more as one array for the batched score kernel
                    counts = [int(p.q_rows.size) for p in probes]
                    host["all"] = np.concatenate([p.q_rows for p in probes]).astype(np.int32)
                    host["off"] = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
                    host["shift"] = np.asarray([p.affix_shift for p in probes], dtype=np.int32)
                dev_rows = self._staging.ship(**host)
                for i, p in enumerate(probes):
                    p.q_rows = dev_rows[f"r{i}"]
                if len(probes) > 1:
                    batch = _ProbeBatch()
                    batch.q_rows, batch.offsets, batch.max_q_rows = dev_rows["all"], dev_rows["off"], max(counts)
                    batch.shifts = dev_rows["shift"] if any(p.affix_shift for p in probes) else None
                    batch.importance, batch.affix_len = importance, affix_len
                    batch.rope_cos, batch.rope_sin = a0.relocation_rope_cos, a0.relocation_rope_sin
                    batch.usable = True
            else:
                for p in probes:
                    p.q_rows = torch.empty(0, dtype=torch.int32, device=self.device)
            self._finish_timing(timing, "anchor_selection_prepare", t_prep)
            for m in self._attn_layers:
                m.probe, m.probe_batch = probes, batch
            t_fwd = self._start_timing()
            self._forward_model(input_ids, position_ids, compute_logits=False, max_pos=max(len(s) for s in seqs))
            self._finish_timing(timing, "anchor_selection_forward", t_fwd)
            self._add_timing_count(timing, "anchor_selection_forward_calls", 1)
            self._add_timing_count(timing, "anchor_selection_sequences", len(seqs))
        finally:
            for m in self._attn_layers:
                m.probe = m.probe_batch = None
            reset_context()
            for seq in reversed(temporarily_allocated):
                if seq.block_table:
                    self.block_manager.deallocate(seq)
            for (seq, table, anchors, rpos, rslots, rsm, sso, mat) in saved:
                seq.block_table, seq.anchor_positions = table, anchors
                seq.recompute_positions, seq.recompute_slot_mapping, seq.read_slot_map = rpos, rslots, rsm
                seq.shared_slot_offset, seq.relocated_affix_materialized = sso, mat
            if workspace:
                self.block_manager.release_prefix_tail(self.shared_prefix_blocks)
                self._relocated_affix_slot_offset = None
        return importance

    def _compute_anchor_positions_batch(self, seqs):
        """Anchor positions (logical, ascending) of each request: influence scores from the
        probe, then radix-select top-k with ties to the lowest index
        (reference: model_runner.py:640-845)."""
        result = [[] for _ in seqs]
        active = [(i, s) for i, s in enumerate(seqs) if s.acache_enabled and s.num_anchor_tokens > 0]
        if not active or active[0][1].affix_len <= 0:
            return result
        act_seqs = [s for _, s in active]
        importance = self.anchor_importance_scores(act_seqs)
        timing = self._active_timing
        t0 = self._start_timing()
        largest = self.config.selection_mode != "bottom"
        ks = {s.num_anchor_tokens for s in act_seqs}
        offsets = self._staging.ship(off=np.asarray([s.affix_start for s in act_seqs], dtype=np.int32))["off"]
        if len(ks) == 1:
            picked = ops.anchor_topk(importance, ks.pop(), largest, offsets).cpu()
            self.d2h_bytes += picked.numel() * 8
            for (i, _), row in zip(active, picked.tolist()):
                result[i] = row
        else:
            for b, (i, s) in enumerate(active):
                row = ops.anchor_topk(importance[b: b + 1], s.num_anchor_tokens, largest, offsets[b: b + 1]).cpu()
                self.d2h_bytes += row.numel() * 8
                result[i] = row[0].tolist()
        self._finish_timing(timing, "anchor_selection_topk", t0)
        return result

    def _prepare_acache(self, seqs):
        toks = self._resolve_declared_prefix_tokens(seqs)
        if not toks:
            return ()
        for seq in seqs:
            seq.enable_acache(len(toks), self.config.anchor_ratio, affix_start=seq.prompt_affix_start,
                              affix_end=seq.prompt_affix_end)
        return toks

    def _select_anchor_positions_batched(self, seqs) -> bool:
        """Anchor selection of several new requests with ragged batched probe forwards instead of
        one forward per request.  A request's scores do not depend on what else is in the batch,
        and relocation inside the kernel gives the bits of the materialised copy the one-request
        probe reads, so the anchors are the ones of the per-request procedure; what that procedure
        does to the allocator (every probe takes blocks from the head of the free list and returns
        them to its tail, around an optional relocation workspace) is replayed on the host
        afterwards from the state before the probes.  Returns False, with nothing changed, when
        the batch cannot be probed this way (then the per-request procedure runs)."""
        bm = self.block_manager
        todo = [s for s in seqs if s.acache_enabled and s.num_anchor_tokens > 0 and s.affix_len > 0]
        if (len(todo) < 2 or self.config.max_num_seqs == 1 or any(s.block_table for s in todo)
                or self._relocated_affix_slot_offset is not None
                or any(s.num_cache_blocks > len(bm.free_block_ids) for s in todo)):
            return False
        # a batch rotates the shared keys inside the attention kernel where the one-request probe
        # reads a materialised copy; over a long span that costs more than the batching saves
        if any(s.affix_start != 0 for s in todo) and self.shared_prefix_len > 2048:
            return False
        state = bm.snapshot()
        budget = max(int(getattr(self.config, "max_num_batched_tokens", 16384)), 1)
        picked = {}
        try:
            i = 0
            while i < len(todo):
                chunk, rows, blocks = [], 0, 0
                while i < len(todo):
                    s = todo[i]
                    n = len(s) - s.affix_len
                    if chunk and (rows + n > budget or blocks + s.num_cache_blocks > len(bm.free_block_ids)):
                        break
                    chunk.append(s)
                    rows, blocks = rows + n, blocks + s.num_cache_blocks
                    i += 1
                for s, anchors in zip(chunk, self._compute_anchor_positions_batch(chunk)):
                    picked[s.seq_id] = anchors
        except torch.OutOfMemoryError:
            bm.restore(state)
            for s in todo:
                s.block_table = []
            return False
        bm.restore(state)
        for s in seqs:
            if s.seq_id not in picked:
                s.set_anchor_positions([])
                continue
            # the allocator traffic of this request's own probe (reference: model_runner.py:684-699,799-821)
            workspace = self._reserve_single_sequence_relocation_workspace(s, force=True)
            bm.allocate(s)
            self._record_kv_cache_usage(self._active_timing)
            bm.deallocate(s)
            if workspace:
                bm.release_prefix_tail(self.shared_prefix_blocks)
                self._relocated_affix_slot_offset = None
            s.set_anchor_positions(picked[s.seq_id])
        return True

    def _select_anchor_positions_for_sequences(self, seqs, prefix_token_ids, allow_kv_cache_resize, minimum_blocks=None):
        """One probe per request, as the reference (model_runner.py:862-907), with its
        out-of-memory recovery: shrink the cache, recompute the affix, retry.  With
        ``config.batch_anchor_selection`` the probes of a batch of new requests run as ragged
        batched forwards first (same anchors, same allocator state afterwards)."""
        if getattr(self.config, "batch_anchor_selection", False) and self._select_anchor_positions_batched(seqs):
            return
        for seq in seqs:
            while True:
                try:
                    seq.set_anchor_positions(self._compute_anchor_positions_batch([seq])[0])
                    break
                except torch.OutOfMemoryError as oom:
                    err = torch.OutOfMemoryError(str(oom))
                gc.collect()
                if self.device.type == "cuda":
                    torch.cuda.empty_cache()
                if not allow_kv_cache_resize or not self._shrink_kv_cache_for_acache(
                        seqs, len(prefix_token_ids), minimum_blocks=minimum_blocks):
                    raise err
                self._ensure_shared_prefix(prefix_token_ids, seqs, minimum_blocks=minimum_blocks)

    def _prepare_admitted_sequences_for_acache(self, seqs, prefix_token_ids, allow_kv_cache_resize):
        if not seqs:
            return
        if self.acache_ready and self.shared_prefix_token_ids != prefix_token_ids:
            raise ValueError("ACache prefix mode requires a consistent shared prefix across active requests.")
        target = int(self.config.num_kvcache_blocks)
        minimum = min(target, self._selection_kv_cache_blocks(seqs, len(prefix_token_ids)))
        try:
            if not self.acache_ready:
                if allow_kv_cache_resize:
                    self._ensure_shared_prefix(prefix_token_ids, seqs, minimum_blocks=minimum)
                else:
                    self._precompute_shared_prefix(list(prefix_token_ids))
            self._select_anchor_positions_for_sequences(seqs, prefix_token_ids, allow_kv_cache_resize, minimum)
        except Exception:
            if allow_kv_cache_resize and self.config.num_kvcache_blocks != target:
                self.allocate_kv_cache(num_blocks=target)
            raise
        if allow_kv_cache_resize and self.config.num_kvcache_blocks != target:
            self.allocate_kv_cache(num_blocks=target)
            self._ensure_shared_prefix(prefix_token_ids, seqs)

    def _finalize_sequence_layout(self, seq):
        seq.finalize_slot_mapping()
        self._materialize_single_sequence_affix(seq)

    def _collect_admissible_sequences(self, prompts, next_prompt_idx, current_batch_size, max_num_seqs):
        """FIFO admission by free blocks and running-set size; stops at the first
        request that does not fit (reference: model_runner.py:960-976)."""
        picked = admissible_prefix(islice(prompts, next_prompt_idx, None), current_batch_size, max_num_seqs,
                                   len(self.block_manager.free_block_ids))
        return picked, next_prompt_idx + len(picked)

    def _admit_sequences_with_acache(self, batched_prompts, new_prompts, prefix_token_ids, allow_kv_cache_resize):
        if not new_prompts:
            return 0
        self._prepare_admitted_sequences_for_acache(new_prompts, prefix_token_ids, allow_kv_cache_resize)
        self._reserve_single_sequence_relocation_workspace(new_prompts[0])
        admitted = 0
        for seq in new_prompts:
            if not self.block_manager.can_allocate(seq):
                break
            self.block_manager.allocate(seq)
            self._record_kv_cache_usage(self._active_timing)
            self._finalize_sequence_layout(seq)
            batched_prompts.append(seq)
            admitted += 1
        return admitted

    # ------------------------------------------------------------------ step metadata
    def _note_attention_work(self, phase, q_lens, k_lens):
        """Algorithmic work of one attention launch of the coming forward, for the optional
        device timers: FLOPs ``4 q kv nh D`` and bytes (K and V read once per KV head, q read
        and the output written once)."""
        nh, hkv, D, _ = self._arch()
        es = self.kv_cache.element_size()
        q = np.asarray(q_lens, dtype=np.float64)
        k = np.asarray(k_lens, dtype=np.float64)
        flops = float((4.0 * q * k * nh * D).sum())
        nbytes = float((2.0 * k * hkv * D * es + 2.0 * q * nh * D * es).sum())
        aa.ATTENTION_PHASE = phase
        aa.ATTENTION_WORK = nbytes if phase == "decode" else flops

    def prepare_block_tables(self, seqs):
        width = max(len(seq.block_table) for seq in seqs)
        table = np.full((len(seqs), width), -1, dtype=np.int32)
        for i, seq in enumerate(seqs):
            table[i, : len(seq.block_table)] = seq.block_table
        return self._staging.ship(t=table)["t"]

    @staticmethod
    def _pick(seqs, active_indices):
        if active_indices is None:
            return list(seqs)
        if torch.is_tensor(active_indices):
            active_indices = active_indices.tolist()
        return [seqs[int(i)] for i in active_indices]

    def prepare_caching(self, seqs, active_indices=None):
        """Full-recompute refresh of the no-reuse baseline: every token of every request
        is a query, K/V go to the request's own blocks (reference: model_runner.py:1010-1068)."""
        ps = self._pick(seqs, active_indices)
        lens = np.asarray([len(s) for s in ps], dtype=np.int64)
        cu = np.zeros(len(ps) + 1, dtype=np.int32)
        cu[1:] = np.cumsum(lens)
        width = max(len(s.block_table) for s in ps)
        table = np.full((len(ps), width), -1, dtype=np.int32)
        for i, s in enumerate(ps):
            table[i, : len(s.block_table)] = s.block_table
        dev = self._staging.ship(
            input_ids=np.concatenate([np.asarray(s.token_ids, dtype=np.int64) for s in ps]),
            positions=np.concatenate([np.arange(n, dtype=np.int64) for n in lens]),
            cu=cu, slots=np.concatenate([s.private_slots() for s in ps]).astype(np.int32),
            gen_starts=(cu[:-1] + np.asarray([s.generation_start for s in ps])).astype(np.int32),
            blk_idx=np.asarray([s.current_block_idx for s in ps], dtype=np.int32), table=table)
        self._last_cu_q_host = cu
        mx = int(lens.max())
        set_context(True, dev["cu"], dev["cu"], None, mx, mx, dev["slots"], dev["table"])
        return dev["input_ids"], dev["positions"], dev["gen_starts"], dev["blk_idx"]

    def prepare_decoding(self, seqs, active_indices=None):
        """Block decode of the baseline (reference: model_runner.py:1070-1114)."""
        ps = self._pick(seqs, active_indices)
        T, bs = self.config.block_length, self.config.cache_block_size
        starts = np.asarray([s.generation_start + s.current_block_idx * T for s in ps], dtype=np.int64)
        pos = starts[:, None] + np.arange(T, dtype=np.int64)[None, :]
        width = max(len(s.block_table) for s in ps)
        table = np.full((len(ps), width), -1, dtype=np.int32)
        for i, s in enumerate(ps):
            table[i, : len(s.block_table)] = s.block_table
        slots = table[np.arange(len(ps))[:, None], pos // bs] * bs + pos % bs
        lens = np.asarray([len(s) for s in ps], dtype=np.int32)
        cu_k = np.zeros(len(ps) + 1, dtype=np.int32)
        cu_k[1:] = np.cumsum(lens)
        dev = self._staging.ship(positions=pos, slots=slots.astype(np.int32).reshape(-1), seqlens=lens, table=table,
                                 cu_q=np.arange(0, (len(ps) + 1) * T, T, dtype=np.int32), cu_k=cu_k)
        # block tables with ragged queries cover the decode form too
        set_context(True, dev["cu_q"], dev["cu_k"], dev["seqlens"], T, int(lens.max()), dev["slots"], dev["table"])
        return dev["positions"]

    def prepare_caching_acache(self, seqs, active_indices=None, use_query_relocation=None):
        """Refresh ("anchor-only recompute") metadata: the queries are the anchors plus the
        request's own tokens, K/V of those rows go to the private slots, attention reads
        every logical position through the slot map (reference: model_runner.py:1295-1395)."""
        ps = self._pick(seqs, active_indices)
        self._configure_affix_relocation(ps)
        materialized = all(getattr(s, "relocated_affix_materialized", False) for s in ps)
        if use_query_relocation is None:
            use_query_relocation = self.config.max_num_seqs != 1
        use_query_relocation = self._affix_relocation_enabled and not materialized and bool(use_query_relocation)
        q_lens = np.asarray([len(s.recompute_positions) for s in ps], dtype=np.int64)
        k_lens = np.asarray([len(s) for s in ps], dtype=np.int64)
        cu_q = np.zeros(len(ps) + 1, dtype=np.int32)
        cu_k = np.zeros(len(ps) + 1, dtype=np.int32)
        cu_q[1:], cu_k[1:] = np.cumsum(q_lens), np.cumsum(k_lens)
        ids, pos, slots, read, shared_lens, shifts, bqs = [], [], [], [], [], [], []
        for b, s in enumerate(ps):
            rp = np.asarray(s.recompute_positions, dtype=np.int64)
            assert len(s.recompute_slot_mapping) == rp.shape[0] and len(s.read_slot_map) == len(s)
            ids.append(np.asarray(s.token_ids, dtype=np.int64)[rp])
            pos.append(rp)
            slots.append(np.asarray(s.recompute_slot_mapping, dtype=np.int32))
            layout, n_shared = self._attention_read_layout(s, use_query_relocation)
            read.append(np.asarray(layout, dtype=np.int32))
            shared_lens.append(n_shared)
            shifts.append(s.affix_start if self._affix_relocation_enabled else 0)
            first = s.generation_start + s.current_block_idx * s.block_length
            hit = np.searchsorted(rp, first)
            bqs.append(cu_q[b] + (int(hit) if hit < rp.shape[0] and rp[hit] == first else s.block_query_start()))
        arrays = dict(input_ids=np.concatenate(ids), positions=np.concatenate(pos), cu_q=cu_q, cu_k=cu_k,
                      kv_seqlens=k_lens.astype(np.int32), slots=np.concatenate(slots), read=np.concatenate(read),
                      bqs=np.asarray(bqs, dtype=np.int32))
        if use_query_relocation:
            arrays["shared_lens"] = np.asarray(shared_lens, dtype=np.int32)
        if not materialized:
            arrays["shifts"] = np.asarray(shifts, dtype=np.int32)
        dev = self._staging.ship(**arrays)
        self._last_cu_q_host = cu_q
        self._note_attention_work("refresh", q_lens, k_lens)
        set_context(True, dev["cu_q"], dev["cu_k"], dev["kv_seqlens"], int(q_lens.max()), int(k_lens.max()),
                    dev["slots"], None, True, dev["read"], dev.get("shared_lens"), dev.get("shifts"))
        return dev["input_ids"], dev["positions"], dev["bqs"]

    def prepare_decoding_acache(self, seqs, active_indices=None, graphs=None):
        """Block-decode metadata: ``[B, block_length]`` queries at the working block's
        positions, K/V written in place at the block's read slots
        (reference: model_runner.py:1397-1471).  ``graphs``: a dict of captured decode forwards;
        the metadata then goes to the fixed buffers of the matching one (made on demand), which
        is left in ``self._decode_graph``."""
        ps = self._pick(seqs, active_indices)
        T = self.config.block_length
        self._configure_affix_relocation(ps)
        materialized = all(getattr(s, "relocated_affix_materialized", False) for s in ps)
        use_qr = self._use_query_side_affix_relocation(materialized)
        k_lens = np.asarray([len(s) for s in ps], dtype=np.int64)
        grouped = self._group_shared_span(ps, materialized, use_qr)
        starts, slots, read, shared_lens, shifts = [], [], [], [], []
        for s in ps:
            st = s.generation_start + s.current_block_idx * T
            starts.append(st)
            slots.append(np.asarray(s.read_slot_map[st: st + T], dtype=np.int32))
            layout, n_shared = attention_read_runs(s)[:2] if grouped else self._attention_read_layout(s, use_qr)
            read.append(np.asarray(layout, dtype=np.int32))
            shared_lens.append(n_shared)
            shifts.append(s.affix_start if self._affix_relocation_enabled else 0)
        cu_k = np.zeros(len(ps) + 1, dtype=np.int32)
        cu_k[1:] = np.cumsum([r.shape[0] for r in read])
        pos = np.asarray(starts, dtype=np.int64)[:, None] + np.arange(T, dtype=np.int64)[None, :]
        arrays = dict(positions=pos, cu_q=np.arange(0, (len(ps) + 1) * T, T, dtype=np.int32), cu_k=cu_k,
                      kv_seqlens=k_lens.astype(np.int32), slots=np.concatenate(slots), read=np.concatenate(read))
        if use_qr or grouped:
            arrays["shared_lens"] = np.asarray(shared_lens, dtype=np.int32)
        if not materialized:
            arrays["shifts"] = np.asarray(shifts, dtype=np.int32)
        staging = self._staging
        self._decode_graph = None
        if graphs is not None:
            key = (len(ps), grouped, tuple(sorted(arrays)))
            graph = graphs.get(key)
            if graph is None or not graph.staging.fits(**arrays):
                # read-map capacity and RoPE table length: powers of two with head-room
                cap = 1 << int(2 * arrays["read"].size - 1).bit_length()
                max_pos = 1 << int(2 * int(k_lens.max()) - 1).bit_length()
                graphs.pop(key, None)
                graph = graphs[key] = _DecodeGraph(self, len(ps), {k: a.dtype for k, a in arrays.items()}, cap, max_pos)
                self._evict_decode_graphs(graphs, keep=key)
            else:
                graphs[key] = graphs.pop(key)      # most recently used last
            if int(k_lens.max()) <= graph.max_pos:
                staging, self._decode_graph = graph.staging, graph
        dev = staging.ship(**arrays)
        self._note_attention_work("decode", [T] * len(ps), k_lens)
        set_context(False, dev["cu_q"], dev["cu_k"], dev["kv_seqlens"], T, int(k_lens.max()), dev["slots"], None, True,
                    dev["read"], dev.get("shared_lens"), dev.get("shifts"))
        get_context().group_shared_span = grouped
        return dev["positions"]

    # Every captured decode forward keeps its own logits tensor ``[rows * block_length, vocab]`` alive
    # (only intermediates are shared between graphs), so the set is bounded: at most this many
    # graphs and this many bytes of logits; the least recently used ones are dropped and captured
    # again if their row count comes back.  The bound stays inside ``acache_memory_reserve_gb``.
    MAX_DECODE_GRAPHS = 8
    MAX_DECODE_GRAPH_LOGITS_BYTES = 2 << 30

    def _evict_decode_graphs(self, graphs, keep):
        hf = self.config.hf_config
        vocab = int(getattr(hf, "embedding_size", None) or getattr(hf, "vocab_size", 0) or 0)
        row_bytes = self.config.block_length * vocab * self.kv_cache.element_size()
        def held(g):   # a graph whose output head returns statistics keeps no logits
            return 0 if isinstance(g.logits, tuple) and g.logits[0] is None else g.tokens.shape[0] * row_bytes

        while len(graphs) > 1:
            total = sum(held(g) for g in graphs.values())
            if len(graphs) <= self.MAX_DECODE_GRAPHS and total <= self.MAX_DECODE_GRAPH_LOGITS_BYTES:
                break
            oldest = next(k for k in graphs if k != keep)
            victim = graphs.pop(oldest)
            if self._graph_with_pending_timers is victim:
                self.harvest_graph_timers()
            if self._decode_graph is victim:
                self._decode_graph = None
            victim.graph = victim.logits = None

    def _graph_stamp(self):
        """What a captured forward has baked in besides its own buffers: the cache, the RoPE
        tables and the shared-span length.  A graph is captured again when any of them changed."""
        a0 = self._attn_layers[0]
        ptr_of = lambda t: t.data_ptr() if t is not None and t.numel() else 0
        return (ptr_of(self.kv_cache), tuple(ptr_of(r.cos) for r in self._rope_caches), a0.shared_prefix_len,
                ptr_of(a0.relocation_rope_cos), ptr_of(a0.relocation_rope_sin))

    def harvest_graph_timers(self):
        """Reads the event times of the last graph replay (it must have completed: call after a
        host synchronisation or, as the next replay does, in stream order before re-recording)."""
        graph = self._graph_with_pending_timers
        if graph is not None and graph.pending_work is not None:
            if _lib.kernel_timers_enabled():
                torch.cuda.current_stream().synchronize()
                _lib.harvest_graph_timers(graph.events, graph.pending_work)
            graph.pending_work = None
        self._graph_with_pending_timers = None

    # ------------------------------------------------------------------ sampling
    def get_transfer_index(self, logits, temperature, remasking, mask_index, x, threshold=0.9):
        """Greedy / Gumbel candidates and the confidence-threshold commit mask, returned
        like the reference does (model_runner.py:2279-2314).  The engine's loops use the
        fused in-place kernel instead; this method serves callers that want the mask."""
        x0 = torch.argmax(add_gumbel_noise(logits, temperature), dim=-1)
        if remasking == "low_confidence":
            lf = logits.float()
            p = torch.exp(torch.gather(lf, -1, x0.unsqueeze(-1)).squeeze(-1) - torch.logsumexp(lf, dim=-1))
        elif remasking == "random":
            p = torch.rand(x0.shape, device=x0.device)
        else:
            raise NotImplementedError(remasking)
        x0 = torch.where(mask_index, x0, x)
        conf = torch.where(mask_index, p, torch.full_like(p, -np.inf))
        transfer = (conf >= threshold) & mask_index
        needs = mask_index.any(dim=1) & ~transfer.any(dim=1)
        rows = torch.where(needs)[0]
        transfer[rows, torch.argmax(conf, dim=1)[rows]] = True
        return x0, transfer

    def _commit(self, logits, working_blocks, rows):
        """Unmask ``working_blocks[rows]`` from ``logits [len(rows)*T, V]`` in place."""
        cfg = self.config
        T = cfg.block_length
        if cfg.temperature == 0 and cfg.remasking == "low_confidence":
            sub = working_blocks.index_select(0, rows).contiguous()
            ops.transfer_tokens(logits, sub, cfg.mask_id, cfg.threshold)
            working_blocks.index_copy_(0, rows, sub)
            return
        sub = working_blocks.index_select(0, rows)
        lg = logits.view(rows.numel(), T, -1)
        x0, ti = self.get_transfer_index(lg, cfg.temperature, cfg.remasking, sub == cfg.mask_id, sub, cfg.threshold)
        working_blocks.index_copy_(0, rows, torch.where(ti, x0, sub))

    def _commit_output(self, logits, stats, working_blocks, rows):
        """Unmask ``working_blocks[rows]`` from a forward's output, whichever form it has."""
        if stats is None:
            return self._commit(logits.reshape(rows.numel() * self.config.block_length, -1), working_blocks, rows)
        x0, conf = stats
        sub = working_blocks.index_select(0, rows).contiguous()
        ops.apply_transfer(x0.reshape(-1), conf.reshape(-1), sub, self.config.mask_id, self.config.threshold)
        working_blocks.index_copy_(0, rows, sub)

    # ------------------------------------------------------------------ generation loops
    @torch.inference_mode()
    def generate_with_dual_cache(self, prompts, arrival_times=None):
        """No-reuse baseline: every refresh recomputes all tokens of the request
        (reference: model_runner.py:1473-1723)."""
        return self._generate(prompts, reuse=False, arrival_times=arrival_times)

    @torch.inference_mode()
    def generate_with_acache(self, prompts, arrival_times=None):
        """Generation with affix-KV reuse (reference: model_runner.py:2032-2277).  With
        ``arrival_times`` the prompts are served as a request stream (see ``_generate``)."""
        timing = self._new_timing("acache", len(prompts))
        self.last_timing = timing if timing is not None else {}
        prev, self._active_timing = self._active_timing, timing
        try:
            t0 = self._start_timing()
            prefix = self._prepare_acache(prompts)
            self._finish_timing(timing, "acache_metadata", t0)
        finally:
            self._active_timing = prev
        if not prefix:
            self._resolve_timing()
            return self.generate_with_dual_cache(prompts, arrival_times)
        return self._generate(prompts, reuse=True, prefix=prefix, timing=timing, arrival_times=arrival_times)

    def _refresh(self, batched, working_blocks, rows_host, reuse, timing):
        """Refresh forward of the requests in ``rows_host`` (indices into ``batched``) in
        chunks of ``recompute_batch_size``; the logits of each request's current block feed
        the first unmasking of that block."""
        cfg = self.config
        T = cfg.block_length
        block_offset = self._block_offset
        for i in range(0, len(rows_host), cfg.recompute_batch_size):
            chunk = rows_host[i: i + cfg.recompute_batch_size]
            seqs = [batched[r] for r in chunk]
            t0 = self._start_timing()
            if reuse:
                input_ids, positions, starts = self.prepare_caching_acache(seqs)
            else:
                input_ids, positions, gen_starts, blk_idx = self.prepare_caching(seqs)
                starts = gen_starts + T * blk_idx
            self._finish_timing(timing, "cache_prepare", t0)
            keep = starts.to(torch.int64).unsqueeze(1) + block_offset
            if self._is_dream_model():
                row_starts = torch.from_numpy(self._last_cu_q_host[:-1].astype(np.int64)).to(self.device)
                keep = self._dream_shift_keep_indices(keep, row_starts)
            keep = keep.flatten()
            t0 = self._start_timing()
            out = self._forward_model(input_ids, positions, logits_keep_indices=keep, max_pos=max(len(s) for s in seqs),
                                      greedy_stats=self._greedy())
            self._finish_timing(timing, "cache_forward", t0)
            self._add_timing_count(timing, "cache_forward_calls", 1)
            self._add_timing_count(timing, "cache_forward_nfe", len(chunk))
            t0 = self._start_timing()
            rows = torch.as_tensor(chunk, dtype=torch.int64, device=self.device)
            if self._is_dream_model():
                # only the block's first token is seeded from the refresh logits
                # (reference: model_runner.py:2114-2118)
                if out.stats is not None:
                    seed = out.stats[0].view(len(chunk), T)[:, 0]
                else:
                    logits = out.logits.view(len(chunk), T, -1)
                    if cfg.temperature > 0:
                        seed = torch.distributions.Categorical(
                            probs=torch.softmax(logits[:, 0].float() / cfg.temperature, dim=-1)).sample()
                    else:
                        seed = logits[:, 0].argmax(dim=-1)
                working_blocks[rows, 0] = seed
            else:
                self._commit_output(out.logits, out.stats, working_blocks, rows)
            self._finish_timing(timing, "cache_update", t0)
            reset_context()

    def _generate(self, prompts, reuse, prefix=(), timing=None, arrival_times=None):
        """Continuous-batching loop shared by both generation modes.  ``arrival_times`` (seconds
        from the start of the call, ascending, one per prompt) turns the hand-over of all prompts
        up front into a request stream: a request is only admissible once it has arrived, and
        admission is also attempted at every block boundary, not only when a request retires."""
        cfg = self.config
        dev = self.device
        T, mask_id = cfg.block_length, cfg.mask_id
        assert cfg.recompute_batch_size > 0, "recompute_batch_size must be larger than 0"
        max_num_seqs = cfg.max_num_seqs if cfg.max_num_seqs > 0 else len(prompts)
        if timing is None:
            timing = self._new_timing("acache" if reuse else "dual_cache", len(prompts))
            self.last_timing = timing if timing is not None else {}
        prev_timing, self._active_timing = self._active_timing, timing
        t_total = self._start_timing()
        self._block_offset = torch.arange(T, device=dev)
        total_nfe = 0
        outputs = [None] * len(prompts)
        index_of = {seq.seq_id: i for i, seq in enumerate(prompts)}
        next_idx = 0
        batched: list[Sequence] = []
        t_begin = time.perf_counter()
        self.last_completion_times = [None] * len(prompts)
        if arrival_times is not None:
            assert len(arrival_times) == len(prompts) and list(arrival_times) == sorted(arrival_times)

        def n_visible():
            if arrival_times is None:
                return len(prompts)
            now = time.perf_counter() - t_begin
            n = next_idx
            while n < len(prompts) and arrival_times[n] <= now:
                n += 1
            return n

        def admit(allow_resize):
            nonlocal next_idx
            visible = prompts if arrival_times is None else prompts[: n_visible()]
            if reuse:
                new, nxt = self._collect_admissible_sequences(visible, next_idx, len(batched), max_num_seqs)
                n_ok = self._admit_sequences_with_acache(batched, new, prefix, allow_kv_cache_resize=allow_resize)
                next_idx = nxt - (len(new) - n_ok)
            else:
                while (next_idx < len(visible) and len(batched) < max_num_seqs
                       and self.block_manager.can_allocate(visible[next_idx])):
                    seq = visible[next_idx]
                    self.block_manager.allocate(seq)
                    self._record_kv_cache_usage(timing)
                    batched.append(seq)
                    next_idx += 1

        try:
            t0 = self._start_timing()
            if arrival_times is not None and prompts and arrival_times[0] > 0:
                time.sleep(max(arrival_times[0] - (time.perf_counter() - t_begin), 0.0))
            admit(True)
            self._finish_timing(timing, "scheduler", t0)
            if not batched and prompts:
                raise RuntimeError("No requests could be admitted under the current ACache KV-cache budget."
                                   if reuse else "No requests could be admitted under the current KV-cache budget.")
            working = torch.full((len(batched), T), mask_id, dtype=torch.int64, device=dev)
            self._refresh(batched, working, list(range(len(batched))), reuse, timing)
            total_nfe += len(batched)
            decode_key = None
            decode_positions = None
            decode_graph = None
            use_graphs = bool(getattr(cfg, "use_cuda_graphs", True)) and dev.type == "cuda"
            # Every decode step commits at least one position per row, so a block needs at
            # most block_length steps unless the model keeps predicting the mask token itself
            # (the reference would then spin forever); stop with an error instead.
            steps_on_key, step_cap = 0, 8 * T + 8
            while batched or next_idx < len(prompts):
                if not batched:
                    # idle replica: wait for the next arrival, then start it like a first batch
                    if arrival_times is None:
                        raise RuntimeError("No requests could be admitted under the current KV-cache budget.")
                    time.sleep(max(arrival_times[next_idx] - (time.perf_counter() - t_begin), 0.0))
                    admit(True)
                    if not batched:
                        raise RuntimeError("No requests could be admitted under the current KV-cache budget.")
                    working = torch.full((len(batched), T), mask_id, dtype=torch.int64, device=dev)
                    self._refresh(batched, working, list(range(len(batched))), reuse, timing)
                    total_nfe += len(batched)
                    decode_key = None
                    continue
                counts = (working == mask_id).sum(dim=1).tolist()  # the step's one host sync
                self.d2h_bytes += 8 * len(counts)
                done_rows = [r for r, c in enumerate(counts) if c == 0]
                if done_rows:
                    t0 = self._start_timing()
                    rows_t = torch.as_tensor(done_rows, dtype=torch.int64, device=dev)
                    finished_tokens = working.index_select(0, rows_t).tolist()
                    self.d2h_bytes += 8 * T * len(done_rows)
                    retired = set()
                    for r, toks in zip(done_rows, finished_tokens):
                        seq = batched[r]
                        st = seq.generation_start + seq.current_block_idx * T
                        seq.token_ids[st: st + T] = toks
                        seq.current_block_idx += 1
                        if seq.current_block_idx >= seq.num_blocks_to_generate:
                            self.block_manager.deallocate(seq)
                            retired.add(r)
                            outputs[index_of[seq.seq_id]] = seq.generated_token_ids
                            self.last_completion_times[index_of[seq.seq_id]] = time.perf_counter() - t_begin
                    working[rows_t] = mask_id
                    newcomers = (arrival_times is not None and len(batched) - len(retired) < max_num_seqs
                                 and n_visible() > next_idx)
                    if retired or newcomers:
                        keep_rows = [r for r in range(len(batched)) if r not in retired]
                        batched = [batched[r] for r in keep_rows]
                        admit(len(batched) == 0)
                        fresh = torch.full((len(batched), T), mask_id, dtype=torch.int64, device=dev)
                        if keep_rows:
                            fresh[: len(keep_rows)] = working.index_select(
                                0, torch.as_tensor(keep_rows, dtype=torch.int64, device=dev))
                        working = fresh
                        counts = [counts[r] if r not in done_rows else T for r in keep_rows] + \
                                 [T] * (len(batched) - len(keep_rows))
                    else:
                        counts = [T if r in set(done_rows) else c for r, c in enumerate(counts)]
                    self._finish_timing(timing, "scheduler", t0)
                    refresh_rows = [r for r, c in enumerate(counts) if c == T]
                    if refresh_rows:
                        self._refresh(batched, working, refresh_rows, reuse, timing)
                        total_nfe += len(refresh_rows)
                        decode_key = None
                        continue
                if not batched:
                    continue
                active = [r for r, c in enumerate(counts) if c > 0]
                if not active:
                    continue
                key = tuple((batched[r].seq_id, batched[r].current_block_idx) for r in active)
                steps_on_key = steps_on_key + 1 if key == decode_key else 0
                if steps_on_key > step_cap:
                    raise RuntimeError("block decoding makes no progress: the model keeps predicting the mask token")
                if key != decode_key:
                    t0 = self._start_timing()
                    decode_key = key
                    sel = [batched[r] for r in active]
                    decode_positions = (self.prepare_decoding_acache(sel, graphs=self._decode_graphs if use_graphs else None)
                                        if reuse else self.prepare_decoding(sel))
                    decode_graph = self._decode_graph if reuse else None
                    decode_rows = torch.as_tensor(active, dtype=torch.int64, device=dev)
                    decode_max_pos = max(len(s) for s in sel)
                    self._finish_timing(timing, "decode_prepare", t0)
                t0 = self._start_timing()
                block_tokens = working.index_select(0, decode_rows) if len(active) != len(batched) else working
                if decode_graph is not None:
                    logits, stats = decode_graph.run(self, block_tokens, decode_positions)
                else:
                    logits, stats = self._decode_forward(block_tokens, decode_positions, decode_max_pos)
                self._finish_timing(timing, "decode_forward", t0)
                self._add_timing_count(timing, "decode_forward_calls", 1)
                self._add_timing_count(timing, "decode_forward_nfe", len(active))
                t0 = self._start_timing()
                self._commit_output(logits, stats, working, decode_rows)
                self._finish_timing(timing, "decode_update", t0)
                total_nfe += len(active)
        finally:
            reset_context()
            self._finish_timing(timing, "total", t_total)
            self._resolve_timing()
            if timing is not None:
                timing["total_nfe"] = int(total_nfe)
            self._active_timing = prev_timing
        _lib.check_device_errors(dev)
        self.harvest_graph_timers()
        return outputs, total_nfe
