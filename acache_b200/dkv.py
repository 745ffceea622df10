"""dKV-Cache decoding (delayed KV refresh) on the paged cache, alone or on top of affix reuse.

Second serving mode of the reference engine (reference: nano-vdllm/model_runner.py:1116-1293
``prepare_dkv_caching`` / ``prepare_dkv_caching_acache``, :1724-2030 ``_dkv_*`` and
``_generate_with_dkv_cache``).  A block is denoised in a fixed number of steps with a fixed
quota of tokens committed per step; a *refresh* step queries every dynamic position of the
request, a *compact* step only the tokens that were still unresolved two steps earlier (their
K/V is refreshed with a delay of one step), everything else is read from the cache.  It reuses
every kernel of the affix-reuse path: ragged queries, K/V scattered to the rows' slots (``-1``
keeps a cached row), attention through the slot map or the block tables.

``DkvMixin`` is mixed into ``ModelRunner``; the method names and signatures are the reference's.
"""
from __future__ import annotations

import numpy as np
import torch

from .utils import add_gumbel_noise, reset_context, set_context


class DkvMixin:
    # ------------------------------------------------------------------ schedules and query sets
    @staticmethod
    def _dkv_transfer_schedule(block_length: int, steps_per_block: int) -> list[int]:
        """Tokens committed at each step of a block: as even as possible, the remainder first."""
        if block_length <= 0 or steps_per_block <= 0:
            raise ValueError("dKV block length and steps per block must be positive.")
        base, remainder = divmod(block_length, steps_per_block)
        return [base + (step < remainder) for step in range(steps_per_block)]

    @staticmethod
    def _dkv_query_positions(seq, delayed_unresolved, step: int, cache_interval: int, refresh_positions=None):
        """LLaDA: refresh at steps 0, 1 and every ``cache_interval``-th step, else the tokens that
        were unresolved two steps ago.  Returns (positions, is_refresh)."""
        refresh = step <= 1 or step % cache_interval == 0
        if refresh:
            if refresh_positions is None:
                refresh_positions = list(range(len(seq)))
            return refresh_positions, True
        if delayed_unresolved is None:
            raise RuntimeError("dKV compact decoding requires the delayed unresolved-token state.")
        return delayed_unresolved, False

    def _dream_dkv_query_positions(self, seq, step: int, cache_interval: int, refresh_positions=None):
        """Dream predicts token j from position j-1: query the predecessors of the unresolved
        tokens, always including those of the current block (absolute positions)."""
        dynamic = set(range(len(seq)) if refresh_positions is None else refresh_positions)
        refresh = step % cache_interval == 0
        mask_id = self.config.mask_id
        predecessors = {(pos - 1) % len(seq) for pos, token in enumerate(seq.token_ids) if token == mask_id}
        queries = dynamic if refresh else dynamic & predecessors
        start = seq.generation_start + seq.current_block_idx * self.config.block_length
        queries = set(queries) | {max(pos - 1, 0) for pos in range(start, start + self.config.block_length)
                                  if seq.token_ids[pos] == mask_id}
        return sorted(queries), refresh

    def _dkv_select_masked_tokens(self, logits: torch.Tensor, temperature: float, remasking: str,
                                  num_transfer_tokens: int):
        """Candidates of the masked positions and the ``num_transfer_tokens`` most confident of
        them per request; confidence = log-probability of the candidate in fp64, as the reference
        computes it."""
        if logits.dim() != 3:
            raise ValueError("dKV masked-token logits must have shape [batch, tokens, vocab].")
        batch_size, num_masked, _ = logits.shape
        if not 0 <= num_transfer_tokens <= num_masked:
            raise ValueError(f"Cannot transfer {num_transfer_tokens} tokens from {num_masked} masked positions.")
        x0 = torch.argmax(add_gumbel_noise(logits, temperature=temperature), dim=-1)
        if num_transfer_tokens == 0:
            return x0, torch.empty((batch_size, 0), dtype=torch.int64, device=logits.device)
        if remasking == "low_confidence":
            flat, flat_x0 = logits.reshape(-1, logits.shape[-1]), x0.reshape(-1)
            confidence = torch.empty(flat_x0.shape, dtype=torch.float64, device=logits.device)
            for lo in range(0, flat.shape[0], 64):   # 64 rows at a time: fp64 copies of a 126k vocabulary are large
                rows = flat[lo: lo + 64].to(torch.float64)
                chosen = torch.gather(rows, -1, flat_x0[lo: lo + 64, None]).squeeze(-1)
                confidence[lo: lo + 64] = chosen - torch.logsumexp(rows, dim=-1)
            confidence = confidence.view_as(x0)
        elif remasking == "random":
            confidence = torch.rand((batch_size, num_masked), device=logits.device)
        else:
            raise NotImplementedError(remasking)
        return x0, torch.topk(confidence, k=num_transfer_tokens, dim=-1).indices

    # ------------------------------------------------------------------ step metadata
    @staticmethod
    def _check_query_positions(seq, row_positions):
        if not row_positions:
            raise ValueError("Every active dKV request must contain a query token.")
        if list(row_positions) != sorted(set(row_positions)):
            raise ValueError("dKV query positions must be sorted and unique.")
        if row_positions[0] < 0 or row_positions[-1] >= len(seq):
            raise ValueError("dKV query position lies outside the logical sequence.")

    def prepare_dkv_caching(self, seqs, query_positions):
        """Ragged dKV queries against every request's own blocks (no affix reuse)."""
        if len(seqs) != len(query_positions):
            raise ValueError("Each dKV sequence must have one query-position list.")
        if sum(len(p) for p in query_positions) == 0:
            raise ValueError("dKV-Cache requires at least one query token per forward pass.")
        bs = self.config.cache_block_size
        ids, pos, slots, offsets = [], [], [], []
        cu_q = np.zeros(len(seqs) + 1, dtype=np.int32)
        cu_k = np.zeros(len(seqs) + 1, dtype=np.int32)
        width = max(len(s.block_table) for s in seqs)
        table = np.full((len(seqs), width), -1, dtype=np.int32)
        for row, (seq, rp) in enumerate(zip(seqs, query_positions)):
            self._check_query_positions(seq, rp)
            rp = np.asarray(rp, dtype=np.int64)
            bt = np.asarray(seq.block_table, dtype=np.int64)
            table[row, : bt.shape[0]] = bt
            offsets.append(int(cu_q[row]))
            ids.append(np.asarray(seq.token_ids, dtype=np.int64)[rp])
            pos.append(rp)
            slots.append((bt[rp // bs] * bs + rp % bs).astype(np.int32))
            cu_q[row + 1] = cu_q[row] + rp.shape[0]
            cu_k[row + 1] = cu_k[row] + len(seq)
        dev = self._staging.ship(input_ids=np.concatenate(ids), positions=np.concatenate(pos), cu_q=cu_q, cu_k=cu_k,
                                 slots=np.concatenate(slots), table=table)
        q_lens, k_lens = np.diff(cu_q), np.diff(cu_k)
        self._note_attention_work("refresh", q_lens, k_lens)
        set_context(True, dev["cu_q"], dev["cu_k"], None, int(q_lens.max()), int(k_lens.max()), dev["slots"], dev["table"])
        return dev["input_ids"], dev["positions"], offsets

    def prepare_dkv_caching_acache(self, seqs, query_positions):
        """Ragged dKV queries against the affix-reuse read layout.  A queried position that has no
        private slot (a frozen affix token, only queried by Dream for its successor's logits)
        gets write slot -1: its cached K/V stays."""
        if len(seqs) != len(query_positions):
            raise ValueError("Each dKV sequence must have one query-position list.")
        if sum(len(p) for p in query_positions) == 0:
            raise ValueError("dKV-Cache requires at least one query token per forward pass.")
        self._configure_affix_relocation(seqs)
        materialized = all(getattr(s, "relocated_affix_materialized", False) for s in seqs)
        use_qr = self._use_query_side_affix_relocation(materialized)
        dream = self._is_dream_model()
        ids, pos, slots, read, shared_lens, shifts, offsets = [], [], [], [], [], [], []
        cu_q = np.zeros(len(seqs) + 1, dtype=np.int32)
        cu_k = np.zeros(len(seqs) + 1, dtype=np.int32)
        for row, (seq, rp) in enumerate(zip(seqs, query_positions)):
            self._check_query_positions(seq, rp)
            cached = getattr(seq, "_dkv_layout", None)    # per request, until its slot layout changes
            if cached is None or cached[0] is not seq.recompute_slot_mapping or cached[1] != use_qr:
                layout, n_shared = self._attention_read_layout(seq, use_qr)
                cached = seq._dkv_layout = (seq.recompute_slot_mapping, use_qr,
                                            dict(zip(seq.recompute_positions, seq.recompute_slot_mapping)),
                                            np.asarray(layout, dtype=np.int32), n_shared)
            slot_of = cached[2]
            try:
                row_slots = [slot_of.get(p, -1) if dream else slot_of[p] for p in rp]
            except KeyError as exc:
                raise ValueError("dKV+ACache cannot query a frozen non-anchor affix token.") from exc
            rp = np.asarray(rp, dtype=np.int64)
            offsets.append(int(cu_q[row]))
            ids.append(np.asarray(seq.token_ids, dtype=np.int64)[rp])
            pos.append(rp)
            slots.append(np.asarray(row_slots, dtype=np.int32))
            read.append(cached[3])
            shared_lens.append(cached[4])
            shifts.append(seq.affix_start if self._affix_relocation_enabled else 0)
            cu_q[row + 1] = cu_q[row] + rp.shape[0]
            cu_k[row + 1] = cu_k[row] + len(seq)
        arrays = dict(input_ids=np.concatenate(ids), positions=np.concatenate(pos), cu_q=cu_q, cu_k=cu_k,
                      slots=np.concatenate(slots), read=np.concatenate(read))
        if use_qr:
            arrays["shared_lens"] = np.asarray(shared_lens, dtype=np.int32)
        if not materialized:
            arrays["shifts"] = np.asarray(shifts, dtype=np.int32)
        dev = self._staging.ship(**arrays)
        q_lens, k_lens = np.diff(cu_q), np.diff(cu_k)
        self._note_attention_work("refresh", q_lens, k_lens)
        set_context(True, dev["cu_q"], dev["cu_k"], None, int(q_lens.max()), int(k_lens.max()), dev["slots"], None, True,
                    dev["read"], dev.get("shared_lens"), dev.get("shifts"))
        return dev["input_ids"], dev["positions"], offsets

    # ------------------------------------------------------------------ generation
    @torch.inference_mode()
    def generate_with_dkv_cache(self, prompts):
        """dKV-Cache decoding on the paged cache (no affix reuse)."""
        return self._generate_with_dkv_cache(prompts, use_acache=False)

    @torch.inference_mode()
    def generate_with_dkv_acache(self, prompts):
        """dKV-Cache decoding with the shared affix read from the cache (anchors recomputed)."""
        return self._generate_with_dkv_cache(prompts, use_acache=True)

    def _generate_with_dkv_cache(self, prompts, use_acache: bool):
        cfg = self.config
        dream = self._is_dream_model()
        mask_id, T = cfg.mask_id, cfg.block_length
        cache_interval = int(cfg.dkv_cache_interval)
        steps = int(cfg.dkv_steps) or int(cfg.gen_length)
        num_blocks = int(cfg.gen_length) // T
        if int(cfg.gen_length) % T != 0:
            raise ValueError("dKV generation length must be divisible by block length.")
        if steps % num_blocks != 0:
            raise ValueError("dKV denoising steps must be divisible by the number of blocks.")
        if cache_interval <= 0:
            raise ValueError("dKV cache interval must be positive.")
        schedule = self._dkv_transfer_schedule(T, steps // num_blocks)
        max_num_seqs = cfg.max_num_seqs if cfg.max_num_seqs > 0 else len(prompts)

        timing = self._new_timing("dkv_acache" if use_acache else "dkv_cache", len(prompts))
        self.last_timing = timing if timing is not None else {}
        prev_timing, self._active_timing = self._active_timing, timing
        t_total = self._start_timing()
        prefix = ()
        if use_acache:
            t0 = self._start_timing()
            prefix = self._prepare_acache(prompts)
            self._finish_timing(timing, "acache_metadata", t0)
            if not prefix:
                use_acache = False
        total_nfe = 0
        outputs = [None] * len(prompts)
        index_of = {seq.seq_id: i for i, seq in enumerate(prompts)}
        next_idx = 0
        try:
            while next_idx < len(prompts):
                t0 = self._start_timing()
                batch: list = []
                if use_acache:
                    new, nxt = self._collect_admissible_sequences(prompts, next_idx, 0, max_num_seqs)
                    admitted = self._admit_sequences_with_acache(batch, new, prefix, allow_kv_cache_resize=True)
                    next_idx = nxt - (len(new) - admitted)
                else:
                    while (next_idx < len(prompts) and len(batch) < max_num_seqs
                           and self.block_manager.can_allocate(prompts[next_idx])):
                        self.block_manager.allocate(prompts[next_idx])
                        self._record_kv_cache_usage(timing)
                        batch.append(prompts[next_idx])
                        next_idx += 1
                self._finish_timing(timing, "scheduler", t0)
                if not batch:
                    raise RuntimeError("No dKV request could be admitted under the current KV-cache budget.")
                total_nfe += self._dkv_denoise_batch(batch, num_blocks, schedule, cache_interval, use_acache, dream, timing)
                t0 = self._start_timing()
                for seq in batch:
                    outputs[index_of[seq.seq_id]] = seq.generated_token_ids
                    self.block_manager.deallocate(seq)
                self._finish_timing(timing, "scheduler", t0)
        finally:
            reset_context()
            self._finish_timing(timing, "total", t_total)
            self._resolve_timing()
            if timing is not None:
                timing["total_nfe"] = int(total_nfe)
            self._active_timing = prev_timing
        from . import _lib

        _lib.check_device_errors(self.device)
        return outputs, total_nfe

    def _dkv_denoise_batch(self, batch, num_blocks, schedule, cache_interval, use_acache, dream, timing) -> int:
        """All blocks of one static batch; returns the number of function evaluations."""
        cfg = self.config
        mask_id, T = cfg.mask_id, cfg.block_length
        nfe = 0
        for block_idx in range(num_blocks):
            for seq in batch:
                seq.current_block_idx = block_idx
            previous_unresolved = [None] * len(batch)
            delayed_unresolved = [None] * len(batch)
            for step, quota in enumerate(schedule):
                query_positions, is_refresh = [], None
                for row, seq in enumerate(batch):
                    dynamic = seq.recompute_positions if use_acache else None
                    if dream:
                        rp, refresh = self._dream_dkv_query_positions(seq, step, cache_interval, dynamic)
                    else:
                        rp, refresh = self._dkv_query_positions(seq, delayed_unresolved[row], step, cache_interval, dynamic)
                    query_positions.append(rp)
                    if is_refresh is None:
                        is_refresh = refresh
                    elif is_refresh != refresh:
                        raise RuntimeError("dKV batch rows disagree on refresh state.")
                t0 = self._start_timing()
                prepare = self.prepare_dkv_caching_acache if use_acache else self.prepare_dkv_caching
                input_ids, positions, offsets = prepare(batch, query_positions)
                self._finish_timing(timing, "cache_prepare", t0)

                # rows whose logits are needed: the masked tokens of the block (Dream: their predecessors)
                mask_positions, logit_rows = [], []
                for row, seq in enumerate(batch):
                    start = seq.generation_start + block_idx * T
                    masked = [p for p in range(start, start + T) if seq.token_ids[p] == mask_id]
                    mask_positions.append(masked)
                    where = {p: offsets[row] + i for i, p in enumerate(query_positions[row])}
                    try:
                        logit_rows.extend(where[max(p - 1, 0) if dream else p] for p in masked)
                    except KeyError as exc:
                        raise RuntimeError("dKV delayed query omitted a currently masked token.") from exc
                num_masked = len(mask_positions[0])
                if any(len(m) != num_masked for m in mask_positions):
                    raise RuntimeError("dKV batch rows have different masked-token counts.")
                keep = self._staging.ship(k=np.asarray(logit_rows, dtype=np.int64))["k"]

                t0 = self._start_timing()
                max_pos = max(len(s) for s in batch)
                logits = self._forward_model(input_ids, positions, logits_keep_indices=keep, max_pos=max_pos).logits
                self._finish_timing(timing, "cache_forward", t0)
                self._add_timing_count(timing, "dkv_refresh_forward_calls" if is_refresh else "dkv_compact_forward_calls", 1)
                self._add_timing_count(timing, "cache_forward_calls", 1)
                self._add_timing_count(timing, "cache_forward_nfe", len(batch))
                nfe += len(batch)

                t0 = self._start_timing()
                x0, selected = self._dkv_select_masked_tokens(logits.view(len(batch), num_masked, -1), cfg.temperature,
                                                              cfg.remasking, quota)
                tokens = torch.gather(x0, 1, selected).tolist() if quota else [[] for _ in batch]
                chosen = selected.tolist()
                self.d2h_bytes += 16 * quota * len(batch)
                for row, seq in enumerate(batch):
                    for idx, tok in zip(chosen[row], tokens[row]):
                        seq.token_ids[mask_positions[row][idx]] = int(tok)
                    start = seq.generation_start + block_idx * T
                    unresolved = [p for p in range(start, seq.generation_end) if seq.token_ids[p] == mask_id]
                    delayed_unresolved[row] = previous_unresolved[row]
                    previous_unresolved[row] = unresolved
                self._finish_timing(timing, "cache_update", t0)
            for seq in batch:
                start = seq.generation_start + block_idx * T
                if mask_id in seq.token_ids[start: start + T]:
                    raise RuntimeError("dKV transfer schedule did not finish the current block.")
        return nfe
