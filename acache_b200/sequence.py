"""Per-request logical layout for affix-KV reuse.

Host-side mirror of the reference request object (reference:
nano-vdllm/sequence.py:13-212).  A request is a token list with three spans:

* the shared *affix* ``[affix_start, affix_end)`` whose K/V lives once in the
  shared slots ``0..A-1`` of the paged cache,
* the *generation span* ``[generation_start, generation_end)`` of mask tokens
  that is denoised block by block,
* everything else (the request's own context).

The request owns ``num_cache_blocks`` private blocks.  Their slots are split,
in block-table order, into ``num_anchor_tokens`` anchor slots followed by one
slot per non-affix position (reference: sequence.py:169-202).

The public attributes are plain Python lists, exactly as in the reference, so
code written against the reference keeps working.  The slot arithmetic itself
is done with numpy and int32 copies are kept next to the lists
(``*_np`` attributes) so the engine can build step metadata without walking
Python lists.
"""
from __future__ import annotations

import math
from enum import Enum, auto
from itertools import count

import numpy as np


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Sequence:
    """One request.  Constructor arguments follow reference sequence.py:16-27."""

    counter = count()

    def __init__(
        self,
        token_ids: list[int],
        block_length: int = 32,
        gen_length: int = 256,
        cache_block_size: int = 256,
        mask_id: int = 126336,
        prompt_affix_len: int = 0,
        prompt_affix_start: int | None = None,
        prompt_affix_end: int | None = None,
        generation_start: int | None = None,
    ):
        self.seq_id = next(Sequence.counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        gen_length = int(gen_length)

        if generation_start is None:
            # completion: the generation span is appended after the prompt
            self.generation_start = self.num_prompt_tokens
            self.token_ids += [mask_id] * gen_length
        else:
            # in-place infill: the span lies inside the given tokens
            g0 = int(generation_start)
            g1 = g0 + gen_length
            if g0 < 0 or g1 < g0 or g1 > self.num_prompt_tokens:
                raise ValueError("Infill generation span must be contained in the provided prompt.")
            self.generation_start = g0
            self.token_ids[g0:g1] = [mask_id] * gen_length
        self.generation_end = self.generation_start + gen_length
        self.num_tokens = len(self.token_ids)

        a0 = 0 if prompt_affix_start is None else int(prompt_affix_start)
        a1 = a0 + int(prompt_affix_len) if prompt_affix_end is None else int(prompt_affix_end)
        if not (0 <= a0 <= a1 <= self.num_tokens):
            raise ValueError("Affix span must be contained in the logical sequence.")
        if self.generation_start < a1 and self.generation_end > a0:
            raise ValueError("Generation and affix spans must not overlap.")
        self.prompt_affix_start = a0
        self.prompt_affix_end = a1
        self.prompt_affix_len = a1 - a0

        self.block_table: list[int] = []
        self.gen_length = gen_length
        self.block_length = block_length
        self.cache_block_size = cache_block_size
        self.mask_id = mask_id
        self.current_block_idx = 0
        self.num_blocks_to_generate = -(-gen_length // block_length)

        self.acache_enabled = False
        self.affix_start = a0
        self.affix_end = a1
        self.affix_len = 0
        self.anchor_positions: list[int] = []
        self.num_anchor_tokens = 0
        self.recompute_positions: list[int] = list(range(self.num_tokens))
        self.recompute_slot_mapping: list[int] = []
        self.read_slot_map: list[int] = []
        self.shared_slot_offset = 0
        self.relocated_affix_materialized = False

    # ---- container protocol -------------------------------------------------
    def __len__(self):
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    # ---- views ---------------------------------------------------------------
    @property
    def is_finished(self):
        return self.status == SequenceStatus.FINISHED

    @property
    def prompt_token_ids(self):
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def generated_token_ids(self):
        return self.token_ids[self.generation_start : self.generation_end]

    @property
    def prompt_affix_token_ids(self):
        return self.token_ids[self.prompt_affix_start : self.prompt_affix_end]

    @property
    def non_affix_positions(self):
        return [*range(self.affix_start), *range(self.affix_end, self.num_tokens)]

    @property
    def num_private_slots(self):
        if not self.acache_enabled:
            return self.num_tokens
        return self.num_anchor_tokens + self.num_tokens - self.affix_len

    @property
    def num_cache_blocks(self):
        return -(-self.num_private_slots // self.cache_block_size)

    @property
    def last_cache_block_num_tokens(self):
        return self.num_private_slots - (self.num_cache_blocks - 1) * self.cache_block_size

    def block(self, i):
        assert 0 <= i < self.num_cache_blocks
        bs = self.cache_block_size
        return self.token_ids[i * bs : (i + 1) * bs]

    # ---- affix reuse ------------------------------------------------------------
    def enable_acache(
        self,
        affix_len: int | None = None,
        anchor_ratio: float = 0.0,
        *,
        affix_start: int | None = None,
        affix_end: int | None = None,
    ):
        """Declare the reusable span and the anchor budget
        ``k = min(ceil(ratio * A), A)`` (reference: sequence.py:126-152)."""
        a0 = self.prompt_affix_start if affix_start is None else int(affix_start)
        if affix_end is not None:
            a1 = int(affix_end)
        elif affix_len is not None:
            a1 = a0 + int(affix_len)
        else:
            a1 = self.prompt_affix_end
        if not (0 <= a0 <= a1 <= self.num_tokens):
            raise ValueError("ACache affix span must be contained in the logical sequence.")
        self.affix_start, self.affix_end = a0, a1
        self.affix_len = a1 - a0
        self.acache_enabled = self.affix_len > 0
        self.num_anchor_tokens = min(math.ceil(anchor_ratio * self.affix_len), self.affix_len)
        self.anchor_positions = []
        self.recompute_positions = list(range(self.num_tokens))
        self.recompute_slot_mapping = []
        self.read_slot_map = []
        self.relocated_affix_materialized = False

    def set_anchor_positions(self, anchor_positions: list[int]):
        """Install the selected anchors (logical positions inside the affix).
        Reference: sequence.py:154-167."""
        chosen = sorted({int(p) for p in anchor_positions})
        if not self.acache_enabled:
            self.anchor_positions = []
            self.num_anchor_tokens = 0
            self.recompute_positions = list(range(self.num_tokens))
            return
        assert all(self.affix_start <= p < self.affix_end for p in chosen)
        assert len(chosen) == min(self.num_anchor_tokens, self.affix_len)
        self.anchor_positions = chosen
        self.num_anchor_tokens = len(chosen)
        self.recompute_positions = sorted(chosen + self.non_affix_positions)

    def private_slots(self) -> np.ndarray:
        """Flat cache slots of the request's own blocks, in block-table order,
        truncated to ``num_private_slots``."""
        bs = self.cache_block_size
        n = self.num_private_slots
        nb = self.num_cache_blocks
        table = np.asarray(self.block_table[:nb], dtype=np.int64)
        slots = (table[:, None] * bs + np.arange(bs, dtype=np.int64)[None, :]).reshape(-1)[:n]
        assert slots.shape[0] == n
        return slots

    def finalize_slot_mapping(self, shared_slot_offset: int = 0):
        """Bind logical positions to cache slots once ``block_table`` is known
        (reference: sequence.py:169-202)."""
        self.shared_slot_offset = shared_slot_offset
        own = self.private_slots()
        if not self.acache_enabled:
            self.recompute_positions = list(range(self.num_tokens))
            self.recompute_slot_mapping = own.tolist()
            self.read_slot_map = own.tolist()
            return

        k = self.num_anchor_tokens
        anchors = np.asarray(self.anchor_positions, dtype=np.int64)
        outside = np.asarray(self.non_affix_positions, dtype=np.int64)
        assert own.shape[0] - k == outside.shape[0]

        read = np.full(self.num_tokens, -1, dtype=np.int64)
        # shared span first, then overwrite the anchors with their private copies
        read[self.affix_start : self.affix_end] = shared_slot_offset + np.arange(self.affix_len)
        read[anchors] = own[:k]
        read[outside] = own[k:]

        rows = np.concatenate([anchors, outside])
        slots = np.concatenate([own[:k], own[k:]])
        order = np.argsort(rows, kind="stable")
        self.recompute_positions = rows[order].tolist()
        self.recompute_slot_mapping = slots[order].tolist()
        self.read_slot_map = read.tolist()

    def block_query_start(self):
        """Row index, inside ``recompute_positions``, of the first token of the
        block currently being denoised (reference: sequence.py:204-206)."""
        first = self.generation_start + self.current_block_idx * self.block_length
        return self.recompute_positions.index(first)

    # Pickling uses the default protocol (the whole attribute dict): a request that crosses a
    # process boundary arrives with its tokens, spans and slot layout intact.
