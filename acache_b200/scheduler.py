"""Request admission for block-wise denoising.

The reference ships a scheduler class with the token-by-token interface of an
autoregressive engine (reference: nano-vdllm/scheduler.py:8-71: ``add``,
``schedule``, ``is_finished``, ``preempt``, ``postprocess``); its engine does
the actual admission inline (reference: nano-vdllm/model_runner.py:960-1003).
This class keeps the interface and implements the engine's admission rule
behind it; the rule itself is ``admissible_prefix`` below, which the engine's own
admission (``ModelRunner._collect_admissible_sequences``) calls too:

* requests wait in FIFO order,
* a request is admitted while the running set is below ``max_num_seqs``
  (0 = unlimited) and the allocator has ``num_cache_blocks`` free blocks for it;
  admission stops at the first request that does not fit (no skipping),
* a request leaves when its last block is denoised; its blocks return to the
  allocator and the next waiting requests are admitted (continuous batching).
"""
from __future__ import annotations

from collections import deque

from .block_manager import BlockManager
from .config import Config
from .sequence import Sequence, SequenceStatus


def admissible_prefix(waiting, n_running: int, max_num_seqs: int, free_blocks: int) -> list[Sequence]:
    """Longest FIFO prefix of ``waiting`` that fits: the running set stays below
    ``max_num_seqs`` and every picked request finds ``num_cache_blocks`` free blocks; stops at
    the first request that does not fit (reference: nano-vdllm/model_runner.py:960-976)."""
    picked = []
    for seq in waiting:
        if n_running + len(picked) >= max_num_seqs or seq.num_cache_blocks > free_blocks:
            break
        picked.append(seq)
        free_blocks -= seq.num_cache_blocks
    return picked


class Scheduler:
    def __init__(self, config: Config, block_manager: BlockManager | None = None):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = getattr(config, "eos", -1)
        self.block_manager = block_manager or BlockManager(config.num_kvcache_blocks, config.kvcache_block_size)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()

    def is_finished(self):
        return not self.waiting and not self.running

    def add(self, seq: Sequence):
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def admissible(self, free_blocks: int | None = None) -> list[Sequence]:
        """Longest FIFO prefix of the waiting queue that fits the block budget and
        the running-set limit; nothing is allocated or dequeued."""
        budget = len(self.block_manager.free_block_ids) if free_blocks is None else free_blocks
        limit = self.max_num_seqs if self.max_num_seqs > 0 else len(self.running) + len(self.waiting)
        return admissible_prefix(self.waiting, len(self.running), limit, budget)

    def schedule(self) -> tuple[list[Sequence], bool]:
        """Returns ``(seqs, is_refresh)``: newly admitted requests (they need a
        refresh forward) if any could be admitted, else the running set (decode)."""
        admitted = []
        for seq in self.admissible():
            if not self.block_manager.can_allocate(seq):
                break
            self.block_manager.allocate(seq)
            seq.status = SequenceStatus.RUNNING
            self.waiting.popleft()
            self.running.append(seq)
            admitted.append(seq)
        if admitted:
            return admitted, True
        assert self.running, "nothing to schedule"
        return list(self.running), False

    def preempt(self, seq: Sequence):
        seq.status = SequenceStatus.WAITING
        if seq.block_table:
            self.block_manager.deallocate(seq)
        if seq in self.running:
            self.running.remove(seq)
        seq.current_block_idx = 0
        self.waiting.appendleft(seq)

    def postprocess(self, seqs: list[Sequence], finished: list[bool]) -> list[bool]:
        """Retire the requests flagged as done and free their blocks."""
        for seq, done in zip(seqs, finished):
            if done:
                seq.status = SequenceStatus.FINISHED
                if seq.block_table:
                    self.block_manager.deallocate(seq)
                self.running.remove(seq)
        return list(finished)
