"""Paged-block allocator for the KV cache.

Mirror of the reference allocator (reference: nano-vdllm/block_manager.py:12-62)
with the same observable order of block ids, because block tables are part of
the parity contract:

* ``allocate`` takes blocks from the head of the free queue,
* ``deallocate`` returns a request's blocks in reverse table order to the tail,
* ``reserve_prefix(n)`` pins ids ``0..n-1`` (shared affix, and the relocation
  workspace right behind it),
* ``release_prefix_tail(n)`` unpins every reserved id ``>= n``, highest first.

The free queue is an insertion-ordered set, so removing a specific id (needed
by ``reserve_prefix``) is O(1) instead of a deque scan.
"""
from __future__ import annotations


class Block:
    __slots__ = ("block_id", "is_free")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.is_free = True


class _FifoIdSet:
    """FIFO queue of unique ints with O(1) membership and removal."""

    def __init__(self, ids=()):
        self._d = dict.fromkeys(ids)

    def __len__(self):
        return len(self._d)

    def __iter__(self):
        return iter(self._d)

    def __contains__(self, x):
        return x in self._d

    def __getitem__(self, i):
        if i == 0:
            return next(iter(self._d))
        return list(self._d)[i]

    def __eq__(self, other):
        return list(self) == list(other)

    def __repr__(self):
        return f"_FifoIdSet({list(self._d)})"

    def append(self, x):
        assert x not in self._d
        self._d[x] = None

    def remove(self, x):
        del self._d[x]

    def popleft(self):
        x = next(iter(self._d))
        del self._d[x]
        return x


class BlockManager:
    def __init__(self, num_blocks: int, cache_block_size: int):
        self.cache_block_size = cache_block_size
        self.blocks: list[Block] = [Block(i) for i in range(num_blocks)]
        self.free_block_ids = _FifoIdSet(range(num_blocks))
        self.used_block_ids: set[int] = set()
        self.reserved_block_ids: set[int] = set()

    # -- single-block primitives ------------------------------------------------
    def _allocate_block(self, block_id: int) -> Block:
        blk = self.blocks[block_id]
        assert blk.is_free, f"Block {block_id} is not free but trying to allocate"
        blk.is_free = False
        self.free_block_ids.remove(block_id)
        self.used_block_ids.add(block_id)
        return blk

    def _deallocate_block(self, block_id: int):
        blk = self.blocks[block_id]
        assert not blk.is_free, f"Block {block_id} is already free but trying to deallocate"
        blk.is_free = True
        self.used_block_ids.remove(block_id)
        self.free_block_ids.append(block_id)

    # -- shared-affix reservation -------------------------------------------------
    def reserve_prefix(self, num_blocks: int):
        for block_id in range(num_blocks):
            if block_id not in self.reserved_block_ids:
                self._allocate_block(block_id)
                self.reserved_block_ids.add(block_id)

    def release_prefix_tail(self, num_blocks: int):
        for block_id in sorted((b for b in self.reserved_block_ids if b >= num_blocks), reverse=True):
            self.reserved_block_ids.remove(block_id)
            self._deallocate_block(block_id)

    # -- whole-state copy (the engine replays the reference's allocator traffic from it) ----------
    def snapshot(self):
        return (list(self.free_block_ids), set(self.used_block_ids), set(self.reserved_block_ids))

    def restore(self, state):
        free, used, reserved = state
        self.free_block_ids = _FifoIdSet(free)
        self.used_block_ids = set(used)
        self.reserved_block_ids = set(reserved)
        for blk in self.blocks:
            blk.is_free = blk.block_id in self.free_block_ids

    # -- per-request ----------------------------------------------------------------
    def can_allocate(self, seq) -> bool:
        return len(self.free_block_ids) >= seq.num_cache_blocks

    def allocate(self, seq):
        assert not seq.block_table
        for _ in range(seq.num_cache_blocks):
            seq.block_table.append(self._allocate_block(self.free_block_ids[0]).block_id)

    def deallocate(self, seq):
        for block_id in reversed(seq.block_table):
            self._deallocate_block(block_id)
        seq.block_table.clear()

    # -- queried by the block scheduler ---------------------------------------------
    def can_append(self, seq) -> bool:
        """A request never grows after admission (its generation span is part of
        its layout from the start), so appending never needs a new block."""
        return True

    def may_append(self, seq):
        return None
