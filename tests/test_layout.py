"""Host-side layout (Sequence / BlockManager / read layout) against vectors
produced by the reference's own classes."""
import pytest

from acache_b200.block_manager import BlockManager
from acache_b200.sequence import Sequence


def _build(case):
    seq = Sequence(case["tokens"], block_length=case["block_length"], gen_length=case["gen_length"],
                   cache_block_size=case["cache_block_size"], mask_id=case["mask_id"], **case["kwargs"])
    seq.enable_acache(anchor_ratio=case["ratio"])
    mgr = BlockManager(case["num_blocks"], case["cache_block_size"])
    mgr.reserve_prefix(case["shared_blocks"])
    seq.set_anchor_positions(case["anchors"])
    mgr.allocate(seq)
    mgr.deallocate(seq)
    mgr.allocate(seq)
    seq.finalize_slot_mapping()
    seq.current_block_idx = case["current_block_idx"]
    return seq, mgr


def test_layout_matches_reference_vectors(layout_cases):
    from acache_b200.model_runner import attention_read_layout

    for case in layout_cases:
        seq, mgr = _build(case)
        out = case["out"]
        for name in ("token_ids", "block_table", "recompute_positions", "recompute_slot_mapping", "read_slot_map",
                     "num_anchor_tokens", "num_private_slots", "num_cache_blocks"):
            assert getattr(seq, name) == out[name], name
        assert seq.block_query_start() == out["block_query_start"]
        assert list(mgr.free_block_ids) == out["free_after"]
        A = seq.affix_len
        packed, n_shared = attention_read_layout(seq, True, A)
        assert packed == out["packed_read"] and n_shared == out["packed_shared"]


def test_read_runs_are_a_reordering_with_holes_at_the_anchors(layout_cases):
    """attention_read_runs keeps exactly the keys of the logical read order: the affix span
    as consecutive slots with -1 at the anchors, then the anchors' private slots, then the rest."""
    import numpy as np

    from acache_b200.model_runner import attention_read_runs

    seen_holes = 0
    for case in layout_cases:
        seq, _ = _build(case)
        layout, n_span, first = attention_read_runs(seq)
        layout = np.asarray(layout)
        logical = np.asarray(seq.read_slot_map)
        assert n_span == seq.affix_len and layout.shape[0] == logical.shape[0] + int((layout == -1).sum())
        assert sorted(layout[layout >= 0].tolist()) == sorted(logical.tolist())
        span = layout[:n_span]
        live = span >= 0
        if live.any() and not live.all():
            # live entries are one run of consecutive slots, holes sit exactly at the anchors
            start = span[live][0] - np.flatnonzero(live)[0]
            assert start == first
            assert (span[live] == start + np.flatnonzero(live)).all()
            holes = (np.flatnonzero(~live) + seq.affix_start).tolist()
            assert holes == seq.anchor_positions
            k = len(holes)
            assert layout[n_span: n_span + k].tolist() == [seq.read_slot_map[p] for p in holes]
            seen_holes += 1
        # second call returns the cached arrays
        again = attention_read_runs(seq)[0]
        assert again is layout or (np.asarray(again) == layout).all()
    assert seen_holes > 10


def test_read_layout_known_answers():
    """reference: nano-vdllm/tests/test_model_runner_acache.py:26-47."""
    from types import SimpleNamespace

    from acache_b200.model_runner import attention_read_layout

    seq = SimpleNamespace(affix_start=2, shared_slot_offset=0, read_slot_map=[8, 9, 0, 10, 2, 11])
    assert attention_read_layout(seq, True, 3) == ([0, 2, 8, 9, 10, 11], 2)
    assert attention_read_layout(seq, False, 3) == ([8, 9, 0, 10, 2, 11], 0)


@pytest.mark.parametrize(
    ("tokens", "a0", "a1", "g0"),
    [([10, 11, 12], 0, 2, None), ([10, 20, 21, 11], 1, 3, None), ([10, 99, 99, 20, 21], 3, 5, 1)],
)
def test_affix_layout_maps_shared_and_private_slots(tokens, a0, a1, g0):
    """reference: nano-vdllm/tests/test_sequence_spans.py:11-45."""
    seq = Sequence(tokens, gen_length=2, block_length=2, cache_block_size=4, mask_id=99,
                   prompt_affix_start=a0, prompt_affix_end=a1, generation_start=g0)
    seq.enable_acache(anchor_ratio=0.5)
    anchor = a1 - 1
    seq.set_anchor_positions([anchor])
    seq.block_table = list(range(2, 2 + seq.num_cache_blocks))
    seq.finalize_slot_mapping(shared_slot_offset=0)
    assert seq.recompute_positions == sorted([anchor] + seq.non_affix_positions)
    assert seq.read_slot_map[a0] == 0
    assert seq.read_slot_map[anchor] != anchor - a0
    assert all(s >= 0 for s in seq.read_slot_map)
    assert seq.block_query_start() == seq.recompute_positions.index(seq.generation_start)


def test_suffix_layout_generates_inside_prompt():
    """reference: nano-vdllm/tests/test_sequence_spans.py:48-61."""
    seq = Sequence([10, 50, 51, 20, 21], gen_length=2, block_length=2, mask_id=99,
                   prompt_affix_start=3, prompt_affix_end=5, generation_start=1)
    assert seq.token_ids == [10, 99, 99, 20, 21]
    assert seq.generated_token_ids == [99, 99]


def test_overlapping_spans_are_rejected():
    with pytest.raises(ValueError):
        Sequence([1, 2, 3, 4], gen_length=2, block_length=2, mask_id=99,
                 prompt_affix_start=1, prompt_affix_end=3, generation_start=2)


def test_release_prefix_tail_returns_workspace_blocks():
    """reference: nano-vdllm/tests/test_sequence_spans.py:76-84."""
    mgr = BlockManager(6, 4)
    mgr.reserve_prefix(4)
    assert list(mgr.free_block_ids) == [4, 5]
    mgr.release_prefix_tail(2)
    assert mgr.reserved_block_ids == {0, 1}
    assert list(mgr.free_block_ids) == [4, 5, 3, 2]
