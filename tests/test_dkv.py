"""dKV-Cache decoding: host-side schedules and query sets against the reference's known
answers, and the CPU restatement against fixtures produced by the reference's HF batch-1
dKV + affix-reuse paths (CPU; the engine itself is compared on the GPU in test_engine_gpu.py)."""
import pytest
import torch

from acache_b200.config import Config
from acache_b200.model_runner import ModelRunner
from acache_b200.sequence import Sequence


def _bare_runner(**cfg):
    runner = object.__new__(ModelRunner)
    runner.config = Config(**cfg)
    return runner


def test_transfer_schedule_known_answers():
    """reference: nano-vdllm/tests/test_model_runner_acache.py:127-129."""
    assert ModelRunner._dkv_transfer_schedule(32, 32) == [1] * 32
    assert ModelRunner._dkv_transfer_schedule(8, 3) == [3, 3, 2]
    assert sum(ModelRunner._dkv_transfer_schedule(32, 5)) == 32
    with pytest.raises(ValueError):
        ModelRunner._dkv_transfer_schedule(8, 0)


def test_llada_query_positions_one_step_delay_and_refresh():
    """reference: nano-vdllm/tests/test_model_runner_acache.py:132-158."""
    seq = Sequence([2, 3], gen_length=4, cache_block_size=8, block_length=4, mask_id=63)
    delayed = [3, 4, 5]
    assert ModelRunner._dkv_query_positions(seq, None, 0, 8) == (list(range(6)), True)
    assert ModelRunner._dkv_query_positions(seq, None, 1, 8) == (list(range(6)), True)
    assert ModelRunner._dkv_query_positions(seq, delayed, 2, 8) == (delayed, False)
    assert ModelRunner._dkv_query_positions(seq, delayed, 8, 8) == (list(range(6)), True)
    dynamic = [0, 2, 3, 4, 5]     # with affix reuse a refresh queries the dynamic positions only
    assert ModelRunner._dkv_query_positions(seq, None, 0, 8, dynamic) == (dynamic, True)
    assert ModelRunner._dkv_query_positions(seq, delayed, 2, 8, dynamic) == (delayed, False)
    with pytest.raises(RuntimeError):
        ModelRunner._dkv_query_positions(seq, None, 2, 8)


def test_dream_query_positions_absolute_predecessors():
    """reference: nano-vdllm/tests/test_dream_dkv.py:19-28."""
    runner = _bare_runner(model_type="dream", mask_id=63, block_length=4)
    seq = Sequence([2, 3], gen_length=4, block_length=4, mask_id=63)
    seq.token_ids[3] = 7
    assert runner._dream_dkv_query_positions(seq, 0, 8) == (list(range(6)), True)
    assert runner._dream_dkv_query_positions(seq, 1, 8) == ([1, 3, 4], False)
    assert runner._dream_dkv_query_positions(seq, 8, 8)[1]
    # position 1 is a frozen affix token but still predicts the masked token 2
    assert runner._dream_dkv_query_positions(seq, 1, 8, [2, 3, 4, 5]) == ([1, 3, 4], False)


def test_low_confidence_selection_uses_a_fixed_quota():
    """reference: nano-vdllm/tests/test_model_runner_acache.py:161-179."""
    runner = _bare_runner()
    logits = torch.tensor([[[5.0, 0.0, 0.0, 0.0], [1.0, 1.0, 1.0, 1.0], [2.0, 1.0, 1.0, 1.0]]])
    x0, selected = runner._dkv_select_masked_tokens(logits, temperature=0.0, remasking="low_confidence",
                                                    num_transfer_tokens=2)
    assert x0.tolist() == [[0, 0, 0]]
    assert set(selected[0].tolist()) == {0, 2}
    x0, selected = runner._dkv_select_masked_tokens(logits, 0.0, "low_confidence", 0)
    assert selected.shape == (1, 0)
    with pytest.raises(ValueError):
        runner._dkv_select_masked_tokens(logits, 0.0, "low_confidence", 4)


@pytest.mark.parametrize("which", ["hf_llada_dkv", "hf_dream_dkv"])
def test_oracle_dkv_matches_hf_reference_fixtures(which, request):
    """Tokens (and the number of denoising forwards) of the reference's HF dKV + affix-reuse
    generation, prefix / infix / suffix, anchor ratios 0, ~1/3 and 1, cache intervals 1-3."""
    from oracle.engine import compute_affix_kv, generate_request_dkv, select_anchors
    from oracle.models import ArchSpec, OracleModel

    meta, weights, arrays = request.getfixturevalue(which)
    arch = ArchSpec(**meta["arch"])
    model = OracleModel(arch, weights, torch.float32)
    for c in meta["cases"]:
        G = c["gen_length"]
        toks = list(c["prompt"]) + ([arch.mask_id] * G if c["generation_start"] is None else [])
        g0 = len(c["prompt"]) if c["generation_start"] is None else c["generation_start"]
        a0, a1 = c["affix_start"], c["affix_end"]
        affix_kv = compute_affix_kv(model, toks[a0:a1])
        anchors, _ = select_anchors(model, affix_kv, toks, a0, a1, c["anchor_ratio"])
        out, nfe = generate_request_dkv(model, toks, g0, G, c["block_length"], c["steps"], c["interval"], affix_kv,
                                        a0, a1, anchors)
        assert out == arrays[c["tag"] + "::tokens"].tolist(), c["tag"]
        assert nfe == c["steps"], c["tag"]
