"""The CPU restatement (oracle/) against fixtures produced by the reference's
own code (tests/golden/make_golden.py).  No GPU needed."""
import numpy as np
import pytest
import torch

from conftest import load_npz
from oracle import attention as oatt
from oracle import kv_ops, sampling, topk
from oracle.engine import compute_affix_kv, generate_request, select_anchors
from oracle.models import ArchSpec, OracleModel


def test_store_kvcache_matches_reference_kernel(triton_ops):
    t = triton_ops
    kc, vc = t["store_kc_in"].clone(), t["store_vc_in"].clone()
    kv_ops.store_kvcache(t["store_key"], t["store_val"], kc, vc, t["store_slots"])
    assert torch.equal(kc, t["store_kc_out"]) and torch.equal(vc, t["store_vc_out"])


def test_materialize_bit_exact_vs_reference_kernel(triton_ops):
    t = triton_ops
    for tag in ("f32", "f16"):
        A, shift, dst = (int(x) for x in t[f"mat_{tag}_meta"])
        k, v = t[f"mat_{tag}_k_in"].clone(), t[f"mat_{tag}_v_in"].clone()
        kv_ops.materialize_relocated_affix(k, v, t["mat_cos"], t["mat_sin"], dst, A, shift)
        assert torch.equal(k, t[f"mat_{tag}_k_out"]), tag
        assert torch.equal(v, t[f"mat_{tag}_v_out"]), tag


def test_attention_modes_vs_reference_kernel(triton_ops):
    t = triton_ops
    spl = int(t["att_shared_prefix_len"])
    for tag, tol in (("f32", 2e-5), ("f16", 4e-3)):
        q, kc, vc = t[f"att_{tag}_q"], t[f"att_{tag}_kc"], t[f"att_{tag}_vc"]
        cu_q, cu_k = t[f"att_{tag}_cu_q"], t[f"att_{tag}_cu_k"]
        plain = oatt.acache_attention(q, kc, vc, cu_q, cu_k, t[f"att_{tag}_logical"])
        key = oatt.acache_attention(q, kc, vc, cu_q, cu_k, t[f"att_{tag}_logical"], None, spl, None,
                                    t[f"att_{tag}_shifts"], t["att_cos"], t["att_sin"])
        qs = oatt.acache_attention(q, kc, vc, cu_q, cu_k, t[f"att_{tag}_packed"], None, spl,
                                   t[f"att_{tag}_shared_lens"], t[f"att_{tag}_shifts"], t["att_cos"], t["att_sin"])
        for name, got in (("plain", plain), ("keyside", key), ("queryside", qs)):
            ref = t[f"att_{tag}_{name}"]
            err = (got.float() - ref.float()).abs().max().item()
            assert err < tol, (tag, name, err)


def test_block_table_attention_vs_reference_kernel(triton_ops):
    t = triton_ops
    got = oatt.baseline_ragged_attention(t["bt_q"], t["bt_kc"], t["bt_vc"], t["bt_cu"], t["bt_cu"], t["bt_tables"])
    assert (got - t["bt_ragged"]).abs().max() < 2e-5
    got = oatt.baseline_decode_attention(t["bt_qd"], t["bt_kc"], t["bt_vc"], t["bt_seqlens"], t["bt_tables"])
    assert (got - t["bt_decode"]).abs().max() < 2e-5


def test_sampling_matches_reference():
    z = load_npz("sampling.npz")
    x0, ti = sampling.get_transfer_index(torch.from_numpy(z["logits"]), torch.from_numpy(z["mask"]),
                                         torch.from_numpy(z["x"]), float(z["threshold"]))
    assert np.array_equal(x0.numpy(), z["x0"]) and np.array_equal(ti.numpy(), z["transfer"])


def test_topk_matches_torch_on_tie_free_scores():
    z = load_npz("topk.npz")
    s = torch.from_numpy(z["scores"])
    assert np.array_equal(topk.anchor_topk(s, int(z["k"]), True).numpy(), z["top"])
    assert np.array_equal(topk.anchor_topk(s, int(z["k"]), False).numpy(), z["bottom"])


def test_topk_tie_rule_is_lowest_index():
    s = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0, 3.0]])
    assert topk.anchor_topk(s, 3, True).tolist() == [[1, 2, 4]]
    assert topk.anchor_topk(s, 2, False).tolist() == [[0, 5]]
    z = torch.zeros(2, 9)
    assert topk.anchor_topk(z, 4, True).tolist() == [[0, 1, 2, 3]] * 2


@pytest.mark.parametrize("which", ["hf_llada", "hf_dream"])
def test_engine_restatement_vs_hf_reference_path(which, request):
    """Anchors, importance scores and final tokens of the reference's HF batch-1
    paths (LLaDA, Dream with GQA; fp32, CPU) for prefix / infix / suffix placement."""
    meta, weights, arrays = request.getfixturevalue(which)
    arch = ArchSpec(**meta["arch"])
    model = OracleModel(arch, weights, torch.float32)
    affix_kv = None
    for case in meta["cases"]:
        prompt = case["prompt"]
        a0, a1 = case["affix_start"], case["affix_end"]
        G = case["gen_length"]
        if case["generation_start"] is None:
            tokens = prompt + [arch.mask_id] * G
            g0 = len(prompt)
        else:
            tokens = list(prompt)
            g0 = case["generation_start"]
        if affix_kv is None:
            affix_kv = compute_affix_kv(model, tokens[a0:a1])
        anchors, scores = select_anchors(model, affix_kv, tokens, a0, a1, case["anchor_ratio"], "top")
        ref_scores = arrays[f"{case['tag']}::importance"]
        assert np.allclose(scores.numpy(), ref_scores, rtol=1e-4, atol=1e-5), case["tag"]
        assert anchors == case["anchors"], case["tag"]
        out, nfe = generate_request(model, affix_kv, tokens, a0, a1, g0, G, case["block_length"], anchors,
                                    case["threshold"])
        assert out == arrays[f"{case['tag']}::tokens"].tolist(), case["tag"]
        assert nfe + 1 == case["nfe_with_probe"], case["tag"]
