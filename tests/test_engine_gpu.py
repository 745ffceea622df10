"""Engine on the GPU against (a) fixtures produced by the reference's HF batch-1 path and
(b) the CPU oracle engine, on tiny random models: anchors bit-exact, greedy tokens
identical, logits within tolerance, block tables as the allocator contract dictates."""
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _llada(arch, weights, dtype):
    from acache_b200.model.configuration import LLaDAConfig
    from acache_b200.model.modeling_llada import LLaDAModelLM

    cfg = LLaDAConfig(d_model=arch.d_model, n_heads=arch.n_heads, n_kv_heads=arch.n_kv_heads, n_layers=arch.n_layers,
                      mlp_hidden_size=arch.ffn, vocab_size=arch.vocab, embedding_size=arch.vocab,
                      rope_theta=arch.rope_theta, rms_norm_eps=arch.rms_eps, activation_type=arch.act,
                      mask_token_id=arch.mask_id, max_sequence_length=256)
    model = LLaDAModelLM(cfg, device=DEV, dtype=dtype, init_params=False)
    missing = model.load_state_dict({k: v.to(dtype) for k, v in weights.items()}, strict=True)
    assert not missing.missing_keys
    return cfg, model.eval().fuse_projections()


def _dream(arch, weights, dtype):
    from acache_b200.model.configuration import DreamConfig
    from acache_b200.model.modeling_dream import DreamModel

    cfg = DreamConfig(hidden_size=arch.d_model, num_attention_heads=arch.n_heads, num_key_value_heads=arch.n_kv_heads,
                      num_hidden_layers=arch.n_layers, intermediate_size=arch.ffn, vocab_size=arch.vocab,
                      rope_theta=arch.rope_theta, rms_norm_eps=arch.rms_eps, hidden_act=arch.act,
                      mask_token_id=arch.mask_id)
    model = DreamModel(cfg, device=DEV, dtype=dtype, init_params=False)
    model.load_state_dict({k: v.to(dtype) for k, v in weights.items()}, strict=True)
    return cfg, model.eval().fuse_projections()


def _serve_config(hf_cfg, arch, kind, dtype, **kw):
    from acache_b200.config import Config

    base = dict(hf_config=hf_cfg, mask_id=arch.mask_id, recompute_batch_size=2, max_num_seqs=3, gen_length=8,
                block_length=4, cache_block_size=8, num_kvcache_blocks=24, temperature=0.0, threshold=0.9,
                enable_acache=True, anchor_ratio=0.25, selection_mode="top", model_type=kind,
                kv_cache_dtype={torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype])
    base.update(kw)
    return Config(**base)


def _sequence(case, arch, block=8):
    from acache_b200.sequence import Sequence

    return Sequence(case["prompt"], block_length=case["block_length"], gen_length=case["gen_length"],
                    cache_block_size=block, mask_id=arch.mask_id, prompt_affix_start=case["affix_start"],
                    prompt_affix_end=case["affix_end"], generation_start=case["generation_start"])


@pytest.mark.parametrize("which,kind", [("hf_llada", "llada"), ("hf_dream", "dream")])
def test_engine_matches_hf_reference_fixtures(which, kind, request):
    """fp32 end to end: anchors and greedy tokens of the reference's HF paths (LLaDA; Dream with
    GQA) for prefix, infix and suffix placement, with the requests mixed in one continuously
    batched run."""
    from acache_b200.model_runner import ModelRunner
    from oracle.models import ArchSpec

    meta, weights, arrays = request.getfixturevalue(which)
    arch = ArchSpec(**meta["arch"])
    hf_cfg, model = (_llada if kind == "llada" else _dream)(arch, weights, torch.float32)
    for thr in (0.9, 0.05):
        cases = [c for c in meta["cases"] if c["threshold"] == thr]
        runner = ModelRunner(model, _serve_config(hf_cfg, arch, kind, torch.float32, threshold=thr))
        seqs = [_sequence(c, arch) for c in cases]
        outs, nfe = runner.generate_with_acache(seqs)
        want_nfe = 0
        for c, seq, out in zip(cases, seqs, outs):
            tag = c["tag"]
            assert seq.anchor_positions == c["anchors"], tag
            want = arrays[f"{tag}::tokens"].tolist()
            assert seq.token_ids == want, tag
            g0 = len(c["prompt"]) if c["generation_start"] is None else c["generation_start"]
            assert out == want[g0: g0 + c["gen_length"]], tag
            want_nfe += c["nfe_with_probe"] - 1
        assert nfe == want_nfe
        # every block went back to the allocator, the shared affix stays pinned
        bm = runner.block_manager
        assert bm.reserved_block_ids == set(range(runner.shared_prefix_blocks))
        assert len(bm.free_block_ids) == len(bm.blocks) - runner.shared_prefix_blocks


def test_importance_scores_match_hf_reference(hf_llada):
    from acache_b200.model_runner import ModelRunner
    from oracle.models import ArchSpec

    meta, weights, arrays = hf_llada
    arch = ArchSpec(**meta["arch"])
    hf_cfg, model = _llada(arch, weights, torch.float32)
    runner = ModelRunner(model, _serve_config(hf_cfg, arch, "llada", torch.float32))
    for c in meta["cases"][::2]:
        seq = _sequence(c, arch)
        toks = runner._prepare_acache([seq])
        runner._precompute_shared_prefix(list(toks))
        scores = runner.anchor_importance_scores([seq]).cpu().numpy()[0]
        assert np.allclose(scores, arrays[f"{c['tag']}::importance"], rtol=2e-4, atol=2e-5), c["tag"]
        assert runner._compute_anchor_positions(seq) == c["anchors"]
        # the probe leaves the allocator as it found it, apart from the rotation of the free list
        assert seq.block_table == []


def _random_requests(rng, arch, n, A, G, mode_cycle, affix):
    reqs = []
    for i in range(n):
        mode = mode_cycle[i % len(mode_cycle)]
        head, tail = rng.randint(1, 9), rng.randint(1, 9)
        body = lambda k: [rng.randint(1, arch.vocab - 2) for _ in range(k)]
        if mode == "prefix":
            toks = affix + body(tail)
            r = dict(affix_start=0, affix_end=A, generation_start=None)
        elif mode == "infix":
            toks = body(head) + affix + body(tail)
            r = dict(affix_start=head, affix_end=head + A, generation_start=None)
        else:
            toks = body(head) + [arch.mask_id] * G + affix
            r = dict(affix_start=head + G, affix_end=head + G + A, generation_start=head)
        r.update(prompt=toks, gen_length=G)
        reqs.append(r)
    return reqs


@pytest.mark.parametrize("kind,nh,hkv", [("llada", 4, 4), ("llada", 4, 2), ("dream", 4, 2)])
@pytest.mark.parametrize("max_num_seqs", [1, 4])
def test_engine_matches_cpu_oracle_fp32(kind, nh, hkv, max_num_seqs):
    """Random tiny models, mixed placements, continuous batching with more requests than
    slots; greedy tokens, anchors and NFE equal the request-at-a-time CPU restatement."""
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.engine import generate_with_acache
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    rng = random.Random(5)
    arch = ArchSpec(kind, n_layers=2, d_model=64, n_heads=nh, n_kv_heads=hkv, ffn=96, vocab=160, rope_theta=10000.0,
                    rms_eps=1e-5 if kind == "llada" else 1e-6, act="silu", mask_id=159)
    weights = random_state_dict(arch, seed=11, std=0.3)
    A, G, T = 13, 8, 4
    affix = [rng.randint(1, 150) for _ in range(A)]
    reqs = _random_requests(rng, arch, 6, A, G, ["infix", "prefix", "suffix"], affix)
    oracle = OracleModel(arch, weights, torch.float32)
    o_req = []
    for r in reqs:
        toks = list(r["prompt"]) + ([arch.mask_id] * G if r["generation_start"] is None else [])
        o_req.append(dict(tokens=toks, affix_start=r["affix_start"], affix_end=r["affix_end"],
                          generation_start=len(r["prompt"]) if r["generation_start"] is None else r["generation_start"],
                          gen_length=G))
    want, want_nfe, want_anchors = generate_with_acache(oracle, o_req, anchor_ratio=0.3, threshold=0.6, block_length=T)

    hf_cfg, model = (_llada if kind == "llada" else _dream)(arch, weights, torch.float32)
    cfg = _serve_config(hf_cfg, arch, kind, torch.float32, threshold=0.6, anchor_ratio=0.3, max_num_seqs=max_num_seqs,
                        num_kvcache_blocks=32, block_length=T, gen_length=G)
    runner = ModelRunner(model, cfg)
    seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                     prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"],
                     generation_start=r["generation_start"]) for r in reqs]
    outs, nfe = runner.generate_with_acache(seqs)
    assert [s.anchor_positions for s in seqs] == want_anchors
    assert outs == want
    assert nfe == want_nfe


@pytest.mark.parametrize("kind,nh,hkv,affix_kinds", [("llada", 4, 4, ["prefix"]), ("llada", 4, 2, ["infix", "suffix"]),
                                                     ("dream", 4, 2, ["prefix", "infix"])])
@pytest.mark.parametrize("grouped", [False, True])
def test_engine_bf16_tensor_core_path_agrees_with_fp32_oracle(kind, nh, hkv, affix_kinds, grouped):
    """bf16 cache and weights, head_dim 128: every step runs the tcgen05 kernels (refresh,
    block decode with the softmax spread over the warps, the grouped two-part kernel when
    ``grouped``, tensor-core influence score).  bf16 rounding may flip a greedy choice between
    near-equal logits, after which the request's later tokens differ too, so this free-running
    check is agreement with the bf16 CPU restatement on most tokens (a wrong kernel gives about
    1/vocab) and nearly all anchors, identical results between two runs, and a clean device
    error flag.  The step-by-step comparison of logits, greedy choices and anchors in bf16 is
    tests/test_engine_parity_gpu.py (teacher-forced, real widths); exactness is checked kernel by
    kernel and end to end in fp32."""
    from acache_b200 import _lib
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.engine import generate_with_acache
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    rng = random.Random(17)
    arch = ArchSpec(kind, n_layers=2, d_model=128 * nh, n_heads=nh, n_kv_heads=hkv, ffn=256, vocab=200,
                    rope_theta=10000.0, rms_eps=1e-5 if kind == "llada" else 1e-6, act="silu", mask_id=199)
    weights = random_state_dict(arch, seed=23, std=0.8)
    A, G, T = 150, 16, 8
    affix = [rng.randint(1, 190) for _ in range(A)]
    reqs = _random_requests(rng, arch, 6, A, G, affix_kinds, affix)
    oracle = OracleModel(arch, weights, torch.bfloat16)    # the same roundings as the served model, on the CPU
    o_req = []
    for r in reqs:
        toks = list(r["prompt"]) + ([arch.mask_id] * G if r["generation_start"] is None else [])
        o_req.append(dict(tokens=toks, affix_start=r["affix_start"], affix_end=r["affix_end"],
                          generation_start=len(r["prompt"]) if r["generation_start"] is None else r["generation_start"],
                          gen_length=G))
    want, _, want_anchors = generate_with_acache(oracle, o_req, anchor_ratio=0.2, threshold=0.6, block_length=T)

    hf_cfg, model = (_llada if kind == "llada" else _dream)(arch, weights, torch.bfloat16)

    def run():
        cfg = _serve_config(hf_cfg, arch, kind, torch.bfloat16, threshold=0.6, anchor_ratio=0.2, max_num_seqs=4,
                            num_kvcache_blocks=40, cache_block_size=64, block_length=T, gen_length=G,
                            group_shared_span=grouped)
        runner = ModelRunner(model, cfg)
        seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=64, mask_id=arch.mask_id,
                         prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"],
                         generation_start=r["generation_start"]) for r in reqs]
        outs, nfe = runner.generate_with_acache(seqs)
        return outs, [s.anchor_positions for s in seqs]

    outs, anchors = run()
    _lib.check_device_errors()
    assert all(arch.mask_id not in o for o in outs)
    tok_total = sum(len(o) for o in want)
    tok_same = sum(int(a == b) for o, w in zip(outs, want) for a, b in zip(o, w))
    anc_total = sum(len(a) for a in want_anchors)
    anc_same = sum(len(set(a) & set(b)) for a, b in zip(anchors, want_anchors))
    print(f"agreement: tokens {tok_same}/{tok_total}, anchors {anc_same}/{anc_total}")
    assert anc_same >= 0.85 * anc_total, (anc_same, anc_total)
    assert tok_same >= 0.8 * tok_total, (tok_same, tok_total)
    again, anchors_again = run()
    assert again == outs and anchors_again == anchors     # deterministic, whichever part arrives second


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graph_replayed_decode_equals_eager_decode(dtype):
    """The block-decode forward replayed from a CUDA graph (step metadata in fixed buffers, one
    graph per number of active rows, reused across blocks and across calls) gives exactly the
    tokens of the eager forward; batch composition changes while requests retire."""
    from acache_b200 import _lib
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.models import ArchSpec, random_state_dict

    rng = random.Random(29)
    arch = ArchSpec("llada", n_layers=2, d_model=256, n_heads=2, n_kv_heads=2, ffn=192, vocab=180, rope_theta=10000.0,
                    rms_eps=1e-5, act="silu", mask_id=179)
    weights = random_state_dict(arch, seed=31, std=0.5)
    A, T = 40, 4
    affix = [rng.randint(1, 170) for _ in range(A)]
    hf_cfg, model = _llada(arch, weights, dtype)

    def run(graphs, runner=None):
        outs = []
        for G in (8, 12):   # two calls on one runner: graphs of the first call are reused by the second
            reqs = _random_requests(random.Random(G), arch, 5, A, G, ["prefix", "infix", "suffix"], affix)
            cfg = _serve_config(hf_cfg, arch, "llada", dtype, threshold=0.7, anchor_ratio=0.25, max_num_seqs=3,
                                num_kvcache_blocks=48, cache_block_size=16, block_length=T, gen_length=G,
                                use_cuda_graphs=graphs)
            runner = runner or ModelRunner(model, cfg)
            runner.config.gen_length = G
            seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=16, mask_id=arch.mask_id,
                             prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"],
                             generation_start=r["generation_start"]) for r in reqs]
            outs.append(runner.generate_with_acache(seqs))
        return outs, runner

    eager, _ = run(False)
    _lib.enable_kernel_timers(True)     # timed operators inside the graph record external events
    try:
        replayed, runner = run(True)
        timers = _lib.kernel_timers()
    finally:
        _lib.enable_kernel_timers(False)
    assert replayed == eager
    assert runner._decode_graphs and all(g.graph is not None for g in runner._decode_graphs.values())
    assert timers["attention_decode"][1] > 0 and timers["attention_decode"][0] > 0.0
    _lib.check_device_errors()


@pytest.mark.parametrize("which,kind", [("hf_llada_dkv", "llada"), ("hf_dream_dkv", "dream")])
def test_dkv_engine_matches_hf_reference_fixtures(which, kind, request):
    """dKV-Cache decoding on top of affix reuse, fp32: the tokens of the reference's HF batch-1
    path for prefix / infix / suffix placement (batched here, three requests per run), anchor
    ratios 0, ~1/3 and 1, cache intervals 1-3; with ratio 1 the plain dKV engine gives the same."""
    from acache_b200.model_runner import ModelRunner
    from oracle.models import ArchSpec

    meta, weights, arrays = request.getfixturevalue(which)
    arch = ArchSpec(**meta["arch"])
    hf_cfg, model = (_llada if kind == "llada" else _dream)(arch, weights, torch.float32)
    grid = sorted({(c["anchor_ratio"], c["interval"]) for c in meta["cases"]})
    for ratio, interval in grid:
        cases = [c for c in meta["cases"] if (c["anchor_ratio"], c["interval"]) == (ratio, interval)]
        G, T, steps = cases[0]["gen_length"], cases[0]["block_length"], cases[0]["steps"]
        cfg = _serve_config(hf_cfg, arch, kind, torch.float32, anchor_ratio=ratio, gen_length=G, block_length=T,
                            dkv_steps=steps, dkv_cache_interval=interval, enable_dkv_cache=True, max_num_seqs=3)
        runner = ModelRunner(model, cfg)
        seqs = [_sequence(c, arch) for c in cases]
        outs, nfe = runner.generate_with_dkv_acache(seqs)
        assert nfe == steps * len(cases)
        for c, seq, out in zip(cases, seqs, outs):
            want = arrays[c["tag"] + "::tokens"].tolist()
            assert seq.token_ids == want, c["tag"]
            g0 = len(c["prompt"]) if c["generation_start"] is None else c["generation_start"]
            assert out == want[g0: g0 + G], c["tag"]
        if ratio == 1.0:   # every affix token recomputed = no reuse at all
            cfg = _serve_config(hf_cfg, arch, kind, torch.float32, gen_length=G, block_length=T, dkv_steps=steps,
                                dkv_cache_interval=interval, enable_dkv_cache=True, enable_acache=False, max_num_seqs=2)
            plain = ModelRunner(model, cfg)
            from acache_b200.sequence import Sequence

            prompts = []
            for c in cases:
                toks = list(c["prompt"])
                prompts.append(Sequence(toks, block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                                        generation_start=c["generation_start"]))
            outs2, nfe2 = plain.generate_with_dkv_cache(prompts)
            assert outs2 == outs and nfe2 == nfe


@pytest.mark.parametrize("kind,nh,hkv", [("llada", 4, 2), ("dream", 4, 2)])
def test_dkv_engine_matches_cpu_oracle_fp32(kind, nh, hkv):
    """Random tiny GQA models, five requests over mixed placements in static batches of three:
    dKV alone and dKV on top of affix reuse against the request-at-a-time CPU restatement."""
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.engine import generate_with_dkv
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    rng = random.Random(41)
    arch = ArchSpec(kind, n_layers=2, d_model=64, n_heads=nh, n_kv_heads=hkv, ffn=96, vocab=160, rope_theta=10000.0,
                    rms_eps=1e-5 if kind == "llada" else 1e-6, act="silu", mask_id=159)
    weights = random_state_dict(arch, seed=13, std=0.3)
    A, G, T, steps, interval = 11, 8, 4, 4, 2
    affix = [rng.randint(1, 150) for _ in range(A)]
    reqs = _random_requests(rng, arch, 5, A, G, ["infix", "prefix", "suffix"], affix)
    oracle = OracleModel(arch, weights, torch.float32)
    o_req = []
    for r in reqs:
        toks = list(r["prompt"]) + ([arch.mask_id] * G if r["generation_start"] is None else [])
        o_req.append(dict(tokens=toks, affix_start=r["affix_start"], affix_end=r["affix_end"],
                          generation_start=len(r["prompt"]) if r["generation_start"] is None else r["generation_start"],
                          gen_length=G))
    hf_cfg, model = (_llada if kind == "llada" else _dream)(arch, weights, torch.float32)
    for ratio in (None, 0.3):
        want, want_nfe = generate_with_dkv(oracle, o_req, T, steps, interval, ratio)
        cfg = _serve_config(hf_cfg, arch, kind, torch.float32, anchor_ratio=ratio or 0.0, gen_length=G, block_length=T,
                            dkv_steps=steps, dkv_cache_interval=interval, enable_dkv_cache=True,
                            enable_acache=ratio is not None, max_num_seqs=3, num_kvcache_blocks=40)
        runner = ModelRunner(model, cfg)
        seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                         prompt_affix_start=r["affix_start"] if ratio is not None else None,
                         prompt_affix_end=r["affix_end"] if ratio is not None else None,
                         generation_start=r["generation_start"]) for r in reqs]
        outs, nfe = (runner.generate_with_dkv_acache if ratio is not None else runner.generate_with_dkv_cache)(seqs)
        assert outs == want, ratio
        assert nfe == want_nfe


def test_reuse_with_every_affix_token_an_anchor_equals_no_reuse_baseline(hf_llada):
    """reference: nano-vdllm/tests/test_model_runner_acache.py:597-687 (ratio 1.0 recomputes
    the whole affix, so the logits equal the full-recompute baseline)."""
    from acache_b200.model_runner import ModelRunner
    from acache_b200.utils import reset_context
    from oracle.models import ArchSpec

    meta, weights, _ = hf_llada
    arch = ArchSpec(**meta["arch"])
    hf_cfg, model = _llada(arch, weights, torch.bfloat16)
    for c in meta["cases"][:6:2]:
        base = ModelRunner(model, _serve_config(hf_cfg, arch, "llada", torch.bfloat16, enable_acache=False))
        seq = _sequence(c, arch)
        base.block_manager.allocate(seq)
        seq.finalize_slot_mapping()
        ids, pos, _, _ = base.prepare_caching([seq])
        want = model(ids, position_ids=pos).logits.float()
        reset_context()
        run = ModelRunner(model, _serve_config(hf_cfg, arch, "llada", torch.bfloat16, anchor_ratio=1.0))
        seq = _sequence(c, arch)
        toks = run._prepare_acache([seq])
        run._precompute_shared_prefix(list(toks))
        seq.set_anchor_positions(list(range(seq.affix_start, seq.affix_end)))
        run.block_manager.allocate(seq)
        seq.finalize_slot_mapping()
        ids, pos, _ = run.prepare_caching_acache([seq])
        got = model(ids, position_ids=pos).logits.float()
        reset_context()
        torch.testing.assert_close(got, want, rtol=5e-2, atol=5e-2)


def test_baseline_generation_equals_reuse_with_full_anchor_ratio_fp32():
    """generate_with_dual_cache against generate_with_acache(ratio 1.0): same tokens."""
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.models import ArchSpec, random_state_dict

    rng = random.Random(9)
    arch = ArchSpec("llada", n_layers=2, d_model=64, n_heads=4, n_kv_heads=4, ffn=96, vocab=160, rope_theta=10000.0,
                    rms_eps=1e-5, act="silu", mask_id=159)
    weights = random_state_dict(arch, seed=4, std=0.3)
    hf_cfg, model = _llada(arch, weights, torch.float32)
    A, G, T = 9, 8, 4
    affix = [rng.randint(1, 150) for _ in range(A)]
    reqs = _random_requests(rng, arch, 4, A, G, ["prefix", "infix", "suffix"], affix)

    def run(reuse):
        cfg = _serve_config(hf_cfg, arch, "llada", torch.float32, threshold=0.5, anchor_ratio=1.0, max_num_seqs=2,
                            num_kvcache_blocks=32, block_length=T, gen_length=G, enable_acache=reuse,
                            group_shared_span=False)  # exact equality needs the same summation order of the keys
        runner = ModelRunner(model, cfg)
        seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                         prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"],
                         generation_start=r["generation_start"]) for r in reqs]
        return (runner.generate_with_acache if reuse else runner.generate_with_dual_cache)(seqs)

    got, nfe_a = run(True)
    want, nfe_b = run(False)
    assert got == want and nfe_a == nfe_b


def test_block_tables_follow_the_allocator_contract():
    """Worked example with the reference's own classes (block 8, 8 blocks, 2-token prefix
    affix, ratio 0.5): the probe of each request rotates the free list, so the two requests
    end up in blocks 3 and 4."""
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.models import ArchSpec, random_state_dict

    arch = ArchSpec("llada", n_layers=1, d_model=64, n_heads=4, n_kv_heads=4, ffn=64, vocab=64, rope_theta=10000.0,
                    rms_eps=1e-5, act="silu", mask_id=63)
    hf_cfg, model = _llada(arch, random_state_dict(arch, seed=1, std=0.2), torch.float32)
    cfg = _serve_config(hf_cfg, arch, "llada", torch.float32, anchor_ratio=0.5, max_num_seqs=4, num_kvcache_blocks=8,
                        block_length=4, gen_length=4, threshold=0.0)
    runner = ModelRunner(model, cfg)
    a = Sequence([2, 3, 4, 5], block_length=4, gen_length=4, cache_block_size=8, mask_id=63, prompt_affix_len=2)
    b = Sequence([2, 3, 4, 6], block_length=4, gen_length=4, cache_block_size=8, mask_id=63, prompt_affix_len=2)
    prefix = runner._prepare_acache([a, b])
    batched = []
    runner._admit_sequences_with_acache(batched, [a, b], prefix, allow_kv_cache_resize=False)
    assert a.block_table == [3] and b.block_table == [4]
    assert list(runner.block_manager.free_block_ids) == [5, 6, 7, 1, 2]
    for seq in (a, b):
        anchor = seq.anchor_positions[0]
        first = seq.block_table[0] * 8
        assert seq.read_slot_map[anchor] == first
        assert seq.read_slot_map[1 - anchor] == 1 - anchor
        assert seq.recompute_slot_mapping == list(range(first, first + 7))


def test_anchor_selection_oom_recovery_is_host_side(hf_llada, monkeypatch):
    """Failure injected on the host: the probe raises OutOfMemoryError once; the engine
    shrinks the cache by 4 blocks, recomputes the affix, retries and restores the size."""
    from acache_b200.model_runner import ModelRunner
    from oracle.models import ArchSpec

    meta, weights, arrays = hf_llada
    arch = ArchSpec(**meta["arch"])
    hf_cfg, model = _llada(arch, weights, torch.float32)
    runner = ModelRunner(model, _serve_config(hf_cfg, arch, "llada", torch.float32))
    real = runner.anchor_importance_scores
    fired = []

    def flaky(seqs):
        if not fired:
            fired.append(1)
            raise torch.OutOfMemoryError("injected")
        return real(seqs)

    monkeypatch.setattr(runner, "anchor_importance_scores", flaky)
    cases = [c for c in meta["cases"] if c["threshold"] == 0.9][:2]
    seqs = [_sequence(c, arch) for c in cases]
    outs, _ = runner.generate_with_acache(seqs)
    assert fired and runner.config.num_kvcache_blocks == 24
    for c, seq in zip(cases, seqs):
        assert seq.token_ids == arrays[f"{c['tag']}::tokens"].tolist()


def test_request_stream_with_arrival_times_gives_the_same_tokens():
    """Requests handed over as a stream (arrival times) instead of all at once: admission happens
    at block boundaries as requests arrive, each request's tokens are unchanged."""
    from acache_b200.dp import poisson_arrival_times
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from oracle.engine import generate_with_acache
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    rng = random.Random(13)
    arch = ArchSpec("llada", n_layers=2, d_model=64, n_heads=4, n_kv_heads=4, ffn=96, vocab=160, rope_theta=10000.0,
                    rms_eps=1e-5, act="silu", mask_id=159)
    weights = random_state_dict(arch, seed=21, std=0.3)
    A, G, T = 11, 8, 4
    affix = [rng.randint(1, 150) for _ in range(A)]
    reqs = _random_requests(rng, arch, 5, A, G, ["prefix", "infix"], affix)
    oracle = OracleModel(arch, weights, torch.float32)
    o_req = [dict(tokens=list(r["prompt"]) + [arch.mask_id] * G, affix_start=r["affix_start"], affix_end=r["affix_end"],
                  generation_start=len(r["prompt"]), gen_length=G) for r in reqs]
    want, want_nfe, _ = generate_with_acache(oracle, o_req, anchor_ratio=0.3, threshold=0.6, block_length=T)
    hf_cfg, model = _llada(arch, weights, torch.float32)
    cfg = _serve_config(hf_cfg, arch, "llada", torch.float32, threshold=0.6, anchor_ratio=0.3, max_num_seqs=3,
                        num_kvcache_blocks=32, block_length=T, gen_length=G)
    runner = ModelRunner(model, cfg)
    seqs = [Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                     prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"]) for r in reqs]
    times = poisson_arrival_times(len(seqs), rate_per_s=40.0, seed=2)
    outs, nfe = runner.generate_with_acache(seqs, arrival_times=times)
    assert outs == want and nfe == want_nfe
    assert all(t is not None and t >= a for t, a in zip(runner.last_completion_times, times))


def test_fused_qkv_projection_path_gives_the_same_logits():
    """The tcgen05 QKV GEMM with fused RoPE + cache scatter, switched on inside the model,
    against the default library-GEMM path: refresh logits agree within bf16 tolerance and the
    K/V written to the cache agree."""
    from acache_b200.model import modeling_common
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from acache_b200.utils import reset_context
    from oracle.models import ArchSpec, random_state_dict

    rng = random.Random(3)
    arch = ArchSpec("llada", n_layers=2, d_model=256, n_heads=2, n_kv_heads=2, ffn=512, vocab=320, rope_theta=500000.0,
                    rms_eps=1e-5, act="silu", mask_id=319)
    weights = random_state_dict(arch, seed=8, std=0.08)
    hf_cfg, model = _llada(arch, weights, torch.bfloat16)
    A, G, T = 40, 8, 4
    affix = [rng.randint(1, 300) for _ in range(A)]
    r = _random_requests(rng, arch, 1, A, G, ["infix"], affix)[0]
    results = []
    for fused in (False, True):
        modeling_common.FUSED_QKV = fused
        try:
            cfg = _serve_config(hf_cfg, arch, "llada", torch.bfloat16, anchor_ratio=0.25, max_num_seqs=2,
                                num_kvcache_blocks=32, block_length=T, gen_length=G)
            runner = ModelRunner(model, cfg)
            seq = Sequence(r["prompt"], block_length=T, gen_length=G, cache_block_size=8, mask_id=arch.mask_id,
                           prompt_affix_start=r["affix_start"], prompt_affix_end=r["affix_end"])
            toks = runner._prepare_acache([seq])
            runner._precompute_shared_prefix(list(toks))
            seq.set_anchor_positions(list(range(seq.affix_start, seq.affix_start + seq.num_anchor_tokens)))
            runner.block_manager.allocate(seq)
            seq.finalize_slot_mapping()
            ids, pos, _ = runner.prepare_caching_acache([seq])
            logits = model(ids, position_ids=pos).logits.float()
            reset_context()
            results.append((logits, runner.kv_cache.float().clone(), list(seq.recompute_slot_mapping)))
        finally:
            modeling_common.FUSED_QKV = False
    (la, ca, slots), (lb, cb, _) = results
    torch.testing.assert_close(lb, la, rtol=5e-2, atol=5e-2)
    flat_a = ca.view(2, arch.n_layers, -1, arch.n_kv_heads, 128)[:, :, slots]
    flat_b = cb.view(2, arch.n_layers, -1, arch.n_kv_heads, 128)[:, :, slots]
    torch.testing.assert_close(flat_b, flat_a, rtol=5e-2, atol=5e-2)
