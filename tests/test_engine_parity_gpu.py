"""Engine against the CPU restatement at the real widths of the three served workloads, in
bf16, teacher-forced: two layers of the LLaDA-8B architecture with an 800-token prefix affix,
two layers of Dream-7B with a 600-token affix inside the prompt (query-side relocation), and
LLaDA with a 2048-token affix behind the generation span.

Every forward of every request (the refresh and the first block-decode steps) is compared
with the restatement's forward of the same request in the same state: after each step the
engine's working block is overwritten with the tokens the restatement committed, so one
flipped greedy choice cannot cascade.  Checked per step:

* logits: max |difference| <= 2e-2 of the restatement's logit range (bf16 tolerance);
* greedy choice: wherever the arg-max differs, the restatement's own margin between the two
  candidates is below that tolerance (the first divergence is printed with its margin);
* K/V rows the forward wrote to the paged cache against the restatement's dense cache;
* the shared affix K/V, and its relocated copy when the affix does not start at 0.

Anchors: the restatement's scores through the top-k operator give exactly its anchors; the
engine's own scores (fp32 accumulation where the reference rounds partial sums to bf16) give
the same set up to swaps between scores closer than one bf16 step at the threshold, and the
margin of every swapped index is printed.
"""
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2


def _rel(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)


def _check_logits(tag, got, want, report):
    """got/want [T, V].  Returns nothing; raises on a difference above tolerance."""
    got, want = got.float().cpu(), want.float().cpu()
    span = (want.max() - want.min()).item()
    err = (got - want).abs().max().item() / span
    report["max_logit_err"] = max(report.get("max_logit_err", 0.0), err)
    assert err <= TOL, f"{tag}: logits differ by {err:.3e} of the logit range"
    ga, wa = got.argmax(-1), want.argmax(-1)
    for r in (ga != wa).nonzero().flatten().tolist():
        margin = (want[r, wa[r]] - want[r, ga[r]]).item() / span
        if "first_divergence" not in report:
            report["first_divergence"] = f"{tag} row {r}: engine {int(ga[r])}, restatement {int(wa[r])}, margin {margin:.2e} of range"
        report["flips"] = report.get("flips", 0) + 1
        assert margin <= TOL, f"{tag} row {r}: arg-max differs with a margin of {margin:.3e} of the logit range"


def _check_stats(tag, x0, conf, want, report):
    """The form greedy unmasking consumes when the output head is fused with the arg-max: token and
    confidence per position against the restatement's logits of the same step."""
    want = want.float().cpu()
    x0, conf = x0.cpu(), conf.float().cpu()
    span = (want.max() - want.min()).item()
    top2 = want.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > TOL * span
    assert torch.equal(x0[clear], want.argmax(-1)[clear]), tag
    picked = want.gather(1, x0[:, None])[:, 0]
    assert ((top2[:, 0] - picked) <= TOL * span).all(), tag          # never a token the restatement ranks far below
    want_conf = torch.exp(top2[:, 0] - torch.logsumexp(want, -1))
    err = (torch.log(conf) - torch.log(want_conf)).abs().max().item()
    report["max_log_conf_err"] = max(report.get("max_log_conf_err", 0.0), err)
    assert err <= 2 * TOL * span, f"{tag}: confidence differs by a factor of e^{err:.3f}"
    report["fused_head_steps"] = report.get("fused_head_steps", 0) + 1


def _build(kind, layers, seed):
    if kind == "llada":
        from acache_b200.model.configuration import LLaDAConfig
        from acache_b200.model.modeling_llada import LLaDAModelLM

        hf = LLaDAConfig.llada_8b()
        hf.n_layers = layers
        model = LLaDAModelLM(hf, device=DEV, dtype=torch.bfloat16, init_params=True, seed=seed).eval()
        head = model.model.transformer["ff_out"].weight
        arch = dict(kind="llada", n_layers=layers, d_model=hf.d_model, n_heads=hf.n_heads, n_kv_heads=hf.n_kv_heads,
                    ffn=hf.ffn_size, vocab=hf.vocab_size, rope_theta=hf.rope_theta, rms_eps=hf.rms_norm_eps,
                    act="silu", mask_id=hf.mask_token_id)
    else:
        from acache_b200.model.configuration import DreamConfig
        from acache_b200.model.modeling_dream import DreamModel

        hf = DreamConfig.dream_7b()
        hf.num_hidden_layers = layers
        model = DreamModel(hf, device=DEV, dtype=torch.bfloat16, init_params=True, seed=seed).eval()
        head = model.lm_head.weight
        arch = dict(kind="dream", n_layers=layers, d_model=hf.hidden_size, n_heads=hf.num_attention_heads,
                    n_kv_heads=hf.num_key_value_heads, ffn=hf.intermediate_size, vocab=hf.vocab_size,
                    rope_theta=hf.rope_theta, rms_eps=hf.rms_norm_eps, act="silu", mask_id=hf.mask_token_id)
    with torch.no_grad():
        head[hf.mask_token_id] = head[0]    # the mask token is never the arg-max (ties go to the lower index)
    from oracle.models import ArchSpec, OracleModel

    weights = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    oracle = OracleModel(ArchSpec(**arch), weights, torch.bfloat16)
    return hf, model.fuse_projections(), oracle


def _run_case(kind, placement, A, ratio, n_req, own_lo, own_hi, G, T, decode_steps, seed, own_gemm=None):
    """``own_gemm``: None = the projections as shipped; True = every projection on this package's
    CTA-pair tcgen05 kernels (fused QKV + RoPE + scatter, gate/up + activation, plain, output head)."""
    from acache_b200.model import modeling_common as mc

    saved = (mc.OWN_QKV, mc.OWN_GATE_UP, mc.OWN_DENSE, mc.OWN_HEAD)
    if own_gemm is not None:
        mc.set_own_gemm(own_gemm)
    try:
        return _run_case_body(kind, placement, A, ratio, n_req, own_lo, own_hi, G, T, decode_steps, seed)
    finally:
        mc.OWN_QKV, mc.OWN_GATE_UP, mc.OWN_DENSE, mc.OWN_HEAD = saved


def _run_case_body(kind, placement, A, ratio, n_req, own_lo, own_hi, G, T, decode_steps, seed):
    from acache_b200 import _lib, ops
    from acache_b200.config import Config
    from acache_b200.model import acache_attention as aa
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence
    from acache_b200.utils import reset_context
    from oracle.engine import _request_kv, compute_affix_kv, request_steps, select_anchors

    hf, model, oracle = _build(kind, 2, seed)
    spec = oracle.spec
    rng = random.Random(seed)
    body = lambda n: [rng.randrange(1, 20000) for _ in range(n)]
    affix = body(A)
    reqs = []
    for _ in range(n_req):
        if placement == "prefix":
            prompt, a0, g0 = affix + body(rng.randint(own_lo, own_hi)), 0, None
        elif placement == "infix":
            head = body(rng.randint(own_lo, own_hi))
            prompt, a0, g0 = head + affix + body(rng.randint(own_lo, own_hi)), len(head), None
        else:   # the affix behind the generation span
            ctx = body(rng.randint(own_lo, own_hi))
            prompt, a0, g0 = ctx + [spec.mask_id] * G + affix, len(ctx) + G, len(ctx)
        reqs.append((prompt, a0, g0))
    Bk = 256
    blocks = -(-A // Bk) * 2 + n_req * (-(-(A + own_hi * 2 + G) // Bk) + 1) + 4
    cfg = Config(hf_config=hf, mask_id=spec.mask_id, recompute_batch_size=n_req, max_num_seqs=n_req, gen_length=G,
                 block_length=T, threshold=0.9, cache_block_size=Bk, num_kvcache_blocks=blocks, enable_acache=True,
                 anchor_ratio=ratio, selection_mode="top", model_type=kind, use_cuda_graphs=False)
    runner = ModelRunner(model, cfg)
    seqs = [Sequence(p, block_length=T, gen_length=G, cache_block_size=Bk, mask_id=spec.mask_id,
                     prompt_affix_start=a0, prompt_affix_end=a0 + A, generation_start=g0) for p, a0, g0 in reqs]
    report = {}
    with torch.inference_mode():
        # ---- shared affix K/V
        prefix = runner._prepare_acache(seqs)
        runner._precompute_shared_prefix(list(prefix))
        affix_kv = compute_affix_kv(oracle, affix)
        k, v = runner._flat_kv()
        report["affix_k_err"], report["affix_v_err"] = _rel(k[:, :A], affix_kv.k), _rel(v[:, :A], affix_kv.v)
        assert report["affix_k_err"] <= TOL and report["affix_v_err"] <= TOL, report

        # ---- anchors
        steps, states = [], []
        for seq in seqs:
            o_anchors, o_scores = select_anchors(oracle, affix_kv, seq.token_ids, seq.affix_start, seq.affix_end, ratio)
            off = torch.tensor([seq.affix_start], dtype=torch.int32, device=DEV)
            fed = ops.anchor_topk(o_scores[None].to(DEV), seq.num_anchor_tokens, True, off)[0].tolist()
            assert fed == o_anchors                      # same scores in, same anchors out
            own_scores = runner.anchor_importance_scores([seq])[0]
            own = ops.anchor_topk(own_scores[None], seq.num_anchor_tokens, True, off)[0].tolist()
            swapped = sorted(set(own) ^ set(o_anchors))
            kth = torch.sort(o_scores, descending=True).values[seq.num_anchor_tokens - 1].item()
            margins = [abs(o_scores[i - seq.affix_start].item() - kth) for i in swapped]
            report["anchor_overlap"] = report.get("anchor_overlap", []) + [f"{len(set(own) & set(o_anchors))}/{len(o_anchors)}"]
            report["swapped_margins"] = report.get("swapped_margins", []) + [
                (i, round(m, 5)) for i, m in zip(swapped, margins)]
            score_err = (own_scores.cpu() - o_scores).abs().max().item()
            report["score_err"] = max(report.get("score_err", 0.0), score_err / (o_scores.max() - o_scores.min()).item())
            # a swap is only legitimate between scores the reference itself cannot tell apart: its
            # per-layer sums are bf16 values, whose spacing at the threshold's magnitude is 2^-7 * kth
            assert all(m <= abs(kth) * 2.0 ** -7 for m in margins), (swapped, margins, kth)
            seq.set_anchor_positions(o_anchors)          # teacher forcing: the rest uses the restatement's anchors
            kv_out = []
            g0 = seq.generation_start
            steps.append(request_steps(oracle, affix_kv, seq.token_ids, seq.affix_start, seq.affix_end, g0, G, T,
                                       o_anchors, 0.9, kv_out=kv_out))
            states.append(kv_out)

        # ---- relocated affix K/V (the materialising kernel at this size)
        if placement != "prefix":
            runner._configure_affix_relocation(seqs)
            a0 = runner._attn_layers[0]
            nb = -(-A // Bk)
            L, _, hkv, D = k.shape
            ks = torch.zeros(L, 2 * nb * Bk, hkv, D, dtype=k.dtype, device=DEV)
            vs = torch.zeros_like(ks)
            ks[:, :A], vs[:, :A] = k[:, :A], v[:, :A]
            shift = seqs[0].affix_start
            aa.relocate_affix_batched(ks, vs, a0.relocation_rope_cos, a0.relocation_rope_sin, A,
                                      torch.tensor([shift], dtype=torch.int32, device=DEV),
                                      dst_slots=torch.tensor([nb * Bk], dtype=torch.int32, device=DEV))
            want = _request_kv(oracle, affix_kv, len(seqs[0]), shift)
            report["relocated_k_err"] = _rel(ks[:, nb * Bk: nb * Bk + A], want.k[:, shift: shift + A])
            assert report["relocated_k_err"] <= TOL, report
            assert torch.equal(vs[:, nb * Bk: nb * Bk + A], v[:, :A])

        # ---- refresh forward of all requests in one ragged batch
        for seq in seqs:
            runner.block_manager.allocate(seq)
            runner._finalize_sequence_layout(seq)
        ids, pos, starts = runner.prepare_caching_acache(seqs)
        keep = starts.to(torch.int64).unsqueeze(1) + torch.arange(T, device=DEV)
        if kind == "dream":
            row_starts = torch.from_numpy(runner._last_cu_q_host[:-1].astype(np.int64)).to(DEV)
            keep = runner._dream_shift_keep_indices(keep, row_starts)
        out = runner._forward_model(ids, pos, logits_keep_indices=keep.flatten(), max_pos=max(len(s) for s in seqs))
        reset_context()
        logits = out.logits.view(len(seqs), T, -1)
        working = torch.empty(len(seqs), T, dtype=torch.int64, device=DEV)
        for b, seq in enumerate(seqs):
            phase, _, want, blk = next(steps[b])
            assert phase == "refresh"
            _check_logits(f"refresh req {b}", logits[b], want, report)
            working[b] = blk.to(DEV)
            kv, rows = states[b][0], states[b][1]
            slots = torch.tensor(seq.recompute_slot_mapping, dtype=torch.int64, device=DEV)
            assert seq.recompute_positions == rows.tolist()
            report["kv_rows_err"] = max(report.get("kv_rows_err", 0.0), _rel(k[:, slots], kv.k[:, rows]),
                                        _rel(v[:, slots], kv.v[:, rows]))
        assert report["kv_rows_err"] <= TOL, report

        # ---- block-decode steps, teacher-forced
        for step in range(decode_steps):
            positions = runner.prepare_decoding_acache(seqs)
            lg = runner._forward_model(working, positions, max_pos=max(len(s) for s in seqs)).logits
            lg = runner._dream_decode_logits(lg)
            _, stats = runner._decode_forward(working, positions, max(len(s) for s in seqs))   # what unmasking consumes
            reset_context()
            for b, seq in enumerate(seqs):
                phase, _, want, blk = next(steps[b])
                assert phase == "decode"
                _check_logits(f"decode step {step} req {b}", lg[b], want, report)
                if stats is not None:
                    _check_stats(f"decode step {step} req {b}", stats[0][b], stats[1][b], want, report)
                working[b] = blk.to(DEV)
    _lib.check_device_errors()
    print(f"parity {kind} {placement} A={A}: {report}")
    return report


@pytest.mark.parametrize("own_gemm", [None, True])
def test_llada_prefix_800_teacher_forced(own_gemm):
    """The benchmark's shape: LLaDA-8B widths, 800-token prefix affix, requests of 64-256 tokens."""
    _run_case("llada", "prefix", A=800, ratio=0.2, n_req=3, own_lo=64, own_hi=256, G=32, T=32, decode_steps=3, seed=5,
              own_gemm=own_gemm)


@pytest.mark.parametrize("own_gemm", [None, True])
def test_dream_infix_600_teacher_forced(own_gemm):
    """Dream-7B widths (28 query heads on 4 KV heads), 600-token affix between a head and a tail of
    32-128 tokens: query-side relocation, shifted logits."""
    _run_case("dream", "infix", A=600, ratio=0.2, n_req=3, own_lo=32, own_hi=128, G=32, T=32, decode_steps=3, seed=6,
              own_gemm=own_gemm)


def test_llada_suffix_2048_teacher_forced():
    """The long-context shape with the affix cut to 2048 tokens so the CPU side stays short: the
    affix behind an 8-token generation span, contexts of 256-1024 tokens, anchor ratio 0.1."""
    _run_case("llada", "suffix", A=2048, ratio=0.1, n_req=2, own_lo=256, own_hi=1024, G=8, T=8, decode_steps=2, seed=7)


def test_llada_infix_4096_teacher_forced():
    """A long affix inside the prompt: the influence score walks it in chunks, decode and refresh
    read a 4096-token shared span through query-side relocation."""
    _run_case("llada", "infix", A=4096, ratio=0.1, n_req=2, own_lo=5, own_hi=300, G=32, T=32, decode_steps=2, seed=8)


def test_graph_replay_equals_eager_at_real_widths_with_fused_projections():
    """Two layers at LLaDA-8B widths, bf16, the shipped projection kernels (fused QKV, gate/up and
    output head with arg-max statistics): the block-decode forward replayed from CUDA graphs gives
    exactly the tokens of the eager forward while the number of active rows changes (five
    requests, three slots), i.e. every buffer a captured kernel uses stays valid across replays
    and across graphs of other row counts."""
    from acache_b200 import _lib
    from acache_b200.config import Config
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence

    hf, model, _ = _build("llada", 2, seed=11)
    rng = random.Random(12)
    A, G, T = 300, 64, 32
    affix = [rng.randrange(1, 20000) for _ in range(A)]
    prompts = [affix + [rng.randrange(1, 20000) for _ in range(rng.randint(20, 200))] for _ in range(5)]

    def run(graphs):
        cfg = Config(hf_config=hf, mask_id=hf.mask_token_id, recompute_batch_size=2, max_num_seqs=3, gen_length=G,
                     block_length=T, threshold=0.9, cache_block_size=256, num_kvcache_blocks=2 + 3 * 3 + 2,
                     enable_acache=True, anchor_ratio=0.2, selection_mode="top", model_type="llada",
                     use_cuda_graphs=graphs)
        runner = ModelRunner(model, cfg)
        seqs = [Sequence(p, block_length=T, gen_length=G, cache_block_size=256, mask_id=hf.mask_token_id,
                         prompt_affix_len=A) for p in prompts]
        outs, nfe = runner.generate_with_acache(seqs)
        return outs, nfe, [s.anchor_positions for s in seqs], runner

    eager = run(False)[:3]
    replayed = run(True)
    assert replayed[:3] == eager
    assert len(replayed[3]._decode_graphs) >= 2          # several row counts were captured
    _lib.check_device_errors()


def test_many_running_requests_grouped_decode_has_no_device_errors():
    """Two layers at LLaDA-8B widths with 48 requests running at once: block decode launches several
    rounds of grouped attention CTAs per layer (48 x 32 heads / 2 = 768 on 296 resident), refresh
    goes through the many-row kernel, and requests finish at different steps.  With grouped and
    with per-request attention the engine takes the same number of forwards and no kernel raises
    the device error flag (a bounded wait that runs out raises it)."""
    from acache_b200 import _lib
    from acache_b200.config import Config
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence

    hf, model, _ = _build("llada", 2, seed=21)
    rng = random.Random(22)
    A, G, T, n = 800, 64, 32, 72
    affix = [rng.randrange(1, 20000) for _ in range(A)]
    prompts = [affix + [rng.randrange(1, 20000) for _ in range(rng.randint(64, 256))] for _ in range(n)]

    def run(grouped):
        cfg = Config(hf_config=hf, mask_id=hf.mask_token_id, recompute_batch_size=8, max_num_seqs=48, gen_length=G,
                     block_length=T, threshold=0.9, cache_block_size=256, num_kvcache_blocks=4 + 48 * 3 + 4,
                     enable_acache=True, anchor_ratio=0.2, selection_mode="top", model_type="llada")
        cfg.group_shared_span = grouped
        runner = ModelRunner(model, cfg)
        seqs = [Sequence(p, block_length=T, gen_length=G, cache_block_size=256, mask_id=hf.mask_token_id,
                         prompt_affix_len=A) for p in prompts]
        outs, nfe = runner.generate_with_acache(seqs)
        _lib.check_device_errors()
        return outs, nfe

    # the two kernels sum in different orders and a random-init model is full of near-ties, so the
    # tokens are not compared here (the kernel tests compare the two forms number by number)
    grouped = run(True)
    plain = run(False)
    assert grouped[1] == plain[1]
    assert [len(o) for o in grouped[0]] == [len(o) for o in plain[0]]
