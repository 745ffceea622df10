"""Generates the golden fixtures in this directory from the reference itself.

Runs only where a checkout of the reference is available (its root is argument 1
or $ACACHE_REFERENCE).  It imports the reference's own Python, read-only, on CPU:

* layout.json       - reference Sequence / BlockManager / _attention_read_layout
                      on seeded random prefix / infix / suffix requests
                      (nano-vdllm/sequence.py, block_manager.py, model_runner.py:275-282)
* triton_ops.npz    - the reference Triton kernels executed by the Triton CPU
                      interpreter (TRITON_INTERPRET=1) in fp32 / fp16:
                      store_kvcache, _materialize_relocated_affix_kernel,
                      _acache_attention_kernel (plain, key-side, query-side),
                      _baseline_ragged/_decode_attention_kernel
* sampling.npz      - reference ModelRunner.get_transfer_index (model_runner.py:2279-2314)
* topk.npz          - torch.topk + sort on tie-free scores (model_runner.py:833-843)
* hf_llada.npz      - the reference HF batch-1 path (llada/generate_ACache.py) on a
                      tiny random LLaDA in fp32: importance scores, anchors, first
                      refresh logits, final tokens, nfe for prefix / infix / suffix
* hf_dream.npz      - the same for Dream (dream/generate_ACache.py), GQA
* hf_llada_dkv.npz  - the reference HF batch-1 dKV + affix-reuse path for LLaDA
                      (llada/eval_dKV_ACache.py generate_with_dkv_anchor_attention), same grid
* hf_dream_dkv.npz  - the reference HF batch-1 dKV + affix-reuse path
                      (dream/generate_dKV_ACache.py) on a tiny random Dream in fp32: final
                      tokens and nfe for prefix / infix / suffix, 3 anchor ratios, 3 intervals

Usage: TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py <reference_root>
"""
import importlib
import importlib.util
import json
import os
import random
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
_ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ACACHE_REFERENCE")
if not _ref_root:
    sys.exit("usage: make_golden.py <reference_root>  (or set ACACHE_REFERENCE)")
REF = Path(_ref_root)
sys.path.insert(0, str(REF / "nano-vdllm"))
sys.path.insert(0, str(HERE.parents[1]))

# flash_attn is imported by the reference attention module but never called here
if importlib.util.find_spec("flash_attn") is None:
    fa = types.ModuleType("flash_attn")
    fa.flash_attn_varlen_func = fa.flash_attn_with_kvcache = None
    sys.modules["flash_attn"] = fa


def rope_table(length, head_dim, theta, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    fr = torch.outer(torch.arange(length, dtype=torch.float32), inv)
    emb = torch.cat((fr, fr), -1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


# --------------------------------------------------------------------------- layout
def make_layout():
    from block_manager import BlockManager
    from model_runner import ModelRunner
    from sequence import Sequence

    rng = random.Random(1234)
    cases = []
    for _ in range(60):
        bs = rng.choice([4, 8, 16, 256])
        A = rng.randint(1, 40)
        head, tail = rng.randint(0, 20), rng.randint(0, 20)
        G = rng.choice([2, 4, 8])
        mode = rng.choice(["prefix", "infix", "suffix"])
        if mode == "prefix":
            toks = [rng.randint(0, 90) for _ in range(A + tail)]
            kw = dict(prompt_affix_start=0, prompt_affix_end=A)
        elif mode == "infix":
            toks = [rng.randint(0, 90) for _ in range(head + A + tail)]
            kw = dict(prompt_affix_start=head, prompt_affix_end=head + A)
        else:
            toks = [rng.randint(0, 90) for _ in range(head + G + A)]
            kw = dict(prompt_affix_start=head + G, prompt_affix_end=head + G + A, generation_start=head)
        ratio = rng.choice([0.0, 0.1, 0.2, 0.5, 1.0])
        seq = Sequence(toks, block_length=2, gen_length=G, cache_block_size=bs, mask_id=99, **kw)
        seq.enable_acache(anchor_ratio=ratio)
        shared_blocks = -(-A // bs)
        mgr = BlockManager(shared_blocks + 40, bs)
        mgr.reserve_prefix(shared_blocks)
        anchors = sorted(rng.sample(range(seq.affix_start, seq.affix_end), seq.num_anchor_tokens))
        seq.set_anchor_positions(anchors)
        # a probe allocation/free before the real one rotates the free list (model_runner.py:693,799-801)
        mgr.allocate(seq)
        mgr.deallocate(seq)
        mgr.allocate(seq)
        seq.finalize_slot_mapping()
        seq.current_block_idx = rng.randrange(seq.num_blocks_to_generate)
        runner = object.__new__(ModelRunner)
        runner.shared_prefix_len = A
        packed, n_shared = runner._attention_read_layout(seq, True)
        cases.append(dict(
            tokens=toks, kwargs=kw, gen_length=G, block_length=2, cache_block_size=bs, mask_id=99, ratio=ratio,
            shared_blocks=shared_blocks, num_blocks=shared_blocks + 40, anchors=anchors,
            current_block_idx=seq.current_block_idx,
            out=dict(token_ids=seq.token_ids, block_table=seq.block_table, recompute_positions=seq.recompute_positions,
                     recompute_slot_mapping=seq.recompute_slot_mapping, read_slot_map=seq.read_slot_map,
                     num_anchor_tokens=seq.num_anchor_tokens, num_private_slots=seq.num_private_slots,
                     num_cache_blocks=seq.num_cache_blocks, block_query_start=seq.block_query_start(),
                     free_after=list(mgr.free_block_ids), packed_read=packed, packed_shared=n_shared),
        ))
    (HERE / "layout.json").write_text(json.dumps(cases))
    print("layout.json", len(cases))


# --------------------------------------------------------------------------- triton kernels
def make_triton_ops():
    att = importlib.import_module("model.attention")
    ak = importlib.import_module("model.acache_attention")
    out = {}
    g = torch.Generator().manual_seed(7)

    def rn(*s, dtype=torch.float32):
        return torch.randn(*s, generator=g).to(dtype)

    # ---- store_kvcache (attention.py:11-41)
    N, H, D, nb, Bk = 9, 2, 32, 4, 8
    key, val = rn(N, H, D), rn(N, H, D)
    kc, vc = rn(nb, Bk, H, D), rn(nb, Bk, H, D)
    slots = torch.tensor([3, -1, 17, 0, 31, 8, -1, 9, 22], dtype=torch.int32)
    out["store_key"], out["store_val"], out["store_kc_in"], out["store_vc_in"], out["store_slots"] = key, val, kc.clone(), vc.clone(), slots
    att.store_kvcache_kernel[(N,)](key, key.stride(0), val, val.stride(0), kc, vc, slots, H * D)
    out["store_kc_out"], out["store_vc_out"] = kc, vc

    # ---- materialise (acache_attention.py:7-128), fp32 and fp16 caches, fp32 tables
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
        L, S, H, D = 2, 40, 2, 64
        A, shift, dst = 11, 5, 24
        k, v = rn(L, S, H, D, dtype=dt), rn(L, S, H, D, dtype=dt)
        cos, sin = rope_table(S, D, 10000.0, torch.float32)
        out[f"mat_{tag}_k_in"], out[f"mat_{tag}_v_in"] = k.clone(), v.clone()
        for l in range(L):
            lk, lv = k[l : l + 1], v[l : l + 1]
            ak._materialize_relocated_affix_kernel[(A * H,)](
                lk, lv, cos, sin, dst, A, shift,
                stride_kl=lk.stride(0), stride_ks=lk.stride(1), stride_kh=lk.stride(2), stride_kd=lk.stride(3),
                stride_vl=lv.stride(0), stride_vs=lv.stride(1), stride_vh=lv.stride(2), stride_vd=lv.stride(3),
                stride_rope_p=cos.stride(0), stride_rope_d=cos.stride(1),
                NUM_KV_HEADS=H, HEAD_DIM=D, BLOCK_D=64, num_warps=4)
        out[f"mat_{tag}_k_out"], out[f"mat_{tag}_v_out"] = k, v
        out[f"mat_{tag}_meta"] = torch.tensor([A, shift, dst])
    out["mat_cos"], out["mat_sin"] = rope_table(40, 64, 10000.0, torch.float32)

    # ---- acache attention (acache_attention.py:338-514), 3 modes x {f32, f16}
    def run_acache(q, kc, vc, cu_q, cu_k, rsm, shared_prefix_len=0, shared_kv_lens=None, shifts=None, cos=None, sin=None):
        nh, D = q.shape[1], q.shape[2]
        Hkv = kc.shape[2]
        B = cu_q.numel() - 1
        max_q = int((cu_q[1:] - cu_q[:-1]).max())
        reloc = shared_prefix_len > 0 and shifts is not None
        qside = reloc and shared_kv_lens is not None
        o = torch.empty_like(q)
        dummy = cu_q
        ak._acache_attention_kernel[(-(-max_q // 16), B, nh)](
            q, kc, vc, rsm, cu_q, cu_k, o,
            shared_kv_lens if shared_kv_lens is not None else dummy,
            shifts if reloc else dummy, cos if reloc else q, sin if reloc else q,
            D ** -0.5, shared_prefix_len,
            stride_qt=q.stride(0), stride_qh=q.stride(1), stride_qd=q.stride(2),
            stride_ks=kc.stride(1), stride_kh=kc.stride(2), stride_kd=kc.stride(3),
            stride_vs=vc.stride(1), stride_vh=vc.stride(2), stride_vd=vc.stride(3),
            stride_ot=o.stride(0), stride_oh=o.stride(1), stride_od=o.stride(2),
            stride_rope_p=cos.stride(0) if reloc else 0, stride_rope_d=cos.stride(1) if reloc else 0,
            kv_group_num=nh // Hkv, HEAD_DIM=D, BLOCK_M=16, BLOCK_N=64, BLOCK_D=D,
            APPLY_RELOCATION=reloc, QUERY_SIDE_RELOCATION=qside, num_warps=4, num_stages=2)
        return o

    for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
        nh, Hkv, D, nb, Bk = 4, 2, 64, 12, 8
        A = 10  # shared span = slots 0..9
        q_lens, kv_lens, shifts_l = [19, 7, 33], [37, 21, 50], [5, 0, 9]
        kc, vc = rn(nb, Bk, Hkv, D, dtype=dt), rn(nb, Bk, Hkv, D, dtype=dt)
        q = rn(sum(q_lens), nh, D, dtype=dt)
        cos, sin = rope_table(64, D, 10000.0, torch.float32)
        cu_q = torch.tensor([0, *np.cumsum(q_lens)], dtype=torch.int32)
        cu_k = torch.tensor([0, *np.cumsum(kv_lens)], dtype=torch.int32)
        pyr = random.Random(5)
        logical, packed, shared_lens = [], [], []
        for kv_len, s in zip(kv_lens, shifts_l):
            private = pyr.sample(range(A, nb * Bk), kv_len)
            anchors = set(pyr.sample(range(s, s + A), 3))
            m = [(p - s) if (s <= p < s + A and p not in anchors) else private[p] for p in range(kv_len)]
            logical += m
            sh = [x for x in m if x < A]
            packed += sh + [x for x in m if x >= A]
            shared_lens.append(len(sh))
        logical_t = torch.tensor(logical, dtype=torch.int32)
        packed_t = torch.tensor(packed, dtype=torch.int32)
        shifts_t = torch.tensor(shifts_l, dtype=torch.int32)
        shl_t = torch.tensor(shared_lens, dtype=torch.int32)
        out[f"att_{tag}_q"], out[f"att_{tag}_kc"], out[f"att_{tag}_vc"] = q, kc, vc
        out[f"att_{tag}_cu_q"], out[f"att_{tag}_cu_k"] = cu_q, cu_k
        out[f"att_{tag}_logical"], out[f"att_{tag}_packed"] = logical_t, packed_t
        out[f"att_{tag}_shifts"], out[f"att_{tag}_shared_lens"] = shifts_t, shl_t
        out[f"att_{tag}_plain"] = run_acache(q, kc, vc, cu_q, cu_k, logical_t)
        out[f"att_{tag}_keyside"] = run_acache(q, kc, vc, cu_q, cu_k, logical_t, A, None, shifts_t, cos, sin)
        out[f"att_{tag}_queryside"] = run_acache(q, kc, vc, cu_q, cu_k, packed_t, A, shl_t, shifts_t, cos, sin)
    out["att_cos"], out["att_sin"] = rope_table(64, 64, 10000.0, torch.float32)
    out["att_shared_prefix_len"] = torch.tensor(10)

    # ---- block-table kernels (acache_attention.py:132-334)
    nh, Hkv, D, nb, Bk = 4, 2, 64, 16, 8
    kc, vc = rn(nb, Bk, Hkv, D), rn(nb, Bk, Hkv, D)
    lens = [21, 40, 9]
    pyr = random.Random(9)
    ids = pyr.sample(range(nb), sum(-(-n // Bk) for n in lens))
    bt = torch.full((3, 5), -1, dtype=torch.int32)
    o = 0
    for i, n in enumerate(lens):
        c = -(-n // Bk)
        bt[i, :c] = torch.tensor(ids[o : o + c], dtype=torch.int32)
        o += c
    cu = torch.tensor([0, *np.cumsum(lens)], dtype=torch.int32)
    q = rn(sum(lens), nh, D)
    res = torch.empty_like(q)
    ak._baseline_ragged_attention_kernel[(-(-max(lens) // 16), 3, nh)](
        q, kc, vc, bt, cu, cu, res, D ** -0.5,
        stride_qt=q.stride(0), stride_qh=q.stride(1), stride_qd=q.stride(2),
        stride_kb=kc.stride(0), stride_ks=kc.stride(1), stride_kh=kc.stride(2), stride_kd=kc.stride(3),
        stride_vb=vc.stride(0), stride_vs=vc.stride(1), stride_vh=vc.stride(2), stride_vd=vc.stride(3),
        stride_bt=bt.stride(0), stride_ot=res.stride(0), stride_oh=res.stride(1), stride_od=res.stride(2),
        kv_group_num=nh // Hkv, BLOCK_SIZE=Bk, HEAD_DIM=D, BLOCK_M=16, BLOCK_N=64, BLOCK_D=D, num_warps=4, num_stages=2)
    out["bt_kc"], out["bt_vc"], out["bt_tables"], out["bt_cu"], out["bt_q"], out["bt_ragged"] = kc, vc, bt, cu, q, res
    T = 4
    qd = rn(3, T, nh, D)
    resd = torch.empty_like(qd)
    sl = torch.tensor(lens, dtype=torch.int32)
    ak._baseline_decode_attention_kernel[(1, 3, nh)](
        qd, kc, vc, sl, bt, resd, D ** -0.5,
        stride_qb=qd.stride(0), stride_qt=qd.stride(1), stride_qh=qd.stride(2), stride_qd=qd.stride(3),
        stride_kb=kc.stride(0), stride_ks=kc.stride(1), stride_kh=kc.stride(2), stride_kd=kc.stride(3),
        stride_vb=vc.stride(0), stride_vs=vc.stride(1), stride_vh=vc.stride(2), stride_vd=vc.stride(3),
        stride_bt=bt.stride(0), stride_ob=resd.stride(0), stride_ot=resd.stride(1), stride_oh=resd.stride(2),
        stride_od=resd.stride(3), kv_group_num=nh // Hkv, QUERY_LEN=T, BLOCK_SIZE=Bk, HEAD_DIM=D,
        BLOCK_M=16, BLOCK_N=64, BLOCK_D=D, num_warps=4, num_stages=2)
    out["bt_qd"], out["bt_seqlens"], out["bt_decode"] = qd, sl, resd

    np.savez_compressed(HERE / "triton_ops.npz", **{k: v.numpy() for k, v in out.items()})
    print("triton_ops.npz", len(out))


# --------------------------------------------------------------------------- sampling + topk
def make_sampling_topk():
    from model_runner import ModelRunner

    runner = object.__new__(ModelRunner)
    g = torch.Generator().manual_seed(11)
    B, T, V = 5, 8, 97
    logits = torch.randn(B, T, V, generator=g) * 3.0
    logits[0, 2, 13] += 12.0  # a confident position
    logits[1, :, 5] += 15.0   # a fully confident row
    x = torch.randint(0, V - 1, (B, T), generator=g)
    mask = torch.rand(B, T, generator=g) < 0.6
    mask[3] = False           # a row without masks
    x = torch.where(mask, torch.full_like(x, V - 1), x)
    x0, ti = runner.get_transfer_index(logits, 0.0, "low_confidence", mask, x, 0.9)
    np.savez_compressed(HERE / "sampling.npz", logits=logits.numpy(), x=x.numpy(), mask=mask.numpy(),
                        x0=x0.numpy(), transfer=ti.numpy(), threshold=np.float32(0.9))
    scores = torch.randn(6, 512, generator=g)
    top = torch.topk(scores, 103, largest=True).indices.sort().values
    bot = torch.topk(scores, 103, largest=False).indices.sort().values
    np.savez_compressed(HERE / "topk.npz", scores=scores.numpy(), top=top.numpy(), bottom=bot.numpy(), k=np.int64(103))
    print("sampling.npz topk.npz")


# --------------------------------------------------------------------------- HF batch-1 path
def make_hf_llada():
    root = REF
    pkg = "acache_hf_llada_model"
    package = types.ModuleType(pkg)
    package.__path__ = [str(root / "llada" / "model")]
    sys.modules[pkg] = package
    cfgm = importlib.import_module(f"{pkg}.configuration_llada")
    mm = importlib.import_module(f"{pkg}.modeling_llada")
    sys.path.insert(0, str(root / "llada"))
    spec = importlib.util.spec_from_file_location("acache_hf_generate", root / "llada" / "generate_ACache.py")
    gen = importlib.util.module_from_spec(spec)
    sys.modules["acache_hf_generate"] = gen
    spec.loader.exec_module(gen)

    from oracle.models import ArchSpec, random_state_dict

    arch = ArchSpec("llada", n_layers=2, d_model=64, n_heads=4, n_kv_heads=4, ffn=96, vocab=128,
                    rope_theta=10000.0, rms_eps=1e-5, act="silu", mask_id=127)
    cfg = cfgm.LLaDAConfig(
        vocab_size=128, embedding_size=128, d_model=64, n_heads=4, n_kv_heads=4, n_layers=2, mlp_hidden_size=96,
        activation_type="silu", block_type="llama", rope=True, rope_theta=10000.0, attention_dropout=0.0,
        residual_dropout=0.0, embedding_dropout=0.0, eos_token_id=0, pad_token_id=0, mask_token_id=127,
        layer_norm_type="rms", weight_tying=False, include_bias=False, flash_attention=False, init_device="cpu")
    model = mm.LLaDAModelLM(cfg).eval()
    sd = random_state_dict(arch, seed=3, std=0.35)
    model.load_state_dict(sd, strict=True)

    pyr = random.Random(21)
    A, G, BL = 12, 8, 4
    affix = [pyr.randint(1, 120) for _ in range(A)]
    layouts = []
    for mode, head, tail in (("prefix", 0, 7), ("infix", 5, 6), ("suffix", 9, 0), ("prefix", 0, 3), ("infix", 2, 9)):
        if mode == "prefix":
            prompt = affix + [pyr.randint(1, 120) for _ in range(tail)]
            kw = dict(affix_start=0, affix_end=A, generation_start=None)
        elif mode == "infix":
            prompt = [pyr.randint(1, 120) for _ in range(head)] + affix + [pyr.randint(1, 120) for _ in range(tail)]
            kw = dict(affix_start=head, affix_end=head + A, generation_start=None)
        else:
            prompt = [pyr.randint(1, 120) for _ in range(head)] + [127] * G + affix
            kw = dict(affix_start=head + G, affix_end=head + G + A, generation_start=head)
        layouts.append((mode, prompt, kw))

    res = {f"w::{k}": v.numpy() for k, v in sd.items()}
    meta = []
    with torch.inference_mode():
        affix_ids = torch.tensor([affix])
        affix_cache = model(affix_ids, use_cache=True).past_key_values
        for i, (mode, prompt, kw) in enumerate(layouts):
            for thr in (0.9, 0.05):
                p = torch.tensor([prompt])
                if kw["generation_start"] is None:
                    x = torch.cat([p, torch.full((1, G), 127)], dim=1)
                else:
                    x = p.clone()
                imp = gen.compute_attention_importance_cross_affix(model, x, affix_cache, mask_id=127,
                                                                   affix_start=kw["affix_start"])
                k = min(gen.ceil_to_int(0.25 * A), A)
                anchors = (gen.select_anchor_tokens(imp, k, "top")[0] + kw["affix_start"]).tolist()
                outx, nfe = gen.generate_with_anchor_attention(
                    model, p, steps=G, gen_length=G, block_length=BL, mask_id=127, threshold=thr,
                    anchor_ratio=0.25, selection_mode="top", precomputed_affix_cache=affix_cache, **kw)
                tag = f"case{i}_thr{thr}"
                res[f"{tag}::importance"] = imp[0].numpy()
                res[f"{tag}::tokens"] = outx[0].numpy()
                meta.append(dict(tag=tag, mode=mode, prompt=prompt, gen_length=G, block_length=BL, threshold=thr,
                                 anchor_ratio=0.25, anchors=anchors, nfe_with_probe=int(nfe), **kw))
    res["meta"] = np.frombuffer(json.dumps(dict(cases=meta, arch=arch.__dict__)).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "hf_llada.npz", **res)
    print("hf_llada.npz", len(meta))


def make_hf_llada_dkv():
    """The reference HF batch-1 dKV + affix-reuse path for LLaDA
    (llada/eval_dKV_ACache.py:75-277 ``generate_with_dkv_anchor_attention``) on the tiny random
    LLaDA of ``make_hf_llada``.  The file's evaluation-harness imports (lm_eval, accelerate) are not
    installed here, so only its three generation functions are compiled, from the file as it
    lies, into a namespace that holds the helpers they import."""
    import ast
    from typing import Optional, Sequence, Tuple

    root = REF
    pkg = "acache_hf_llada_model"
    if pkg not in sys.modules:
        package = types.ModuleType(pkg)
        package.__path__ = [str(root / "llada" / "model")]
        sys.modules[pkg] = package
    cfgm = importlib.import_module(f"{pkg}.configuration_llada")
    mm = importlib.import_module(f"{pkg}.modeling_llada")
    sys.path.insert(0, str(root / "llada"))

    def load(name, filename):
        spec = importlib.util.spec_from_file_location(name, root / "llada" / filename)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module

    gen_acache = load("acache_hf_generate", "generate_ACache.py")
    gen_plain = load("acache_hf_generate_plain", "generate.py")
    source = (root / "llada" / "eval_dKV_ACache.py").read_text()
    wanted = {"_dkv_transfer_schedule", "_full_cache_with_static_affix", "generate_with_dkv_anchor_attention"}
    tree = ast.parse(source)
    tree.body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    assert {n.name for n in tree.body} == wanted
    ns = dict(torch=torch, Optional=Optional, Sequence=Sequence, Tuple=Tuple,
              KVCache=Sequence[Tuple[torch.Tensor, torch.Tensor]], add_gumbel_noise=gen_plain.add_gumbel_noise,
              ceil_to_int=gen_acache.ceil_to_int,
              compute_attention_importance_cross_affix=gen_acache.compute_attention_importance_cross_affix,
              select_anchor_tokens=gen_acache.select_anchor_tokens)
    exec(compile(ast.fix_missing_locations(tree), str(root / "llada" / "eval_dKV_ACache.py"), "exec"), ns)
    generate = ns["generate_with_dkv_anchor_attention"]

    from oracle.models import ArchSpec, random_state_dict

    arch = ArchSpec("llada", n_layers=2, d_model=64, n_heads=4, n_kv_heads=4, ffn=96, vocab=128,
                    rope_theta=10000.0, rms_eps=1e-5, act="silu", mask_id=127)
    cfg = cfgm.LLaDAConfig(
        vocab_size=128, embedding_size=128, d_model=64, n_heads=4, n_kv_heads=4, n_layers=2, mlp_hidden_size=96,
        activation_type="silu", block_type="llama", rope=True, rope_theta=10000.0, attention_dropout=0.0,
        residual_dropout=0.0, embedding_dropout=0.0, eos_token_id=0, pad_token_id=0, mask_token_id=127,
        layer_norm_type="rms", weight_tying=False, include_bias=False, flash_attention=False, init_device="cpu")
    model = mm.LLaDAModelLM(cfg).eval()
    sd = random_state_dict(arch, seed=9, std=0.35)
    model.load_state_dict(sd, strict=True)

    pyr = random.Random(35)
    A, G, BL, STEPS = 7, 8, 4, 8
    affix = [pyr.randint(1, 120) for _ in range(A)]
    res = {f"w::{k}": v.numpy() for k, v in sd.items()}
    meta = []
    with torch.inference_mode():
        cache = model(torch.tensor([affix]), use_cache=True).past_key_values
        for mode, head, tail in (("prefix", 0, 5), ("infix", 3, 4), ("suffix", 4, 0)):
            if mode == "prefix":
                prompt = affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=0, affix_end=A, generation_start=None)
            elif mode == "infix":
                prompt = [pyr.randint(1, 120) for _ in range(head)] + affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=head, affix_end=head + A, generation_start=None)
            else:
                prompt = [pyr.randint(1, 120) for _ in range(head)] + [127] * G + affix
                kw = dict(affix_start=head + G, affix_end=head + G + A, generation_start=head)
            x = torch.tensor([prompt])
            for ratio in (0.0, 0.3, 1.0):
                for interval in (1, 2, 3):
                    tokens, nfe = generate(model, x, steps=STEPS, gen_length=G, block_length=BL, temperature=0.,
                                           remasking="low_confidence", mask_id=127, selection_mode="top",
                                           drop_non_anchor=False, anchor_ratio=ratio, dkv_cache_interval=interval,
                                           precomputed_affix_cache=cache, **kw)
                    tag = f"{mode}_r{ratio}_i{interval}"
                    res[f"{tag}::tokens"] = tokens[0].numpy()
                    meta.append(dict(tag=tag, mode=mode, prompt=prompt, gen_length=G, block_length=BL, steps=STEPS,
                                     anchor_ratio=ratio, interval=interval, nfe=int(nfe), **kw))
    res["meta"] = np.frombuffer(json.dumps(dict(cases=meta, arch=arch.__dict__)).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "hf_llada_dkv.npz", **res)
    print("hf_llada_dkv.npz", len(meta))


def _hf_dream_modules():
    """(configuration module, modeling module, generate_ACache module, loader) of the reference's
    HF Dream path."""
    root = REF / "dream"
    pkg = "acache_hf_dream_model"
    package = types.ModuleType(pkg)
    package.__path__ = [str(root / "model")]
    sys.modules[pkg] = package
    # the installed transformers no longer ships the plain RoPE initialiser the reference's HF
    # Dream model looks up by the name "default": inv_freq[j] = theta^(-2j/D), no scaling
    from transformers import modeling_rope_utils as _mru

    def _default_rope(config, device=None, **_):
        dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        inv = 1.0 / (config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float().to(device) / dim))
        return inv, 1.0

    _mru.ROPE_INIT_FUNCTIONS.setdefault("default", _default_rope)
    cfgm = importlib.import_module(f"{pkg}.configuration_dream")
    mm = importlib.import_module(f"{pkg}.modeling_dream")

    def load(name, filename):
        spec = importlib.util.spec_from_file_location(name, root / filename)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return module

    # the reference scripts import their model code as the top-level package ``model``
    sys.modules["model.generation_utils_block"] = importlib.import_module(f"{pkg}.generation_utils_block")
    sys.modules["model.modeling_dream"] = mm
    if "generate_ACache" not in sys.modules or getattr(sys.modules["generate_ACache"], "__name__", "") != "acache_hf_dream_generate":
        sys.modules["generate_ACache"] = load("acache_hf_dream_generate", "generate_ACache.py")
    return cfgm, mm, sys.modules["generate_ACache"], load


def _tiny_hf_dream(cfgm, mm, seed, n_kv_heads=4):
    from oracle.models import ArchSpec, random_state_dict

    arch = ArchSpec("dream", n_layers=2, d_model=64, n_heads=4, n_kv_heads=n_kv_heads, ffn=128, vocab=128,
                    rope_theta=10000.0, rms_eps=1e-6, act="silu", mask_id=127)
    cfg = cfgm.DreamConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=n_kv_heads, max_position_embeddings=64,
                           mask_token_id=127, pad_token_id=0, rope_theta=10000.0, rms_norm_eps=1e-6)
    model = mm.DreamModel(cfg).eval()
    sd = random_state_dict(arch, seed=seed, std=0.35)
    missing = model.load_state_dict(sd, strict=False)
    assert not missing.unexpected_keys and all("rotary" in k or "inv_freq" in k for k in missing.missing_keys), missing
    return arch, model, sd


def make_hf_dream():
    """The reference HF batch-1 affix-reuse path for Dream (dream/generate_ACache.py) on a tiny
    random GQA Dream in fp32: importance scores, anchors, final tokens, nfe."""
    cfgm, mm, gen, _ = _hf_dream_modules()
    arch, model, sd = _tiny_hf_dream(cfgm, mm, seed=7, n_kv_heads=2)
    pyr = random.Random(23)
    A, G, BL = 12, 8, 4
    affix = [pyr.randint(1, 120) for _ in range(A)]
    res = {f"w::{k}": v.numpy() for k, v in sd.items()}
    meta = []
    with torch.inference_mode():
        affix_cache = model(torch.tensor([affix]), use_cache=True).past_key_values
        for i, (mode, head, tail) in enumerate((("prefix", 0, 7), ("infix", 5, 6), ("suffix", 9, 0), ("infix", 2, 9))):
            if mode == "prefix":
                prompt = affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=0, affix_end=A, generation_start=None)
            elif mode == "infix":
                prompt = [pyr.randint(1, 120) for _ in range(head)] + affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=head, affix_end=head + A, generation_start=None)
            else:
                prompt = [pyr.randint(1, 120) for _ in range(head)] + [127] * G + affix
                kw = dict(affix_start=head + G, affix_end=head + G + A, generation_start=head)
            for thr in (0.9, 0.05):
                p = torch.tensor([prompt])
                x = torch.cat([p, torch.full((1, G), 127)], dim=1) if kw["generation_start"] is None else p.clone()
                imp = gen.compute_attention_importance_cross_affix(model, x, affix_cache, mask_id=127,
                                                                   affix_start=kw["affix_start"])
                k = min(gen.ceil_to_int(0.25 * A), A)
                anchors = (gen.select_anchor_tokens(imp, k, "top")[0] + kw["affix_start"]).tolist()
                outx, nfe = gen.generate_with_anchor_attention(
                    model, p, steps=G, gen_length=G, block_length=BL, mask_id=127, threshold=thr,
                    anchor_ratio=0.25, selection_mode="top", precomputed_affix_cache=affix_cache, **kw)
                tag = f"case{i}_thr{thr}"
                res[f"{tag}::importance"] = imp[0].numpy()
                res[f"{tag}::tokens"] = outx[0].numpy()
                meta.append(dict(tag=tag, mode=mode, prompt=prompt, gen_length=G, block_length=BL, threshold=thr,
                                 anchor_ratio=0.25, anchors=anchors, nfe_with_probe=int(nfe), **kw))
    res["meta"] = np.frombuffer(json.dumps(dict(cases=meta, arch=arch.__dict__)).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "hf_dream.npz", **res)
    print("hf_dream.npz", len(meta))


def make_hf_dream_dkv():
    """The reference HF batch-1 dKV + affix-reuse path (dream/generate_dKV_ACache.py) on a tiny
    random Dream in fp32: final tokens and NFE for prefix / infix / suffix placement, several
    anchor ratios and cache intervals (the cases of the reference's own
    nano-vdllm/tests/test_dream_dkv.py:60-111, run here on CPU in fp32)."""
    cfgm, mm, _, load = _hf_dream_modules()
    gen = load("acache_hf_dream_dkv", "generate_dKV_ACache.py")
    arch, model, sd = _tiny_hf_dream(cfgm, mm, seed=5)

    pyr = random.Random(33)
    A, G, BL, STEPS = 6, 8, 4, 8
    affix = [pyr.randint(1, 120) for _ in range(A)]
    res = {f"w::{k}": v.numpy() for k, v in sd.items()}
    meta = []
    with torch.inference_mode():
        for mode, head, tail in (("prefix", 0, 5), ("infix", 3, 4), ("suffix", 4, 0)):
            if mode == "prefix":
                prompt = affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=0, affix_end=A, generation_start=None)
            elif mode == "infix":
                prompt = [pyr.randint(1, 120) for _ in range(head)] + affix + [pyr.randint(1, 120) for _ in range(tail)]
                kw = dict(affix_start=head, affix_end=head + A, generation_start=None)
            else:
                prompt = [pyr.randint(1, 120) for _ in range(head)] + [127] * G + affix
                kw = dict(affix_start=head + G, affix_end=head + G + A, generation_start=head)
            x = torch.tensor([prompt])
            cache = model(x[:, kw["affix_start"]: kw["affix_end"]], use_cache=True).past_key_values
            for ratio in (0.0, 0.34, 1.0):
                for interval in (1, 2, 3):
                    tokens, nfe = gen.generate_with_dkv_anchor_attention(
                        model, x, steps=STEPS, gen_length=G, block_length=BL, temperature=0., remasking="low_confidence",
                        mask_id=127, selection_mode="top", drop_non_anchor=False, anchor_ratio=ratio,
                        dkv_cache_interval=interval, precomputed_affix_cache=cache, **kw)
                    tag = f"{mode}_r{ratio}_i{interval}"
                    res[f"{tag}::tokens"] = tokens[0].numpy()
                    meta.append(dict(tag=tag, mode=mode, prompt=prompt, gen_length=G, block_length=BL, steps=STEPS,
                                     anchor_ratio=ratio, interval=interval, nfe=int(nfe), **kw))
    res["meta"] = np.frombuffer(json.dumps(dict(cases=meta, arch=arch.__dict__)).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "hf_dream_dkv.npz", **res)
    print("hf_dream_dkv.npz", len(meta))


if __name__ == "__main__":
    which = sys.argv[2:] or ["layout", "triton", "sampling", "hf", "dream", "dkv"]
    if "dream" in which:
        make_hf_dream()
    if "dkv" in which:
        make_hf_llada_dkv()
        make_hf_dream_dkv()
    if "layout" in which:
        make_layout()
    if "triton" in which:
        make_triton_ops()
    if "sampling" in which:
        make_sampling_topk()
    if "hf" in which:
        make_hf_llada()
