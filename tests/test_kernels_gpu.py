"""CUDA kernels (through the C ABI) against the CPU oracle and the reference-generated
golden vectors.  Bit-exact for data movement, rotation and index selection; stated
tolerances for the floating-point contractions."""
import numpy as np
import pytest
import torch

from conftest import load_npz

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from acache_b200 import _lib, ops
    from acache_b200.model import acache_attention as aa
    from acache_b200.model import attention as att

    return _lib, ops, aa, att


def _rope(length, D, theta=10000.0, dtype=torch.float32):
    from oracle.rope import rope_table

    c, s = rope_table(length, D, theta, dtype)
    return c, s


# ----------------------------------------------------------------------------- store
def test_store_kvcache_golden(triton_ops):
    _lib, ops, aa, att = _ops()
    t = triton_ops
    kc, vc = t["store_kc_in"].to(DEV), t["store_vc_in"].to(DEV)
    att.store_kvcache(t["store_key"].to(DEV), t["store_val"].to(DEV), kc, vc, t["store_slots"].to(DEV))
    assert torch.equal(kc.cpu(), t["store_kc_out"]) and torch.equal(vc.cpu(), t["store_vc_out"])
    _lib.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_store_kvcache_random(dtype):
    from oracle import kv_ops

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(0)
    N, H, D, nb, Bk = 300, 8, 128, 6, 256
    key = torch.randn(N, H, D, generator=g).to(dtype)
    val = torch.randn(N, H, D, generator=g).to(dtype)
    kc = torch.randn(nb, Bk, H, D, generator=g).to(dtype)
    vc = torch.randn(nb, Bk, H, D, generator=g).to(dtype)
    slots = torch.randperm(nb * Bk, generator=g)[:N].to(torch.int32)
    slots[::7] = -1
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    # strided rows: key/value are slices of a fused projection output
    fused = torch.zeros(N, 3, H, D, dtype=dtype, device=DEV)
    fused[:, 1], fused[:, 2] = key.to(DEV), val.to(DEV)
    att.store_kvcache(fused[:, 1], fused[:, 2], kc_d, vc_d, slots.to(DEV))
    kv_ops.store_kvcache(key, val, kc, vc, slots)
    assert torch.equal(kc_d.cpu(), kc) and torch.equal(vc_d.cpu(), vc)
    _lib.check_device_errors()


def test_store_kvcache_flags_bad_slot_without_faulting():
    _lib, ops, aa, att = _ops()
    key = torch.ones(2, 1, 16, device=DEV)
    kc = torch.zeros(1, 4, 1, 16, device=DEV)
    vc = torch.zeros_like(kc)
    att.store_kvcache(key, key, kc, vc, torch.tensor([1, 99], dtype=torch.int32, device=DEV))
    with pytest.raises(_lib.AcacheError):
        _lib.check_device_errors()
    assert kc[0, 1].eq(1).all() and kc[0, 0].eq(0).all()


def test_empty_inputs_are_noops():
    _lib, ops, aa, att = _ops()
    kc = torch.zeros(1, 4, 1, 16, device=DEV)
    att.store_kvcache(torch.zeros(0, 1, 16, device=DEV), torch.zeros(0, 1, 16, device=DEV), kc, kc.clone(),
                      torch.zeros(0, dtype=torch.int32, device=DEV))
    out = ops.anchor_topk(torch.zeros(0, 8, device=DEV), 3)
    assert out.shape == (0, 3)
    q = torch.zeros(0, 2, 16, device=DEV)
    cu = torch.zeros(1, dtype=torch.int32, device=DEV)
    o = aa.acache_attention(q, kc.expand(1, 4, 1, 16).contiguous(), kc.clone(), cu, cu,
                            torch.zeros(0, dtype=torch.int32, device=DEV), max_seqlen_q=0)
    assert o.shape == q.shape


# ----------------------------------------------------------------------------- relocation
def test_materialize_golden_bit_exact(triton_ops):
    _lib, ops, aa, att = _ops()
    t = triton_ops
    for tag in ("f32", "f16"):
        A, shift, dst = (int(x) for x in t[f"mat_{tag}_meta"])
        k, v = t[f"mat_{tag}_k_in"].to(DEV), t[f"mat_{tag}_v_in"].to(DEV)
        aa.materialize_relocated_affix(k, v, t["mat_cos"].to(DEV), t["mat_sin"].to(DEV), dst, A, shift)
        assert torch.equal(k.cpu(), t[f"mat_{tag}_k_out"]), tag
        assert torch.equal(v.cpu(), t[f"mat_{tag}_v_out"]), tag
    _lib.check_device_errors()


@pytest.mark.parametrize("dtype,table_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                                (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16)])
def test_relocation_batched_block_tables_bit_exact(dtype, table_dtype):
    """Micro-op configuration: 2 layers, 8 KV heads, head_dim 128, blocks of 256, a
    512-token affix, 4 requests with shifts 0 / U[64,1024], RoPE theta 5e5."""
    from oracle import kv_ops

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(1)
    L, H, D, Bk, A, R = 2, 8, 128, 256, 512, 4
    nb = 2 + 2 * R
    k = torch.randn(L, nb * Bk, H, D, generator=g).to(dtype)
    v = torch.randn(L, nb * Bk, H, D, generator=g).to(dtype)
    cos, sin = _rope(1100, D, 500000.0, table_dtype)
    shifts = [0] + torch.randint(64, 1025, (R - 1,), generator=g).tolist()
    perm = (torch.randperm(nb - 2, generator=g) + 2).tolist()
    tables = [perm[2 * r: 2 * r + 2] for r in range(R)]
    kd, vd = k.to(DEV), v.to(DEV)
    aa.relocate_affix_batched(kd, vd, cos.to(DEV), sin.to(DEV), A,
                              torch.tensor(shifts, dtype=torch.int32, device=DEV),
                              dst_block_tables=torch.tensor(tables, dtype=torch.int32, device=DEV), block_size=Bk)
    kv_ops.relocate_affix_batched(k, v, cos, sin, tables, shifts, A, Bk)
    assert torch.equal(kd.cpu(), k) and torch.equal(vd.cpu(), v)
    _lib.check_device_errors()


def test_relocation_ragged_affix_and_single_form():
    from oracle import kv_ops

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(2)
    L, S, H, D = 3, 64, 2, 64
    k = torch.randn(L, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(L, S, H, D, generator=g).to(torch.bfloat16)
    cos, sin = _rope(S, D)
    kd, vd = k.to(DEV), v.to(DEV)
    aa.materialize_relocated_affix(kd, vd, cos.to(DEV), sin.to(DEV), 12, 7, 5)
    kv_ops.materialize_relocated_affix(k, v, cos, sin, 12, 7, 5)
    assert torch.equal(kd.cpu(), k) and torch.equal(vd.cpu(), v)


def test_relocation_roundtrip_property():
    """Relocating by +s and then rotating back by -s recovers K within bf16 rounding;
    V is copied exactly.  Size-independent check used at full cache sizes."""
    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(3)
    L, H, D, Bk, A = 4, 8, 128, 256, 1024
    k = torch.randn(L, 3 * A, H, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(L, 3 * A, H, D, generator=g).to(torch.bfloat16).to(DEV)
    cos, sin = _rope(2048, D, 500000.0)
    cos, sin = cos.to(DEV), sin.to(DEV)
    src_k, src_v = k[:, :A].clone(), v[:, :A].clone()
    aa.materialize_relocated_affix(k, v, cos, sin, A, A, 777)
    assert torch.equal(v[:, A: 2 * A], src_v)
    # norms are preserved by a rotation
    n0 = src_k.float().norm(dim=-1)
    n1 = k[:, A: 2 * A].float().norm(dim=-1)
    assert torch.allclose(n0, n1, rtol=1e-2, atol=1e-2)
    rot = k[:, A: 2 * A].float()
    half = D // 2
    back = rot * cos[777] - torch.cat((-rot[..., half:], rot[..., :half]), -1) * sin[777]
    assert (back - src_k.float()).abs().max() < 0.05


# ----------------------------------------------------------------------------- rope + store
@pytest.mark.parametrize("kind", ["llada", "dream"])
def test_rope_store_matches_oracle(kind):
    from oracle import kv_ops
    from oracle.rope import dream_rope_qk, llada_rope_qk

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(4)
    n, nh, hkv, D, nb, Bk = 77, 8, 2, 128, 3, 64
    dt = torch.bfloat16
    q = torch.randn(n, nh, D, generator=g).to(dt)
    k = torch.randn(n, hkv, D, generator=g).to(dt)
    v = torch.randn(n, hkv, D, generator=g).to(dt)
    pos = torch.randint(0, 500, (n,), generator=g)
    kc = torch.zeros(nb, Bk, hkv, D, dtype=dt)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * Bk, generator=g)[:n].to(torch.int32)
    slots[5] = -1
    theta = 500000.0
    if kind == "llada":
        q_ref, k_ref = llada_rope_qk(q, k, pos, theta)
        cos, sin = _rope(512, D, theta, torch.float32)
    else:
        q_ref, k_ref = dream_rope_qk(q, k, pos, theta)
        cos, sin = _rope(512, D, theta, dt)
    kv_ops.store_kvcache(k_ref, v, kc, vc, slots)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    kcd, vcd = torch.zeros_like(kc, device=DEV), torch.zeros_like(vc, device=DEV)
    ops.rope_store(qd, kd, vd, pos.to(DEV), cos.to(DEV), sin.to(DEV), kcd, vcd, slots.to(DEV))
    assert torch.equal(qd.cpu(), q_ref) and torch.equal(kd.cpu(), k_ref)
    assert torch.equal(kcd.cpu(), kc) and torch.equal(vcd.cpu(), vc)
    _lib.check_device_errors()


# ----------------------------------------------------------------------------- top-k
def test_topk_golden_and_ties():
    from oracle import topk as otopk

    _lib, ops, aa, att = _ops()
    z = load_npz("topk.npz")
    s = torch.from_numpy(z["scores"]).to(DEV)
    assert np.array_equal(ops.anchor_topk(s, int(z["k"]), True).cpu().numpy(), z["top"])
    assert np.array_equal(ops.anchor_topk(s, int(z["k"]), False).cpu().numpy(), z["bottom"])
    t = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0, 3.0]], device=DEV)
    assert ops.anchor_topk(t, 3, True).tolist() == [[1, 2, 4]]
    assert ops.anchor_topk(t, 2, False).tolist() == [[0, 5]]
    assert ops.anchor_topk(torch.zeros(2, 9, device=DEV), 4, True).tolist() == [[0, 1, 2, 3]] * 2
    off = torch.tensor([10, 20], dtype=torch.int32, device=DEV)
    assert ops.anchor_topk(torch.zeros(2, 9, device=DEV), 2, True, off).tolist() == [[10, 11], [20, 21]]
    g = torch.Generator().manual_seed(5)
    for A, k in ((1, 1), (33, 33), (800, 160), (1024, 7), (1025, 103), (8192, 820), (60000, 5000)):
        for quant in (False, True):
            sc = torch.randn(3, A, generator=g)
            if quant:  # duplicate-heavy: many equal scores straddle the cut
                sc = (sc * 2).round() / 2
            sc[0, 0] = float("-inf")
            for largest in (True, False):
                got = ops.anchor_topk(sc.to(DEV), k, largest).cpu()
                assert torch.equal(got, otopk.anchor_topk(sc, k, largest)), (A, k, quant, largest)


# ----------------------------------------------------------------------------- importance
@pytest.mark.parametrize("nh,hkv,D,A,nq,shift,dt", [
    (4, 4, 64, 37, 9, 0, torch.bfloat16), (8, 2, 128, 300, 70, 13, torch.bfloat16),
    (4, 2, 32, 64, 5, 3, torch.float32), (32, 32, 128, 800, 256, 0, torch.bfloat16),
    # long affixes: cut into chunks walked by separate CTAs, two launches
    (32, 32, 128, 5000, 8, 40, torch.bfloat16), (8, 2, 128, 2500, 200, 0, torch.bfloat16),
    (4, 4, 64, 2049, 3, 5, torch.float16)])
def test_anchor_importance_vs_oracle(nh, hkv, D, A, nq, shift, dt):
    from oracle.importance import layer_importance, relocate_keys

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(6)
    n = nq + 11
    q = torch.randn(n, nh, D, generator=g).to(dt)
    kc = torch.randn(A + 20, hkv, D, generator=g).to(dt)
    rows = torch.randperm(n, generator=g)[:nq].sort().values.to(torch.int32)
    cos, sin = _rope(64, D)
    kk = relocate_keys(kc[:A], cos, sin, shift) if shift else kc[:A]
    ref = layer_importance(q[rows.long()], kk, D ** -0.5, exact=True)
    imp = torch.zeros(A, device=DEV)
    for _ in range(2):  # accumulates across calls (layers)
        ops.anchor_importance(q.to(DEV), rows.to(DEV), kc.to(DEV)[:A], shift, cos.to(DEV), sin.to(DEV), D ** -0.5, imp)
    got = imp.cpu() / 2
    assert torch.allclose(got, ref, rtol=2e-3, atol=1e-4), (got - ref).abs().max()
    assert abs(float(got.sum()) - nq * nh) < 1e-2 * nq * nh  # softmax rows sum to one


@pytest.mark.parametrize("nh,hkv,D,A,counts,shifts,dt", [
    (32, 32, 128, 800, [32, 32, 7, 0, 256, 31], None, torch.bfloat16),       # a request without mask rows
    (8, 2, 128, 300, [70, 5, 129], [13, 0, 40], torch.bfloat16),             # GQA, rotated keys, two row tiles
    (4, 4, 64, 2048, [3, 9], [5, 5], torch.float16),                         # the longest unchunked affix
    (28, 4, 128, 600, [32] * 9, [17, 90, 33, 64, 0, 1, 2, 3, 127], torch.bfloat16)])
def test_anchor_importance_batched_has_the_bits_of_the_per_request_call(nh, hkv, D, A, counts, shifts, dt):
    """All requests of a probe batch in one launch against one launch per request: same bits,
    also when the scores accumulate over several calls (layers)."""
    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(16)
    n = sum(counts) + 23
    q = torch.randn(n, nh, D, generator=g).to(dt).to(DEV)
    kc = torch.randn(A + 20, hkv, D, generator=g).to(dt).to(DEV)
    cos, sin = (t.to(DEV) for t in _rope(128, D))
    perm = torch.randperm(n, generator=g)[: sum(counts)]
    rows, off = [], [0]
    for c in counts:
        rows.append(perm[off[-1]: off[-1] + c].sort().values.to(torch.int32))
        off.append(off[-1] + c)
    ref = torch.zeros(len(counts), A, device=DEV)
    got = torch.zeros(len(counts), A, device=DEV)
    all_rows = torch.cat(rows).to(DEV)
    offsets = torch.tensor(off, dtype=torch.int32, device=DEV)
    dev_shifts = None if shifts is None else torch.tensor(shifts, dtype=torch.int32, device=DEV)
    for _ in range(2):
        for r, rr in enumerate(rows):
            ops.anchor_importance(q, rr.to(DEV), kc[:A], 0 if shifts is None else shifts[r], cos, sin, D ** -0.5, ref[r])
        assert ops.anchor_importance_batched(q, all_rows, offsets, max(counts), kc[:A], dev_shifts, cos, sin,
                                             D ** -0.5, got)
    assert torch.equal(got, ref)
    for r, c in enumerate(counts):
        assert abs(float(got[r].sum()) - 2 * c * nh) <= 1e-2 * max(2 * c * nh, 1)
    _lib.check_device_errors()


def test_anchor_importance_batched_declines_what_only_the_per_request_call_takes():
    _lib, ops, aa, att = _ops()
    off = torch.tensor([0, 2, 4], dtype=torch.int32, device=DEV)
    rows = torch.arange(4, dtype=torch.int32, device=DEV)
    imp = torch.zeros(2, 2049, device=DEV)
    q = torch.zeros(4, 4, 64, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(2049, 4, 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.anchor_importance_batched(q, rows, off, 2, kc, None, None, None, 0.125, imp)   # chunked affix
    q32, k32 = torch.zeros(4, 4, 64, device=DEV), torch.zeros(100, 4, 64, device=DEV)
    assert not ops.anchor_importance_batched(q32, rows, off, 2, k32, None, None, None, 0.125, imp[:, :100].contiguous())
    assert float(imp.abs().sum()) == 0.0
    _lib.check_device_errors()


# ----------------------------------------------------------------------------- attention
def _tol(dt):
    return {torch.float32: 2e-5, torch.float16: 4e-3, torch.bfloat16: 2e-2}[dt]


def _assert_close(got, ref, dt, tag=None):
    """Tolerance of the dtype applied twice: the largest difference must stay below it in
    absolute terms AND relative to the largest reference magnitude (max relative error 2e-2 for
    bf16), so outputs that are small as a whole are not passed by the absolute bound alone."""
    got, ref = got.detach().cpu().float(), ref.detach().cpu().float()
    if got.numel() == 0:
        return
    tol = _tol(dt)
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err < tol, (tag, err)
    assert err <= tol * max(scale, 1e-30), (tag, err, scale, err / max(scale, 1e-30))


def test_attention_golden_all_modes(triton_ops):
    _lib, ops, aa, att = _ops()
    t = {k: v.to(DEV) for k, v in triton_ops.items() if k.startswith("att_")}
    spl = int(t["att_shared_prefix_len"])
    for tag, tol in (("f32", 2e-5), ("f16", 4e-3)):
        args = (t[f"att_{tag}_q"], t[f"att_{tag}_kc"], t[f"att_{tag}_vc"], t[f"att_{tag}_cu_q"], t[f"att_{tag}_cu_k"])
        plain = aa.acache_attention(*args, t[f"att_{tag}_logical"])
        key = aa.acache_attention(*args, t[f"att_{tag}_logical"], None, spl, None, t[f"att_{tag}_shifts"],
                                  t["att_cos"], t["att_sin"])
        qs = aa.acache_attention(*args, t[f"att_{tag}_packed"], None, spl, t[f"att_{tag}_shared_lens"],
                                 t[f"att_{tag}_shifts"], t["att_cos"], t["att_sin"])
        for name, got in (("plain", plain), ("keyside", key), ("queryside", qs)):
            err = (got.float() - t[f"att_{tag}_{name}"].float()).abs().max().item()
            assert err < tol, (tag, name, err)
    _lib.check_device_errors()


def test_block_table_attention_golden(triton_ops):
    _lib, ops, aa, att = _ops()
    t = {k: v.to(DEV) for k, v in triton_ops.items() if k.startswith("bt_")}
    got = aa.baseline_ragged_attention(t["bt_q"], t["bt_kc"], t["bt_vc"], t["bt_cu"], t["bt_cu"], t["bt_tables"])
    assert (got - t["bt_ragged"]).abs().max() < 2e-5
    got = aa.baseline_decode_attention(t["bt_qd"], t["bt_kc"], t["bt_vc"], t["bt_seqlens"], t["bt_tables"])
    assert (got - t["bt_decode"]).abs().max() < 2e-5


def _random_case(g, dt, nh, hkv, D, Bk, nb, q_lens, kv_lens, A=0, shifts=None):
    """Random paged cache + per-request slot maps; with A > 0 the slots 0..A-1 are a
    shared span placed at logical [shift, shift + A) of every request, minus a few anchors."""
    import random

    pyr = random.Random(int(torch.randint(0, 1 << 30, (1,), generator=g)))
    kc = torch.randn(nb, Bk, hkv, D, generator=g).to(dt)
    vc = torch.randn(nb, Bk, hkv, D, generator=g).to(dt)
    q = torch.randn(sum(q_lens), nh, D, generator=g).to(dt)
    logical, packed, shared_lens = [], [], []
    for i, n in enumerate(kv_lens):
        private = pyr.sample(range(A, nb * Bk), n)
        if A:
            s = shifts[i]
            anchors = set(pyr.sample(range(s, s + A), max(1, A // 5)))
            m = [(p - s) if (s <= p < s + A and p not in anchors) else private[p] for p in range(n)]
        else:
            m = private
        logical += m
        sh = [x for x in m if x < A]
        packed += sh + [x for x in m if x >= A]
        shared_lens.append(len(sh))
    cu_q = torch.tensor([0, *np.cumsum(q_lens)], dtype=torch.int32)
    cu_k = torch.tensor([0, *np.cumsum(kv_lens)], dtype=torch.int32)
    return q, kc, vc, cu_q, cu_k, torch.tensor(logical, dtype=torch.int32), torch.tensor(packed, dtype=torch.int32), \
        torch.tensor(shared_lens, dtype=torch.int32)


@pytest.mark.parametrize("dt,nh,hkv,D", [
    (torch.bfloat16, 8, 8, 128), (torch.bfloat16, 28, 4, 128), (torch.float16, 4, 2, 64),
    (torch.float16, 4, 2, 160), (torch.float32, 4, 4, 16), (torch.bfloat16, 4, 4, 16)])
def test_attention_random_vs_oracle(dt, nh, hkv, D):
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(7)
    Bk, nb, A = 16, 40, 48
    q_lens, kv_lens, shifts = [70, 1, 33, 130], [200, 90, 64, 333], [9, 0, 16, 101]
    q, kc, vc, cu_q, cu_k, logical, packed, shl = _random_case(g, dt, nh, hkv, D, Bk, nb, q_lens, kv_lens, A, shifts)
    cos, sin = _rope(512, D)
    sh_t = torch.tensor(shifts, dtype=torch.int32)
    d = lambda x: x.to(DEV)
    tol = _tol(dt)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, logical)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(logical))
    _assert_close(got, ref, dt)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, logical, None, A, None, sh_t, cos, sin)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(logical), None, A, None, d(sh_t), d(cos), d(sin))
    _assert_close(got, ref, dt)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, packed, None, A, shl, sh_t, cos, sin)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(packed), None, A, d(shl), d(sh_t), d(cos), d(sin),
                              max_seqlen_q=max(q_lens), max_seqlen_k=max(kv_lens))
    _assert_close(got, ref, dt)
    _lib.check_device_errors()


def test_materialised_equals_key_side_relocation_bitwise():
    """reference: nano-vdllm/tests/test_attention_kernels.py:168-234."""
    _lib, ops, aa, att = _ops()
    torch.manual_seed(0)
    L, S, nh, hkv, D = 1, 32, 4, 2, 64
    q_len, kv_len, a0, A, dst = 5, 13, 7, 3, 24
    dt = torch.bfloat16
    q = torch.randn(q_len, nh, D, device=DEV, dtype=dt)
    k = torch.randn(L, S, hkv, D, device=DEV, dtype=dt)
    v = torch.randn_like(k)
    cos, sin = (x.to(DEV) for x in _rope(S, D))
    key_slots = list(range(A, A + kv_len))
    for lp, pos in enumerate(range(a0, a0 + A)):
        key_slots[pos] = lp
    cu_q = torch.tensor([0, q_len], device=DEV, dtype=torch.int32)
    cu_k = torch.tensor([0, kv_len], device=DEV, dtype=torch.int32)
    shifts = torch.tensor([a0], device=DEV, dtype=torch.int32)
    key_side = aa.acache_attention(q, k[0].view(4, 8, hkv, D), v[0].view(4, 8, hkv, D), cu_q, cu_k,
                                   torch.tensor(key_slots, device=DEV, dtype=torch.int32),
                                   shared_prefix_len=A, affix_shifts=shifts, rope_cos=cos, rope_sin=sin)
    aa.materialize_relocated_affix(k, v, cos, sin, dst, A, a0)
    mat_slots = list(key_slots)
    for lp, pos in enumerate(range(a0, a0 + A)):
        mat_slots[pos] = dst + lp
    mat = aa.acache_attention(q, k[0].view(4, 8, hkv, D), v[0].view(4, 8, hkv, D), cu_q, cu_k,
                              torch.tensor(mat_slots, device=DEV, dtype=torch.int32))
    assert torch.equal(mat, key_side)


# ----------------------------------------------------------------------------- block ops
@pytest.mark.parametrize("cols", [64, 4096, 3584, 1000])
def test_rmsnorm_matches_reference_flow(cols):
    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(8)
    x = (torch.randn(37, cols, generator=g) * 3).to(torch.bfloat16)
    w = torch.randn(cols, generator=g).to(torch.bfloat16)
    xf = x.float()
    ref = w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16)
    got = ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-5).cpu()
    # the fp32 mean is reduced in a different order: allow one bf16 ulp on a few elements
    diff = (got.float() - ref.float()).abs()
    assert (diff <= ref.float().abs() * 2 ** -7 + 1e-6).all()
    assert (diff > 0).float().mean() < 0.01


def test_add_rmsnorm_equals_add_then_rmsnorm():
    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(18)
    for cols in (64, 4096, 3584):
        x = (torch.randn(33, cols, generator=g) * 3).to(torch.bfloat16).to(DEV)
        d = torch.randn(33, cols, generator=g).to(torch.bfloat16).to(DEV)
        w = torch.randn(cols, generator=g).to(torch.bfloat16).to(DEV)
        want_x = x + d
        want_y = ops.rmsnorm(want_x, w, 1e-5)
        got_y = ops.add_rmsnorm(x, d, w, 1e-5)
        assert torch.equal(x, want_x) and torch.equal(got_y, want_y)


@pytest.mark.parametrize("act", ["silu", "relu", "gelu"])
def test_act_mul(act):
    import torch.nn.functional as F

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(9)
    a = (torch.randn(5, 1003, generator=g) * 2).to(torch.bfloat16)
    b = torch.randn(5, 1003, generator=g).to(torch.bfloat16)
    ref = {"silu": F.silu, "relu": F.relu, "gelu": F.gelu}[act](a) * b
    got = ops.act_mul(a.to(DEV), b.to(DEV), act).cpu()
    diff = (got.float() - ref.float()).abs()
    assert (diff <= ref.float().abs() * 2 ** -7 + 1e-6).all()


def test_transfer_tokens_golden_and_random():
    from oracle import sampling

    _lib, ops, aa, att = _ops()
    z = load_npz("sampling.npz")
    logits, x, mask = torch.from_numpy(z["logits"]), torch.from_numpy(z["x"]), torch.from_numpy(z["mask"])
    mask_id = int(x[mask][0])
    blocks = x.clone().to(DEV)
    ops.transfer_tokens(logits.to(DEV), blocks, mask_id, float(z["threshold"]))
    want = torch.where(torch.from_numpy(z["transfer"]), torch.from_numpy(z["x0"]), x)
    assert torch.equal(blocks.cpu(), want)
    g = torch.Generator().manual_seed(10)
    B, T, V = 16, 32, 126464
    lg = (torch.randn(B * T, V, generator=g) * 2).to(torch.bfloat16)
    lg[torch.arange(0, B * T, 3), torch.randint(0, V, (len(range(0, B * T, 3)),), generator=g)] += 14.0
    xb = torch.full((B, T), 126336, dtype=torch.int64)
    xb[:, ::5] = 7
    x0, ti = sampling.get_transfer_index(lg.view(B, T, V), xb == 126336, xb, 0.9)
    want = torch.where(ti, x0, xb)
    blocks = xb.clone().to(DEV)
    ops.transfer_tokens(lg.to(DEV), blocks, 126336, 0.9)
    assert torch.equal(blocks.cpu(), want)


# ----------------------------------------------------------------------------- tensor-core attention
@pytest.mark.parametrize("dt,nh,hkv,D,q_lens,kv_lens", [
    (torch.bfloat16, 32, 32, 128, [32, 32, 32], [1216, 1120, 1312]),          # block decode, MHA
    (torch.bfloat16, 28, 4, 128, [32, 32], [1112, 920]),                      # block decode, GQA 7
    (torch.bfloat16, 8, 8, 128, [480, 672, 1], [1120, 1312, 65]),             # refresh
    (torch.float16, 14, 2, 64, [129, 300], [64, 577]),                        # head_dim 64, GQA 7
    (torch.bfloat16, 4, 4, 128, [5, 0, 9], [3, 10, 0]),                       # empty / tiny requests
    (torch.bfloat16, 4, 2, 128, [600, 130], [700, 1500]),                     # 1200 virtual rows: CTA pairs, a ragged second request
])
def test_attention_tensor_core_shapes(dt, nh, hkv, D, q_lens, kv_lens):
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(11)
    Bk = 64
    nb = (sum(kv_lens) + 200) // Bk + 4
    A = 40
    shifts = [17, 0, 33][: len(q_lens)]
    q, kc, vc, cu_q, cu_k, logical, packed, shl = _random_case(g, dt, nh, hkv, D, Bk, nb, q_lens, kv_lens, 0, None)
    d = lambda x: x.to(DEV)
    tol = _tol(dt)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, logical)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(logical), max_seqlen_q=max(q_lens))
    live = torch.cat([torch.full((n,), float(k > 0)) for n, k in zip(q_lens, kv_lens)]).bool()
    _assert_close(got.cpu()[live], ref[live], dt)
    if min(kv_lens) > A + 40:
        q, kc, vc, cu_q, cu_k, logical, packed, shl = _random_case(g, dt, nh, hkv, D, Bk, nb, q_lens, kv_lens, A, shifts)
        cos, sin = _rope(2048, D)
        sh_t = torch.tensor(shifts, dtype=torch.int32)
        ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, packed, None, A, shl, sh_t, cos, sin)
        got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(packed), None, A, d(shl), d(sh_t), d(cos),
                                  d(sin), max_seqlen_q=max(q_lens), max_seqlen_k=max(kv_lens))
        _assert_close(got, ref, dt)
    _lib.check_device_errors()


def test_attention_tensor_core_growing_scores_and_block_tables():
    """Scores that grow tile after tile force the accumulator rescale path; K/V addressed
    through block tables (baseline kernels' form)."""
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(12)
    dt, nh, hkv, D, Bk = torch.bfloat16, 4, 2, 128, 16
    lens = [700, 333]
    nblk = [-(-n // Bk) for n in lens]
    nb = sum(nblk) + 3
    ids = torch.randperm(nb, generator=g).tolist()
    bt = torch.full((2, max(nblk)), -1, dtype=torch.int32)
    o = 0
    for i, c in enumerate(nblk):
        bt[i, :c] = torch.tensor(ids[o: o + c], dtype=torch.int32)
        o += c
    kc = torch.randn(nb, Bk, hkv, D, generator=g)
    vc = torch.randn(nb, Bk, hkv, D, generator=g).to(dt)
    q = torch.randn(sum(lens), nh, D, generator=g).to(dt)
    # make later keys of request 0 much larger: the running maximum keeps jumping
    for j in range(lens[0]):
        kc[bt[0, j // Bk], j % Bk] *= 1.0 + 6.0 * j / lens[0]
    kc = kc.to(dt)
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32)
    ref = oatt.baseline_ragged_attention(q, kc, vc, cu, cu, bt)
    got = aa.baseline_ragged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), cu.to(DEV), cu.to(DEV), bt.to(DEV),
                                       max_seqlen_q=max(lens))
    _assert_close(got, ref, torch.bfloat16)
    qd = q[:64].reshape(2, 32, nh, D)
    sl = torch.tensor(lens, dtype=torch.int32)
    ref = oatt.baseline_decode_attention(qd, kc, vc, sl, bt)
    got = aa.baseline_decode_attention(qd.to(DEV), kc.to(DEV), vc.to(DEV), sl.to(DEV), bt.to(DEV))
    _assert_close(got, ref, torch.bfloat16)
    _lib.check_device_errors()


def _runs_case(g, dt, nh, hkv, D, Bk, nb, A, q_lens, own_lens, hole_every=5, nan_fill=True):
    """Shared span = slots 0..A-1; every request reads it as one run with holes (-1) where an
    'anchor' has a private copy, then the private copies, then its own tokens, all private
    slots being consecutive from a block boundary.  Returns the run layout and the same keys
    without holes in logical order."""
    kc = torch.randn(nb, Bk, hkv, D, generator=g).to(dt)
    vc = torch.randn(nb, Bk, hkv, D, generator=g).to(dt)
    q = torch.randn(sum(q_lens), nh, D, generator=g).to(dt)
    runs, logical, n_span = [], [], []
    next_block = -(-A // Bk)
    for own in own_lens:
        holes = list(range(2, A, hole_every)) if hole_every else []
        k = len(holes)
        base = next_block * Bk
        next_block += -(-(k + own) // Bk)
        assert next_block <= nb
        span = list(range(A))
        log = list(range(A))
        for i, h in enumerate(holes):
            span[h] = -1
            log[h] = base + i
        private = list(range(base, base + k + own))
        runs += span + private
        logical += log + private[k:]
        n_span.append(A)
    if nan_fill:  # rows a hole stands for and rows past the last used slot hold NaN: they must not leak
        flat_k, flat_v = kc.view(-1, hkv, D), vc.view(-1, hkv, D)
        for h in (range(2, A, hole_every) if hole_every else []):
            flat_k[h], flat_v[h] = float("nan"), float("nan")
        flat_k[next_block * Bk:], flat_v[next_block * Bk:] = float("nan"), float("nan")
        used = torch.zeros(nb * Bk, dtype=torch.bool)
        used[torch.tensor([x for x in runs if x >= 0])] = True
        used[:A] = True
        flat_k[~used], flat_v[~used] = float("nan"), float("nan")
    ql = torch.tensor([0, *np.cumsum(q_lens)], dtype=torch.int32)
    holes_n = len(range(2, A, hole_every)) if hole_every else 0
    cu_runs = torch.tensor([0, *np.cumsum([A + holes_n + o for o in own_lens])], dtype=torch.int32)
    cu_log = torch.tensor([0, *np.cumsum([A + o for o in own_lens])], dtype=torch.int32)
    return q, kc, vc, ql, cu_runs, torch.tensor(runs, dtype=torch.int32), cu_log, \
        torch.tensor(logical, dtype=torch.int32), torch.tensor(n_span, dtype=torch.int32)


@pytest.mark.parametrize("dt,nh,hkv,D,A,q_lens,own_lens", [
    (torch.bfloat16, 32, 32, 128, 800, [32, 32, 32], [96, 300, 511]),     # block decode, MHA, 800-token affix
    (torch.bfloat16, 28, 4, 128, 600, [32, 32], [64, 257]),               # GQA 7
    (torch.float16, 4, 2, 64, 130, [70, 3], [10, 200]),                    # head_dim 64, ragged queries
    (torch.bfloat16, 4, 4, 128, 64, [5, 9], [0, 1]),                       # one full span tile, (almost) nothing else
    (torch.float32, 4, 4, 32, 100, [7, 40], [30, 5]),                      # CUDA-core kernel, same contract
])
def test_attention_slot_runs_with_holes(dt, nh, hkv, D, A, q_lens, own_lens):
    """The run layout (consecutive slots read as runs, -1 = key that takes no part) gives
    the same attention as the logical order; dead rows never leak, even when they hold NaN."""
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(21)
    Bk = 256
    nb = -(-A // Bk) + sum(-(-(A // 5 + 1 + o) // Bk) for o in own_lens) + 1
    q, kc, vc, cu_q, cu_runs, runs, cu_log, logical, n_span = _runs_case(g, dt, nh, hkv, D, Bk, nb, A, q_lens, own_lens)
    d = lambda x: x.to(DEV)
    tol = _tol(dt)
    ref = oatt.acache_attention(q, torch.nan_to_num(kc), torch.nan_to_num(vc), cu_q, cu_log, logical)
    assert torch.isfinite(ref.float()).all()
    # oracle agrees with itself across the two layouts (holes are handled the same way)
    ref_runs = oatt.acache_attention(q, torch.nan_to_num(kc), torch.nan_to_num(vc), cu_q, cu_runs, runs)
    assert (ref_runs.float() - ref.float()).abs().max() < tol
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), max_seqlen_q=max(q_lens))
    assert torch.isfinite(got.float()).all()
    _assert_close(got, ref, dt)
    # run split: the private part starts a fresh tile (all of its tiles are whole runs)
    got2 = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), None, 0, d(n_span),
                               max_seqlen_q=max(q_lens))
    assert torch.isfinite(got2.float()).all()
    _assert_close(got2, ref, dt)
    _lib.check_device_errors()


def test_attention_slot_runs_query_side_and_edges():
    """Query-side relocation over a run layout; a tile of holes only; a run that ends at the
    last slot of the cache (the last tile reaches past it); a run that starts at an odd slot."""
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(22)
    dt, nh, hkv, D, Bk, A = torch.bfloat16, 8, 8, 128, 256, 300
    q, kc, vc, cu_q, cu_runs, runs, cu_log, logical, n_span = _runs_case(
        g, dt, nh, hkv, D, Bk, 6, A, [32, 40], [100, 37], nan_fill=False)
    d = lambda x: x.to(DEV)
    cos, sin = _rope(2048, D)
    shifts = torch.tensor([11, 140], dtype=torch.int32)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_runs, runs, None, A, n_span, shifts, cos, sin)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), None, A, d(n_span), d(shifts), d(cos),
                              d(sin), max_seqlen_q=40, max_seqlen_k=600)
    _assert_close(got, ref, torch.bfloat16)

    # hand-made map, tile by tile: [64 holes] [run 7..70 (odd start)] [64 scattered rows]
    # [the last 40 slots of the cache: a run whose last tile reaches past the end]
    nslots = 6 * Bk
    m = [-1] * 64 + list(range(7, 71)) + [5, 900, 333] + list(range(100, 161)) + list(range(nslots - 40, nslots))
    cu_k = torch.tensor([0, len(m)], dtype=torch.int32)
    cu_q1 = torch.tensor([0, 32], dtype=torch.int32)
    mm = torch.tensor(m, dtype=torch.int32)
    ref = oatt.acache_attention(q[:32], kc, vc, cu_q1, cu_k, mm)
    got = aa.acache_attention(d(q[:32]), d(kc), d(vc), d(cu_q1), d(cu_k), d(mm), max_seqlen_q=32)
    _assert_close(got, ref, torch.bfloat16)
    # nothing but holes: zeros
    mm = torch.full((130,), -1, dtype=torch.int32)
    cu_k = torch.tensor([0, 130], dtype=torch.int32)
    got = aa.acache_attention(d(q[:32]), d(kc), d(vc), d(cu_q1), d(cu_k), d(mm), max_seqlen_q=32)
    assert torch.equal(got.cpu().float(), torch.zeros(32, nh, D))
    _lib.check_device_errors()


@pytest.mark.parametrize("dt,nh,hkv,D,A,q_lens,own_lens,shifts", [
    (torch.bfloat16, 32, 32, 128, 800, [32] * 6, [96, 300, 511, 64, 130, 257], None),        # block decode, MHA; 6 = 4 + 2
    (torch.bfloat16, 8, 8, 128, 200, [32, 7, 0, 32, 1, 32, 32, 32, 5], [50, 0, 9, 300, 1, 70, 64, 65, 2], None),
    (torch.bfloat16, 28, 4, 128, 300, [4, 4, 3, 4, 4], [64, 257, 10, 0, 90], None),           # GQA 7: 4 x 7 = 28 rows
    (torch.float16, 4, 2, 64, 130, [16, 16, 9], [10, 200, 33], [5, 77, 140]),                 # head_dim 64, query-side
    (torch.bfloat16, 8, 8, 128, 100, [32, 32, 32, 32], [40, 41, 42, 43], [3, 3, 900, 0]),     # query-side, MHA
])
def test_attention_grouped_shared_span(dt, nh, hkv, D, A, q_lens, own_lens, shifts):
    """The grouped block-decode kernel (shared span staged once per four requests, parts folded
    by the second arrival) against the oracle and the per-request kernel."""
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(31)
    Bk = 256
    nb = -(-A // Bk) + sum(-(-(A // 5 + 1 + o) // Bk) for o in own_lens) + 1
    q, kc, vc, cu_q, cu_runs, runs, cu_log, logical, n_span = _runs_case(g, dt, nh, hkv, D, Bk, nb, A, q_lens, own_lens)
    d = lambda x: x.to(DEV)
    tol = _tol(dt)
    kw = {}
    args = [None, 0, n_span]
    if shifts is not None:
        cos, sin = _rope(2048, D)
        sh = torch.tensor(shifts, dtype=torch.int32)
        args = [None, A, n_span, sh, cos, sin]
        kw = dict(max_seqlen_k=1024)
    ref = oatt.acache_attention(q, torch.nan_to_num(kc), torch.nan_to_num(vc), cu_q, cu_runs, runs, *args)
    dargs = [d(x) if torch.is_tensor(x) else x for x in args]
    plain = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), *dargs, max_seqlen_q=max(q_lens), **kw)
    launches = _lib.LAUNCHES
    for _ in range(3):  # the scratch is reused as it was left
        got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), *dargs, max_seqlen_q=max(q_lens),
                                  group_shared_span=True, **kw)
        assert torch.isfinite(got.float()).all()
        _assert_close(got, ref, dt)
        assert (got.float() - plain.float()).abs().max() < tol
    assert _lib.LAUNCHES == launches + 3
    _lib.check_device_errors()


def test_attention_grouped_declines_and_reports():
    """More than 32 rows per request: the plain kernel answers.  Requests of a group that name
    different spans: reported through the error flag, nothing faults, and the next call works."""
    from acache_b200._lib import AcacheError
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(32)
    dt, nh, hkv, D, Bk, A = torch.bfloat16, 8, 8, 128, 256, 128
    q, kc, vc, cu_q, cu_runs, runs, cu_log, logical, n_span = _runs_case(
        g, dt, nh, hkv, D, Bk, 8, A, [40, 33], [20, 30], nan_fill=False)
    d = lambda x: x.to(DEV)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_runs, runs)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), None, 0, d(n_span), max_seqlen_q=40,
                              group_shared_span=True)
    _assert_close(got, ref, torch.bfloat16)
    _lib.check_device_errors()

    q, kc, vc, cu_q, cu_runs, runs, cu_log, logical, n_span = _runs_case(
        g, dt, nh, hkv, D, Bk, 8, A, [32, 32], [20, 30], nan_fill=False)
    bad = runs.clone()
    second = int(cu_runs[1])
    bad[second: second + A][bad[second: second + A] >= 0] += 256        # request 1 names another span
    aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(bad), None, 0, d(n_span), max_seqlen_q=32,
                        group_shared_span=True)
    with pytest.raises(AcacheError, match="same shared span"):
        _lib.check_device_errors()
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_runs, runs)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_runs), d(runs), None, 0, d(n_span), max_seqlen_q=32,
                              group_shared_span=True)
    _assert_close(got, ref, torch.bfloat16)
    _lib.check_device_errors()


def test_attention_many_rows_reports_bad_slots_and_holes():
    """The 256-row kernel (requests of more than 128 virtual rows; CTA pairs from 1024): read-map
    entries outside the cache are skipped and reported, the next call works; entries of -1 are
    keys that take no part; a request whose keys are all holes gets zeros."""
    from acache_b200._lib import AcacheError
    from oracle import attention as oatt

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(41)
    dt, nh, hkv, D, Bk = torch.bfloat16, 4, 2, 128, 64
    q_lens, kv_lens = [300, 520, 140], [333, 700, 65]           # 600 / 1040 / 280 virtual rows
    nb = sum(kv_lens) // Bk + 8
    q, kc, vc, cu_q, cu_k, logical, packed, shl = _random_case(g, dt, nh, hkv, D, Bk, nb, q_lens, kv_lens, 0, None)
    d = lambda x: x.to(DEV)
    ref = oatt.acache_attention(q, kc, vc, cu_q, cu_k, logical)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(logical), max_seqlen_q=max(q_lens))
    _assert_close(got, ref, dt)
    _lib.check_device_errors()

    bad = logical.clone()
    bad[int(cu_k[1]) + 77] = nb * Bk + 5                          # one key of request 1 lies outside the cache
    aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(bad), max_seqlen_q=max(q_lens))
    with pytest.raises(AcacheError):
        _lib.check_device_errors()
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(logical), max_seqlen_q=max(q_lens))
    _assert_close(got, ref, dt)
    _lib.check_device_errors()

    holes = logical.clone()
    holes[int(cu_k[0]): int(cu_k[1]): 3] = -1                     # every third key of request 0 takes no part
    holes[int(cu_k[2]): int(cu_k[3])] = -1                        # request 2 sees nothing at all
    keep = torch.ones(int(cu_k[3]), dtype=torch.bool)
    keep[int(cu_k[0]): int(cu_k[1]): 3] = False
    keep[int(cu_k[2]): int(cu_k[3])] = False
    kept = logical[keep]
    cu_kept = torch.tensor([0, int(keep[: int(cu_k[1])].sum()), int(keep[: int(cu_k[2])].sum()), int(keep.sum())],
                           dtype=torch.int32)
    live_rows = int(cu_q[2])
    ref = oatt.acache_attention(q[:live_rows], kc, vc, cu_q[:3], cu_kept[:3], kept)
    got = aa.acache_attention(d(q), d(kc), d(vc), d(cu_q), d(cu_k), d(holes), max_seqlen_q=max(q_lens))
    _assert_close(got[:live_rows], ref, dt)
    assert torch.equal(got[live_rows:].cpu().float(), torch.zeros(q_lens[2], nh, D))
    _lib.check_device_errors()


# ----------------------------------------------------------------------------- fused QKV GEMM
@pytest.mark.parametrize("kind,n,hidden,nh,hkv", [("llada", 300, 512, 4, 4), ("dream", 77, 448, 7, 1),
                                                   ("llada", 512, 4096, 32, 32)])
def test_qkv_rope_scatter_matches_unfused_path(kind, n, hidden, nh, hkv):
    """tcgen05 GEMM with the fused bias + RoPE + cache-scatter epilogue against the unfused
    sequence (fp32 reference GEMM rounded to bf16, oracle RoPE, oracle scatter).  The only
    difference allowed is the accumulation order of the projection (bf16 tolerance 2e-2)."""
    from oracle import kv_ops
    from oracle.rope import dream_rope_qk, llada_rope_qk

    _lib, ops, aa, att = _ops()
    g = torch.Generator().manual_seed(20)
    D, dt = 128, torch.bfloat16
    N = (nh + 2 * hkv) * D
    x = torch.randn(n, hidden, generator=g).to(dt)
    w = (torch.randn(N, hidden, generator=g) * hidden ** -0.5).to(dt)
    bias = (torch.randn(N, generator=g) * 0.1).to(dt) if kind == "dream" else None
    pos = torch.randint(0, 900, (n,), generator=g)
    nb, Bk = n // 64 + 2, 64
    slots = torch.randperm(nb * Bk, generator=g)[:n].to(torch.int32)
    slots[3] = -1
    theta = 500000.0
    ref = x.float() @ w.float().T
    if bias is not None:
        ref = ref + bias.float()
    ref = ref.to(dt)
    q_ref, k_ref, v_ref = ref[:, : nh * D].view(n, nh, D), ref[:, nh * D: (nh + hkv) * D].view(n, hkv, D), \
        ref[:, (nh + hkv) * D:].view(n, hkv, D)
    if kind == "llada":
        q_ref, k_ref = llada_rope_qk(q_ref, k_ref, pos, theta)
        cos, sin = _rope(1024, D, theta, torch.float32)
    else:
        q_ref, k_ref = dream_rope_qk(q_ref, k_ref, pos, theta)
        cos, sin = _rope(1024, D, theta, dt)
    kc, vc = torch.zeros(nb, Bk, hkv, D, dtype=dt), torch.zeros(nb, Bk, hkv, D, dtype=dt)
    kv_ops.store_kvcache(k_ref, v_ref, kc, vc, slots)
    kcd, vcd = torch.zeros_like(kc, device=DEV), torch.zeros_like(vc, device=DEV)
    q = ops.qkv_rope_scatter(x.to(DEV), w.to(DEV), None if bias is None else bias.to(DEV), nh, hkv, D, pos.to(DEV),
                             cos.to(DEV), sin.to(DEV), kcd, vcd, slots.to(DEV))
    tol = 3e-2
    assert (q.cpu().float() - q_ref.float()).abs().max() < tol
    assert (kcd.cpu().float() - kc.float()).abs().max() < tol
    assert (vcd.cpu().float() - vc.float()).abs().max() < tol
    # rows with slot -1 and unused slots stay untouched
    assert float(kcd.cpu().float().abs().sum(dim=(-1, -2)).view(-1)[~torch.isin(torch.arange(nb * Bk), slots.long())].sum()) == 0
    _lib.check_device_errors()
