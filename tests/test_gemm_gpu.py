"""The CTA-pair tcgen05 projections against plain fp32 references of the same operators (a
floating-point kernel: the reference is the fp32 product rounded the way the unfused operator
chain rounds it; tolerance = one bf16 step of accumulation-order noise, stated per test)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (rows, in, out): ragged row counts, row blocks that are partly or wholly outside the matrix,
# column counts that are not a multiple of the tile, one real projection shape
SHAPES = [(300, 512, 384), (77, 448, 272), (1, 64, 64), (700, 256, 1040), (512, 4096, 4096), (513, 128, 2048)]
TILES = [(0, 0), (1, 64), (1, 256), (2, 128), (2, 176), (1, 112)]


def _ops():
    from acache_b200 import _lib, ops

    _lib.load()
    return _lib, ops


def _close(got, ref, what):
    """bf16 operands, fp32 accumulation on both sides: results may differ by one rounding step of
    the output (2^-8 relative) where the two summation orders straddle a rounding boundary."""
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = ref.abs().max().item()
    torch.testing.assert_close(got, ref, rtol=2 ** -7, atol=2 ** -8 * scale, msg=lambda m: f"{what}: {m}")


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("n,k,m_out", SHAPES)
def test_linear_matches_fp32_reference(n, k, m_out, tile):
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(n + k)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(m_out, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    b = torch.randn(m_out, generator=g).to(torch.bfloat16) if n % 2 else None
    ref = x.float() @ w.float().T
    if b is not None:
        ref = ref + b.float()
    ops.GEMM_TILE = tile
    try:
        got = ops.linear(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV))
    finally:
        ops.GEMM_TILE = (0, 0)
    _close(got, ref.to(torch.bfloat16), f"linear {n}x{k}x{m_out} tile {tile}")
    _lib.check_device_errors()


@pytest.mark.parametrize("tile", [(0, 0), (1, 256), (2, 256), (1, 112)])
@pytest.mark.parametrize("n,k,m_out,splits", [(300, 1024, 384, 3), (77, 576, 272, 2), (1, 512, 64, 8), (512, 4096, 4096, 0),
                                              (512, 12288, 4096, 0), (513, 1152, 2048, 5), (256, 4096, 4096, 0), (256, 4096, 4096, 4)])
def test_linear_partials_sum_to_the_projection(n, k, m_out, splits, tile):
    """The fp32 slices of the K range add up to the fp32 product (tolerance: fp32 summation-order
    noise, 1e-4 of the largest entry); a slice count of 0 takes the launch's own plan."""
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(n + k)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(m_out, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    parts = ops.linear_partials(x.to(DEV), w.to(DEV), splits, tile)
    want = splits or ops.linear_partials_splits(n, k, m_out)
    assert parts.shape == (want, n, m_out) and parts.dtype == torch.float32
    if splits == 0:               # the launch plan: only long K ranges with few output tiles are sliced
        assert want == {(512, 4096): 1, (512, 12288): 2, (256, 4096): 1}[(n, k)]
    torch.testing.assert_close(parts.sum(0).cpu(), ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())
    if want > 1:                  # every slice carries its own part of the K range
        k_per = -(-(-(-k // 64)) // want) * 64
        ref0 = x[:, :k_per].float() @ w[:, :k_per].float().T
        torch.testing.assert_close(parts[0].cpu(), ref0, rtol=1e-4, atol=1e-4 * ref.abs().max().item())
    _lib.check_device_errors()


def test_linear_partials_rejects_an_empty_slice():
    _lib, ops = _ops()
    x = torch.zeros(16, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        ops.linear_partials(x, w, 3)          # two k blocks cannot feed three slices
    assert ops.linear_partials(x, w, 2).shape == (2, 16, 64)
    _lib.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,cols,splits", [(37, 4096, 4), (512, 4096, 2), (5, 1024, 1), (9, 3584, 3)])
def test_add_rmsnorm_takes_fp32_slices_bit_exactly(n, cols, splits, dtype):
    """``add_rmsnorm`` on the slices = the slices summed in order in fp32, rounded to the model
    dtype, then the ordinary fused add + normalisation: same bits in x and in y."""
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(n + cols)
    x = torch.randn(n, cols, generator=g).to(dtype).to(DEV)
    parts = torch.randn(splits, n, cols, generator=g).to(DEV)
    wt = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).to(DEV)
    acc = torch.zeros(n, cols, device=DEV)
    for s in range(splits):
        acc = acc + parts[s]
    x_ref = x.clone()
    y_ref = ops.add_rmsnorm(x_ref, acc.to(dtype), wt, 1e-5)
    x_got = x.clone()
    y_got = ops.add_rmsnorm(x_got, parts, wt, 1e-5)
    assert torch.equal(x_got, x_ref) and torch.equal(y_got, y_ref)
    # strided slices: rows of a wider buffer
    wide = torch.randn(splits, n, cols + 64, generator=g).to(DEV)
    view = wide[:, :, 32:32 + cols]
    acc = torch.zeros(n, cols, device=DEV)
    for s in range(splits):
        acc = acc + view[s]
    x_ref = x.clone()
    y_ref = ops.add_rmsnorm(x_ref, acc.to(dtype), wt, 1e-5)
    x_got = x.clone()
    y_got = ops.add_rmsnorm(x_got, view, wt, 1e-5)
    assert torch.equal(x_got, x_ref) and torch.equal(y_got, y_ref)
    _lib.check_device_errors()


def test_linear_takes_strided_rows_and_fp16():
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(3)
    big = torch.randn(200, 640, generator=g).to(torch.float16).to(DEV)
    x = big[:, 128:384]                      # rows 640 elements apart, 256 used
    w = (torch.randn(96, 256, generator=g) / 16).to(torch.float16).to(DEV)
    got = ops.linear(x, w)
    ref = (x.float() @ w.float().T).to(torch.float16)
    _close(got, ref, "strided fp16")
    _lib.check_device_errors()


@pytest.mark.parametrize("tile", [(0, 0), (2, 112), (1, 256)])
@pytest.mark.parametrize("n,k,f,act", [(300, 512, 768, "silu"), (64, 256, 136, "gelu"), (512, 4096, 12288, "silu")])
def test_linear_swiglu_matches_the_separate_operators(n, k, f, act, tile):
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(f)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(f, k, generator=g) * k ** -0.5).to(torch.bfloat16).to(DEV)
    wu = (torch.randn(f, k, generator=g) * k ** -0.5).to(torch.bfloat16).to(DEV)
    gate = (x.float() @ wg.float().T).to(torch.bfloat16)
    up = (x.float() @ wu.float().T).to(torch.bfloat16)
    fn = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu}[act]
    ref = (fn(gate.float()).to(torch.bfloat16).float() * up.float()).to(torch.bfloat16)
    ops.GEMM_TILE = tile
    try:
        got = ops.linear_swiglu(x, ops.interleave_rows(wg, wu), act)
    finally:
        ops.GEMM_TILE = (0, 0)
    # a one-step difference in gate or up moves the product by up to two steps
    got, ref = got.float().cpu(), ref.float().cpu()
    torch.testing.assert_close(got, ref, rtol=2 ** -6, atol=2 ** -7 * ref.abs().max().item())
    _lib.check_device_errors()


@pytest.mark.parametrize("tile", [(0, 0), (2, 176), (1, 64)])
@pytest.mark.parametrize("kind,n,hidden,nh,hkv", [("llada", 300, 512, 4, 4), ("dream", 77, 448, 7, 1),
                                                   ("llada", 512, 4096, 32, 32)])
def test_linear_qkv_rope_scatter_matches_unfused_path(kind, n, hidden, nh, hkv, tile):
    """Interleaved-weight QKV projection with bias + RoPE + cache scatter in the epilogue against
    the unfused sequence (fp32 product rounded to bf16, CPU restatement of RoPE and of the
    scatter)."""
    from oracle import kv_ops
    from oracle.rope import dream_rope_qk, llada_rope_qk, rope_table

    _lib, ops = _ops()
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
        cos, sin = rope_table(1024, D, theta, torch.float32)
    else:
        q_ref, k_ref = dream_rope_qk(q_ref, k_ref, pos, theta)
        cos, sin = rope_table(1024, D, theta, dt)
    kc, vc = torch.zeros(nb, Bk, hkv, D, dtype=dt), torch.zeros(nb, Bk, hkv, D, dtype=dt)
    kv_ops.store_kvcache(k_ref, v_ref, kc, vc, slots)
    kcd, vcd = torch.zeros_like(kc, device=DEV), torch.zeros_like(vc, device=DEV)
    ops.GEMM_TILE = tile
    try:
        q = ops.linear_qkv_rope_scatter(x.to(DEV), ops.interleave_heads(w).to(DEV),
                                        None if bias is None else ops.interleave_heads(bias).to(DEV), nh, hkv, D,
                                        pos.to(DEV), cos.to(DEV), sin.to(DEV), kcd, vcd, slots.to(DEV))
    finally:
        ops.GEMM_TILE = (0, 0)
    tol = 3e-2      # one bf16 step of the projection, carried through the rotation
    assert (q.cpu().float() - q_ref.float()).abs().max() < tol
    assert (kcd.cpu().float() - kc.float()).abs().max() < tol
    assert (vcd.cpu().float() - vc.float()).abs().max() < tol
    unused = ~torch.isin(torch.arange(nb * Bk), slots.long())
    assert float(kcd.cpu().float().abs().sum(dim=(-1, -2)).view(-1)[unused].sum()) == 0
    _lib.check_device_errors()


@pytest.mark.parametrize("n,k,vocab", [(96, 256, 5008), (512, 4096, 126464)])
def test_linear_argmax_matches_logits_then_argmax(n, k, vocab):
    """Output head fused with the greedy statistics against logits -> arg-max / logsumexp:
    identical choices wherever the top two logits are not within a rounding step, confidence
    within a few per cent: the two paths round the logits from differently ordered fp32 sums, and one bf16 step of the maximum logit (2^-8 of its magnitude) moves the confidence by that much."""
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(vocab)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(vocab, k, generator=g) * k ** -0.5).to(torch.bfloat16).to(DEV)
    w[7] = w[3]                                   # equal logits: the lower index must win
    logits = (x.float() @ w.float().T).to(torch.bfloat16)
    want = logits.argmax(-1)
    lf = logits.float()
    want_conf = torch.exp(lf.max(-1).values - torch.logsumexp(lf, -1))
    x0, conf = ops.linear_argmax(x, w)
    top2 = lf.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 ** -6 * top2[:, 0].abs()
    assert clear.float().mean() > 0.5
    assert torch.equal(x0[clear], want[clear])
    picked = lf.gather(1, x0[:, None])[:, 0]
    assert ((top2[:, 0] - picked) <= 2 ** -6 * top2[:, 0].abs() + 1e-6).all()
    assert not (x0 == 7).any()
    torch.testing.assert_close(conf[clear], want_conf[clear], rtol=6e-2, atol=1e-6)
    _lib.check_device_errors()


def test_act_mul_halves_equals_act_mul_on_the_two_halves():
    """One projection over the concatenated gate / up weights followed by the activation kernel on
    its halves gives the bits of the two separate projections followed by ``act_mul``."""
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(9)
    x = torch.randn(77, 2 * 136, generator=g).to(torch.bfloat16).to(DEV)
    want = ops.act_mul(x[:, :136].contiguous(), x[:, 136:].contiguous(), "silu")
    assert torch.equal(ops.act_mul_halves(x, "silu"), want)
    wide = torch.randn(50, 400, generator=g).to(torch.float16).to(DEV)[:, :272]     # rows 400 elements apart
    want = ops.act_mul(wide[:, :136].contiguous(), wide[:, 136:].contiguous(), "gelu")
    assert torch.equal(ops.act_mul_halves(wide, "gelu"), want)


def test_apply_transfer_is_the_commit_rule_of_transfer_tokens():
    """Statistics in, blocks edited in place: the same result as ``transfer_tokens`` on the logits
    the statistics came from (threshold commits, forced commit of the most confident position)."""
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(10)
    R, T, V, mask = 6, 8, 96, 95
    logits = (torch.randn(R * T, V, generator=g) * 4).to(torch.bfloat16).to(DEV)
    logits[:, mask] = -30.0
    blocks = torch.full((R, T), mask, dtype=torch.int64)
    blocks[0, :] = 3                      # nothing left to unmask
    blocks[1, ::2] = 5                    # partly unmasked
    for thr in (0.3, 0.999):
        a, b = blocks.clone().to(DEV), blocks.clone().to(DEV)
        x0, conf = ops.transfer_tokens(logits, a, mask, thr)
        ops.apply_transfer(x0.reshape(-1).contiguous(), conf.reshape(-1).contiguous(), b, mask, thr)
        assert torch.equal(a, b)
        assert (a[0] == 3).all() and (a[1, ::2] == 5).all()
