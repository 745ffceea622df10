"""The allocation-free variant of the anchor influence score (collected last on purpose:
a run that stops at the first failure has then already run everything else).

It exists for hosts that cannot allocate device memory when they call in - a runtime that
owns the whole GPU through its own arena, a plugin that is handed nothing but its input and
output buffers - so the test drives it straight through the C ABI with buffers made up
front and compares it with the ordinary entry point, twice in a row because both calls use
the same fixed scratch array inside the library."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, nq, nh, hkv, D, A, dt=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    n = nq + 7
    q = torch.randn(n, nh, D, generator=g).to(dt).to(DEV)
    kc = torch.randn(A, hkv, D, generator=g).to(dt).to(DEV)
    rows = torch.randperm(n, generator=g)[:nq].sort().values.to(torch.int32).to(DEV)
    return q, kc, rows


def test_static_scratch_variant_matches_the_allocating_entry_point_twice():
    from acache_b200 import _lib
    from acache_b200._lib import check, dtype_code, ptr, stream_ptr
    from acache_b200.model.modeling_common import build_rope_table

    lib = _lib.load()
    cos, sin = build_rope_table(64, 128, 500000.0, torch.float32, DEV)
    # two different problems back to back: the second must not see leftovers of the first
    for seed, (nq, nh, hkv, A, shift) in enumerate([(70, 8, 2, 300, 13), (33, 4, 4, 129, 0)]):
        D = 128
        q, kc, rows = _inputs(seed, nq, nh, hkv, D, A)
        want = torch.zeros(A, device=DEV)
        got = torch.zeros(A, device=DEV)
        nbytes = lib.acache_anchor_importance_scratch_bytes(nq, nh, A)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        args = (ptr(q), q.stride(0), ptr(rows), nq, nh, hkv, D, dtype_code(q.dtype), ptr(kc), kc.stride(0), A, shift,
                ptr(cos), ptr(sin), cos.stride(0), cos.shape[0], dtype_code(cos.dtype), D ** -0.5)
        check(lib.acache_anchor_importance(*args, ptr(want), ptr(scratch), nbytes, None, stream_ptr()), "importance")
        check(lib.acache_anchor_importance_static(*args, ptr(got), None, stream_ptr()), "importance_static")
        torch.cuda.synchronize()
        # same kernels, same summation order: the tolerance of the score tests is more than enough
        assert torch.allclose(got, want, rtol=2e-3, atol=1e-4)
        assert torch.equal(got, want)
        assert float(got.sum()) > 0


def test_static_scratch_variant_refuses_oversized_requests():
    from acache_b200 import _lib
    from acache_b200._lib import ptr

    lib = _lib.load()
    cap = lib.acache_anchor_importance_static_scratch_bytes()
    assert cap == 8 << 20
    # 64 query tiles x 32 heads x 8192 affix tokens of fp32 partial sums is far beyond 8 MiB
    nq, nh, A = 2048, 32, 8192
    assert lib.acache_anchor_importance_scratch_bytes(nq, nh, A) > cap
    imp = torch.zeros(A, device=DEV)
    dummy = torch.zeros(16, device=DEV)
    rc = lib.acache_anchor_importance_static(ptr(dummy), 0, ptr(dummy), nq, nh, nh, 128, 2, ptr(dummy), 0, A, 0, None,
                                             None, 0, 0, 0, 1.0, ptr(imp), None, None)
    assert rc == -4
    assert lib.acache_status_string(rc) == b"size beyond a fixed limit"
    assert float(imp.abs().sum()) == 0.0


def test_python_wrapper_of_the_static_variant():
    from acache_b200 import ops

    q, kc, rows = _inputs(5, 40, 4, 2, 64, 200)
    a = torch.zeros(200, device=DEV)
    b = torch.zeros(200, device=DEV)
    ops.anchor_importance(q, rows, kc, 0, None, None, 0.125, a)
    ops.anchor_importance_noalloc(q, rows, kc, 0, None, None, 0.125, b)
    assert torch.equal(a, b)
    with pytest.raises(OverflowError):
        big_q = torch.zeros(4096, 32, 64, device=DEV, dtype=torch.bfloat16)
        ops.anchor_importance_noalloc(big_q, torch.arange(4096, dtype=torch.int32, device=DEV),
                                      torch.zeros(8192, 32, 64, device=DEV, dtype=torch.bfloat16), 0, None, None, 0.125,
                                      torch.zeros(8192, device=DEV))
