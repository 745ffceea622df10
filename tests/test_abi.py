"""The C-ABI library loads and exports every symbol the public header declares.
No compute call is made, so this runs without a GPU."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "acache_b200.h").read_text()
    return sorted(set(re.findall(r"^ACACHE_API [\w\s\*]+?\b(acache_\w+)\(", text, flags=re.M)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("acache_store_kvcache", "acache_relocate_affix", "acache_anchor_topk", "acache_anchor_importance",
                 "acache_attention", "acache_paged_attention", "acache_rope_store", "acache_transfer_tokens"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from acache_b200 import _lib

    assert _lib.LIB_PATH.exists(), "build the library first: python -m acache_b200.build"
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in _declared():
        assert hasattr(lib, name), name
    assert sorted(_lib.EXPORTED_SYMBOLS) == _declared()
    assert _lib.load().acache_abi_version() >= 1
    assert _lib.load().acache_status_string(-1) == b"invalid argument"


def test_argument_validation_needs_no_gpu():
    from acache_b200 import _lib

    lib = _lib.load()
    # bad dtype / negative sizes are rejected before any CUDA call
    assert lib.acache_store_kvcache(None, 0, None, 0, None, None, None, 4, 16, 8, 99, None, None) == -1
    assert lib.acache_anchor_topk(None, -1, 4, 4, 1, 1, None, None, None) == -1
    assert lib.acache_anchor_topk(None, 0, 4, 4, 1, 1, None, None, None) == 0
    assert lib.acache_anchor_importance_scratch_bytes(33, 4, 100) == 2 * 4 * 100 * 4


def test_launch_plans_and_new_entry_points_validate_without_a_gpu():
    """Host-side arithmetic of the library: the K-slicing plan of the plain projections and the
    scratch size / argument checks of the batched influence score."""
    from acache_b200 import _lib

    lib = _lib.load()
    plan = lib.acache_linear_partials_splits
    assert plan(512, 12288, 4096) == 2      # block decode of 16 requests, feed-forward output: 32 tiles x 2 slices
    assert plan(256, 12288, 4096) == 4      # 8 requests: 16 tiles x 4 slices of 48 k blocks
    assert plan(512, 4096, 4096) == 1       # K too short for a slice of 48 k blocks
    assert plan(2304, 12288, 4096) == 1     # a refresh chunk has enough whole tiles
    assert plan(1024, 18944, 3584) == 1     # Dream block decode: 56 whole tiles
    assert plan(0, 128, 64) == 1 and plan(16, 128, 64) == 1
    assert lib.acache_linear_partials(None, 0, 4, 128, None, 64, 2, None, 17, 0, 0, None, None) == -1   # slice count
    assert lib.acache_linear_partials(None, 0, 0, 128, None, 64, 2, None, 2, 0, 0, None, None) == 0     # no rows
    assert lib.acache_anchor_importance_batched_scratch_bytes(3, 33, 4, 100) == 3 * 2 * 4 * 100 * 4
    assert lib.acache_anchor_importance_batched_scratch_bytes(0, 33, 4, 100) == 0
    args = [None, 0, None, None, 2, 4, 4, 3, 64, 2, None, 0, 10, None, None, None, 0, 0, 0, 0.125, None, 10, None, 0,
            None, None]
    assert lib.acache_anchor_importance_batched(*args) == -1          # heads not a multiple of KV heads
    args[7] = 4
    args[4] = 0
    assert lib.acache_anchor_importance_batched(*args) == 0           # no requests: nothing to do
    args[4] = 2
    assert lib.acache_anchor_importance_batched(*args) == -1          # null pointers
    args[21] = 9
    assert lib.acache_anchor_importance_batched(*args) == -1          # score rows shorter than the affix
