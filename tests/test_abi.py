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
