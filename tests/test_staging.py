"""Host-side packing of the step metadata (CPU): the one-copy staging buffer and its
fixed-layout variant that captured decode forwards read from."""
import numpy as np
import torch

from acache_b200.model_runner import _Staging, _StaticStaging


def _arrays(n_rows, read_len, T=4, with_shifts=True):
    rng = np.random.default_rng(n_rows * 1000 + read_len)
    a = dict(positions=rng.integers(0, 500, (n_rows, T)).astype(np.int64),
             cu_q=np.arange(0, (n_rows + 1) * T, T, dtype=np.int32),
             cu_k=np.arange(n_rows + 1, dtype=np.int32) * (read_len // n_rows),
             kv_seqlens=rng.integers(1, 99, n_rows).astype(np.int32),
             slots=rng.integers(0, 999, n_rows * T).astype(np.int32),
             read=rng.integers(-1, 999, read_len).astype(np.int32))
    if with_shifts:
        a["shifts"] = rng.integers(0, 50, n_rows).astype(np.int32)
    return a


def test_staging_round_trips_every_array():
    st = _Staging(torch.device("cpu"))
    arrays = _arrays(3, 30)
    dev = st.ship(**arrays)
    for k, a in arrays.items():
        assert dev[k].shape == a.shape and np.array_equal(dev[k].numpy(), a), k
        assert dev[k].data_ptr() % (8 if a.dtype == np.int64 else 4) == 0
    assert st.h2d_bytes >= sum(a.nbytes for a in arrays.values())


def test_static_staging_keeps_addresses_and_checks_capacity():
    counter = _Staging(torch.device("cpu"))
    first = _arrays(3, 30)
    caps = {k: (a.dtype, {"read": 64}.get(k, a.size)) for k, a in first.items()}
    st = _StaticStaging(torch.device("cpu"), caps, counter)
    dev1 = st.ship(**first)
    where = {k: v.data_ptr() for k, v in dev1.items()}
    second = _arrays(3, 57)                       # another request mix: longer read map, same rows
    assert st.fits(**second)
    dev2 = st.ship(**second)
    for k, a in second.items():
        assert dev2[k].data_ptr() == where[k], k      # a captured kernel keeps reading the right place
        assert np.array_equal(dev2[k].numpy(), a), k
        assert dev2[k].data_ptr() % 8 == 0 or a.dtype != np.int64
    assert counter.h2d_bytes == sum(a.nbytes for a in first.values()) + sum(a.nbytes for a in second.values())
    assert not st.fits(**_arrays(3, 65))              # read map longer than the capacity
    assert not st.fits(**_arrays(3, 30, with_shifts=False))   # another set of arrays = another layout
    assert not st.fits(**_arrays(4, 40))              # more rows


def test_decode_graph_cache_is_bounded():
    """The set of captured decode forwards is bounded by count and by the bytes of logits they
    keep alive; the least recently used ones go first and the newest always stays."""
    from types import SimpleNamespace

    import torch

    from acache_b200.model_runner import ModelRunner

    r = ModelRunner.__new__(ModelRunner)
    r.config = SimpleNamespace(block_length=32, hf_config=SimpleNamespace(embedding_size=126464, vocab_size=126464))
    r.kv_cache = torch.empty(1, dtype=torch.bfloat16)
    r._graph_with_pending_timers = r._decode_graph = None
    graph = lambda rows: SimpleNamespace(tokens=torch.empty(rows, 32), graph=object(), logits=object())
    graphs = {}
    for rows in range(1, 13):            # small graphs: the count bound applies
        graphs[rows] = graph(rows)
        r._evict_decode_graphs(graphs, keep=rows)
    assert list(graphs) == list(range(5, 13))
    big = {}
    for rows in (64, 63, 62, 61, 60):    # 0.5 GB of logits each: the byte bound applies
        big[rows] = graph(rows)
        r._evict_decode_graphs(big, keep=rows)
    assert list(big) == [63, 62, 61, 60]
    lone = {64: graph(6400)}             # one oversized graph is still kept (it is the one in use)
    r._evict_decode_graphs(lone, keep=64)
    assert list(lone) == [64]
