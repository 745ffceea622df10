"""Host-side logic of data-parallel serving on CPU: two gloo ranks, a stand-in engine.
(The engine itself needs a GPU; the sharding, the affix broadcast and the result gather do not.)"""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from acache_b200.dp import broadcast_shared_affix, poisson_arrival_times, serve_sharded, shard_round_robin


class FakeRunner:
    """Stores the affix K/V like the engine does and 'generates' a function of the request."""

    def __init__(self, layers=2, hkv=2, D=4):
        self.device = torch.device("cpu")
        self.kv_cache = torch.zeros(2, layers, 4, 8, hkv, D)
        self._layers, self._hkv, self._D = layers, hkv, D
        self.installed = None
        self.computed = False

    def _arch(self):
        return self._hkv, self._hkv, self._D, self._layers

    def _precompute_shared_prefix(self, tokens):
        self.computed = True
        n = len(tokens)
        base = torch.tensor(tokens, dtype=torch.float32).view(1, 1, n, 1, 1)
        self._packed = base.expand(2, self._layers, n, self._hkv, self._D).contiguous() + torch.arange(2).view(2, 1, 1, 1, 1)

    def export_shared_prefix_kv(self):
        return self._packed

    def load_shared_prefix_kv(self, tokens, packed):
        self.installed = (list(tokens), packed.clone())

    def generate_with_acache(self, seqs, arrival_times=None):
        assert arrival_times is None or len(arrival_times) == len(seqs)
        return [[s * 10, s * 10 + 1] for s in seqs], 3 * len(seqs)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        runner = FakeRunner()
        affix = [5, 6, 7]
        nbytes = broadcast_shared_affix(runner, affix, src=0)
        assert nbytes == 2 * 2 * 3 * 2 * 4 * 4
        if rank == 0:
            assert runner.computed and runner.installed is None
        else:
            assert not runner.computed
            toks, packed = runner.installed
            assert toks == affix and packed[0, 0, :, 0, 0].tolist() == [5.0, 6.0, 7.0] and packed[1, 1, 2, 1, 3] == 8.0
        requests = list(range(7))
        times = poisson_arrival_times(7, rate_per_s=50.0, seed=1)
        outs, nfe = serve_sharded(runner, requests, times)
        assert outs == [[r * 10, r * 10 + 1] for r in requests] and nfe == 21
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_two_rank_affix_broadcast_and_sharded_serving():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(0) and ret.get(1)


def test_round_robin_and_poisson_helpers():
    assert shard_round_robin(list(range(10)), 1, 4) == [1, 5, 9]
    t = poisson_arrival_times(100, 10.0, seed=3)
    assert t[0] == 0.0 and t == sorted(t) and len(t) == 100
    assert 5.0 < t[-1] < 20.0  # about n / rate
    assert t == poisson_arrival_times(100, 10.0, seed=3)
