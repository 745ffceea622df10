"""Data-parallel serving: one engine replica per GPU, requests sharded round-robin, the
shared affix K/V computed once and broadcast to every replica.

The reference runs one process per GPU through ``accelerate`` and every process recomputes
the affix itself (reference: nano-vdllm/eval_llada.py:172-216, :314-320); it has no
collective.  Here the only exchange of the path is that broadcast (NCCL over NVLink on
GPUs; the same code runs over gloo for the host-side tests); nothing is exchanged per step.
"""
from __future__ import annotations

import random

import torch
import torch.distributed as dist


def shard_round_robin(items, rank: int, world_size: int):
    """Items ``rank, rank + world_size, ...`` (the order inside a shard is the arrival order)."""
    return list(items[rank::world_size])


def poisson_arrival_times(n: int, rate_per_s: float, seed: int = 0) -> list[float]:
    """Arrival times (seconds, ascending, first one at 0) of a Poisson process with the given
    rate: exponential inter-arrival gaps from a seeded generator."""
    rng = random.Random(seed)
    t, out = 0.0, []
    for i in range(n):
        if i:
            t += rng.expovariate(rate_per_s)
        out.append(t)
    return out


def broadcast_shared_affix(runner, affix_tokens, src: int = 0, group=None):
    """Rank ``src`` runs the affix forward and packs its K/V ``[2, layers, A, kv_heads, head_dim]``;
    every other rank receives the buffer and installs it in blocks ``0..ceil(A/Bk)-1`` of its own
    cache.  Returns the number of payload bytes."""
    rank = dist.get_rank(group)
    if rank == src:
        runner._precompute_shared_prefix(list(affix_tokens))
        packed = runner.export_shared_prefix_kv()
    else:
        _, hkv, D, layers = runner._arch()
        packed = torch.empty(2, layers, len(affix_tokens), hkv, D, dtype=runner.kv_cache.dtype, device=runner.device)
    dist.broadcast(packed, src=src, group=group)
    if rank != src:
        runner.load_shared_prefix_kv(list(affix_tokens), packed)
    return packed.numel() * packed.element_size()


def serve_sharded(runner, all_sequences, arrival_times=None, group=None):
    """Serves this rank's round-robin shard of ``all_sequences`` (optionally as a stream with
    per-request ``arrival_times``) and gathers ``(global index, generated tokens)`` on every rank.
    Returns ``(outputs in global order, total nfe over all ranks)``."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    mine = shard_round_robin(list(range(len(all_sequences))), rank, world)
    seqs = [all_sequences[i] for i in mine]
    times = None if arrival_times is None else [arrival_times[i] for i in mine]
    outs, nfe = runner.generate_with_acache(seqs, arrival_times=times) if seqs else ([], 0)
    gathered = [None] * world
    dist.all_gather_object(gathered, (mine, outs, nfe), group=group)
    result = [None] * len(all_sequences)
    total = 0
    for idx, o, n in gathered:
        total += n
        for i, tokens in zip(idx, o):
            result[i] = tokens
    return result, total
