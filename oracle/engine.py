"""Request-at-a-time CPU restatement of generation with affix-KV reuse.

Restates, for one request, what the reference engine does for every request of a
batch (requests only share the read-only affix K/V, so batching does not change
a request's tokens): reference nano-vdllm/model_runner.py:492-541 (affix forward
alone at positions 0..A-1, K cached post-RoPE), :640-845 (anchor-selection probe
and top-k), :2032-2277 (refresh at every new block, block decoding until no mask
is left), :56-66,2091-2118 (Dream's shifted logits and seed token); same
algorithm as the HF batch-1 path, reference llada/generate_ACache.py:311-629.
"""
import math

import torch

from .importance import relocate_keys
from .models import KVState, OracleModel
from .rope import rope_table
from .sampling import get_transfer_index
from .topk import anchor_topk


def compute_affix_kv(model: OracleModel, affix_tokens):
    """K/V of the affix run alone (reference: model_runner.py:492-541)."""
    A = len(affix_tokens)
    kv = KVState(model.spec, A, model.dtype)
    t = torch.tensor(affix_tokens, dtype=torch.long)
    pos = torch.arange(A)
    model.forward_rows(t, pos, kv, pos)
    return kv


def _relocation_tables(model: OracleModel, length):
    # LLaDA keeps fp32 tables, Dream casts them to the cache dtype
    # (reference: model_runner.py:258-271)
    dt = torch.float32 if model.spec.kind == "llada" else model.dtype
    return rope_table(length, model.spec.head_dim, model.spec.rope_theta, dt)


def _request_kv(model, affix_kv, total_len, affix_start):
    """Dense logical cache of a request with the shared affix relocated into
    [affix_start, affix_start + A) (key-side relocation semantics)."""
    A = affix_kv.k.shape[1]
    kv = KVState(model.spec, total_len, model.dtype)
    cos, sin = _relocation_tables(model, max(total_len, affix_start + 1))
    for l in range(model.spec.n_layers):
        k = affix_kv.k[l]
        if affix_start != 0:
            k = relocate_keys(k, cos, sin, affix_start)
        kv.k[l, affix_start : affix_start + A] = k
        kv.v[l, affix_start : affix_start + A] = affix_kv.v[l]
    return kv


def select_anchors(model, affix_kv, tokens, affix_start, affix_end, anchor_ratio, selection_mode="top", exact=False):
    """Returns (anchor logical positions, fp32 scores [A])."""
    A = affix_end - affix_start
    k = min(math.ceil(anchor_ratio * A), A)
    n = len(tokens)
    outside = torch.tensor([*range(affix_start), *range(affix_end, n)], dtype=torch.long)
    tok = torch.tensor(tokens, dtype=torch.long)
    kv = _request_kv(model, affix_kv, n, affix_start)
    acc = torch.zeros(A, dtype=torch.float32)
    probe = {"mask_rows": tok[outside] == model.spec.mask_id, "affix": slice(affix_start, affix_end), "acc": acc,
             "exact": exact}
    if k > 0:
        model.forward_rows(tok[outside], outside, kv, outside, probe=probe)
    idx = anchor_topk(acc[None], k, largest=(selection_mode != "bottom"))[0]
    return (idx + affix_start).tolist(), acc


def request_steps(model, affix_kv, tokens, affix_start, affix_end, generation_start, gen_length, block_length,
                  anchors, threshold=0.9, kv_out=None):
    """Generator over the forwards of one request, in order.  Yields
    ``(phase, block index, logits [block_length, vocab], block tokens after the commit)`` with
    phase 'refresh' (forward over anchors + own tokens, reference: model_runner.py:2091-2118) or
    'decode' (forward over the working block, reference: model_runner.py:2196-2271).  The
    logits are the ones unmasking sees (Dream's already shifted).  ``kv_out``: a list that
    receives the request's dense logical cache and the row set of the refresh, for callers
    that compare cache contents."""
    spec = model.spec
    n = len(tokens)
    x = torch.tensor(tokens, dtype=torch.long)
    kv = _request_kv(model, affix_kv, n, affix_start)
    anchors = sorted(anchors)
    rows = torch.tensor(sorted(set(anchors) | set(range(affix_start)) | set(range(affix_end, n))), dtype=torch.long)
    if kv_out is not None:
        kv_out.extend([kv, rows])
    row_of = {int(p): i for i, p in enumerate(rows.tolist())}
    for b in range(-(-gen_length // block_length)):
        s = generation_start + b * block_length
        e = s + block_length
        first = row_of[s]
        keep = torch.arange(first, first + block_length)
        if spec.kind == "dream":
            keep = torch.clamp(keep, min=1) - 1  # logits of the preceding row (reference: model_runner.py:63-66)
        logits = model.forward_rows(x[rows], rows, kv, rows, logits_rows=keep)
        blk = x[s:e].clone()
        if spec.kind == "dream":
            blk[0] = torch.argmax(logits[0])
        else:
            x0, ti = get_transfer_index(logits[None], (blk == spec.mask_id)[None], blk[None], threshold)
            blk = torch.where(ti[0], x0[0], blk)
        x[s:e] = blk
        yield "refresh", b, logits, x[s:e].clone()
        pos = torch.arange(s, e)
        while bool((x[s:e] == spec.mask_id).any()):
            logits = model.forward_rows(x[s:e], pos, kv, pos, logits_rows=torch.arange(block_length))
            if spec.kind == "dream":
                logits = torch.cat([logits[:1], logits[:-1]], dim=0)
            blk = x[s:e].clone()
            x0, ti = get_transfer_index(logits[None], (blk == spec.mask_id)[None], blk[None], threshold)
            x[s:e] = torch.where(ti[0], x0[0], blk)
            yield "decode", b, logits, x[s:e].clone()
    if kv_out is not None:
        kv_out.append(x.tolist())


def generate_request(model, affix_kv, tokens, affix_start, affix_end, generation_start, gen_length, block_length,
                     anchors, threshold=0.9, trace=None):
    """Denoise one request.  ``tokens`` already contains the mask span.
    Returns (tokens list, nfe)."""
    x = list(tokens)
    nfe = 0
    for phase, b, logits, blk in request_steps(model, affix_kv, tokens, affix_start, affix_end, generation_start,
                                               gen_length, block_length, anchors, threshold):
        nfe += 1
        if trace is not None:
            trace.append((phase, b, logits.clone()))
        s = generation_start + b * block_length
        x[s: s + block_length] = blk.tolist()
    return x, nfe


def generate_with_acache(model, requests, anchor_ratio, selection_mode="top", threshold=0.9, block_length=32):
    """requests: list of dicts {tokens (with masks), affix_start, affix_end,
    generation_start, gen_length}.  All share the same affix tokens.
    Returns (list of generated spans, total nfe, list of anchor lists)."""
    r0 = requests[0]
    affix_tokens = r0["tokens"][r0["affix_start"] : r0["affix_end"]]
    affix_kv = compute_affix_kv(model, affix_tokens)
    outs, anchors_all, nfe = [], [], 0
    for r in requests:
        anchors, _ = select_anchors(model, affix_kv, r["tokens"], r["affix_start"], r["affix_end"], anchor_ratio,
                                    selection_mode)
        toks, n = generate_request(model, affix_kv, r["tokens"], r["affix_start"], r["affix_end"],
                                   r["generation_start"], r["gen_length"], block_length, anchors, threshold)
        outs.append(toks[r["generation_start"] : r["generation_start"] + r["gen_length"]])
        anchors_all.append(anchors)
        nfe += n
    return outs, nfe, anchors_all


# ------------------------------------------------------------------------------------------
# dKV-Cache decoding, one request at a time (reference: nano-vdllm/model_runner.py:1724-2030).
def dkv_transfer_schedule(block_length, steps_per_block):
    base, rem = divmod(block_length, steps_per_block)
    return [base + (s < rem) for s in range(steps_per_block)]


def generate_request_dkv(model, tokens, generation_start, gen_length, block_length, steps, cache_interval,
                         affix_kv=None, affix_start=0, affix_end=0, anchors=None):
    """Denoise one request with delayed KV refresh.  ``affix_kv`` given: the shared affix is read
    from the cache and only the anchors and the request's own tokens are dynamic.  Temperature 0,
    low-confidence remasking (confidence in fp64).  Returns (tokens list, nfe)."""
    spec = model.spec
    mask_id, dream = spec.mask_id, spec.kind == "dream"
    n = len(tokens)
    x = list(tokens)
    if affix_kv is not None:
        kv = _request_kv(model, affix_kv, n, affix_start)
        dynamic = sorted(set(anchors) | set(range(affix_start)) | set(range(affix_end, n)))
    else:
        kv = KVState(spec, n, model.dtype)
        dynamic = list(range(n))
    dyn = set(dynamic)
    num_blocks = gen_length // block_length
    schedule = dkv_transfer_schedule(block_length, steps // num_blocks)
    generation_end = generation_start + gen_length
    nfe = 0
    for b in range(num_blocks):
        start = generation_start + b * block_length
        previous = delayed = None
        for step, quota in enumerate(schedule):
            if dream:
                refresh = step % cache_interval == 0
                pred = {(p - 1) % n for p, t in enumerate(x) if t == mask_id}
                q = set(dyn if refresh else dyn & pred)
                q |= {max(p - 1, 0) for p in range(start, start + block_length) if x[p] == mask_id}
                positions = sorted(q)
            else:
                refresh = step <= 1 or step % cache_interval == 0
                positions = list(dynamic) if refresh else list(delayed)
            masked = [p for p in range(start, start + block_length) if x[p] == mask_id]
            where = {p: i for i, p in enumerate(positions)}
            rows = torch.tensor([where[max(p - 1, 0) if dream else p] for p in masked], dtype=torch.long)
            pos_t = torch.tensor(positions, dtype=torch.long)
            write = torch.tensor([p if p in dyn else -1 for p in positions], dtype=torch.long)
            logits = model.forward_rows(torch.tensor([x[p] for p in positions], dtype=torch.long), pos_t, kv, write,
                                        logits_rows=rows)
            nfe += 1
            x0 = torch.argmax(logits, dim=-1)
            if quota:
                l64 = logits.to(torch.float64)
                conf = torch.gather(l64, -1, x0[:, None]).squeeze(-1) - torch.logsumexp(l64, dim=-1)
                for idx in torch.topk(conf, k=quota).indices.tolist():
                    x[masked[idx]] = int(x0[idx])
            unresolved = [p for p in range(start, generation_end) if x[p] == mask_id]
            delayed, previous = previous, unresolved
    return x, nfe


def generate_with_dkv(model, requests, block_length, steps, cache_interval, anchor_ratio=None, selection_mode="top"):
    """``anchor_ratio`` None: dKV-Cache alone (every request keeps a full cache of its own);
    otherwise dKV-Cache on top of affix reuse.  Returns (generated spans, total nfe)."""
    affix_kv = None
    if anchor_ratio is not None:
        r0 = requests[0]
        affix_kv = compute_affix_kv(model, r0["tokens"][r0["affix_start"]: r0["affix_end"]])
    outs, nfe = [], 0
    for r in requests:
        anchors = None
        if affix_kv is not None:
            anchors, _ = select_anchors(model, affix_kv, r["tokens"], r["affix_start"], r["affix_end"], anchor_ratio,
                                        selection_mode)
        toks, n = generate_request_dkv(model, r["tokens"], r["generation_start"], r["gen_length"], block_length, steps,
                                       cache_interval, affix_kv, r["affix_start"], r["affix_end"], anchors)
        outs.append(toks[r["generation_start"]: r["generation_start"] + r["gen_length"]])
        nfe += n
    return outs, nfe
