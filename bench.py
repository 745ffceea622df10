"""Benchmark of generation with affix-KV reuse.

Default workload (per GPU; weak scaling): LLaDA-8B architecture, random-init bf16, prefix
placement, a shared 800-token affix plus 16 ragged requests of uniform [64, 256] tokens,
gen/steps/block = 256/256/32, confidence threshold 0.9, anchor_ratio 0.2.  Synthetic token
ids, fixed seeds.  One step = one ``generate_with_acache`` call over the batch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|cfg3|cfg4|cfg5]

``--workload`` selects one of the other served configurations (``cfg2`` is the default and the
benchmark): ``cfg3`` Dream-7B architecture, batch 32, a 600-token affix between a head and a tail of
32-128 tokens; ``cfg4`` LLaDA-8B, batch 64, an 8192-token affix behind contexts of 1024-4096 tokens,
gen/steps/block 8/8/8, anchor ratio 0.1; ``cfg5`` 1024 requests of the default shape arriving as a
Poisson stream, sharded round-robin over the replicas, at most 64 running per GPU (strong scaling).

Prints ONE JSON line on rank 0.  ``value`` is generated tok/s over all GPUs timed with CUDA
events around K steps (affix K/V resident from the warm-up, request objects prebuilt);
``e2e`` is the same metric by wall clock from raw host token lists to host token lists
(request construction, every host-to-device metadata copy and device-to-host token read
included).  ``roofline`` is the dominant kernel of this package in the timed region, timed
live with CUDA events.  ``--impl reference`` times the CPU restatement of the reference's
path on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

AFFIX_LEN, BATCH, GEN, BLOCK, THRESHOLD, RATIO = 800, 16, 256, 32, 0.9, 0.2
REQ_LO, REQ_HI = 64, 256
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch at the default
# workload's shape, from a profiler capture of that shape (not measured by this program)
PROFILED_DECODE_ATTENTION_DRAM_BYTES = 170.3e6
WORKLOAD = ("LLaDA-8B arch random-init bf16, prefix affix 800 tok + 16 ragged requests U[64,256], "
            "gen/steps/block 256/256/32, thr 0.9, anchor_ratio 0.2")

# model family, affix placement, affix length, range of the request's own spans, requests per
# GPU, generated tokens, block length, anchor ratio, refresh chunk
WORKLOADS = {
    "cfg2": dict(model="llada", placement="prefix", affix=800, own=(64, 256), batch=16, gen=256, block=32, ratio=0.2,
                 chunk=4, text=WORKLOAD, metric="generated tok/s/box LLaDA-8B-arch bs16 affix reuse"),
    "cfg3": dict(model="dream", placement="infix", affix=600, own=(32, 128), batch=32, gen=256, block=32, ratio=0.2,
                 chunk=4, text=("Dream-7B arch random-init bf16, 600-token affix between a head and a tail of U[32,128] "
                                "tokens, batch 32, gen/steps/block 256/256/32, thr 0.9, anchor_ratio 0.2"),
                 metric="generated tok/s/box Dream-7B-arch bs32 infix affix reuse"),
    "cfg4": dict(model="llada", placement="suffix", affix=8192, own=(1024, 4096), batch=64, gen=8, block=8, ratio=0.1,
                 chunk=4, text=("LLaDA-8B arch random-init bf16, 8192-token affix behind contexts of U[1024,4096] tokens, "
                                "batch 64, gen/steps/block 8/8/8, thr 0.9, anchor_ratio 0.1, paged KV block 256"),
                 metric="generated tok/s/box LLaDA-8B-arch bs64 long suffix affix reuse"),
    "cfg5": dict(model="llada", placement="prefix", affix=800, own=(64, 256), batch=64, gen=256, block=32, ratio=0.2,
                 chunk=4, total=1024, rate_per_gpu=8.0,
                 text=("LLaDA-8B arch random-init bf16, prefix affix 800 tok, 1024 ragged requests U[64,256] as a Poisson "
                       "stream, round-robin over the replicas, at most 64 running per GPU, gen/steps/block 256/256/32, "
                       "thr 0.9, anchor_ratio 0.2"),
                 metric="generated tok/s/box LLaDA-8B-arch request stream affix reuse"),
}


def make_requests(seed: int, vocab: int, mask_id: int, n: int, affix_len: int = AFFIX_LEN, own=(REQ_LO, REQ_HI),
                  spans: int = 1):
    """Raw host token lists: (affix tokens, list of the requests' own spans).  ``spans`` = 2
    gives (head, tail) pairs for an affix inside the prompt."""
    rng = random.Random(seed)

    def tok():
        t = rng.randrange(1, vocab - 1)
        return t if t != mask_id else t - 1

    affix = [tok() for _ in range(affix_len)]
    if spans == 1:
        return affix, [[tok() for _ in range(rng.randint(*own))] for _ in range(n)]
    return affix, [tuple([tok() for _ in range(rng.randint(*own))] for _ in range(spans)) for _ in range(n)]


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


# ----------------------------------------------------------------------------- CPU arm
_CPU_MODELS: dict = {}


def cpu_reference_sample(layers: int = 2, n_requests: int = 4, gen_length: int = BLOCK, seed: int = 0):
    """The CPU restatement of the reference path (oracle/) on a bounded sample of the default
    workload: the LLaDA-8B architecture truncated to ``layers`` layers in fp32, the 800-token
    affix, ``n_requests`` requests, ``gen_length`` generated tokens each (one block).  Time is
    extrapolated linearly in the parameter count to 32 layers.  Returns a dict."""
    import torch

    from oracle.engine import compute_affix_kv, generate_request, select_anchors
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    # a launcher for several ranks pins every process to one OpenMP thread; this arm runs alone
    # on rank 0 and may use the whole host
    torch.set_num_threads(max(os.cpu_count() or 1, 1))
    full_layers = 32
    if layers not in _CPU_MODELS:   # built once per process: drawing 1.4 G random weights takes longer than a sample
        arch = ArchSpec("llada", n_layers=layers, d_model=4096, n_heads=32, n_kv_heads=32, ffn=12288, vocab=126464,
                        rope_theta=500000.0, rms_eps=1e-5, act="silu", mask_id=126336)
        _CPU_MODELS[layers] = OracleModel(arch, random_state_dict(arch, seed=0, std=0.02), torch.float32)
    model = _CPU_MODELS[layers]
    arch = model.spec
    affix, tails = make_requests(seed, arch.vocab, arch.mask_id, n_requests)
    with torch.inference_mode():
        affix_kv = compute_affix_kv(model, affix)  # resident affix, as in the GPU arm's steady state
        t0 = time.perf_counter()
        nfe = 0
        for tail in tails:
            tokens = affix + tail + [arch.mask_id] * gen_length
            anchors, _ = select_anchors(model, affix_kv, tokens, 0, len(affix), RATIO)
            _, n = generate_request(model, affix_kv, tokens, 0, len(affix), len(affix) + len(tail), gen_length, BLOCK,
                                    anchors, THRESHOLD)
            nfe += n
        dt = time.perf_counter() - t0
    per_layer = 4 * 4096 * 4096 + 3 * 4096 * 12288
    head = 4096 * 126464
    scale = (full_layers * per_layer + head) / (layers * per_layer + head)
    tok_s_sample = n_requests * gen_length / dt
    return dict(value=tok_s_sample / scale, unit="tok/s", cores=torch.get_num_threads(), kind="port", extrapolated=True,
                sample=(f"{n_requests} request(s) x {gen_length} generated tokens (1 block) of the workload, affix K/V "
                        f"resident, architecture truncated to {layers} of {full_layers} layers in fp32 on CPU: "
                        f"{dt:.1f} s, {nfe} forwards; tok/s extrapolated by the parameter-count ratio {scale:.2f} "
                        f"(attention, probe and sampling cost do not scale with the parameter count, so this is an "
                        f"indication, not a like-for-like measurement)"),
                seconds=dt)


def run_reference(args):
    """The CPU restatement of the reference path on the host cores.  However many steps are asked
    for, the bounded sample (about 10 s of CPU work) is timed at most three times, so the arm ends
    within two minutes at any N; under a multi-rank launcher rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    steps = max(args.steps, 1)
    timed = min(steps, 3)
    warm = 1 if args.warmup > 0 else 0
    vals, t_begin = [], time.perf_counter()
    for i in range(warm + timed):
        base = cpu_reference_sample(seed=i)
        if i >= warm:
            vals.append(base)
        if time.perf_counter() - t_begin > 75.0 and vals:
            break
    value = sum(v["value"] for v in vals) / len(vals)
    secs = sum(v["seconds"] for v in vals) / len(vals)
    base = dict(vals[-1], value=value)
    base.pop("seconds")
    base["sample"] += f"; the sample was timed {len(vals)} time(s) after {warm} warm-up pass(es), whatever --steps says"
    line = dict(impl="reference", metric=wl["metric"], value=value, unit="tok/s",
                n_gpus=args.gpus, steps=steps, warmup=args.warmup, ms_per_step=secs * 1e3,
                higher_is_better=True, scaling="strong" if args.workload == "cfg5" else "weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config={"workload": wl["text"], "batch_per_gpu": wl["batch"], "layers": 32, "parallelism": f"dp{args.gpus}",
                        "l2": "weights (16 GB) and K/V re-read every step exceed the 126 MB L2"},
                note=("CPU restatement of the reference path (oracle/) on the host cores, on a bounded sample of the "
                      "LLaDA-8B prefix workload; see cpu_baseline.sample"),
                cpu_baseline=base, e2e={"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                gpu_launches=0)
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def build_model(wl, dev, layers=0):
    """Random-init bf16 model of the workload's architecture; returns (hf config, model, kind)."""
    import torch

    if wl["model"] == "llada":
        from acache_b200.model.configuration import LLaDAConfig
        from acache_b200.model.modeling_llada import LLaDAModelLM

        hf = LLaDAConfig.llada_8b()
        if layers:
            hf.n_layers = layers
        model = LLaDAModelLM(hf, device=dev, dtype=torch.bfloat16, init_params=True, seed=1234).eval()
        head = model.model.transformer["ff_out"].weight
    else:
        from acache_b200.model.configuration import DreamConfig
        from acache_b200.model.modeling_dream import DreamModel

        hf = DreamConfig.dream_7b()
        if layers:
            hf.num_hidden_layers = layers
        model = DreamModel(hf, device=dev, dtype=torch.bfloat16, init_params=True, seed=1234).eval()
        head = model.lm_head.weight
    with torch.no_grad():  # the mask token must never be the arg-max (see oracle/models.py:random_state_dict)
        head[hf.mask_token_id] = head[0]
    model.fuse_projections()
    return hf, model


def build_sequences(wl, hf, affix, spans):
    """Request objects of the workload's placement from raw host token lists."""
    from acache_b200.sequence import Sequence

    A, G, T, mask = len(affix), wl["gen"], wl["block"], hf.mask_token_id
    seqs = []
    for sp in spans:
        if wl["placement"] == "prefix":
            seqs.append(Sequence(affix + sp, block_length=T, gen_length=G, cache_block_size=256, mask_id=mask,
                                 prompt_affix_len=A))
        elif wl["placement"] == "infix":
            head, tail = sp
            seqs.append(Sequence(head + affix + tail, block_length=T, gen_length=G, cache_block_size=256, mask_id=mask,
                                 prompt_affix_start=len(head), prompt_affix_end=len(head) + A))
        else:   # context, generation span, then the affix
            seqs.append(Sequence(sp + [mask] * G + affix, block_length=T, gen_length=G, cache_block_size=256,
                                 mask_id=mask, prompt_affix_start=len(sp) + G, prompt_affix_end=len(sp) + G + A,
                                 generation_start=len(sp)))
    return seqs


def cache_blocks(wl, batch, dev):
    """Blocks for the shared affix plus ``batch`` requests of the largest size, bounded by what
    the device has free (the engine admits by free blocks, so fewer blocks only lower the
    number of requests in flight)."""
    import torch

    A, (lo, hi), G = wl["affix"], wl["own"], wl["gen"]
    own_max = hi * (2 if wl["placement"] == "infix" else 1)
    anchors = -(-int(wl["ratio"] * A * 1000) // 1000)
    per_request = -(-(anchors + own_max + G) // 256)
    want = -(-A // 256) * (2 if wl["placement"] != "prefix" else 1) + per_request * batch + 4
    layers, hkv = (32, 32) if wl["model"] == "llada" else (28, 4)
    block_bytes = 2 * layers * 256 * hkv * 128 * 2
    free, _ = torch.cuda.mem_get_info(dev)
    fit = int((free - (12 << 30)) // block_bytes)      # leave room for activations, logits and graphs
    return max(min(want, fit), -(-A // 256) + per_request + 1)


def subpath_timings(peaks):
    """Kernels of the path that the default workload exercises little or not at all, timed alone
    at the shapes of the other configurations: CUDA events, L2 flushed between launches, 50
    launches each.  Bandwidth-bound ones against the measured copy bandwidth, the refresh
    attention against the measured burst bf16 rate (it is timed in isolation)."""
    import torch

    from acache_b200 import microbench as mb

    cases = [
        ("relocate_affix_cfg3", "relocate_dream_infix", "Dream-7B, 600-token affix, 32 requests, all 28 layers, one launch"),
        ("relocate_affix_cfg4", "relocate_llada_8192_1req", "LLaDA-8B, 8192-token affix, 1 request, 8 of 32 layers per launch"),
        ("relocate_affix_cfg1", "relocate_cfg1_fp32", "2 layers, 8 KV heads, fp32, 512-token affix, 4 requests"),
        ("attention_refresh_cfg2", "attention_refresh_llada", "4 requests x 576 query rows, kv 1120-1312, 32 heads"),
        ("rope_store_decode", "rope_store_decode_llada", "512 rows, 32 + 32 heads"),
        ("rope_store_refresh", "rope_store_refresh_llada", "2304 rows, 32 + 32 heads"),
        ("transfer_tokens", "transfer_tokens_llada", "512 rows x 126464 logits"),
    ]
    flush = mb._flush_buffer()
    out = {}
    for name, case, shape in cases:
        build, bound = mb.CASES[case]
        fn, work = build()
        sec = mb._time(fn, 50, flush)
        if bound == "tensor":
            achieved, peak, unit = work["flops"] / sec / 1e12, peaks["bf16_tflops"], "TFLOP/s"
        else:
            achieved, peak, unit = work["bytes"] / sec / 1e9, peaks["hbm_gbs"], "GB/s"
        out[name] = dict(shape=shape, us=sec * 1e6, bound=bound, achieved=achieved, peak=peak, unit=unit,
                         frac=achieved / peak, launches=50)
        del fn
        torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from acache_b200 import _lib
    from acache_b200.config import Config
    from acache_b200.model_runner import ModelRunner

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    if args.projections != "default":
        from acache_b200.model import modeling_common

        modeling_common.set_own_gemm(args.projections == "own")
        if args.projections not in ("own", "library"):
            on = set(args.projections.split(","))
            assert on <= {"qkv", "gate_up", "dense", "dense_sliced", "head"}, on
            modeling_common.OWN_QKV, modeling_common.OWN_GATE_UP = "qkv" in on, "gate_up" in on
            modeling_common.OWN_DENSE = True if "dense" in on else ("sliced" if "dense_sliced" in on else False)
            modeling_common.OWN_HEAD = "head" in on

    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl["batch"] = args.batch
    batch, G, T, A = wl["batch"], wl["gen"], wl["block"], wl["affix"]
    hf, model = build_model(wl, dev, args.layers)
    n_layers = getattr(hf, "n_layers", getattr(hf, "num_hidden_layers", 0))
    cfg = Config(hf_config=hf, mask_id=hf.mask_token_id, recompute_batch_size=wl["chunk"], max_num_seqs=batch,
                 gen_length=G, block_length=T, threshold=THRESHOLD, cache_block_size=256,
                 num_kvcache_blocks=cache_blocks(wl, batch, dev), enable_acache=True, anchor_ratio=wl["ratio"],
                 selection_mode="top", model_type=wl["model"], profile_timing=True)
    if args.group_shared_span >= 0:
        cfg.group_shared_span = bool(args.group_shared_span)
    if args.mode == "dkv_acache":      # second serving mode of the engine: delayed KV refresh on top of affix reuse
        cfg.enable_dkv_cache, cfg.dkv_steps, cfg.dkv_cache_interval = True, G, 8
    if args.mode == "dual_cache":      # the no-reuse baseline: every request keeps its own copy of the affix
        cfg.enable_acache = False
        cfg.num_kvcache_blocks = batch * -(-(A + 2 * wl["own"][1] + G) // 256) + 4
    runner = ModelRunner(model, cfg)
    generate = {"acache": runner.generate_with_acache, "dkv_acache": runner.generate_with_dkv_acache,
                "dual_cache": runner.generate_with_dual_cache}[args.mode]
    n_spans = 2 if wl["placement"] == "infix" else 1

    def host_inputs(step, n=batch):
        # every rank (replica) serves its own shard of requests; the affix is common
        affix, _ = make_requests(0, hf.vocab_size, hf.mask_token_id, 0, A)
        _, spans = make_requests(1000 + step * world + rank, hf.vocab_size, hf.mask_token_id, n, A, wl["own"], n_spans)
        return affix, spans

    def build(affix, spans):
        return build_sequences(wl, hf, affix, spans)

    # shared affix: computed on rank 0, broadcast to the other replicas over NCCL
    affix, _ = host_inputs(0, 0)
    bcast_ms = bcast_bytes = None
    if world > 1:
        nh, hkv, D, L = runner._arch()
        if rank == 0:
            runner._precompute_shared_prefix(affix)
            packed = runner.export_shared_prefix_kv()
        else:
            packed = torch.empty(2, L, len(affix), hkv, D, dtype=torch.bfloat16, device=dev)
        dist.broadcast(torch.zeros(1, device=dev), src=0)     # sets the communicator up outside the timed copy
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(packed, src=0)
        e1.record()
        torch.cuda.synchronize()
        bcast_ms, bcast_bytes = e0.elapsed_time(e1), packed.numel() * packed.element_size()
        if rank != 0:
            runner.load_shared_prefix_kv(affix, packed)
        del packed

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if args.workload == "cfg5":
        return run_stream(args, wl, hf, runner, rank, world, dev, sync_all, bcast_ms, bcast_bytes)

    _lib.enable_kernel_timers(True)   # on during warm-up too: graphs captured there carry their timing events
    for w in range(args.warmup):
        a, t = host_inputs(10_000 + w)
        generate(build(a, t))

    # ---- device-timed region: K steps, requests prebuilt
    prebuilt = [build(*host_inputs(s)) for s in range(args.steps)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _lib.enable_kernel_timers(True)   # starts the accumulation over
    launches0 = _lib.LAUNCHES
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    nfe = 0
    recompute_ms, recompute_calls = 0.0, 0
    sections = {}
    for seqs in prebuilt:
        outs, n = generate(seqs)
        nfe += n
        recompute_ms += runner.last_timing.get("cache_forward", 0.0) * 1e3
        recompute_calls += runner.last_timing.get("cache_forward_calls", 0)
        for k, v in runner.last_timing.items():
            if isinstance(v, float) and not k.startswith("kv_cache"):
                sections[k] = sections.get(k, 0.0) + v * 1e3 / args.steps
        assert all(o is not None and len(o) == G for o in outs)
    e1.record()
    sync_all()
    dev_ms = e0.elapsed_time(e1)
    launches = _lib.LAUNCHES - launches0
    timers = _lib.kernel_timers()
    _lib.enable_kernel_timers(False)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end-to-end region: raw host lists in, host lists out, wall clock
    h2d0, d2h0 = runner._staging.h2d_bytes, runner.d2h_bytes
    sync_all()
    t0 = time.perf_counter()
    for s in range(args.steps):
        a, t = host_inputs(5_000 + s)
        outs, _ = generate(build(a, t))
        assert all(isinstance(o, list) and len(o) == G for o in outs)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = (runner._staging.h2d_bytes - h2d0) / args.steps
    d2h = (runner.d2h_bytes - d2h0) / args.steps

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    counts = torch.tensor([float(launches), h2d, d2h], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    dev_ms, e2e_ms = times.tolist()
    launches, h2d, d2h = int(counts[0].item()), counts[1].item(), counts[2].item()
    tokens = args.steps * batch * G * world

    if rank == 0:
        peaks = measured_peaks()
        roof = None
        if timers:
            name = max(timers, key=lambda k: timers[k][0])
            ms, n, work = timers[name]
            if name == "attention_decode":
                achieved = work / (ms * 1e-3) / 1e9
                roof = dict(kernel=name, bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                            frac=achieved / peaks["hbm_gbs"], traffic=None, launches=n, avg_us=ms * 1e3 / n,
                            algorithmic_bytes_per_launch=work / n, peak_source=peaks["source"])
                if args.workload == "cfg2" and batch == BATCH:
                    # not measured here: DRAM bytes of one launch from a profiler capture of this shape; they
                    # are below the algorithmic bytes because L2 serves the shared affix after its first reader
                    dram = PROFILED_DECODE_ATTENTION_DRAM_BYTES
                    roof["traffic_profile"] = dict(bytes=dram, source="ncu capture of the same shape",
                                                   frac_of_peak_on_these_bytes=dram / (ms * 1e-3 / n) / 1e9 / peaks["hbm_gbs"])
            else:
                achieved = work / (ms * 1e-3) / 1e12
                roof = dict(kernel=name, bound="tensor", achieved=achieved, peak=peaks["bf16_tflops_sustained"],
                            unit="TFLOP/s", frac=achieved / peaks["bf16_tflops_sustained"], traffic=None, launches=n,
                            avg_us=ms * 1e3 / n, peak_source=peaks["source"])
            roof["share_of_step"] = ms / dev_ms
            roof["other_timed"] = {k: dict(ms=v[0], launches=v[1]) for k, v in timers.items() if k != name}
        cpu = subpaths = None
        if world == 1 and args.mode == "acache" and args.workload == "cfg2":
            if not args.no_subpaths:
                del prebuilt
                subpaths = subpath_timings(peaks)
            if not args.no_cpu_baseline:
                cpu = cpu_reference_sample()
                cpu.pop("seconds")
        metric = wl["metric"]
        workload = wl["text"]
        if args.mode != "acache":   # not the benchmark: another serving mode of the engine on the same requests
            metric += {"dkv_acache": " + dKV-Cache decoding", "dual_cache": " OFF (no-reuse baseline)"}[args.mode]
            workload += {"dkv_acache": ", dKV steps = gen length, cache interval 8",
                         "dual_cache": ", every request recomputes the affix"}[args.mode]
        line = dict(
            metric=metric, value=tokens / (dev_ms * 1e-3), unit="tok/s",
            n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
            config={"workload": workload, "batch_per_gpu": batch, "layers": n_layers, "parallelism": f"dp{world}",
                    "kv_cache_blocks": cfg.num_kvcache_blocks, "projections": args.projections,
                    "l2": "weights (15-16 GB) and K/V re-read every step exceed the 126 MB L2"},
            clocks=clocks,
            e2e={"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            gpu_launches=launches, roofline=roof, cpu_baseline=cpu,
            anchor_recompute_ms=recompute_ms / max(recompute_calls, 1), nfe_per_step=nfe / args.steps,
            affix_broadcast_ms=bcast_ms,
            affix_broadcast_gbs=(bcast_bytes / (bcast_ms * 1e-3) / 1e9) if bcast_ms else None,
            sections_ms_per_step={k: round(v, 2) for k, v in sections.items()}, subpaths=subpaths)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_stream(args, wl, hf, runner, rank, world, dev, sync_all, bcast_ms, bcast_bytes):
    """cfg5: ``total`` requests arrive as one Poisson stream (rate = 8 requests per second per
    replica, so that the replicas stay saturated), request i goes to replica i mod N with its
    own arrival time, every replica batches continuously up to 64 running requests.  One step =
    one pass over the whole stream; the time is the wall clock from the first arrival to the last
    completion (arrivals are wall-clock events), max over ranks.  Strong scaling: the stream is
    the same at every N."""
    import torch
    import torch.distributed as dist

    from acache_b200 import _lib
    from acache_b200.dp import poisson_arrival_times, shard_round_robin

    total, G = wl["total"], wl["gen"]
    rate = wl["rate_per_gpu"] * world
    affix, _ = make_requests(0, hf.vocab_size, hf.mask_token_id, 0, wl["affix"])

    def shard(step):
        _, spans = make_requests(2000 + step, hf.vocab_size, hf.mask_token_id, total, wl["affix"], wl["own"])
        times = poisson_arrival_times(total, rate, seed=step)
        mine = shard_round_robin(list(range(total)), rank, world)
        return build_sequences(wl, hf, affix, [spans[i] for i in mine]), [times[i] for i in mine]

    for w in range(min(args.warmup, 1)):     # one short pass warms the kernels and captures the decode graphs
        seqs, _ = shard(100 + w)
        runner.generate_with_acache(seqs[: 2 * wl["batch"]])
    steps = max(args.steps, 1)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES
    h2d0, d2h0 = runner._staging.h2d_bytes, runner.d2h_bytes
    wall, lat, nfe = 0.0, [], 0
    for s in range(steps):
        seqs, times = shard(s)
        sync_all()
        t0 = time.perf_counter()
        outs, n = runner.generate_with_acache(seqs, arrival_times=times)
        torch.cuda.synchronize()
        wall += time.perf_counter() - t0
        nfe += n
        assert all(o is not None and len(o) == G for o in outs)
        lat += [c - a for c, a in zip(runner.last_completion_times, times)]
    clocks = sampler.stop() if rank == 0 else None
    stats = torch.tensor([wall * 1e3], dtype=torch.float64, device=dev)
    counts = torch.tensor([float(_lib.LAUNCHES - launches0), (runner._staging.h2d_bytes - h2d0) / steps,
                           (runner.d2h_bytes - d2h0) / steps, float(nfe)], dtype=torch.float64, device=dev)
    lat_t = torch.tensor(lat, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
        sizes = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([lat_t.numel()], dtype=torch.int64, device=dev))
        pad = int(max(x.item() for x in sizes))
        buf = torch.full((pad,), float("nan"), dtype=torch.float64, device=dev)
        buf[: lat_t.numel()] = lat_t
        gathered = [torch.empty_like(buf) for _ in range(world)]
        dist.all_gather(gathered, buf)
        lat_t = torch.cat(gathered)
        lat_t = lat_t[~torch.isnan(lat_t)]
    if rank == 0:
        wall_ms = stats[0].item()
        tok_s = steps * total * G / (wall_ms * 1e-3)
        q = torch.quantile(lat_t, torch.tensor([0.5, 0.99], dtype=torch.float64, device=dev)).tolist()
        line = dict(
            metric=wl["metric"], value=tok_s, unit="tok/s", n_gpus=world, steps=steps, warmup=min(args.warmup, 1),
            ms_per_step=wall_ms / steps, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16",
            data="synthetic",
            config={"workload": wl["text"], "requests": total, "max_running_per_gpu": wl["batch"],
                    "arrival_rate_per_s": rate, "layers": getattr(hf, "n_layers", 0), "parallelism": f"dp{world}",
                    "timing": "wall clock from the first arrival to the last completion, max over ranks",
                    "l2": "weights (16 GB) and K/V re-read every step exceed the 126 MB L2"},
            clocks=clocks,
            e2e={"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": counts[1].item(),
                 "d2h_bytes_per_step": counts[2].item()},
            gpu_launches=int(counts[0].item()), roofline=None, cpu_baseline=None,
            completion_latency_s={"p50": q[0], "p99": q[1]}, nfe_per_step=counts[3].item() / steps,
            affix_broadcast_ms=bcast_ms,
            affix_broadcast_gbs=(bcast_bytes / (bcast_ms * 1e-3) / 1e9) if bcast_ms else None)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS),
                    help="cfg2 = the benchmark (default); the other served configurations")
    ap.add_argument("--batch", type=int, default=0, help="requests per GPU (default: the workload's)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the architecture")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-subpaths", action="store_true")
    ap.add_argument("--projections", default="default",
                    help="debug only: 'own' / 'library' = every projection on this package's GEMM kernels / on the "
                         "library GEMM; or a comma list out of qkv,gate_up,dense,dense_sliced,head naming the ones "
                         "on this package's kernels (dense_sliced: the plain projections only where their K range "
                         "is cut into slices; the default is qkv,gate_up,dense_sliced,head)")
    ap.add_argument("--group-shared-span", type=int, default=-1, choices=[-1, 0, 1],
                    help="block-decode attention serves two requests of a KV head per CTA (-1: the engine's default)")
    ap.add_argument("--mode", default="acache", choices=["acache", "dkv_acache", "dual_cache"],
                    help="acache = the benchmark; the other serving modes of the engine on the same workload")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
