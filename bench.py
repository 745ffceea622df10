"""Benchmark of generation with affix-KV reuse.

Workload (per GPU; weak scaling): LLaDA-8B architecture, random-init bf16, prefix
placement, a shared 800-token affix plus 16 ragged requests of uniform [64, 256] tokens,
gen/steps/block = 256/256/32, confidence threshold 0.9, anchor_ratio 0.2.  Synthetic token
ids, fixed seeds.  One step = one ``generate_with_acache`` call over the batch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

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
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch at this workload's
# shape (profiler capture summarised in profiles/attention_tc_decode_llada.md)
NCU_DECODE_ATTENTION_DRAM_BYTES = 171.0e6
WORKLOAD = ("LLaDA-8B arch random-init bf16, prefix affix 800 tok + 16 ragged requests U[64,256], "
            "gen/steps/block 256/256/32, thr 0.9, anchor_ratio 0.2")


def make_requests(seed: int, vocab: int, mask_id: int, n: int, affix_len: int = AFFIX_LEN):
    """Raw host token lists: (affix tokens, list of request tails)."""
    rng = random.Random(seed)

    def tok():
        t = rng.randrange(1, vocab - 1)
        return t if t != mask_id else t - 1

    affix = [tok() for _ in range(affix_len)]
    tails = [[tok() for _ in range(rng.randint(REQ_LO, REQ_HI))] for _ in range(n)]
    return affix, tails


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
def cpu_reference_sample(layers: int = 2, n_requests: int = 4, gen_length: int = BLOCK, seed: int = 0):
    """The CPU restatement of the reference path (oracle/) on a bounded sample of the
    workload: the LLaDA-8B architecture truncated to ``layers`` layers in fp32, the 800-token
    affix, ``n_requests`` requests, ``gen_length`` generated tokens each (one block).  Time is
    extrapolated linearly in the parameter count to 32 layers.  Returns a dict."""
    import torch

    from oracle.engine import compute_affix_kv, generate_request, select_anchors
    from oracle.models import ArchSpec, OracleModel, random_state_dict

    full_layers = 32
    arch = ArchSpec("llada", n_layers=layers, d_model=4096, n_heads=32, n_kv_heads=32, ffn=12288, vocab=126464,
                    rope_theta=500000.0, rms_eps=1e-5, act="silu", mask_id=126336)
    sd = random_state_dict(arch, seed=seed, std=0.02)
    model = OracleModel(arch, sd, torch.float32)
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
    return dict(value=tok_s_sample / scale, unit="tok/s", cores=torch.get_num_threads(), kind="port",
                sample=(f"{n_requests} request(s) x {gen_length} generated tokens (1 block) of the workload, affix K/V "
                        f"resident, architecture truncated to {layers} of {full_layers} layers in fp32 on CPU: "
                        f"{dt:.1f} s, {nfe} forwards; tok/s extrapolated by the parameter-count ratio {scale:.2f}"),
                seconds=dt)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(args.steps, 1)
    vals = []
    base = None
    for i in range(min(args.warmup, 1) + steps):
        base = cpu_reference_sample(seed=i)
        if i >= min(args.warmup, 1):
            vals.append(base)
    value = sum(v["value"] for v in vals) / len(vals)
    secs = sum(v["seconds"] for v in vals) / len(vals)
    base = dict(base, value=value)
    base.pop("seconds")
    line = dict(impl="reference", metric="generated tok/s/box LLaDA-8B-arch bs16 affix reuse", value=value, unit="tok/s",
                n_gpus=args.gpus, steps=steps, warmup=min(args.warmup, 1), ms_per_step=secs * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config={"workload": WORKLOAD, "batch_per_gpu": BATCH, "layers": 32, "parallelism": f"dp{args.gpus}",
                        "l2": "weights (16 GB) and K/V re-read every step exceed the 126 MB L2"},
                note="CPU restatement of the reference path (oracle/) on the host cores; see cpu_baseline.sample",
                cpu_baseline=base, e2e={"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                gpu_launches=0)
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    from acache_b200 import _lib
    from acache_b200.config import Config
    from acache_b200.model.configuration import LLaDAConfig
    from acache_b200.model.modeling_llada import LLaDAModelLM
    from acache_b200.model_runner import ModelRunner
    from acache_b200.sequence import Sequence

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    hf = LLaDAConfig.llada_8b()
    if args.layers:
        hf.n_layers = args.layers
    model = LLaDAModelLM(hf, device=dev, dtype=torch.bfloat16, init_params=True, seed=1234).eval()
    with torch.no_grad():  # the mask token must never be the arg-max (see oracle/models.py:random_state_dict)
        w = model.model.transformer["ff_out"].weight
        w[hf.mask_token_id] = w[0]
    model.fuse_projections()
    shared_blocks = -(-AFFIX_LEN // 256)
    cfg = Config(hf_config=hf, mask_id=hf.mask_token_id, recompute_batch_size=4, max_num_seqs=args.batch,
                 gen_length=GEN, block_length=BLOCK, threshold=THRESHOLD, cache_block_size=256,
                 num_kvcache_blocks=shared_blocks + 3 * args.batch + 4, enable_acache=True, anchor_ratio=RATIO,
                 selection_mode="top", model_type="llada", profile_timing=True)
    if args.mode == "dkv_acache":      # second serving mode of the engine: delayed KV refresh on top of affix reuse
        cfg.enable_dkv_cache, cfg.dkv_steps, cfg.dkv_cache_interval = True, GEN, 8
    if args.mode == "dual_cache":      # the no-reuse baseline: every request keeps its own copy of the affix
        cfg.enable_acache = False
        cfg.num_kvcache_blocks = args.batch * -(-(AFFIX_LEN + REQ_HI + GEN) // 256) + 4
    runner = ModelRunner(model, cfg)
    generate = {"acache": runner.generate_with_acache, "dkv_acache": runner.generate_with_dkv_acache,
                "dual_cache": runner.generate_with_dual_cache}[args.mode]

    def host_inputs(step):
        # every rank (replica) serves its own shard of requests; the affix is common
        affix, _ = make_requests(0, hf.vocab_size, hf.mask_token_id, 0)
        _, tails = make_requests(1000 + step * world + rank, hf.vocab_size, hf.mask_token_id, args.batch)
        return affix, tails

    def build(affix, tails):
        return [Sequence(affix + t, block_length=BLOCK, gen_length=GEN, cache_block_size=256, mask_id=hf.mask_token_id,
                         prompt_affix_len=len(affix)) for t in tails]

    # shared affix: computed on rank 0, broadcast to the other replicas over NCCL
    affix, _ = host_inputs(0)
    bcast_ms = None
    if world > 1:
        if rank == 0:
            runner.block_manager  # noqa: B018
            runner._precompute_shared_prefix(affix)
            packed = runner.export_shared_prefix_kv()
        else:
            nh, hkv, D, L = runner._arch()
            packed = torch.empty(2, L, len(affix), hkv, D, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(packed, src=0)
        e1.record()
        torch.cuda.synchronize()
        bcast_ms = e0.elapsed_time(e1)
        if rank != 0:
            runner.load_shared_prefix_kv(affix, packed)
        del packed

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

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
        assert all(o is not None and len(o) == GEN for o in outs)
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
        assert all(isinstance(o, list) and len(o) == GEN for o in outs)
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
    tokens = args.steps * args.batch * GEN * world

    if rank == 0:
        peaks = measured_peaks()
        roof = None
        if timers:
            name = max(timers, key=lambda k: timers[k][0])
            ms, n, work = timers[name]
            if name == "attention_decode":
                achieved = work / (ms * 1e-3) / 1e9
                # DRAM bytes per launch from the profiler capture of this shape (16 requests):
                # profiles/attention_tc_decode_llada.md; below the algorithmic bytes because the
                # shared affix is served by L2 after its first reader
                traffic = NCU_DECODE_ATTENTION_DRAM_BYTES if args.batch == BATCH else None
                roof = dict(kernel=name, bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                            frac=achieved / peaks["hbm_gbs"], traffic=traffic, launches=n, avg_us=ms * 1e3 / n,
                            algorithmic_bytes_per_launch=work / n, peak_source=peaks["source"])
            else:
                achieved = work / (ms * 1e-3) / 1e12
                roof = dict(kernel=name, bound="tensor", achieved=achieved, peak=peaks["bf16_tflops_sustained"],
                            unit="TFLOP/s", frac=achieved / peaks["bf16_tflops_sustained"], traffic=None, launches=n,
                            avg_us=ms * 1e3 / n, peak_source=peaks["source"])
            roof["share_of_step"] = ms / dev_ms
            roof["other_timed"] = {k: dict(ms=v[0], launches=v[1]) for k, v in timers.items() if k != name}
        cpu = None
        if world == 1 and not args.no_cpu_baseline and args.mode == "acache":
            cpu = cpu_reference_sample()
            cpu.pop("seconds")
        metric = "generated tok/s/box LLaDA-8B-arch bs16 affix reuse"
        workload = WORKLOAD
        if args.mode != "acache":   # not the benchmark: another serving mode of the engine on the same requests
            metric += {"dkv_acache": " + dKV-Cache decoding", "dual_cache": " OFF (no-reuse baseline)"}[args.mode]
            workload += {"dkv_acache": ", dKV steps 256, cache interval 8", "dual_cache": ", every request recomputes the affix"}[args.mode]
        line = dict(
            metric=metric, value=tokens / (dev_ms * 1e-3), unit="tok/s",
            n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
            config={"workload": workload, "batch_per_gpu": args.batch, "layers": hf.n_layers, "parallelism": f"dp{world}",
                    "l2": "weights (16 GB) and K/V re-read every step exceed the 126 MB L2"},
            clocks=clocks,
            e2e={"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            gpu_launches=launches, roofline=roof, cpu_baseline=cpu,
            anchor_recompute_ms=recompute_ms / max(recompute_calls, 1), nfe_per_step=nfe / args.steps,
            affix_broadcast_ms=bcast_ms, sections_ms_per_step={k: round(v, 2) for k, v in sections.items()})
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH, help="requests per GPU (the workload is 16)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the architecture")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--mode", default="acache", choices=["acache", "dkv_acache", "dual_cache"],
                    help="acache = the benchmark; the other serving modes of the engine on the same workload")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
