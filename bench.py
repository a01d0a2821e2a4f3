"""Benchmark of the decode hot path (one process per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

A step is one decode step of one layer: `PagedDecodeWrapper.run()` over a synthetic batch whose
packed KV cache is resident in HBM. The default workload is the Qwen3-8B-shaped INT2 case:
batch 32, 32 query / 8 KV heads, head_dim 128, page 64, seq_lens uniform in [4096, 32768],
random page table, K with per-channel log-normal magnitudes, q = e4m3(8 q). With N > 1 every
rank decodes its own batch of the same shape (independent serving replicas: weak scaling, no
collective on the data path). Prints one JSON line.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PAGE = 64
WORKLOADS = {
    # name: bits, batch, hq, hkv, d, (lo, hi) seq range, distribution, outlier K, cpu sample
    "c1": dict(bits=4, batch=2, hq=32, hkv=8, d=128, seq=(128, 128), dist="uniform",
               outliers=False, identity=True, q_scale=1.0),
    "c2": dict(bits=2, batch=32, hq=32, hkv=8, d=128, seq=(4096, 32768), dist="uniform",
               outliers=True, identity=False, q_scale=8.0),
    "c2-int4": dict(bits=4, batch=32, hq=32, hkv=8, d=128, seq=(4096, 32768), dist="uniform",
                    outliers=True, identity=False, q_scale=8.0),
    "c3-b1": dict(bits=2, batch=1, hq=32, hkv=8, d=128, seq=(100352, 100352), dist="uniform",
                  outliers=True, identity=False, q_scale=8.0),
    "c3-b4": dict(bits=2, batch=4, hq=32, hkv=8, d=128, seq=(100352, 100352), dist="uniform",
                  outliers=True, identity=False, q_scale=8.0),
    "c3-b16": dict(bits=2, batch=16, hq=32, hkv=8, d=128, seq=(100352, 100352), dist="uniform",
                   outliers=True, identity=False, q_scale=8.0),
    "c3-b64": dict(bits=2, batch=64, hq=32, hkv=8, d=128, seq=(100352, 100352), dist="uniform",
                   outliers=True, identity=False, q_scale=8.0),
    "c5-int2": dict(bits=2, batch=256, hq=64, hkv=8, d=64, seq=(64, 131072), dist="loguniform",
                    outliers=False, identity=False, q_scale=8.0),
    "c5-int4": dict(bits=4, batch=256, hq=64, hkv=8, d=64, seq=(64, 131072), dist="loguniform",
                    outliers=False, identity=False, q_scale=8.0),
    "small": dict(bits=2, batch=16, hq=32, hkv=8, d=128, seq=(8192, 16384), dist="uniform",
                  outliers=True, identity=False, q_scale=8.0),
}


def seq_lens_of(cfg, seed):
    rng = np.random.default_rng(seed)
    lo, hi = cfg["seq"]
    if lo == hi:
        return np.full(cfg["batch"], lo, dtype=np.int64)
    if cfg["dist"] == "loguniform":
        return np.round(np.exp(rng.uniform(math.log(lo), math.log(hi), cfg["batch"]))).astype(np.int64)
    return rng.integers(lo, hi + 1, cfg["batch"]).astype(np.int64)


def algorithmic_bytes(cfg, seq):
    """Packed K and V codes + scale records of every token, q and out, page-table entries."""
    d, bits, hkv, hq, b = cfg["d"], cfg["bits"], cfg["hkv"], cfg["hq"], cfg["batch"]
    per_token_head = 2 * d * bits // 8 + 16
    pages = int(sum(-(-int(n) // PAGE) for n in seq))
    return int(seq.sum()) * hkv * per_token_head + b * hq * d * (1 + 2) + 4 * pages


# DRAM bytes (read + write) of one decode launch from an ncu capture of the same command
# (profiles/decode_kernel_c2_int2.md, profiles/decode_kernel_c2_int4.md); other workloads have
# no capture.
NCU_TRAFFIC = {"c2": 401_548_800, "c2-int4": 716_985_600}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()            # nvidia-smi needs ~0.1-1 s before its first line
            while not self.samples and time.time() - t0 < 5.0:
                time.sleep(0.02)
            self.primed = len(self.samples)
        except Exception:
            self.proc = None
        return self

    def under_load(self):
        """Samples taken since the sampler was primed (the idle first lines are dropped)."""
        return len(self.samples) - getattr(self, "primed", 0)

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.samples[getattr(self, "primed", 0):]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "timed region, continued with untimed repeats of the same step until "
                          "nvidia-smi (100 ms period) has sampled it 4 times"}


def build_gpu_case(cfg, device, seed):
    """The workload on the device, written through the library's own append."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = seq_lens_of(cfg, seed)
    pages = [-(-int(n) // PAGE) for n in seq]
    total = sum(pages)
    rng = np.random.default_rng(seed + 1)
    order = np.arange(total) if cfg["identity"] else rng.permutation(total)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    indices = order.astype(np.int32)
    layout = QuantKVLayout.create(bits=cfg["bits"], head_dim=cfg["d"], num_kv_heads=cfg["hkv"],
                                  device=device)
    cache = layout.allocate(total)
    g = torch.Generator(device=device).manual_seed(seed)
    mult = torch.exp(torch.randn(1, cfg["hkv"], cfg["d"], device=device, generator=g)) \
        if cfg["outliers"] else None
    for b, n in enumerate(seq):
        n = int(n)
        k = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
        if mult is not None:
            k = k * mult
        v = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
        t = torch.arange(n, device=device)
        pg = torch.from_numpy(indices[indptr[b]:indptr[b + 1]]).to(device).long()
        slots = pg[t // PAGE] * PAGE + t % PAGE
        cache.append(k.to(torch.bfloat16), v.to(torch.bfloat16), slots)
    q = (torch.randn(cfg["batch"], cfg["hq"], cfg["d"], device=device, generator=g)
         * cfg["q_scale"]).clamp(-448, 448).to(torch.float8_e4m3fn)
    ws = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    w = PagedDecodeWrapper(ws)
    w.plan(torch.from_numpy(indptr).to(device), torch.from_numpy(indices).to(device),
           torch.from_numpy(seq.astype(np.int32)), cfg["hq"], layout,
           sm_scale=cfg["d"] ** -0.5 / cfg["q_scale"])
    torch.cuda.synchronize(device)
    if cache.last_status() != 0:
        raise RuntimeError(f"cache writer reported status {cache.last_status()}")
    return dict(seq=seq, cache=cache, wrapper=w, q=q, layout=layout, indptr=indptr,
                indices=indices)


def cpu_reference_step(cfg, seed, budget_tokens):
    """One decode step of the CPU path (oracle read-back + fp32 softmax attention in torch) on a
    bounded sample of the workload; returns (seconds, kv tokens in the sample, requests)."""
    from oracle import CpuPools, ref_append, ref_attention, ref_dequantize
    seq = seq_lens_of(cfg, seed)
    sample, used = [], 0
    for n in seq:
        n = int(min(n, max(PAGE, budget_tokens - used)))
        sample.append(n)
        used += n
        if used >= budget_tokens:
            break
    pages = [-(-n // PAGE) for n in sample]
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    indices = np.arange(sum(pages), dtype=np.int32)
    pools = CpuPools(sum(pages), cfg["hkv"], cfg["d"], cfg["bits"])
    g = torch.Generator().manual_seed(seed)
    for b, n in enumerate(sample):
        k = torch.randn(n, cfg["hkv"], cfg["d"], generator=g).bfloat16()
        v = torch.randn(n, cfg["hkv"], cfg["d"], generator=g).bfloat16()
        ref_append(pools, k, v, np.arange(n) + int(indptr[b]) * PAGE)
    q = torch.randn(len(sample), cfg["hq"], cfg["d"], generator=g).to(torch.float8_e4m3fn)
    sm = cfg["d"] ** -0.5

    def step():
        kv = ref_dequantize(pools, indptr, indices, sample)
        for b in range(len(sample)):
            ref_attention(q[b].float(), kv[b][0], kv[b][1], sm)
    return step, used, len(sample)


def run_reference(args, cfg):
    """The CPU implementation of the path, timed on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    seq = seq_lens_of(cfg, args.seed)
    # Size the sample so that warm-up plus timed steps end within about three minutes: a probe
    # on 2048 tokens gives the host's rate, the cost being linear in KV tokens.
    probe, probe_tokens, _ = cpu_reference_step(cfg, args.seed, 2048)
    probe()
    t0 = time.perf_counter()
    probe()
    rate = probe_tokens / max(time.perf_counter() - t0, 1e-6)
    budget = int(rate * 180.0 / (args.steps + args.warmup))
    step, tokens, reqs = cpu_reference_step(cfg, args.seed,
                                            max(1024, min(args.cpu_tokens, budget)))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    full = dt * float(seq.sum()) / tokens          # linear in KV tokens
    value = cfg["batch"] / full
    sample = f"{reqs} requests, {tokens} KV tokens of {int(seq.sum())}, scaled linearly in tokens"
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": value,
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": full * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, cfg, seq),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def run_cache_op(args, cfg):
    """The cache writer or the read-back kernel alone (one GPU): algorithmic GB/s from CUDA
    events over `steps` launches on 131,072 tokens of the workload's head shape (inputs and
    outputs together exceed L2)."""
    from foscar_b200 import QuantKVLayout
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    tokens, hkv, d, bits = 131072, cfg["hkv"], cfg["d"], cfg["bits"]
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device=device)
    pages = tokens // PAGE
    cache = layout.allocate(pages)
    g = torch.Generator(device=device).manual_seed(args.seed)
    k = torch.randn(tokens, hkv, d, device=device, generator=g).to(torch.bfloat16)
    v = torch.randn(tokens, hkv, d, device=device, generator=g).to(torch.bfloat16)
    slots = torch.randperm(pages, device=device, generator=g).repeat_interleave(PAGE) * PAGE \
        + torch.arange(PAGE, device=device).repeat(pages)
    packed = tokens * hkv * (2 * d * bits // 8 + 16)
    dense = tokens * hkv * 2 * d * 2
    if args.op == "append":
        def step():
            cache.append(k, v, slots)
        moved = dense + packed + tokens * 8
    else:
        cache.append(k, v, slots)
        k_out, v_out = torch.empty_like(k), torch.empty_like(v)
        indptr = torch.tensor([0, pages], dtype=torch.int32, device=device)
        indices = (slots[::PAGE] // PAGE).to(torch.int32)
        lens = torch.tensor([tokens], dtype=torch.int32, device=device)
        out_indptr = torch.tensor([0], dtype=torch.int32, device=device)

        def step():
            cache.dequantize(k_out, v_out, indptr, indices, lens, out_indptr)
        moved = dense + packed + pages * 4
    for _ in range(args.warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / args.steps
    peak, kind = measured_peak()
    gbs = moved / ms / 1e6
    print(json.dumps({"metric": f"{args.op}_gb_per_s", "value": gbs, "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "higher_is_better": True, "dtype": f"int{bits} codes, f32 scales",
                      "data": "synthetic",
                      "config": {"workload": f"{args.op}: {tokens} tokens x {hkv} KV heads x "
                                             f"head_dim {d}, INT{bits}, random pages"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                                   "frac": gbs / peak, "of": kind, "traffic": None,
                                   "algorithmic_bytes": moved},
                      "device_status": cache.last_status()}))


def run_sequence_split(args, cfg):
    """One batch, every context split page-aligned over the ranks: each rank caches and decodes
    its token range, one NCCL all_gather brings the (o, lse) pairs into local memory, a local
    kernel merges them. Strong scaling: `value` is the batch's tokens/s at N GPUs."""
    import torch.distributed as dist
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, parallel
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    seq = seq_lens_of(cfg, args.seed)
    ranges = [parallel.split_sequence(int(n), rank, world) for n in seq]
    mine = np.array([b - a for a, b in ranges], dtype=np.int64)
    pages = [-(-int(n) // PAGE) for n in mine]
    total = max(sum(pages), 1)
    rng = np.random.default_rng(args.seed + 1 + rank)
    indices = rng.permutation(total).astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    layout = QuantKVLayout.create(bits=cfg["bits"], head_dim=cfg["d"], num_kv_heads=cfg["hkv"],
                                  device=device)
    cache = layout.allocate(total)
    g = torch.Generator(device=device).manual_seed(args.seed + rank)
    for b, n in enumerate(mine):
        n = int(n)
        if n == 0:
            continue
        k = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
        v = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
        t = torch.arange(n, device=device)
        pg = torch.from_numpy(indices[indptr[b]:indptr[b + 1]]).to(device).long()
        cache.append(k.to(torch.bfloat16), v.to(torch.bfloat16), pg[t // PAGE] * PAGE + t % PAGE)
    q = (torch.randn(cfg["batch"], cfg["hq"], cfg["d"], device=device,
                     generator=torch.Generator(device=device).manual_seed(args.seed))
         * cfg["q_scale"]).clamp(-448, 448).to(torch.float8_e4m3fn)
    w = PagedDecodeWrapper(torch.empty(256 << 20, dtype=torch.uint8, device=device))
    w.plan(torch.from_numpy(indptr).to(device), torch.from_numpy(indices).to(device),
           torch.from_numpy(mine.astype(np.int32)), cfg["hq"], layout,
           sm_scale=cfg["d"] ** -0.5 / cfg["q_scale"], o_data_type=torch.float32)
    out = torch.empty(cfg["batch"], cfg["hq"], cfg["d"], dtype=torch.bfloat16, device=device)

    def step():
        if world > 1:
            parallel.sequence_split_decode(w, q, cache, out=out)
        else:
            w.run(q, cache, out=torch.empty(cfg["batch"], cfg["hq"], cfg["d"], device=device))

    for _ in range(args.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    if rank == 0:
        peak, kind = measured_peak()
        moved = algorithmic_bytes(cfg, seq)
        gbs = moved / ms / 1e6
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": cfg["batch"] / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "us_per_step": ms * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": f"e4m3 x int{cfg['bits']} codes, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{args.workload}, every context split over {world} GPUs "
                                   f"(page-aligned ranges; all_gather of (o, lse) + local merge)",
                       "parallelism": f"sequence split x{world}"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak * world, "unit": "GB/s",
                         "frac": gbs / (peak * world), "of": kind, "traffic": None,
                         "algorithmic_bytes": moved},
            "device_status": w.last_status()}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def workload_config(args, cfg, seq):
    return {"workload": f"{args.workload}: INT{cfg['bits']} paged GQA decode, batch {cfg['batch']}, "
                        f"{cfg['hq']}/{cfg['hkv']} heads, head_dim {cfg['d']}, page 64, seq_lens "
                        f"{cfg['seq'][0]}..{cfg['seq'][1]} ({int(seq.sum())} KV tokens per GPU), "
                        f"random page table, token-wise asymmetric groups, q fp8 e4m3",
            "l2": "inputs larger than L2 (packed cache streamed once per step)",
            "parallelism": f"dp{args.gpus} (independent batches per GPU, no collective)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-tokens", type=int, default=16384,
                    help="KV tokens in the CPU baseline's bounded sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--split", default="none", choices=["none", "sequence", "heads"],
                    help="sequence: ONE batch whose every context is split page-aligned over the "
                         "ranks (strong scaling; one all_gather of (o, lse) per step). heads: ONE "
                         "batch whose KV heads (and their query heads) are dealt out to the ranks "
                         "(tensor parallel, strong scaling, no collective)")
    ap.add_argument("--op", default="decode", choices=["decode", "append", "dequantize"],
                    help="decode: the headline step. append / dequantize: the cache writer or the "
                         "read-back kernel alone on a slice of the workload, as GB/s")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args, cfg)
    if args.op != "decode":
        return run_cache_op(args, cfg)
    if args.split == "sequence":
        return run_sequence_split(args, cfg)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    by_heads = args.split == "heads"
    if by_heads:
        # every rank decodes the same requests (same lengths: same seed) for its own KV heads
        from foscar_b200 import parallel
        hq, hkv = parallel.shard_kv_heads(cfg["hq"], cfg["hkv"], rank, world)
        cfg = dict(cfg, hq=hq.stop - hq.start, hkv=hkv.stop - hkv.start)
    case = build_gpu_case(cfg, device, args.seed + (0 if by_heads else 17 * rank))
    w, cache, q, seq = case["wrapper"], case["cache"], case["q"], case["seq"]
    b, hq, d = cfg["batch"], cfg["hq"], cfg["d"]
    out = torch.empty(b, hq, d, dtype=torch.bfloat16, device=device)
    q_host = q.cpu().view(torch.uint8).pin_memory()
    out_host = torch.empty(b, hq, d, dtype=torch.bfloat16).pin_memory()
    q_stage = torch.empty_like(q)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident timing: value (decode + merge) and the decode kernel alone
    for _ in range(args.warmup):
        w.run(q, cache, out=out)
    torch.cuda.synchronize(device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches0 = w.launches
    barrier()
    with ClockSampler(local) as clocks:
        t_all0 = torch.cuda.Event(enable_timing=True)
        t_all1 = torch.cuda.Event(enable_timing=True)
        t_all0.record()
        for i in range(args.steps):
            starts[i].record()
            w.run(q, cache, out=out)
            ends[i].record()
        t_all1.record()
        barrier()
        launches = w.launches - launches0
        # A timed region of a few milliseconds falls between two nvidia-smi samples: keep the
        # same step running, untimed, until the sampler has seen the GPU under this load.
        t_load = time.time()
        while clocks.proc is not None and clocks.under_load() < 4 and time.time() - t_load < 3.0:
            for _ in range(200):
                w.run(q, cache, out=out)
            torch.cuda.synchronize(device)
    total_ms = t_all0.elapsed_time(t_all1)
    decode_ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, ends)]))
    step_ms = total_ms / args.steps

    # ---- end to end through the public API with host buffers
    for _ in range(3):
        q_stage.view(torch.uint8).copy_(q_host, non_blocking=True)
        w.run(q_stage, cache, out=out)
        out_host.copy_(out, non_blocking=True)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        q_stage.view(torch.uint8).copy_(q_host, non_blocking=True)
        w.run(q_stage, cache, out=out)
        out_host.copy_(out, non_blocking=True)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps

    stats = torch.tensor([step_ms, e2e_ms, decode_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    step_ms, e2e_ms, decode_ms = (float(x) for x in stats.cpu())
    status = w.last_status()
    if rank == 0:
        peak, peak_kind = measured_peak()
        abytes = algorithmic_bytes(cfg, seq)
        achieved = abytes / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": "decode_tokens_per_s",
            "value": (1 if by_heads else world) * b / (step_ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "us_per_step": step_ms * 1e3, "higher_is_better": True,
            "scaling": "strong" if by_heads else "weak", "vs_baseline": None,
            "dtype": "e4m3 x int%d codes, f32 accumulate"
            % cfg["bits"], "data": "synthetic", "config": workload_config(args, cfg, seq),
            "hbm_gbs": abytes / (step_ms * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "of": peak_kind,
                         "traffic": NCU_TRAFFIC.get(args.workload),
                         "kernel": "decode_kernel", "kernel_us": decode_ms * 1e3,
                         "algorithmic_bytes": abytes, "frac_of_8tbs_nominal": achieved / 8000.0},
            "e2e": {"value": (1 if by_heads else world) * b / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "us_per_step": e2e_ms * 1e3, "h2d_bytes_per_step": int(q_host.numel()),
                    "d2h_bytes_per_step": int(out_host.numel() * 2)},
            "gpu_launches": launches, "clocks": clocks.summary(), "device_status": status,
            "plan": {"kv_splits": w.kv_splits, "reduction": w.reduction},
        }
        if by_heads:
            line["config"]["parallelism"] = (
                f"kv-head tensor parallel x{world}: {cfg['hkv']} KV heads per GPU, the same "
                f"batch on every GPU, no collective")
        if not args.no_cpu_baseline and world == 1:   # the CPU leg is an N=1 figure
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            step, tokens, reqs = cpu_reference_step(cfg, args.seed, args.cpu_tokens)
            step()
            t0 = time.perf_counter()
            n = 0
            while n < 3 or (time.perf_counter() - t0 < 10.0 and n < 50):
                step()
                n += 1
            dt = (time.perf_counter() - t0) / n
            full = dt * float(seq.sum()) / tokens
            line["cpu_baseline"] = {
                "value": b / full, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"{reqs} requests, {tokens} KV tokens of {int(seq.sum())}, scaled "
                          f"linearly in tokens; oracle read-back + fp32 softmax attention (torch)"}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
