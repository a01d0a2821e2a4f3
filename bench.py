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
    "c4": dict(bits=4, batch=64, hq=16, hkv=2, d=256, seq=(256, 65536), dist="loguniform",
               outliers=True, identity=False, q_scale=8.0, k_channel=True),
    "c4-token": dict(bits=4, batch=64, hq=16, hkv=2, d=256, seq=(256, 65536), dist="loguniform",
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
    """Packed K and V codes + scale records of every token, q and out, page-table entries.
    Records: 16 bytes per (token, KV head), or with K per channel over a page the token's V pair
    (8) plus the page's channel rows spread over its 64 tokens (2 * D * 4 / 64)."""
    d, bits, hkv, hq, b = cfg["d"], cfg["bits"], cfg["hkv"], cfg["hq"], cfg["batch"]
    records = 8 + 2 * d * 4 // PAGE if cfg.get("k_channel") else 16
    per_token_head = 2 * d * bits // 8 + records
    pages = int(sum(-(-int(n) // PAGE) for n in seq))
    return int(seq.sum()) * hkv * per_token_head + b * hq * d * (1 + 2) + 4 * pages


# DRAM bytes (read + write) of one decode launch of the named workload, from a separate ncu
# capture of this command at its default arguments (not a figure of this run): reported as
# `traffic` only when the run's arguments are those of the capture.
CAPTURED_TRAFFIC = {"c2": 402_309_888, "c2-int4": 717_094_656, "c5-int2": 2_161_422_448,
                    "c4": 443_171_840}


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


def build_gpu_case(cfg, device, seed, q_len=1):
    """The workload on the device, written through the library's own append."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = seq_lens_of(cfg, seed)
    pages = [-(-int(n) // PAGE) for n in seq]
    total = sum(pages)
    rng = np.random.default_rng(seed + 1)
    order = np.arange(total) if cfg["identity"] else rng.permutation(total)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    indices = order.astype(np.int32)
    kch = bool(cfg.get("k_channel"))
    layout = QuantKVLayout.create(bits=cfg["bits"], head_dim=cfg["d"], num_kv_heads=cfg["hkv"],
                                  device=device, k_quant=("channel", PAGE) if kch else None)
    cache = layout.allocate(total)
    g = torch.Generator(device=device).manual_seed(seed)
    mult = torch.exp(torch.randn(1, cfg["hkv"], cfg["d"], device=device, generator=g)) \
        if cfg["outliers"] else None
    chunk = 1 << 18     # tokens written per append (bounds the bf16 staging)
    for b, n in enumerate(seq):
        n = int(n)
        pg_all = torch.from_numpy(indices[indptr[b]:indptr[b + 1]]).to(device)
        for a in range(0, n, chunk):
            m = min(chunk, n - a)
            rows = -(-m // PAGE) * PAGE if kch else m     # whole pages for the page writer
            k = torch.randn(rows, cfg["hkv"], cfg["d"], device=device, generator=g)
            if mult is not None:
                k = k * mult
            v = torch.randn(rows, cfg["hkv"], cfg["d"], device=device, generator=g)
            if kch:
                pages = pg_all[a // PAGE:a // PAGE + rows // PAGE].int().contiguous()
                valid = torch.full((rows // PAGE,), PAGE, dtype=torch.int32, device=device)
                valid[-1] = m - (rows - PAGE)
                cache.append_page_groups(k.to(torch.bfloat16), v.to(torch.bfloat16), pages, valid)
            else:
                t = torch.arange(a, a + m, device=device)
                slots = pg_all.long()[t // PAGE] * PAGE + t % PAGE
                cache.append(k.to(torch.bfloat16), v.to(torch.bfloat16), slots)
    q_shape = (cfg["batch"], cfg["hq"], cfg["d"]) if q_len == 1 else \
        (cfg["batch"], q_len, cfg["hq"], cfg["d"])
    q = (torch.randn(*q_shape, device=device, generator=g)
         * cfg["q_scale"]).clamp(-448, 448).to(torch.float8_e4m3fn)
    ws = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    w = PagedDecodeWrapper(ws)
    w.plan(torch.from_numpy(indptr).to(device), torch.from_numpy(indices).to(device),
           torch.from_numpy(seq.astype(np.int32)), cfg["hq"], layout,
           sm_scale=cfg["d"] ** -0.5 / cfg["q_scale"], q_len_per_req=q_len)
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
    sample = (f"{reqs} requests, {tokens} KV tokens of {int(seq.sum())}: a timed step is one "
              f"decode of that sample ({dt * 1e3:.1f} ms); value = batch / (that time scaled "
              f"linearly in KV tokens to the whole batch, {full:.2f} s); N(0,1) K without outlier "
              f"channels on an identity page table (the timing does not depend on the values)")
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": value,
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "whole_batch_ms_per_step": full * 1e3,
            "higher_is_better": True, "scaling": "weak",
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


def _event_ms(step, steps, warmup, device, barrier):
    """Milliseconds per step from CUDA events on the launching stream, after `warmup` steps."""
    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def _max_over_ranks(ms, dist, device):
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _request_rows(cfg, seed, b, n, device):
    """K, V bf16 [n, HKV, D] of request b: the same rows on whichever rank generates them."""
    g = torch.Generator(device=device).manual_seed(seed * 100003 + b)
    k = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
    if cfg["outliers"]:
        k = k * torch.exp(torch.randn(1, cfg["hkv"], cfg["d"], device=device, generator=g))
    v = torch.randn(n, cfg["hkv"], cfg["d"], device=device, generator=g)
    return k.to(torch.bfloat16), v.to(torch.bfloat16)


def _cache_of_ranges(cfg, seed, ranges, device, rng_seed):
    """A cache holding token range [a, b) of every request, with its plan inputs."""
    from foscar_b200 import QuantKVLayout
    mine = np.array([b - a for a, b in ranges], dtype=np.int64)
    pages = [-(-int(n) // PAGE) for n in mine]
    total = max(sum(pages), 1)
    indices = np.random.default_rng(rng_seed).permutation(total).astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    layout = QuantKVLayout.create(bits=cfg["bits"], head_dim=cfg["d"], num_kv_heads=cfg["hkv"],
                                  device=device)
    cache = layout.allocate(total)
    for b, (lo, hi) in enumerate(ranges):
        if hi <= lo:
            continue
        k, v = _request_rows(cfg, seed, b, cfg["seq"][1], device)
        t = torch.arange(hi - lo, device=device)
        pg = torch.from_numpy(indices[indptr[b]:indptr[b + 1]]).to(device).long()
        cache.append(k[lo:hi], v[lo:hi], pg[t // PAGE] * PAGE + t % PAGE)
    return layout, cache, indptr, indices, mine


def measure_sequence_split(cfg, seed, steps, warmup, dist, device, rank, world):
    """ONE batch whose every context is split page-aligned over the ranks: each rank caches and
    decodes its token range; the (o, lse) rows are exchanged and merged by the library's
    one-launch exchange (peer stores, flags; foscar_b200.parallel.SequenceSplitExchange); a step
    (decode launch + exchange launch) is replayed from a CUDA graph, at one GPU too. Rank 0
    also decodes request 0 unsplit and reports the largest difference of its rows. Uniform
    lengths only (the long-context workloads). Returns (ms per step over ranks, max abs error)."""
    from foscar_b200 import PagedDecodeWrapper, parallel
    n = cfg["seq"][1]
    ranges = [parallel.split_sequence(n, rank, world) for _ in range(cfg["batch"])]
    layout, cache, indptr, indices, mine = _cache_of_ranges(cfg, seed, ranges, device,
                                                            seed + 1 + rank)
    q = (torch.randn(cfg["batch"], cfg["hq"], cfg["d"], device=device,
                     generator=torch.Generator(device=device).manual_seed(seed))
         * cfg["q_scale"]).clamp(-448, 448).to(torch.float8_e4m3fn)
    sm = cfg["d"] ** -0.5 / cfg["q_scale"]
    w = PagedDecodeWrapper(torch.empty(256 << 20, dtype=torch.uint8, device=device))
    w.plan(torch.from_numpy(indptr).to(device), torch.from_numpy(indices).to(device),
           torch.from_numpy(mine.astype(np.int32)), cfg["hq"], layout, sm_scale=sm,
           o_data_type=torch.float32 if world > 1 else torch.bfloat16)
    shape = (cfg["batch"], cfg["hq"], cfg["d"])
    out = torch.zeros(shape, dtype=torch.bfloat16, device=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    if world > 1:
        ex = parallel.SequenceSplitExchange(*shape, device=device)
        scratch = (torch.empty(shape, dtype=torch.float32, device=device),
                   torch.empty(shape[:2], dtype=torch.float32, device=device))

        def step():
            parallel.sequence_split_decode(w, q, cache, out=out, exchange=ex, scratch=scratch)
    else:
        def step():
            w.run(q, cache, out=out)
    # the step as a CUDA graph (decode launch + exchange launch): at these step times the
    # host's dispatch of two launches would otherwise be what is measured
    for _ in range(3):
        step()
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    barrier()
    ms = _max_over_ranks(_event_ms(graph.replay, steps, warmup, device, barrier), dist, device)
    status = w.last_status() | (ex.last_status() if world > 1 else 0)
    err = None
    if rank == 0:
        # request 0 unsplit on this GPU
        one = dict(cfg, batch=1)
        lay1, cache1, ip1, ix1, _ = _cache_of_ranges(one, seed, [(0, n)], device, seed + 99)
        w1 = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device=device))
        w1.plan(torch.from_numpy(ip1).to(device), torch.from_numpy(ix1).to(device),
                torch.tensor([n], dtype=torch.int32), cfg["hq"], lay1, sm_scale=sm)
        ref = w1.run(q[:1].contiguous(), cache1)
        torch.cuda.synchronize(device)
        err = float((out[0].float() - ref[0].float()).abs().max().item())
    return ms, err, status


def measure_head_split(cfg, seed, steps, warmup, dist, device, rank, world):
    """ONE batch whose KV heads (and their query heads) are dealt out to the ranks: every rank
    caches and decodes the same requests for its own heads; no collective on the data path.
    Rank 0 checks one request of its output against fp32 attention over the cache's own
    read-back rows (the reference's GPU test metric) and reports the relative L2 error.
    Returns (ms per step over ranks, rel-L2, status)."""
    from foscar_b200 import parallel
    hq, hkv = parallel.shard_kv_heads(cfg["hq"], cfg["hkv"], rank, world)
    mine = dict(cfg, hq=len(hq), hkv=len(hkv))
    case = build_gpu_case(mine, device, seed)
    w, cache, q = case["wrapper"], case["cache"], case["q"]
    out = torch.empty(mine["batch"], mine["hq"], mine["d"], dtype=torch.bfloat16, device=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    ms = _max_over_ranks(_event_ms(lambda: w.run(q, cache, out=out), steps, warmup, device,
                                   barrier), dist, device)
    rel = None
    if rank == 0:
        seq, indptr, indices = case["seq"], case["indptr"], case["indices"]
        b = int(np.argmin(np.where(seq >= 512, seq, 1 << 30)))      # a short request
        n = int(seq[b])
        k_back = torch.empty(n, mine["hkv"], mine["d"], dtype=torch.bfloat16, device=device)
        v_back = torch.empty_like(k_back)
        pages = torch.from_numpy(indices[indptr[b]:indptr[b + 1]].copy()).to(device)
        cache.dequantize(k_back, v_back,
                         torch.tensor([0, pages.numel()], dtype=torch.int32, device=device), pages,
                         torch.tensor([n], dtype=torch.int32, device=device),
                         torch.tensor([0], dtype=torch.int32, device=device))
        g = mine["hq"] // mine["hkv"]
        kb = k_back.float().repeat_interleave(g, dim=1)
        vb = v_back.float().repeat_interleave(g, dim=1)
        sm = mine["d"] ** -0.5 / mine["q_scale"]
        p = torch.softmax(torch.einsum("hd,nhd->hn", q[b].float(), kb) * sm, dim=-1)
        want = torch.einsum("hn,nhd->hd", p, vb)
        rel = float(((out[b].float() - want).norm() / want.norm()).item())
    return ms, rel, w.last_status()


def run_split(args, cfg):
    """`--split sequence|heads`: one batch over all the ranks (strong scaling)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    fn = measure_sequence_split if args.split == "sequence" else measure_head_split
    ms, check, status = fn(cfg, args.seed, args.steps, args.warmup, dist, device, rank, world)
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": cfg["batch"] / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "us_per_step": ms * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": f"e4m3 x int{cfg['bits']} codes, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{args.workload} as ONE batch over {world} GPUs",
                       "parallelism": f"{args.split} split x{world}"},
            "check": {"what": "request 0 vs its unsplit decode on one GPU (max abs)"
                      if args.split == "sequence" else
                      "one request vs fp32 attention over the cache's read-back (rel L2)",
                      "value": check},
            "device_status": status}))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def split_extras(args, dist, device, rank, world):
    """The two partitions of the path across GPUs, timed in the run's own process group and
    attached to its JSON line: the serving sweep shape dealt out by KV heads, and the
    100,352-token context split by sequence at batch 1 and 16. Each entry carries this run's
    time at `world` GPUs and rank 0's time for the whole batch on one GPU."""
    steps, warm = min(args.steps, 20), 3
    extras = {}

    def both(fn, cfg):
        ms_n, check, status = fn(cfg, args.seed, steps, warm, dist, device, rank, world)
        ms_1 = None
        if dist is not None:
            dist.barrier()
        if rank == 0:
            ms_1, _, _ = fn(cfg, args.seed, steps, warm, None, device, 0, 1)
        if dist is not None:
            dist.barrier()
        torch.cuda.empty_cache()
        if rank != 0:
            return None
        return {"us_per_step": ms_n * 1e3, "tokens_per_s": cfg["batch"] / (ms_n * 1e-3),
                "us_per_step_1gpu": ms_1 * 1e3, "speedup_vs_1gpu": ms_1 / ms_n,
                "check": check, "device_status": status}

    if WORKLOADS["c5-int2"]["hkv"] % world == 0:
        extras["tp_heads"] = {"c5-int2": both(measure_head_split, WORKLOADS["c5-int2"]),
                              "check": "rel L2 of one request vs fp32 attention over the "
                                       "cache's read-back rows"}
    extras["seq_split"] = {"c3-b1": both(measure_sequence_split, WORKLOADS["c3-b1"]),
                           "c3-b16": both(measure_sequence_split, WORKLOADS["c3-b16"]),
                           "check": "max abs of request 0 vs its unsplit decode on one GPU"}
    return extras


def workload_config(args, cfg, seq):
    return {"workload": f"{args.workload}: INT{cfg['bits']} paged GQA decode, batch {cfg['batch']}, "
                        f"{cfg['hq']}/{cfg['hkv']} heads, head_dim {cfg['d']}, page 64, seq_lens "
                        f"{cfg['seq'][0]}..{cfg['seq'][1]} ({int(seq.sum())} KV tokens per GPU), "
                        f"random page table, "
                        + ("K per channel over a page and V per token" if cfg.get("k_channel")
                           else "token-wise asymmetric groups") + ", q fp8 e4m3"
                        + (f", {args.q_len} query tokens per request" if args.q_len > 1 else ""),
            "l2": "inputs larger than L2 (packed cache streamed once per step)",
            "parallelism": f"dp{args.gpus} (independent batches per GPU, no collective)"}


def cache_op_figures(cfg, device, seed):
    """The cache writer and the read-back kernel alone on 131,072 tokens of the workload's head
    shape: algorithmic GB/s from CUDA events (inputs and outputs exceed L2)."""
    from foscar_b200 import QuantKVLayout
    tokens, hkv, d, bits = 131072, cfg["hkv"], cfg["d"], cfg["bits"]
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device=device)
    pages = tokens // PAGE
    cache = layout.allocate(pages)
    g = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn(tokens, hkv, d, device=device, generator=g).to(torch.bfloat16)
    v = torch.randn(tokens, hkv, d, device=device, generator=g).to(torch.bfloat16)
    slots = torch.randperm(pages, device=device, generator=g).repeat_interleave(PAGE) * PAGE \
        + torch.arange(PAGE, device=device).repeat(pages)
    packed = tokens * hkv * (2 * d * bits // 8 + 16)
    dense = tokens * hkv * 2 * d * 2
    k_out, v_out = torch.empty_like(k), torch.empty_like(v)
    indptr = torch.tensor([0, pages], dtype=torch.int32, device=device)
    indices = (slots[::PAGE] // PAGE).to(torch.int32)
    lens = torch.tensor([tokens], dtype=torch.int32, device=device)
    out_indptr = torch.tensor([0], dtype=torch.int32, device=device)

    def sync():
        torch.cuda.synchronize(device)
    ms_a = _event_ms(lambda: cache.append(k, v, slots), 10, 3, device, sync)
    ms_d = _event_ms(lambda: cache.dequantize(k_out, v_out, indptr, indices, lens, out_indptr),
                     10, 3, device, sync)
    return {"append_gbs": (dense + packed + tokens * 8) / ms_a / 1e6, "append_ms": ms_a,
            "dequantize_gbs": (dense + packed + pages * 4) / ms_d / 1e6, "dequantize_ms": ms_d,
            "shape": f"{tokens} tokens x {hkv} KV heads x head_dim {d}, INT{bits}, random pages"}


GRID_SHAPES = {"hq32-hkv8-d128": (32, 8, 128), "hq8-hkv1-d128": (8, 1, 128),
               "hq16-hkv2-d64": (16, 2, 64)}
# The reference's published B200 kernel times, us (benchmarks/decode_latency.csv of the
# reference, quoted in its README.md:165-172, 185-192, 220-227): (INT2, INT4) per (shape, batch,
# context).
GRID_PUBLISHED = {}
for _shape, _batch, _int2, _int4 in (
        ("hq32-hkv8-d128", 1, (15.3, 36.7, 62.4, 114.3), (17.6, 44.2, 74.8, 135.6)),
        ("hq32-hkv8-d128", 8, (62.5, 218.3, 399.1, 758.1), (75.1, 251.9, 456.2, 865.7)),
        ("hq8-hkv1-d128", 1, (12.9, 18.2, 22.4, 29.4), (12.2, 18.4, 22.6, 31.6)),
        ("hq8-hkv1-d128", 8, (17.3, 37.5, 63.2, 114.8), (18.8, 44.2, 72.9, 126.3)),
        ("hq16-hkv2-d64", 1, (12.0, 17.0, 22.1, 32.1), (11.8, 17.6, 23.4, 36.6)),
        ("hq16-hkv2-d64", 8, (20.0, 51.0, 89.5, 168.4), (22.0, 59.6, 107.9, 206.1))):
    for _ctx, _a, _b in zip((32768, 131072, 262144, 524288), _int2, _int4):
        GRID_PUBLISHED[(_shape, _batch, _ctx)] = (_a, _b)


def run_grid(args):
    """The reference's own benchmark grid with its protocol (benchmarks/timer.py:35-50,
    benchmarks/run_bench.py:53-81 there): K, V ~ N(0,1), token-wise groups over the whole head,
    f32 records, random page permutation, q = e4m3(8 q) with sm_scale / 8; a 1 GiB write before
    every timed call (cold L2), 5 warm-up + 5 timed calls, the median of the decode launch's
    device time. Prints one JSON object with a row per cell."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=device)
    g = torch.Generator(device=device).manual_seed(0)
    rows = []
    for name, (hq, hkv, d) in GRID_SHAPES.items():
        # one block of random tokens, written again and again: timing does not read values
        blk = 65536
        k = torch.randn(blk, hkv, d, device=device, generator=g).to(torch.bfloat16)
        v = torch.randn(blk, hkv, d, device=device, generator=g).to(torch.bfloat16)
        for bits in (2, 4):
            layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device=device)
            for batch in (1, 8):
                for ctx in (32768, 131072, 262144, 524288):
                    pages_per = ctx // PAGE
                    total = batch * pages_per
                    cache = layout.allocate(total)
                    order = torch.randperm(total, device=device, generator=g)
                    for a in range(0, total * PAGE, blk):
                        m = min(blk, total * PAGE - a)      # (32K contexts are half a block)
                        t = torch.arange(a, a + m, device=device)
                        cache.append(k[:m], v[:m], order[t // PAGE] * PAGE + t % PAGE)
                    q = (torch.randn(batch, hq, d, device=device, generator=g) * 8.0) \
                        .clamp(-448, 448).to(torch.float8_e4m3fn)
                    w = PagedDecodeWrapper(torch.empty(256 << 20, dtype=torch.uint8,
                                                       device=device))
                    indptr = torch.arange(batch + 1, dtype=torch.int32) * pages_per
                    w.plan(indptr.to(device), order.to(torch.int32),
                           torch.full((batch,), ctx, dtype=torch.int32), hq, layout,
                           sm_scale=d ** -0.5 / 8.0)
                    out = torch.empty(batch, hq, d, dtype=torch.bfloat16, device=device)
                    times = []
                    for i in range(10):
                        flush.fill_(i)
                        e0 = torch.cuda.Event(enable_timing=True)
                        e1 = torch.cuda.Event(enable_timing=True)
                        e0.record()
                        w.run(q, cache, out=out)
                        e1.record()
                        torch.cuda.synchronize(device)
                        if i >= 5:
                            times.append(e0.elapsed_time(e1) * 1e3)
                    us = float(np.median(times))
                    moved = batch * ctx * hkv * (2 * d * bits // 8 + 16)
                    pub = GRID_PUBLISHED.get((name, batch, ctx))
                    rows.append({"shape": name, "bits": bits, "batch": batch, "ctx": ctx,
                                 "us": us, "tbs": moved / us / 1e6,
                                 "published_us": None if pub is None else pub[bits // 4],
                                 "status": w.last_status()})
                    del cache, w
                    torch.cuda.empty_cache()
    print(json.dumps({"grid": rows, "protocol": "1 GiB write before every timed call; 5 warm-up "
                      "+ 5 timed; median of CUDA-event time around the decode launch (the merge "
                      "of split units runs inside it)"}))


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
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the writer / read-back figures (N = 1) and the head-split and "
                         "sequence-split runs (N > 1) attached to the line")
    ap.add_argument("--split", default="none", choices=["none", "sequence", "heads"],
                    help="sequence: ONE batch whose every context is split page-aligned over the "
                         "ranks (strong scaling; one exchange of (o, lse) per step). heads: ONE "
                         "batch whose KV heads (and their query heads) are dealt out to the ranks "
                         "(tensor parallel, strong scaling, no collective)")
    ap.add_argument("--op", default="decode", choices=["decode", "append", "dequantize"],
                    help="decode: the headline step. append / dequantize: the cache writer or the "
                         "read-back kernel alone on a slice of the workload, as GB/s")
    ap.add_argument("--q-len", type=int, default=1,
                    help="query tokens per request (speculative step); tokens/s counts them all")
    ap.add_argument("--grid", action="store_true",
                    help="the reference's own benchmark grid with its cold-L2 protocol (one GPU)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args, cfg)
    if args.grid:
        return run_grid(args)
    if args.op != "decode":
        return run_cache_op(args, cfg)
    if args.split != "none":
        return run_split(args, cfg)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    case = build_gpu_case(cfg, device, args.seed + 17 * rank, args.q_len)
    w, cache, q, seq = case["wrapper"], case["cache"], case["q"], case["seq"]
    b, hq, d = cfg["batch"], cfg["hq"], cfg["d"]
    out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)
    q_host = q.cpu().view(torch.uint8).pin_memory()
    out_host = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()
    q_stage = torch.empty_like(q)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident timing: the step (one launch: decode with the merge of split units
    # inside it), and that launch's own device time from an event pair around every step
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
    default_args = args.seed == 0 and args.workload in CAPTURED_TRAFFIC and args.q_len == 1
    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        abytes = algorithmic_bytes(cfg, seq)
        achieved = abytes / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": "decode_tokens_per_s", "value": world * b * args.q_len / (step_ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "us_per_step": step_ms * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 x int%d codes, f32 accumulate"
            % cfg["bits"], "data": "synthetic", "config": workload_config(args, cfg, seq),
            "hbm_gbs": abytes / (step_ms * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "of": peak_kind,
                         "traffic": CAPTURED_TRAFFIC[args.workload] if default_args else None,
                         "traffic_from": "a separate ncu capture of this command's decode launch "
                                         "(dram__bytes_read.sum + dram__bytes_write.sum), not "
                                         "measured by this run" if default_args else None,
                         "kernel": "decode_wide_kernel" if cfg["d"] == 256 else "decode_kernel",
                         "kernel_us": decode_ms * 1e3,
                         "algorithmic_bytes": abytes, "frac_of_8tbs_nominal": achieved / 8000.0},
            "e2e": {"value": world * b * args.q_len / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "us_per_step": e2e_ms * 1e3, "h2d_bytes_per_step": int(q_host.numel()),
                    "d2h_bytes_per_step": int(out_host.numel() * 2)},
            "gpu_launches": launches, "clocks": clocks.summary(), "device_status": status,
            "plan": {"kv_splits": w.kv_splits, "reduction": w.reduction},
        }
    del case, w, cache
    torch.cuda.empty_cache()
    if not args.no_extras:
        if world > 1:
            extras = split_extras(args, dist, device, rank, world)
            if rank == 0:
                line.update(extras)
        elif rank == 0:
            line["cache_ops"] = cache_op_figures(cfg, device, args.seed)
    if rank == 0:
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
                "sample": f"{reqs} requests, {tokens} KV tokens of {int(seq.sum())}: {dt * 1e3:.1f} "
                          f"ms per step of the sample, scaled linearly in KV tokens to the whole "
                          f"batch; oracle read-back + fp32 softmax attention (torch); N(0,1) K "
                          f"without outlier channels on an identity page table (the timing does "
                          f"not depend on the values)"}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
