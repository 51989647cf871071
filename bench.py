"""Benchmark of the hash-code top-k block retrieval path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one decode-step retrieval of ONE decoder layer for a whole batch:
    encode the query heads and the new K token of every request (into the paged code cache), one launch
                                                                         (ucmr_hash_encode_decode_step)
    Hamming scan of every cached token + exact top-k per (request, kv head)   (ucmr_hamming_topk)
on synthetic data of the shapes the workload names.  "Tokens scored" = cached KV positions scanned.

Headline workload `llama3_8b_decode16` (benchmark config 1): batch 16, 131072 tokens per request,
8 kv heads, 32 query heads, head_dim 128, 128-bit codes, block 128, top-k 16 blocks, first 1 and last 2
blocks forced, block score = sum of distances (mean * BS * G).  Four layers' code caches (256 MiB each)
are resident and the steps rotate over them, so every timed scan reads data that is not in L2.
With N > 1 (launched by torch.distributed.run) every rank runs that workload on its own GPU (independent
replicas, no collective: requests are data-parallel) and rank 0 reports the aggregate.

The K timed steps are repeated `reps` times (each repetition bracketed by a barrier and events, at least 50 ms
of device time in total) and the median repetition is reported, so a short K does not make the number a
single-sample measurement.

The same run appends, under the key `configs`, the other benchmark configurations, each checked against the CPU
oracle outside its timed region (`parity`):
    N = 1: single_request_32k (config 0), paged_gather_b64 (config 2, with a roofline object for the gather kernel),
           llama3_70b_tp and million_token_sharded on one rank;
    N > 1: llama3_70b_tp split by kv head over the N ranks (no collective) and million_token_sharded over N ranks
           with both exchanges (peer-memory stores + flag wait, and one NCCL all-gather).

`--impl reference` times the reference's CPU implementation of the path (the C restatement of its algorithm under
oracle/, all host threads; beside it, on a sub-sample, its own compiled C++ retrieval backend and its torch
formulation) on the headline workload, rank 0 only.  That arm does not load the CUDA library.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, seq_len, Hkv, Hq, D, bits, BS, k, layers resident
    "llama3_8b_decode16": dict(B=16, seq=131072, Hkv=8, Hq=32, D=128, bits=128, BS=128, k=16, layers=4),
}
MUST_SELECT = (0, -2, -1)

# The other benchmark configs.  They use Bernoulli(0.5) code bits directly (the scan's cost does not depend on the
# values); the decode-step encode of the queries / new keys is part of the step where the config has keys.
EXTRA_WORKLOADS = {
    # config 0: one request, codes given, latency
    "single_request_32k": dict(B=1, seq=32768, Hkv=8, Hq=32, D=128, bits=128, BS=128, k=64, layers=40),
    # config 2: decode step + physical gather of the selected K/V blocks, ragged batch, 200k-block pool
    "paged_gather_b64": dict(B=64, Hkv=8, Hq=32, D=128, bits=128, BS=128, k=32, pool_blocks=200000,
                             seq_lo=8192, seq_hi=131072, layers=2),
    # config 3: tensor parallel by kv head, no collective; rank r owns Hkv/N kv heads and their query heads
    "llama3_70b_tp": dict(B=8, seq=262144, Hkv=8, Hq=64, D=128, bits=128, BS=128, k=32, layers=4),
    # config 4: sequence sharded over the ranks, local candidates -> exchange -> merge
    "million_token_sharded": dict(B=2, seq=4194304, Hkv=8, Hq=32, D=128, bits=256, BS=64, k=256, layers=2),
}
# What every timed step here may promise the scan about kernels still in flight before it: none writes sequence
# lengths or block tables, and the only code-cache write is the decode-step encode of one new key per request, into
# the request's last block (ucmr.h: UCMR_FLAG_INPUTS_STABLE, UCMR_FLAG_CACHE_APPEND_ONLY).
STABLE = dict(inputs_stable=True, cache_append_only=True)
MIN_TIMED_MS = 50.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self._stop = threading.Event()
        self.thread = None
        self.max_mhz = None
        self.error = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            uuid = None
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if vis:
                tok = vis.split(",")[self.index].strip()
                if tok.isdigit():
                    idx = int(tok)
                else:
                    uuid = tok
            h = nv.nvmlDeviceGetHandleByUUID(uuid) if uuid else nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
            while not self._stop.is_set():
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                r = int(get_reasons(h))
                for name, bit in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(self.period)
            nv.nvmlShutdown()
        except Exception as exc:  # NVML missing: report it, do not fail the benchmark
            self.error = repr(exc)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=5)
        out = {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.error:
            out["error"] = self.error
        return out


class Ranks:
    """The process group of this run (one process per GPU) and its barrier / max-over-ranks helpers."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = None

    def init(self):
        import torch
        import torch.distributed as dist
        self.dev = torch.device(f"cuda:{self.local_rank}")
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        """Element-wise max (or min) over the ranks of a list of floats."""
        import torch
        import torch.distributed as dist
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
        return [float(v) for v in t.cpu()]

    def close(self):
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


MAX_REPS = 400


def timed_reps(run_k, ranks: Ranks, min_ms: float = MIN_TIMED_MS, max_reps: int = 0, host_clock: bool = False):
    """Times `run_k()` (which enqueues exactly K steps) `reps` times, each repetition between a barrier + synchronize
    on both sides, with CUDA events on the current stream (or the host clock around enqueue + synchronize when
    `host_clock`).  Each repetition's time is the max over the ranks; returns the median repetition and the spread.
    `reps` is chosen so that the repetitions add up to at least `min_ms` (the same on every rank)."""
    import torch

    def one():
        ranks.barrier()
        if host_clock:
            t0 = time.perf_counter()
            run_k()
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_k()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        return ms

    est = ranks.reduce([one()])[0]                       # also one more warm-up pass
    reps = int(min(max_reps or MAX_REPS, max(3, math.ceil(min_ms / max(est, 1e-3)))))
    times = ranks.reduce([one() for _ in range(reps)])
    ranks.barrier()
    return dict(ms=float(np.median(times)), reps=reps, ms_min=float(min(times)), ms_max=float(max(times)))


def capture_graphs(step, layers, warm=True):
    """One CUDA graph per resident layer of `step(layer)` (no allocation, no host sync inside)."""
    import torch
    side = torch.cuda.Stream()
    graphs = []
    with torch.cuda.stream(side):
        if warm:
            for layer in range(layers):
                step(layer)
            torch.cuda.synchronize()
        for layer in range(layers):
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph, stream=side):
                step(layer)
            graphs.append(gph)
    torch.cuda.synchronize()
    return graphs


def new_retrieval(B, Hout, k, dev, physical=None):
    import torch
    from unified_cache_management_b200 import ops
    return ops.Retrieval(physical=torch.empty((B, Hout, k), dtype=torch.int32, device=dev) if physical is None else physical,
                         logical=torch.empty((B, Hout, k), dtype=torch.int32, device=dev), scores=None,
                         valid_count=torch.empty((B,), dtype=torch.int32, device=dev),
                         new_seq_lens=torch.empty((B,), dtype=torch.int32, device=dev))


def u32(t):
    return t.contiguous().cpu().numpy().view(np.uint32)


def rand_codes(shape, dev, gen):
    import torch
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=gen)


# ----------------------------------------------------------------------------------------------
# headline workload construction (device)
# ----------------------------------------------------------------------------------------------
def build_workload(cfg, dev, seed=1):
    """Paged code caches filled by the encode kernel from synthetic bf16 keys (prefill), plus the per-step inputs.
    Returns a dict of device tensors and the timing of the bulk encode (K launches of one 1 Mi-row chunk back to back
    between one event pair, arguments prepared once outside)."""
    import torch
    from unified_cache_management_b200 import ops
    B, seq, Hkv, Hq, D, BS, L = cfg["B"], cfg["seq"], cfg["Hkv"], cfg["Hq"], cfg["D"], cfg["BS"], cfg["layers"]
    W = cfg["bits"] // 32
    mb = seq // BS
    NB = B * mb + 8
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    R = (torch.randn((D, cfg["bits"]), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    bt = torch.randperm(NB, device=dev, generator=g)[:B * mb].to(torch.int32).view(B, mb).contiguous()
    seq_lens = torch.full((B,), seq, dtype=torch.int32, device=dev)
    caches = [torch.zeros((NB, BS, Hkv, W), dtype=torch.int32, device=dev) for _ in range(L)]
    pos = torch.arange(seq, device=dev)
    for layer in range(L):
        for b in range(B):
            slots = bt[b].to(torch.int64)[pos // BS] * BS + (pos % BS)
            g.manual_seed(seed * 1000003 + layer * 4099 + b * 17)
            k = torch.randn((seq, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
            ops.hash_encode_and_cache(k, slots, caches[layer], R)
            del k
    q = torch.randn((L, B, Hq, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k_new = torch.randn((L, B, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    last_slot = (bt[:, mb - 1].to(torch.int64) * BS + (BS - 1)).contiguous()
    return dict(R=R, bt=bt, seq_lens=seq_lens, caches=caches, q=q, k_new=k_new, last_slot=last_slot, NB=NB, mb=mb, W=W)


def time_bulk_encode(cfg, wl, dev, iters, peaks):
    """The prefill encode kernel alone: `iters` launches of one request's keys (seq x Hkv rows, bf16) into a scratch
    code cache, back to back between one event pair; four key buffers rotate so that the input is not L2-resident."""
    import torch
    from unified_cache_management_b200 import ops
    seq, Hkv, D, BS, W = cfg["seq"], cfg["Hkv"], cfg["D"], cfg["BS"], wl["W"]
    rows = seq * Hkv
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    keys = [torch.randn((seq, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16) for _ in range(4)]
    scratch = torch.zeros((seq // BS, BS, Hkv, W), dtype=torch.int32, device=dev)
    slots = torch.arange(seq, device=dev, dtype=torch.int64)
    # one CUDA graph per key buffer, so that the host-side argument set-up of a launch is not in the timed loop
    graphs = capture_graphs(lambda i: ops.hash_encode_and_cache(keys[i], slots, scratch, wl["R"]), 4)
    for i in range(4):
        graphs[i].replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        graphs[i % 4].replay()
    e1.record()
    torch.cuda.synchronize()
    t = e0.elapsed_time(e1) / iters * 1e-3
    nbytes = rows * (D * 2 + W * 4)
    flops = 2.0 * rows * D * cfg["bits"]
    return {"bound": "hbm", "kernel": "encode_tc_kernel (tcgen05 bf16 x bf16 -> sign bits, paged code-cache epilogue)",
            "achieved": nbytes / t / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": nbytes / t / 1e9 / peaks["hbm_gbs"],
            "traffic": None, "rows_per_launch": rows, "algorithmic_bytes_per_launch": nbytes, "launch_us_mean": t * 1e6,
            "launches_timed": iters, "tflops": flops / t / 1e12,
            "frac_of_bf16_peak": flops / t / 1e12 / peaks.get("bf16_tflops", 1590.0)}


def time_reference_gpu(cfg, wl, dev, iters=30):
    """Times the reference project's own CUDA path for the same shape, compiled unmodified for this GPU (the
    prebuilt module under oracle/_ref/hamming_cuda, if present): HammingScoreContiCUDA, then the torch tail
    min -> topk -> sort -> gather of its cuda_hamming_topk.  Scan and selection only, no encode.  The codes are
    handed over permuted into that kernel's [Hkv][BS][W] block indexing.  Returns None when the module is absent."""
    import torch
    from oracle import build_oracle
    mod = build_oracle.load_ref_cuda()
    if mod is None:
        return None
    B, Hkv, Hq, BS, k, L = cfg["B"], cfg["Hkv"], cfg["Hq"], cfg["BS"], cfg["k"], cfg["layers"]
    W, mb = wl["W"], wl["mb"]
    refs = [c.permute(0, 2, 1, 3).contiguous().view(c.shape) for c in wl["caches"]]
    q = torch.randint(-2**31, 2**31 - 1, (B, 1, Hq, W), dtype=torch.int32, device=dev)

    def run(layer):
        out = mod.hamming_score(refs[layer], q, wl["bt"], wl["seq_lens"], mb * BS, BS, 2 * BS, True)
        blk = torch.min(out.view(out.shape[0], out.shape[-1] // BS, BS), dim=-1)[0]
        ind = torch.topk(blk, k=k, dim=-1, largest=False)[1]
        ind = torch.sort(ind, dim=-1, descending=False)[0]
        return torch.gather(wl["bt"], dim=-1, index=ind)

    for i in range(5):
        run(i % L)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        run(i % L)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    e0.record()
    for i in range(iters):
        mod.hamming_score(refs[i % L], q, wl["bt"], wl["seq_lens"], mb * BS, BS, 2 * BS, True)
    e1.record()
    torch.cuda.synchronize()
    ms_k = e0.elapsed_time(e1) / iters
    del refs
    return {"what": "reference HammingScoreContiKernel (unmodified, compiled for sm_100) + torch min/topk/sort/gather, "
                    "same shape, block-min selection over all kv heads, no encode",
            "ms_per_step": ms, "value": B * cfg["seq"] / (ms * 1e-3), "unit": "tokens/s",
            "scan_kernel_ms": ms_k, "scan_kernel_gbs": B * cfg["seq"] * Hkv * W * 4 / (ms_k * 1e-3) / 1e9,
            "iters": iters}


def scan_bytes(B, tokens, Hkv, Hq, W, mb, Hout):
    """Algorithmic bytes of one scan launch: codes + query codes + block table + block scores out."""
    return tokens * Hkv * W * 4 + B * Hq * W * 4 + B * mb * 4 + B * Hout * mb * 4


# ----------------------------------------------------------------------------------------------
# CPU arm (test infrastructure under oracle/ used as the timed CPU baseline; never on the product path)
# ----------------------------------------------------------------------------------------------
def cpu_inputs(cfg, seed=1):
    """Host-side inputs of the headline workload for the CPU arm, made with numpy only: Bernoulli code bits for one
    layer's cache (the scan's cost does not depend on the values), a permuted block table, bf16 N(0,1) queries / new
    keys and the bf16 projection."""
    from oracle import oracle as O
    B, seq, Hkv, Hq, D, BS = cfg["B"], cfg["seq"], cfg["Hkv"], cfg["Hq"], cfg["D"], cfg["BS"]
    W, mb = cfg["bits"] // 32, seq // BS
    NB = B * mb + 8
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 2**32, size=(NB, BS, Hkv, W), dtype=np.uint32)
    bt = rng.permutation(NB)[:B * mb].astype(np.int32).reshape(B, mb)
    sl = np.full((B,), seq, dtype=np.int32)
    r = O.f32_to_bf16_bits((rng.standard_normal((D, cfg["bits"])) / np.sqrt(D)).astype(np.float32))
    q = O.f32_to_bf16_bits(rng.standard_normal((B, Hq, D)).astype(np.float32))
    kn = O.f32_to_bf16_bits(rng.standard_normal((B, Hkv, D)).astype(np.float32))
    return codes, bt, sl, r, q, kn


def cpu_step_factory(cfg, host, n_req):
    """One CPU step on the first n_req requests with the C restatement of the reference algorithm."""
    from oracle import oracle as O
    from oracle import oracle_c as OC
    codes, bt_all, sl_all, r, q, kn = host
    bt = np.ascontiguousarray(bt_all[:n_req])
    sl = np.ascontiguousarray(sl_all[:n_req])

    def step():
        OC.hash_encode(kn[:n_req], r)
        qc = OC.hash_encode(q[:n_req], r)
        return OC.hamming_topk(codes, qc, bt, sl, cfg["k"], O.REDUCE_SUM, False, must_select=MUST_SELECT)

    return step


def time_cpu(cfg, host, budget_s=12.0, max_steps=5):
    """Times the CPU arm on a bounded sample: as many requests as fit in about budget_s/max_steps per step."""
    from oracle import oracle_c as OC
    OC.use_all_cores()
    probe = cpu_step_factory(cfg, host, 1)
    t0 = time.perf_counter()
    probe()
    t1 = time.perf_counter() - t0
    n_req = int(max(1, min(cfg["B"], (budget_s / max_steps) / max(t1, 1e-6))))
    step = cpu_step_factory(cfg, host, n_req)
    times = []
    for _ in range(max_steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if sum(times) > budget_s:
            break
    best = min(times)
    return dict(value=n_req * cfg["seq"] / best, unit="tokens/s", cores=OC.num_threads(), kind="port",
                sample=f"{n_req} of {cfg['B']} requests x {cfg['seq']} tokens, one layer, best of {len(times)} steps "
                       f"({best * 1e3:.1f} ms per step), C restatement of the reference algorithm with OpenMP")


def time_reference_backend(cfg, host, n_blocks=4096):
    """The reference's own CPU retrieval backend (hash_retrieval_backend.cpp:321-420, compiled unmodified into
    oracle/_ref): min over a block's tokens of the popcount distance over all heads' bytes, one worker thread per
    submitted request.  Timed on a sub-sample: `n_blocks` blocks per request, one request per host thread."""
    from oracle import build_oracle
    mod = build_oracle.load_ref()
    if mod is None:
        return {"unavailable": "reference backend not built (no reference checkout where build() ran)"}
    codes = host[0]
    NB, BS, Hkv, W = codes.shape
    dim = Hkv * W * 4
    cores = sorted(os.sched_getaffinity(0))
    n_req = len(cores)
    n_blocks = min(n_blocks, NB)
    data = np.ascontiguousarray(codes[:n_blocks]).view(np.uint8).reshape(n_blocks, BS, dim)
    rng = np.random.default_rng(3)
    query = rng.integers(0, 256, size=(n_req, dim), dtype=np.uint8)
    idx = np.tile(np.arange(n_blocks, dtype=np.int32), (n_req, 1))
    backend = mod.HashRetrievalWorkerBackend(data, {0: cores})
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        rids = [backend.submit(query[i:i + 1], cfg["k"], idx[i:i + 1]) for i in range(n_req)]
        for rid in rids:
            backend.wait(rid)
        dt = time.perf_counter() - t0
        for rid in rids:
            backend.get_result(rid)
        best = dt if best is None else min(best, dt)
    del backend
    return {"value": n_req * n_blocks * BS / best, "unit": "tokens/s", "cores": n_req, "kind": "reference",
            "what": "HashRetrievalWorkerBackend of the reference, compiled unmodified: block score = min over tokens, "
                    "all kv heads as one code",
            "sample": f"{n_req} requests (one per worker thread) x {n_blocks} blocks x {BS} tokens, best of 3 "
                      f"({best * 1e3:.1f} ms)"}


def time_torch_formulation(cfg, host, n_blocks=256):
    """The reference's torch formulation of the same retrieval (hash_retrieval_worker.py:102-119): codes unpacked to
    +-1, einsum against the unpacked query, max over a block's tokens, topk, sort, index - on the host cores through
    torch.  Sub-sample: one request x `n_blocks` blocks (the unpacked keys take 32x the packed bytes)."""
    import torch
    codes = host[0]
    NB, BS, Hkv, W = codes.shape
    dim = Hkv * W * 4
    n_blocks = min(n_blocks, NB)
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    raw = torch.from_numpy(np.ascontiguousarray(codes[:n_blocks]).view(np.uint8).reshape(n_blocks, BS, dim).copy())
    masks = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8)

    def unpack(x):   # bytes -> +-1 floats, LSB first (HashEncoder._unpack_hash)
        bits = (x.unsqueeze(-1) & masks) > 0
        return bits.reshape(*x.shape[:-1], -1).to(torch.float32) * 2 - 1

    keys = unpack(raw)                                           # [n_blocks, BS, bits]
    qv = unpack(torch.randint(0, 256, (1, dim), dtype=torch.uint8))
    idx = torch.arange(n_blocks).view(1, -1)
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        data_indexed = keys[idx.flatten()].reshape(1, n_blocks, BS, keys.shape[-1])
        scores = torch.einsum("td,tnjd->tnj", qv, data_indexed)
        blocks = torch.max(scores, dim=-1).values
        top = torch.topk(blocks, min(cfg["k"], n_blocks), dim=-1).indices.sort(dim=-1).values
        _ = idx[torch.arange(1)[:, None], top]
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": n_blocks * BS / best, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "what": "torch formulation of the reference's retrieval (unpack to +-1, einsum, max, topk, sort), float32",
            "sample": f"1 request x {n_blocks} blocks x {BS} tokens, keys unpacked beforehand, best of 3 "
                      f"({best * 1e3:.1f} ms)"}


# ----------------------------------------------------------------------------------------------
# the other benchmark configs
# ----------------------------------------------------------------------------------------------
def _graph_timing(step, layers, K, W, ranks, use_graph=True):
    """Warm-up, optional graph capture per layer, then `timed_reps` of K steps.  Returns (timing dict, launch mode)."""
    for i in range(W):
        step(i % layers)
    ranks.barrier()
    mode = "one CUDA graph per layer-step"
    run = step
    if use_graph:
        try:
            graphs = capture_graphs(step, layers, warm=False)
            run = lambda layer: graphs[layer].replay()
            for i in range(W):
                run(i % layers)
        except Exception as exc:  # noqa: BLE001
            mode = f"stream-ordered launches from Python ({exc})"
            run = step
    else:
        mode = "stream-ordered launches from Python"
    ranks.barrier()

    def run_k():
        for i in range(K):
            run(i % layers)

    return timed_reps(run_k, ranks), mode


def suite_single_request(ranks, K, W, peaks):
    """Config 0: one request of 32768 tokens, codes given, scan + top-64.  40 layer caches of 4 MiB rotate (more than
    L2).  Latency per step; parity of layer 0 against the oracle."""
    import torch
    from oracle import oracle as O
    from oracle import oracle_c as OC
    from unified_cache_management_b200 import ops
    cfg = EXTRA_WORKLOADS["single_request_32k"]
    dev = ranks.dev
    B, seq, Hkv, Hq, BS, k, L = cfg["B"], cfg["seq"], cfg["Hkv"], cfg["Hq"], cfg["BS"], cfg["k"], cfg["layers"]
    Wd, mb = cfg["bits"] // 32, cfg["seq"] // cfg["BS"]
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    caches = [rand_codes((mb, BS, Hkv, Wd), dev, g) for _ in range(L)]
    q = rand_codes((B, Hq, Wd), dev, g)
    bt = torch.randperm(mb, device=dev, generator=g).to(torch.int32).view(B, mb)
    sl = torch.full((B,), seq, dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    out = new_retrieval(B, Hkv, k, dev)

    def step(layer):
        ops.hamming_topk(caches[layer], q, bt, sl, k, reduce="sum", must_select=MUST_SELECT, workspace=ws, out=out,
                         want_scores=False, **STABLE)

    step(0)
    torch.cuda.synchronize()
    ref = OC.hamming_topk(u32(caches[0]), u32(q), bt.cpu().numpy(), sl.cpu().numpy(), k, O.REDUCE_SUM, False,
                          must_select=MUST_SELECT)
    parity = "ok" if np.array_equal(out.physical.cpu().numpy(), ref["physical"]) and \
        np.array_equal(out.logical.cpu().numpy(), ref["logical"]) else "MISMATCH"
    t, mode = _graph_timing(step, L, K, W, ranks)
    ms = t["ms"] / K
    return {"config": 0, "ms_per_step": ms, "latency_us": ms * 1e3, "tokens_per_s": seq / (ms * 1e-3), "steps": K,
            "reps": t["reps"], "parity": parity, "launch": mode, "gpu_launches_per_step": 2,
            "algorithmic_bytes": scan_bytes(B, seq, Hkv, Hq, Wd, mb, Hkv),
            "shape": {kk: vv for kk, vv in cfg.items() if kk != "layers"}}


def suite_paged_gather(ranks, K, W, peaks):
    """Config 2: ragged batch of 64 over a 200000-block pool; step = scan + selection over all kv heads + gather of the
    selected K/V blocks.  One layer's K and V pools (52.4 GB each, content unspecified) are resident."""
    import torch
    from oracle import oracle as O
    from oracle import oracle_c as OC
    from unified_cache_management_b200 import ops
    cfg = EXTRA_WORKLOADS["paged_gather_b64"]
    dev = ranks.dev
    B, Hkv, Hq, D, BS, k, L, NB = cfg["B"], cfg["Hkv"], cfg["Hq"], cfg["D"], cfg["BS"], cfg["k"], cfg["layers"], cfg["pool_blocks"]
    Wd = cfg["bits"] // 32
    need_gib = (2 * NB * BS * Hkv * D * 2 + L * NB * BS * Hkv * Wd * 4) / 2**30 + 6
    free_gib = torch.cuda.mem_get_info(dev)[0] / 2**30
    if free_gib < need_gib:
        return {"config": 2, "skipped": f"needs {need_gib:.0f} GiB of device memory, {free_gib:.0f} GiB free"}
    gs = torch.Generator().manual_seed(2)
    seq = (torch.randint(cfg["seq_lo"] // BS, cfg["seq_hi"] // BS + 1, (B,), generator=gs) * BS).to(torch.int32)
    nblk = (seq // BS).tolist()
    mb = cfg["seq_hi"] // BS
    perm = torch.randperm(NB, generator=gs)[: sum(nblk)].to(torch.int32)
    bt = torch.zeros((B, mb), dtype=torch.int32)
    off = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[off: off + nblk[b]]
        off += nblk[b]
    bt_d, seq_d = bt.to(dev), seq.to(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    caches = [rand_codes((NB, BS, Hkv, Wd), dev, g) for _ in range(L)]
    kp = torch.empty((NB, BS, Hkv, D), dtype=torch.bfloat16, device=dev)
    vp = torch.empty((NB, BS, Hkv, D), dtype=torch.bfloat16, device=dev)
    q = rand_codes((B, Hq, Wd), dev, g)
    ws = ops.new_workspace(B, Hkv, mb, dev, True)
    ret = new_retrieval(B, 1, k, dev)
    ok = torch.empty((B, k * BS, Hkv, D), dtype=torch.bfloat16, device=dev)
    ov = torch.empty_like(ok)
    tokens = int(seq.sum())

    def step(layer):
        ops.hamming_topk(caches[layer], q, bt_d, seq_d, k, reduce="sum", reduce_kvhead=True, must_select=MUST_SELECT,
                         workspace=ws, out=ret, want_scores=False, **STABLE)
        ops.gather_kv(kp, vp, ret.physical.view(B, k), ok, ov)

    step(0)
    torch.cuda.synchronize()
    ref = OC.hamming_topk(u32(caches[0]), u32(q), bt.numpy(), seq.numpy(), k, O.REDUCE_SUM, True, must_select=MUST_SELECT)
    sel = ret.physical.view(B, k)
    good = np.array_equal(sel.cpu().numpy(), ref["physical"].reshape(B, k))
    for b in (0, B // 2, B - 1):   # gathered bytes against a plain indexed read of the pool
        idx = sel[b].to(torch.int64)
        good = good and torch.equal(ok[b].view(k, BS, Hkv, D).view(torch.int16), kp[idx].view(torch.int16)) \
            and torch.equal(ov[b].view(k, BS, Hkv, D).view(torch.int16), vp[idx].view(torch.int16))
    t, mode = _graph_timing(step, L, K, W, ranks)
    ms = t["ms"] / K
    # the gather kernel alone: different selections rotate so that the source blocks are not L2-resident
    sels = [torch.randperm(NB, device=dev, generator=g)[:B * k].to(torch.int32).view(B, k).contiguous() for _ in range(8)]
    n_g = max(K, 20)
    for i in range(3):
        ops.gather_kv(kp, vp, sels[i], ok, ov)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n_g):
        ops.gather_kv(kp, vp, sels[i % 8], ok, ov)
    e1.record()
    torch.cuda.synchronize()
    tg = e0.elapsed_time(e1) / n_g * 1e-3
    gbytes = 2 * 2 * B * k * BS * Hkv * D * 2
    sb = scan_bytes(B, tokens, Hkv, Hq, Wd, mb, 1)
    del kp, vp, ok, ov, caches
    torch.cuda.empty_cache()
    return {"config": 2, "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "steps": K, "reps": t["reps"],
            "parity": "ok" if good else "MISMATCH", "launch": mode, "gpu_launches_per_step": 3, "tokens_per_step": tokens,
            "algorithmic": {"scan_bytes": sb, "gather_bytes": gbytes},
            "step_gbs": (sb + gbytes) / (ms * 1e-3) / 1e9,
            "roofline_gather": {"bound": "hbm", "kernel": "bulk_copy_kernel (paged K/V gather, cp.async.bulk g->s->g)",
                                "achieved": gbytes / tg / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": gbytes / tg / 1e9 / peaks["hbm_gbs"], "traffic": None,
                                "algorithmic_bytes_per_launch": gbytes, "launch_us_mean": tg * 1e6, "launches_timed": n_g},
            "shape": {kk: vv for kk, vv in cfg.items() if kk != "layers"}}


def suite_tp(ranks, K, W, peaks):
    """Config 3: tensor parallel by kv head over the ranks of this run, no collective: rank r owns Hkv/N kv heads of
    every request and their query heads.  Step = decode-step encode (this rank's query heads and new key rows) + scan +
    top-32 per kv head.  Every rank checks its own heads against the oracle."""
    import torch
    from oracle import oracle as O
    from oracle import oracle_c as OC
    from unified_cache_management_b200 import ops
    cfg = EXTRA_WORKLOADS["llama3_70b_tp"]
    dev, world, rank = ranks.dev, ranks.world, ranks.rank
    if cfg["Hkv"] % world != 0:
        return {"config": 3, "skipped": f"{cfg['Hkv']} kv heads do not divide over {world} ranks"}
    B, seq, D, BS, k, L = cfg["B"], cfg["seq"], cfg["D"], cfg["BS"], cfg["k"], cfg["layers"]
    Hkv, Hq = cfg["Hkv"] // world, cfg["Hq"] // world
    Wd, mb = cfg["bits"] // 32, seq // BS
    NB = B * mb
    g = torch.Generator(device=dev)
    g.manual_seed(300 + rank)
    caches = [rand_codes((NB, BS, Hkv, Wd), dev, g) for _ in range(L)]
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, mb).contiguous()
    sl = torch.full((B,), seq, dtype=torch.int32, device=dev)
    R = (torch.randn((D, cfg["bits"]), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    qf = torch.randn((L, B, Hq, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    kn = torch.randn((L, B, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    last_slot = (bt[:, mb - 1].to(torch.int64) * BS + (BS - 1)).contiguous()
    q_codes = torch.empty((B, Hq, Wd), dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    out = new_retrieval(B, Hkv, k, dev)

    def step(layer):
        ops.hash_encode_decode_step(qf[layer], kn[layer], last_slot, caches[layer], R, q_codes_out=q_codes)
        ops.hamming_topk(caches[layer], q_codes, bt, sl, k, reduce="sum", must_select=MUST_SELECT, workspace=ws, out=out,
                         want_scores=False, **STABLE)

    step(0)
    torch.cuda.synchronize()
    ref = OC.hamming_topk(u32(caches[0]), u32(q_codes), bt.cpu().numpy(), sl.cpu().numpy(), k, O.REDUCE_SUM, False,
                          must_select=MUST_SELECT)
    good = np.array_equal(out.physical.cpu().numpy(), ref["physical"]) and \
        np.array_equal(out.logical.cpu().numpy(), ref["logical"])
    good = ranks.reduce([1.0 if good else 0.0], op="min")[0] == 1.0
    t, mode = _graph_timing(step, L, K, W, ranks)
    ms = t["ms"] / K
    sb = scan_bytes(B, B * seq, Hkv, Hq, Wd, mb, Hkv)
    return {"config": 3, "ranks": world, "kv_heads_per_rank": Hkv, "query_heads_per_rank": Hq, "ms_per_step": ms,
            "tokens_per_s": B * seq / (ms * 1e-3), "steps": K, "reps": t["reps"], "scaling": "strong",
            "parity": "ok" if good else "MISMATCH", "parity_checked_on": f"all {world} rank(s), own heads vs oracle",
            "launch": mode, "gpu_launches_per_step": 3, "collective": None,
            "algorithmic": {"scan_bytes_per_gpu": sb, "exchange_bytes": 0},
            "scan_roofline_us_per_gpu": sb / (peaks["hbm_gbs"] * 1e9) * 1e6,
            "shape": {kk: vv for kk, vv in cfg.items() if kk != "layers"}}


def suite_sharded(ranks, K, W, peaks, exchanges=("p2p", "nccl")):
    """Config 4: sequence shards over the ranks of this run: every rank scans its contiguous range of blocks of both
    requests, selects its local top-256 per kv head as (score, id) records, the records are exchanged and merged.
    One rank: candidates + merge without an exchange.  Rank 0 rebuilds the whole problem on the host (every rank's
    codes come from a seed) and compares the merged ids with the unsharded oracle."""
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from oracle import oracle_c as OC
    from unified_cache_management_b200 import ops, sharded
    cfg = EXTRA_WORKLOADS["million_token_sharded"]
    dev, world, rank = ranks.dev, ranks.world, ranks.rank
    B, seq_total, Hkv, Hq, BS, k, L = cfg["B"], cfg["seq"], cfg["Hkv"], cfg["Hq"], cfg["BS"], cfg["k"], cfg["layers"]
    Wd = cfg["bits"] // 32
    nblk_total = seq_total // BS
    if nblk_total % world != 0:
        return {"config": 4, "skipped": f"{nblk_total} blocks do not divide over {world} ranks"}
    per = nblk_total // world
    NB = B * per
    kl = min(k, per)

    def rank_inputs(r, layer):
        g = torch.Generator(device=dev)
        g.manual_seed(4000 + 16 * r + layer)
        codes = rand_codes((NB, BS, Hkv, Wd), dev, g)
        g.manual_seed(4900 + r)
        bt_r = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, per).contiguous()
        return codes, bt_r

    caches = []
    for layer in range(L):
        c, bt_local = rank_inputs(rank, layer)
        caches.append(c)
    g = torch.Generator(device=dev)
    g.manual_seed(44)
    q = rand_codes((B, Hq, Wd), dev, g)                      # the same on every rank
    seq_g = torch.full((B,), seq_total, dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, per, dev)
    scale = 1.0 / (BS * (Hq // Hkv))
    plan = sharded.shard_plan(seq_g, BS, nblk_total, world, rank)
    o_s = torch.empty((B, Hkv, k), dtype=torch.float32, device=dev)
    o_i = torch.empty((B, Hkv, k), dtype=torch.int32, device=dev)
    st_word = torch.zeros(1, dtype=torch.int32, device=dev)

    # the unsharded oracle on rank 0 (layer 0)
    want = None
    if rank == 0:
        full_codes = np.empty((world * NB, BS, Hkv, Wd), dtype=np.uint32)
        full_bt = np.empty((B, nblk_total), dtype=np.int32)
        for r in range(world):
            c, bt_r = (caches[0], bt_local) if r == 0 else rank_inputs(r, 0)
            full_codes[r * NB:(r + 1) * NB] = u32(c)
            full_bt[:, r * per:(r + 1) * per] = bt_r.cpu().numpy() + r * NB
            del c
        OC.use_all_cores()
        want = OC.hamming_topk(full_codes, u32(q), full_bt, seq_g.cpu().numpy(), k, O.REDUCE_SUM, False,
                               must_select=MUST_SELECT)["logical"]
        del full_codes
    torch.cuda.empty_cache()
    ranks.barrier()

    def check():
        """Merged ids of layer 0: equal to the oracle on rank 0 and identical on every rank."""
        torch.cuda.synchronize()
        mine = o_i.cpu().numpy()
        good = 1.0
        if rank == 0:
            good = 1.0 if np.array_equal(mine, want) else 0.0
        digest = float(int(np.bitwise_xor.reduce(mine.astype(np.int64).ravel() * 2654435761 % (2**31))))
        lo, hi = ranks.reduce([digest], "min")[0], ranks.reduce([digest], "max")[0]
        return ranks.reduce([good], "min")[0] == 1.0 and lo == hi

    results = {}
    sb = scan_bytes(B, B * per * BS, Hkv, Hq, Wd, per, Hkv)
    if world == 1:
        def step(layer):
            cs, ci = ops.topk_candidates(caches[layer], q, bt_local, plan.seq_lens_local, seq_g, kl, 0, scale,
                                         reduce="sum", must_select=MUST_SELECT, workspace=ws, **STABLE,
                                         out_scores=cand_s, out_ids=cand_i)
            ops.merge_topk(cs.unsqueeze(0), ci.unsqueeze(0), k, out_scores=o_s, out_ids=o_i)
        cand_s = torch.empty((B, Hkv, kl), dtype=torch.float32, device=dev)
        cand_i = torch.empty((B, Hkv, kl), dtype=torch.int32, device=dev)
        step(0)
        good = check()
        t, mode = _graph_timing(step, L, K, W, ranks)
        results["one_rank"] = {"ms_per_step": t["ms"] / K, "reps": t["reps"], "parity": "ok" if good else "MISMATCH",
                               "launch": mode, "gpu_launches_per_step": 3, "exchange_bytes_per_rank": 0}
    else:
        for kind in exchanges:
            if kind == "p2p":
                ex = sharded.PeerExchange(B, Hkv, kl, dev)

                def step(layer):
                    sharded.sharded_hamming_topk_p2p(caches[layer], q, bt_local, seq_g, k, BS, nblk_total, scale, ex,
                                                     reduce="sum", must_select=MUST_SELECT, workspace=ws, plan=plan,
                                                     status=st_word, **STABLE, out_scores=o_s, out_ids=o_i)
                what = "peer-memory stores from the selection kernel + flag wait in the merge kernel (no collective); " \
                       "step number counted in a device word, so the captured step replays correctly"
                use_graph, launches = True, 3
            else:
                gbuf = torch.empty((world * 2, B, Hkv, kl), dtype=torch.int32, device=dev)
                sbuf = torch.empty((2, B, Hkv, kl), dtype=torch.int32, device=dev)

                def step(layer):
                    s_, i_ = sharded.sharded_hamming_topk(caches[layer], q, bt_local, seq_g, k, BS, nblk_total, scale,
                                                          reduce="sum", must_select=MUST_SELECT, workspace=ws,
                                                          gather_buffer=gbuf, send_buffer=sbuf, plan=plan,
                                                          **STABLE, out_scores=o_s, out_ids=o_i)
                what = "one NCCL all-gather of (score, id) records, stream-ordered launches (a captured all-gather did " \
                       "not complete on this pool)"
                use_graph, launches = False, 4
            ranks.barrier()
            o_i.fill_(-9)
            step(0)
            good = check()
            t, mode = _graph_timing(step, L, K, W, ranks, use_graph=use_graph)
            torch.cuda.synchronize()
            o_i.fill_(-9)
            ranks.barrier()
            step(0)                      # once more after the timed loop: the exchange must still be in step
            good = check() and good
            good = good and ranks.reduce([float(int(st_word.item()))], "max")[0] == 0.0
            results[kind] = {"ms_per_step": t["ms"] / K, "reps": t["reps"], "parity": "ok" if good else "MISMATCH",
                             "exchange": what, "launch": mode, "gpu_launches_per_step": launches,
                             "exchange_bytes_per_rank": 2 * B * Hkv * kl * 4 * (world - 1)}
            ranks.barrier()
    best = min(v["ms_per_step"] for v in results.values())
    return {"config": 4, "ranks": world, "blocks_per_rank": per, "ms_per_step": best,
            "tokens_per_s": B * seq_total / (best * 1e-3), "steps": K, "scaling": "strong",
            "parity": "ok" if all(v["parity"] == "ok" for v in results.values()) else "MISMATCH",
            "parity_checked_on": "rank 0 vs the unsharded oracle on the whole problem; ids identical on all ranks",
            "exchanges": results, "algorithmic": {"scan_bytes_per_gpu": sb},
            "scan_roofline_us_per_gpu": sb / (peaks["hbm_gbs"] * 1e9) * 1e6,
            "shape": {kk: vv for kk, vv in cfg.items() if kk != "layers"}}


def run_config_suite(ranks, K, W, peaks, only=None):
    """The other benchmark configs, run by every rank of this launch; returns the `configs` object (rank 0's view)."""
    import torch
    out = {}
    plan = []
    if ranks.world == 1:
        plan += [("single_request_32k", suite_single_request), ("paged_gather_b64", suite_paged_gather)]
    plan += [("llama3_70b_tp", suite_tp), ("million_token_sharded", suite_sharded)]
    for name, fn in plan:
        if only is not None and name != only:
            continue
        try:
            out[name] = fn(ranks, K, W, peaks)
        except Exception as exc:  # noqa: BLE001  (one config failing must not lose the headline line)
            out[name] = {"error": repr(exc)[:300]}
        torch.cuda.empty_cache()
        ranks.barrier()
    return out


# ----------------------------------------------------------------------------------------------
# small single-kernel cases for profiler captures (inputs above L2 size, a few hundred MB on the device)
# ----------------------------------------------------------------------------------------------
def run_profile_case(what: str) -> None:
    """Three launches of one kernel on a small case: `ncu -k regex:<kernel> -s 1 -c 1 python bench.py --ncu-case X`."""
    import torch
    from unified_cache_management_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(0)

    def rnd_codes(shape):
        return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=g)

    scan_cases = {
        # name: B, Hkv, Hq, W, BS, seq, k, reduce
        "scan": (8, 8, 32, 4, 128, 131072, 16, "sum"),          # half of the headline batch: 134 MB
        "select": (8, 8, 32, 4, 128, 131072, 16, "sum"),
        "scan_min": (8, 8, 32, 4, 128, 131072, 16, "min"),
        "scan_256bit": (2, 8, 32, 8, 64, 262144, 256, "sum"),   # million-token shard shape
        "scan_mla": (16, 1, 64, 18, 64, 131072, 32, "min"),     # MLA: 576-bit codes, 64 query codes: 151 MB
        "scan_bs16": (8, 8, 32, 4, 16, 131072, 128, "sum"),     # vLLM's default block size
        "scan_bs32": (8, 8, 32, 4, 32, 131072, 64, "sum"),
        "scan_tp8": (8, 1, 8, 4, 128, 262144, 32, "sum"),       # config 3 at tp = 8: 33.5 MB per layer
    }
    if what in scan_cases:
        B, Hkv, Hq, W, BS, seq, k, red = scan_cases[what]
        mb = seq // BS
        codes = rnd_codes((B * mb, BS, Hkv, W))
        q = rnd_codes((B, Hq, W))
        bt = torch.randperm(B * mb, device=dev, generator=g).to(torch.int32).view(B, mb)
        sl = torch.full((B,), seq, dtype=torch.int32, device=dev)
        ws = ops.new_workspace(B, Hkv, mb, dev)
        for _ in range(3):
            ops.hamming_topk(codes, q, bt, sl, k, reduce=red, must_select=MUST_SELECT, workspace=ws)
    elif what == "encode":
        x = torch.randn((65536, 8, 128), device=dev, dtype=torch.bfloat16)          # 134 MB of keys
        r = (torch.randn((128, 128), device=dev) / 128 ** 0.5).to(torch.bfloat16)
        out = torch.empty((65536, 8, 4), dtype=torch.int32, device=dev)
        for _ in range(3):
            ops.hash_encode(x, r, out=out)
    elif what == "encode_cache":
        x = torch.randn((65536, 8, 128), device=dev, dtype=torch.bfloat16)          # 134 MB of keys into a paged cache
        r = (torch.randn((128, 128), device=dev) / 128 ** 0.5).to(torch.bfloat16)
        cache = torch.zeros((512, 128, 8, 4), dtype=torch.int32, device=dev)
        perm = torch.randperm(512, device=dev, generator=g)
        pos = torch.arange(65536, device=dev)
        slots = (perm[pos // 128] * 128 + pos % 128).to(torch.int64)
        for _ in range(3):
            ops.hash_encode_and_cache(x, slots, cache, r)
    elif what == "encode_wide":
        x = torch.randn((262144, 512), device=dev, dtype=torch.bfloat16)            # MLA latent vectors: 268 MB
        r = (torch.randn((512, 512), device=dev) / 512 ** 0.5).to(torch.bfloat16)
        out = torch.empty((262144, 16), dtype=torch.int32, device=dev)
        for _ in range(3):
            ops.hash_encode(x, r, out=out)
    elif what == "encode_step":
        xq = torch.randn((16, 32, 128), device=dev, dtype=torch.bfloat16)
        xk = torch.randn((16, 8, 128), device=dev, dtype=torch.bfloat16)
        r = (torch.randn((128, 128), device=dev) / 128 ** 0.5).to(torch.bfloat16)
        cache = torch.zeros((64, 128, 8, 4), dtype=torch.int32, device=dev)
        slots = torch.arange(16, device=dev, dtype=torch.int64) * 128
        for _ in range(3):
            ops.hash_encode_decode_step(xq, xk, slots, cache, r)
    elif what == "gather":
        nbp = 2000                                                                   # 2 x 524 MB pools
        kp = torch.randn((nbp, 128, 8, 128), device=dev, dtype=torch.bfloat16)
        vp = torch.randn((nbp, 128, 8, 128), device=dev, dtype=torch.bfloat16)
        sel = torch.randperm(nbp, device=dev, generator=g)[:16 * 32].to(torch.int32).view(16, 32)
        ok = torch.empty((16, 32 * 128, 8, 128), device=dev, dtype=torch.bfloat16)
        ov = torch.empty_like(ok)
        for _ in range(3):
            ops.gather_kv(kp, vp, sel, ok, ov)
    else:
        raise SystemExit(f"unknown --ncu-case {what}")
    torch.cuda.synchronize()
    print("ok", what)


# ----------------------------------------------------------------------------------------------
# where one decode step spends its time: device-timer stamps taken inside the kernels (trace build of the library)
# ----------------------------------------------------------------------------------------------
TIMELINE_POINTS = [
    ("encode", 0, "encode: entry"), ("encode", 1, "encode: dependency wait passed"), ("encode", 2, "encode: inputs staged"),
    ("encode", 3, "encode: end"),
    ("scan", 0, "scan: entry"), ("scan", 1, "scan: work items counted"), ("scan", 2, "scan: first item resolved"),
    ("scan", 3, "scan: first copy issued"), ("scan", 4, "scan: dependency wait passed"), ("scan", 5, "scan: first block landed"),
    ("scan", 6, "scan: first item scored"), ("scan", 7, "scan: first warp out of items"),
    ("select", 0, "select: entry"), ("select", 1, "select: dependency wait passed"), ("select", 2, "select: keys staged"),
    ("select", 3, "select: threshold known"), ("select", 4, "select: chosen blocks listed"), ("select", 5, "select: end"),
]


def run_timeline(shape: str) -> None:
    """One decode step (encode -> scan -> selection, one CUDA graph per layer) replayed back to back; after each of a
    few runs the stamps of the last step are read back.  Times are relative to the encode kernel's entry, thread 0
    of CTA 0 of each kernel.  decode16 = the headline shape, tp8 = config 3 as one of 8 ranks sees it."""
    trace_lib = os.path.join(ROOT, "unified_cache_management_b200", "libucmr_b200_trace.so")
    if not os.path.exists(trace_lib):
        raise SystemExit("no trace build: run  python -m unified_cache_management_b200.build --trace")
    os.environ["UCMR_LIBRARY"] = trace_lib
    import torch
    from unified_cache_management_b200 import ops
    dev = torch.device("cuda:0")
    B, Hkv, Hq, seq, BS, k, L = (16, 8, 32, 131072, 128, 16, 4) if shape == "decode16" else (8, 1, 8, 262144, 128, 32, 8)
    D, Wd = 128, 4
    mb = seq // BS
    NB = B * mb
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    caches = [rand_codes((NB, BS, Hkv, Wd), dev, g) for _ in range(L)]
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, mb).contiguous()
    sl = torch.full((B,), seq, dtype=torch.int32, device=dev)
    R = (torch.randn((D, 32 * Wd), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    qf = torch.randn((L, B, Hq, D), device=dev, generator=g).to(torch.bfloat16)
    kn = torch.randn((L, B, Hkv, D), device=dev, generator=g).to(torch.bfloat16)
    slots = (bt[:, mb - 1].to(torch.int64) * BS + (BS - 1)).contiguous()
    qc = torch.empty((B, Hq, Wd), dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    out = new_retrieval(B, Hkv, k, dev)

    def step(layer):
        ops.hash_encode_decode_step(qf[layer], kn[layer], slots, caches[layer], R, q_codes_out=qc)
        ops.hamming_topk(caches[layer], qc, bt, sl, k, reduce="sum", must_select=MUST_SELECT, workspace=ws, out=out,
                         want_scores=False, **STABLE)

    graphs = capture_graphs(step, L)
    runs = []
    for trial in range(5):
        for i in range(16 + trial):
            graphs[i % L].replay()
        torch.cuda.synchronize()
        tables = {u: ops.trace_read(u) for u in ("encode", "scan", "select")}
        t0 = tables["encode"][0]
        runs.append([(tables[u][i] - t0) / 1e3 for u, i, _ in TIMELINE_POINTS])
    med = [sorted(r[i] for r in runs)[len(runs) // 2] for i in range(len(TIMELINE_POINTS))]
    for (u, i, name), v, lo, hi in zip(TIMELINE_POINTS, med, [min(r[j] for r in runs) for j in range(len(med))],
                                       [max(r[j] for r in runs) for j in range(len(med))]):
        print(f"{name:34s} {v:8.2f} us   ({lo:.2f} .. {hi:.2f})")
    print(json.dumps({"timeline": shape, "unit": "us after the encode kernel's entry (median of 5 runs)",
                      "points": {name: round(v, 2) for (_, _, name), v in zip(TIMELINE_POINTS, med)}}))


SHARD_TIMELINE_POINTS = [
    ("scan", 0, "scan: entry"), ("scan", 3, "scan: first copy issued"), ("scan", 7, "scan: first warp out of items"),
    ("select", 0, "select: entry"), ("select", 1, "select: dependency wait passed"), ("select", 5, "select: records stored"),
    ("select", 6, "select: records fenced"), ("select", 13, "select: dependency wait passed (last CTA)"),
    ("select", 11, "select: records stored (last CTA)"), ("select", 12, "select: records fenced (last CTA)"),
    ("select", 7, "select: step number published"),
    ("select", 8, "merge: entry"), ("select", 9, "merge: every rank's step number seen"), ("select", 2, "merge: keys staged"),
    ("select", 3, "merge: threshold known"), ("select", 10, "merge: merged"),
]


def run_shard_timeline() -> None:
    """Config 4 over the ranks of this launch (torchrun), peer-memory exchange, one CUDA graph per layer-step: every
    rank prints where its step spends its time, relative to its own scan's entry (the device timers of different
    GPUs are not comparable).  "merge: every rank's step number seen" minus "merge: entry" is the time a rank waits
    for the slowest peer's records."""
    trace_lib = os.path.join(ROOT, "unified_cache_management_b200", "libucmr_b200_trace.so")
    if not os.path.exists(trace_lib):
        raise SystemExit("no trace build: run  python -m unified_cache_management_b200.build --trace")
    os.environ["UCMR_LIBRARY"] = trace_lib
    import torch
    from unified_cache_management_b200 import ops, sharded
    ranks = Ranks()
    ranks.init()
    cfg = EXTRA_WORKLOADS["million_token_sharded"]
    dev, world, rank = ranks.dev, ranks.world, ranks.rank
    if world < 2:
        raise SystemExit("--timeline shards needs at least two ranks (torchrun)")
    B, seq_total, Hkv, Hq, BS, k, L = cfg["B"], cfg["seq"], cfg["Hkv"], cfg["Hq"], cfg["BS"], cfg["k"], cfg["layers"]
    Wd, nblk_total = cfg["bits"] // 32, cfg["seq"] // cfg["BS"]
    per = nblk_total // world
    NB, kl = B * per, min(k, per)
    g = torch.Generator(device=dev)
    g.manual_seed(4000 + rank)
    caches = [rand_codes((NB, BS, Hkv, Wd), dev, g) for _ in range(L)]
    bt_local = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, per).contiguous()
    g.manual_seed(44)
    q = rand_codes((B, Hq, Wd), dev, g)
    seq_g = torch.full((B,), seq_total, dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, per, dev)
    plan = sharded.shard_plan(seq_g, BS, nblk_total, world, rank)
    o_s = torch.empty((B, Hkv, k), dtype=torch.float32, device=dev)
    o_i = torch.empty((B, Hkv, k), dtype=torch.int32, device=dev)
    st_word = torch.zeros(1, dtype=torch.int32, device=dev)
    ex = sharded.PeerExchange(B, Hkv, kl, dev)

    def step(layer):
        sharded.sharded_hamming_topk_p2p(caches[layer], q, bt_local, seq_g, k, BS, nblk_total, 1.0 / (BS * (Hq // Hkv)), ex,
                                         reduce="sum", must_select=MUST_SELECT, workspace=ws, plan=plan, status=st_word,
                                         out_scores=o_s, out_ids=o_i, **STABLE)

    for i in range(4):
        step(i % L)
    ranks.barrier()
    graphs = capture_graphs(step, L, warm=False)
    runs = []
    for trial in range(5):
        ranks.barrier()
        for i in range(16):
            graphs[i % L].replay()
        torch.cuda.synchronize()
        tables = {u: ops.trace_read(u) for u in ("scan", "select")}
        t0 = tables["scan"][0]
        runs.append([(tables[u][i] - t0) / 1e3 for u, i, _ in SHARD_TIMELINE_POINTS])
    med = [sorted(r[i] for r in runs)[len(runs) // 2] for i in range(len(SHARD_TIMELINE_POINTS))]
    line = {"timeline": "shards", "rank": rank, "ranks": world, "status_word": int(st_word.item()),
            "unit": "us after this rank's scan entry (median of 5 runs)",
            "points": {name: round(v, 2) for (_, _, name), v in zip(SHARD_TIMELINE_POINTS, med)}}
    for r in range(world):   # one rank after the other, rank 0 last
        ranks.barrier()
        if rank == (r + 1) % world:
            print(json.dumps(line), flush=True)
    ranks.close()


# ----------------------------------------------------------------------------------------------
def run_reference_arm(args, cfg, config, ranks):
    """The reference's CPU implementation of the path on the headline workload.  Loads nothing of the CUDA library:
    the inputs are made with numpy."""
    if ranks.rank != 0:
        return
    from oracle import oracle_c as OC
    W, K = max(args.warmup, 3), max(args.steps, 1)
    host = cpu_inputs(cfg)
    OC.use_all_cores()
    probe = cpu_step_factory(cfg, host, 1)
    t0 = time.perf_counter()
    probe()
    t1 = time.perf_counter() - t0
    n_req = int(max(1, min(cfg["B"], 1.0 / max(t1, 1e-6))))   # about a second per step at most
    step = cpu_step_factory(cfg, host, n_req)
    for _ in range(W):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(K):
        step()
        done += 1
        if time.perf_counter() - t0 > 150.0:   # keep the whole run within a few minutes
            break
    dt = time.perf_counter() - t0
    val = n_req * cfg["seq"] * done / dt
    sample = f"{n_req} of {cfg['B']} requests x {cfg['seq']} tokens per step, one layer, Bernoulli code bits"
    side = {}
    for name, fn in (("reference_backend", time_reference_backend), ("torch_formulation", time_torch_formulation)):
        try:
            side[name] = fn(cfg, host)
        except Exception as exc:  # noqa: BLE001
            side[name] = {"error": repr(exc)[:200]}
    print(json.dumps({"impl": "reference", "metric": "tokens_scored_per_sec", "value": val, "unit": "tokens/s",
                      "n_gpus": args.gpus, "steps": done, "warmup": W, "ms_per_step": dt / done * 1e3,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32",
                      "data": "synthetic", "config": config,
                      "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": OC.num_threads(), "kind": "port",
                                       "sample": sample, **side},
                      "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3_8b_decode16", choices=sorted(WORKLOADS) + sorted(EXTRA_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="headline workload only")
    ap.add_argument("--max-reps", type=int, default=400,
                    help="upper bound of the repetitions of a timed region (a profiler run wants few)")
    ap.add_argument("--exchange", default="both", choices=["both", "p2p", "nccl"],
                    help="million_token_sharded on several GPUs: how the candidate records travel")
    ap.add_argument("--timeline", default=None, choices=["decode16", "tp8", "shards"],
                    help="print where the time of one decode step goes (device-timer stamps inside the three kernels) "
                         "and exit; needs the trace build: python -m unified_cache_management_b200.build --trace")
    ap.add_argument("--ncu-case", default=None,
                    help="run a small single-kernel case for a profiler capture and exit "
                         "(scan, scan_min, scan_256bit, scan_mla, scan_bs16, scan_bs32, scan_tp8, select, encode, "
                         "encode_cache, encode_wide, encode_step, gather)")
    args = ap.parse_args()

    if args.ncu_case:
        run_profile_case(args.ncu_case)
        return
    if args.timeline == "shards":
        run_shard_timeline()
        return
    if args.timeline:
        run_timeline(args.timeline)
        return
    global MAX_REPS
    MAX_REPS = max(3, args.max_reps)

    ranks = Ranks()
    cfg = dict(WORKLOADS["llama3_8b_decode16"])
    W = max(args.warmup, 3)
    K = max(args.steps, 1)
    world = ranks.world
    config = dict(workload="llama3_8b_decode16", batch=cfg["B"], seq_len=cfg["seq"], kv_heads=cfg["Hkv"],
                  query_heads=cfg["Hq"], head_dim=cfg["D"], hash_bits=cfg["bits"], block_size=cfg["BS"],
                  topk_blocks=cfg["k"], must_select_blocks=list(MUST_SELECT), block_reduce="sum",
                  selection="per kv head", layers_resident=cfg["layers"],
                  l2="steps rotate over resident layer caches: inputs larger than L2",
                  parallelism=f"dp{world} (independent replicas, no collective)")

    if args.impl == "reference":
        if args.workload != "llama3_8b_decode16":
            if ranks.rank == 0:
                print(json.dumps({"impl": "reference",
                                  "unavailable": f"the CPU arm is wired for the headline workload only, not {args.workload}"}))
            return
        run_reference_arm(args, cfg, config, ranks)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the retrieval kernels)")
    ranks.init()
    dev, rank = ranks.dev, ranks.rank
    from unified_cache_management_b200 import ops
    peaks, peak_kind = _peaks()

    if args.workload in EXTRA_WORKLOADS:       # one of the other configs on its own, same JSON contract
        exch = ("p2p", "nccl") if args.exchange == "both" else (args.exchange,)
        fn = {"single_request_32k": suite_single_request, "paged_gather_b64": suite_paged_gather,
              "llama3_70b_tp": suite_tp}.get(args.workload)
        sampler = ClockSampler(ranks.local_rank)
        sampler.start()
        res = fn(ranks, K, W, peaks) if fn else suite_sharded(ranks, K, W, peaks, exchanges=exch)
        clocks = sampler.stop()
        if rank == 0:
            ms = res.get("ms_per_step")
            print(json.dumps({
                "metric": "tokens_scored_per_sec", "value": res.get("tokens_per_s"), "unit": "tokens/s", "n_gpus": world,
                "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True,
                "scaling": res.get("scaling", "weak"), "vs_baseline": None, "dtype": "u32", "data": "synthetic",
                "config": dict(workload=args.workload, l2="steps rotate over resident layer caches"),
                "gpu_launches": (res.get("gpu_launches_per_step") or 3) * K, "clocks": clocks, "detail": res}))
        ranks.close()
        return

    # ------------------------------------------------------------------ headline: config 1
    wl = build_workload(cfg, dev, seed=1 + rank)
    L = cfg["layers"]
    Wd, mb = wl["W"], wl["mb"]
    tokens_per_step = cfg["B"] * cfg["seq"]
    ws = ops.new_workspace(cfg["B"], cfg["Hkv"], mb, dev)
    q_codes = torch.empty((cfg["B"], cfg["Hq"], Wd), dtype=torch.int32, device=dev)
    out = new_retrieval(cfg["B"], cfg["Hkv"], cfg["k"], dev)

    def step(layer):
        ops.hash_encode_decode_step(wl["q"][layer], wl["k_new"][layer], wl["last_slot"], wl["caches"][layer], wl["R"],
                                    q_codes_out=q_codes)
        ops.hamming_topk(wl["caches"][layer], q_codes, wl["bt"], wl["seq_lens"], cfg["k"], reduce="sum",
                         must_select=MUST_SELECT, workspace=ws, out=out, want_scores=False, **STABLE)

    graphs = capture_graphs(step, L)
    for i in range(W):
        graphs[i % L].replay()
    sampler = ClockSampler(ranks.local_rank)
    sampler.start()

    def run_k():
        for i in range(K):
            graphs[i % L].replay()

    timing = timed_reps(run_k, ranks)
    ms_total = timing["ms"]

    # dominant kernel alone (the scan): K back-to-back launches on the current stream between one event pair, same
    # rotation over the layer caches, repeated like the step
    scores = torch.empty((cfg["B"], cfg["Hkv"], mb), dtype=torch.int32, device=dev)

    def scan_k():
        for i in range(K):
            ops.block_scores(wl["caches"][i % L], q_codes, wl["bt"], wl["seq_lens"], reduce="sum", out=scores,
                             **STABLE)

    for _ in range(2):
        scan_k()
    scan_t = timed_reps(scan_k, ranks)
    scan_ms_mean = scan_t["ms"] / K
    # the same launch as a CUDA graph of its own, replayed back to back: launches of different replays do not
    # overlap, so this is the duration of one launch including its own prologue and drain
    scan_graphs = capture_graphs(lambda layer: ops.block_scores(wl["caches"][layer], q_codes, wl["bt"], wl["seq_lens"],
                                                                reduce="sum", out=scores, **STABLE), L)

    def scan_iso_k():
        for i in range(K):
            scan_graphs[i % L].replay()

    scan_ms_isolated = timed_reps(scan_iso_k, ranks)["ms"] / K

    # end to end with HOST buffers: a step's inputs (q and the new keys, bf16) sit in page-locked host memory
    # and the selected block ids must land in page-locked host memory; the host waits for them every step.
    # The encode kernel reads the host inputs across the bus itself and the select kernel writes the ids to
    # the host buffer itself (unified addressing), so the transfers are inside the kernels of the step's CUDA
    # graph and no separate copy is enqueued.  Every step re-reads its inputs from host memory.
    q_pin = wl["q"].cpu().pin_memory()
    k_pin = wl["k_new"].cpu().pin_memory()
    res_host = torch.empty((cfg["B"], cfg["Hkv"], cfg["k"]), dtype=torch.int32).pin_memory()
    out_host = new_retrieval(cfg["B"], cfg["Hkv"], cfg["k"], dev, physical=res_host)

    def host_step(layer):
        ops.hash_encode_decode_step(q_pin[layer], k_pin[layer], wl["last_slot"], wl["caches"][layer], wl["R"],
                                    q_codes_out=q_codes)
        ops.hamming_topk(wl["caches"][layer], q_codes, wl["bt"], wl["seq_lens"], cfg["k"], reduce="sum",
                         must_select=MUST_SELECT, workspace=ws, out=out_host, want_scores=False, **STABLE)

    e2e_graphs = capture_graphs(host_step, L)

    def e2e_k():
        for i in range(K):
            e2e_graphs[i % L].replay()
            torch.cuda.current_stream().synchronize()     # the host reads the ids of every step

    for i in range(W):
        e2e_graphs[i % L].replay()
    torch.cuda.synchronize()
    e2e_t = timed_reps(e2e_k, ranks, host_clock=True)
    e2e_ms = e2e_t["ms"]
    clocks = sampler.stop()
    h2d = q_pin[0].numel() * 2 + k_pin[0].numel() * 2
    d2h = res_host.numel() * 4
    status = ops.workspace_status(ws)

    # checker legs, outside every timed region: both paths of the timed step against the CPU oracle (layer 0)
    parity = None
    if rank == 0:
        from oracle import oracle as O
        from oracle import oracle_c as OC
        OC.use_all_cores()
        graphs[0].replay()
        torch.cuda.synchronize()
        dev_ids = out.physical.cpu().numpy()
        e2e_graphs[0].replay()
        torch.cuda.synchronize()
        ref = OC.hamming_topk(u32(wl["caches"][0]), u32(q_codes), wl["bt"].cpu().numpy(), wl["seq_lens"].cpu().numpy(),
                              cfg["k"], O.REDUCE_SUM, False, must_select=MUST_SELECT)
        good = np.array_equal(dev_ids, ref["physical"]) and np.array_equal(res_host.numpy(), ref["physical"]) and \
            np.array_equal(out.logical.cpu().numpy(), ref["logical"])
        parity = "ok" if good else "MISMATCH"

    roofline_encode = time_bulk_encode(cfg, wl, dev, max(K, 20), peaks) if rank == 0 and world == 1 else None
    line = None
    if rank == 0:
        scan_t_s = scan_ms_mean * 1e-3
        sb = scan_bytes(cfg["B"], tokens_per_step, cfg["Hkv"], cfg["Hq"], Wd, mb, cfg["Hkv"])
        achieved = sb / scan_t_s / 1e9
        line = {
            "metric": "tokens_scored_per_sec", "value": world * tokens_per_step * K / (ms_total * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": config, "reps": timing["reps"],
            "rep_ms_per_step_min_max": [timing["ms_min"] / K, timing["ms_max"] / K],
            "timing": "K steps per repetition between barrier + events, median of `reps` repetitions, max over ranks",
            "per_gpu": tokens_per_step * K / (ms_total * 1e-3),
            "retrieval_latency_us": ms_total / K * 1e3, "parity": parity,
            "roofline": {"bound": "hbm", "kernel": "scan_ring_kernel (Hamming scan)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "frac_of_8tbs_spec": achieved / 8000.0,
                         # ncu (one launch of the half-batch case, 134.5 MB algorithmic): 134,328,576 B read +
                         # 3,549,440 B written = 1.025 x algorithmic; traffic grows with the blocks scanned, so the
                         # full launch is that ratio times its own algorithmic bytes.
                         "traffic": int(round(1.025 * sb)),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a half-batch launch, scaled by blocks scanned",
                         "algorithmic_bytes_per_launch": sb,
                         "launch_us_mean": scan_t_s * 1e6, "launches_timed": K * scan_t["reps"],
                         "launch_us_isolated": scan_ms_isolated * 1e3,
                         "note": "launch_us_mean: K launches back to back on one stream, where a launch sets itself up "
                                 "while its predecessor drains (programmatic dependent launch), as consecutive layers "
                                 "do; launch_us_isolated: the launch as a CUDA graph of its own, replays do not overlap"},
            "e2e": {"value": world * tokens_per_step * K / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / K, "reps": e2e_t["reps"],
                    "rep_ms_per_step_min_max": [e2e_t["ms_min"] / K, e2e_t["ms_max"] / K],
                    "transfer": "kernels read the pinned host inputs and write the ids to pinned host memory "
                                "themselves (unified addressing); host waits for every step"},
            "gpu_launches": 3 * K, "device_status_word": status, "clocks": clocks,
        }
        if roofline_encode is not None:
            line["roofline_encode"] = roofline_encode
        if not args.no_cpu_baseline and world == 1:   # baselines are timed on one rank with the box to itself
            ref_gpu = time_reference_gpu(cfg, wl, dev)
            if ref_gpu is not None:
                line["reference_gpu_kernel"] = ref_gpu
            host = cpu_inputs(cfg)
            base = time_cpu(cfg, host)
            for name, fn in (("reference_backend", time_reference_backend), ("torch_formulation", time_torch_formulation)):
                try:
                    base[name] = fn(cfg, host)
                except Exception as exc:  # noqa: BLE001
                    base[name] = {"error": repr(exc)[:200]}
            line["cpu_baseline"] = base
            del host
    # free the headline workload before the other configs (config 2 alone needs 112 GB)
    del wl, graphs, scan_graphs, e2e_graphs, scores
    torch.cuda.empty_cache()
    ranks.barrier()
    if not args.no_configs:
        suite = run_config_suite(ranks, K, W, peaks)
        if rank == 0:
            line["configs"] = suite
            rf = suite.get("paged_gather_b64", {}).get("roofline_gather")
            if rf:
                line["roofline_gather"] = rf
    if rank == 0:
        print(json.dumps(line))
    ranks.close()


if __name__ == "__main__":
    main()
