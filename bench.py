"""Benchmark of the decode-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the batched long-context config): a Qwen3-8B-shaped decode layer — batch 8 per GPU,
context 32768 per sequence, 32 query / 8 KV heads, head_dim 128, bf16 queries, 16-token pages
laid out by a seeded random permutation, the KV cache pre-quantized from N(0,1) data by the
cache-write kernel — and one step = one decode-attention pass over 36 layers (36 distinct layer
caches, 335 MB each: every launch streams far more than L2 holds).  Metric: decode-attention
tokens/s (batch x GPUs / step time).  With N > 1 every GPU runs its own batch (sequences are
independent: no collective on the data path, weak scaling).

Prints ONE JSON line (rank 0).  `value` is timed on the device with inputs resident in HBM
(CUDA-graph replay of the 36 launches); `e2e` is the same step through the package's
public API with host buffers: the step's queries and new K/V rows are copied from pinned host
memory, the new rows are written into the cache, and the outputs are copied back, all inside
the timed region.  `roofline` is for the decode kernel alone, timed per launch with CUDA events
recorded by the library around that kernel.  `parity` compares layer 0's output of the timed
workload with the CPU oracle (the run fails if the bar is missed).  `cpu_baseline` / `--impl
reference` time the reference's CPU path on full 32768-token sequence passes of the same data:
its torch calls restated (oracle/torch_cpu_path.py, all torch threads) and, beside it under
`port`, the C restatement on all host threads.

Further sections of the same line: `mixed` (64 mixed-length sequences, sharded over the GPUs by
sequence) and `kv_split` (one 1,048,576-token sequence with 8 queries, KV axis split over the
GPUs, partials exchanged by the kernels themselves and, for comparison, by an NCCL all-gather),
each with its own oracle parity check; with N > 1 also `strong` (the stated batch of 8 split
over the GPUs by sequence and by KV head), and `short_chunk` (8 new tokens per sequence over batch
8 x 32768 cached tokens through the causal wide-tile kernel, against the same tokens as decode
rows).  `--sections none` leaves them out.

Other lines on request: `--workload config3 | config4 | sweep` (the parity-test shapes, timed) and
`--workload head_sizes` (cache write, decode and bulk dequantization for head sizes 64 and 256 beside
128, each against its algorithmic bytes, with oracle parity on a slice).
"""
from __future__ import annotations

import argparse
import json
import math
import os

# stdout carries the one JSON line: NCCL prints its version banner (debug levels VERSION and WARN) and its other
# messages to stdout unless told where to write them, and it honours the file only above level VERSION
if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "WARN"
os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

HQ, HKV, D, PAGE, SLOT = 32, 8, 128, 16, 80
ALG_BYTES_PER_TOKEN_HEAD = 136  # K (64 code + 4 norm bytes) + V (64 + 4)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--num-ctas", type=int, default=0)
    ap.add_argument("--c4-tokens", type=int, default=1_048_576,
                    help="--workload config4: tokens of the sequence (a smaller case for a profiler capture)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="config4 on several GPUs: partials exchanged by the kernels themselves (peer stores + "
                         "flags) or by an NCCL all-gather")
    ap.add_argument("--sections", default="all",
                    help="comma list of the extra sections of the config-1 line: mixed, kv_split, strong, short_chunk; all | none")
    ap.add_argument("--workload", default="config1", choices=["config1", "config3", "config4", "sweep", "head_sizes"],
                    help="config1 (default, the headline): batch 8 x 32k per GPU; config3: 64 mixed lengths sharded by "
                         "sequence; config4: one 1M-token sequence, KV axis split over the GPUs, NCCL merge; "
                         "head_sizes: write / decode / dequantization for head sizes 64 and 256")
    return ap.parse_args()


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (C restatement of the reference's torch CPU path) on a bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_decode_rate(cache_np, block_table_np, q_np, signs_np, ctx_sample: int, threads: int, reps: int = 1):
    """KV token-heads per second of the CPU dequant-attention path, `threads` sequences in
    parallel (`reps` rounds of them), each attending `ctx_sample` tokens of the real quantized cache."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import tq_oracle
    nseq = q_np.shape[0]
    lens = np.full(1, ctx_sample, np.int32)

    def one(i):
        b = i % nseq
        return tq_oracle.decode_paged(q_np[b:b + 1], cache_np, block_table_np[b:b + 1], lens, signs_np,
                                      1.0 / math.sqrt(D))
    one(0)
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, range(threads * reps)))
    dt = time.perf_counter() - t0
    return threads * reps * ctx_sample * HKV / dt, dt


def cpu_model() -> str:
    try:
        for ln in Path("/proc/cpuinfo").read_text().splitlines():
            if ln.startswith("model name"):
                return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def torch_decode_rate(cache_np, block_table_np, q_np, signs_np, ctx: int, passes: int):
    """KV token-heads per second of the reference's torch CPU path (oracle/torch_cpu_path.py), one
    full `ctx`-token sequence per pass, torch's own intra-op threads; returns (rate, seconds)."""
    from oracle import torch_cpu_path, tq_oracle
    cen, _ = tq_oracle.codebook(D, 4)
    cache = torch.from_numpy(cache_np)
    bt = torch.from_numpy(block_table_np)
    q = torch.from_numpy(q_np)
    signs = torch.from_numpy(signs_np)
    cen = torch.from_numpy(cen)
    nseq = q.shape[0]
    lens = [ctx]
    t0 = time.perf_counter()
    for i in range(passes):
        b = i % nseq
        torch_cpu_path.decode_attention(q[b:b + 1], cache, bt[b:b + 1], lens, signs, cen, 1.0 / math.sqrt(D))
    dt = time.perf_counter() - t0
    return passes * ctx * HKV / dt, dt


def torch_write_rate(k, v, slots, signs, num_blocks: int, reps: int = 1):
    """Tokens per second of the reference's torch CPU quantizer + pack + scatter."""
    from oracle import torch_cpu_path, tq_oracle
    _, bnd = tq_oracle.codebook(D, 4)
    bnd = torch.from_numpy(bnd)
    cache = torch.zeros((2, num_blocks, PAGE, HKV, SLOT), dtype=torch.uint8)
    t0 = time.perf_counter()
    for _ in range(reps):
        torch_cpu_path.write_kv_cache(cache, k, v, signs, bnd, slots)
    dt = time.perf_counter() - t0
    return k.shape[0] * reps / dt, dt


def oracle_parity(got, want, what: str) -> dict:
    """The parity bar of the tests, evaluated inside the benchmark: per element
    |got - want| <= 2e-3 + 1e-2 |want| and relative (Frobenius) <= 1e-2 must hold or the run fails;
    the strict reading (max-abs <= 2e-3) is reported beside it."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    ok = bool((err <= 2e-3 + 1e-2 * np.abs(want)).all() and rel <= 1e-2)
    res = {"against": "CPU oracle (dequant-attention restatement) on the same bytes", "what": what,
           "max_abs": float(err.max()), "rel": rel, "strict_2e-3": bool(err.max() <= 2e-3), "ok": ok,
           "ref_max_abs": float(np.abs(want).max()), "ref_rms": float(np.sqrt((want ** 2).mean()))}
    if not ok:
        print(json.dumps({"parity_failure": res}), flush=True)
        raise SystemExit(f"parity bar missed: {res}")
    return res


def cpu_write_rate(k_np, v_np, slots_np, signs_np, num_blocks: int, threads: int, reps: int = 1):
    """Tokens per second of the CPU cache write (the C port of the torch quantizer + pack + scatter),
    `threads` chunks of the sample in parallel (ctypes releases the GIL)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import tq_oracle
    cache = np.zeros((2, num_blocks, PAGE, HKV, SLOT), np.uint8)
    n = k_np.shape[0]
    chunks = [(i * n // threads, (i + 1) * n // threads) for i in range(threads)]

    def one(c):
        a, b = c
        tq_oracle.write_kv_cache(cache, k_np[a:b], v_np[a:b], signs_np, slots_np[a:b], D)
    one((0, min(n, 16)))
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, chunks * reps))
    dt = time.perf_counter() - t0
    return n * reps / dt, dt


def synthetic_host_cache(ctx: int, batch: int, seed: int):
    """A host-side quantized cache for the CPU arm when no GPU copy is at hand (reference arm)."""
    from oracle import tq_oracle
    from turboquant_b200 import synthetic
    case = synthetic.decode_case(seed=seed, seq_lens=[ctx] * batch, dtype=torch.bfloat16)
    signs = synthetic.make_signs(D, 42).numpy()
    cache = np.zeros((2, case.num_blocks, PAGE, HKV, SLOT), np.uint8)
    tq_oracle.write_kv_cache(cache, case.k.float().numpy(), case.v.float().numpy(), signs,
                             case.slot_mapping.numpy(), D)
    return cache, case.block_table.numpy(), case.q.float().numpy(), signs


def cpu_arm(cache_np, bt_np, q_np, signs_np, ctx: int, layers: int, torch_passes: int, port_reps: int):
    """Both CPU figures on full `ctx`-token sequence passes of one layer's quantized cache,
    as tokens/s of the whole `layers`-layer step: the torch path (the named baseline) and the C port."""
    threads = os.cpu_count() or 1
    per_token = ctx * HKV * layers                        # KV token-heads one decode token attends
    t_rate, t_dt = torch_decode_rate(cache_np, bt_np, q_np, signs_np, ctx, torch_passes)
    p_rate, p_dt = cpu_decode_rate(cache_np, bt_np, q_np, signs_np, ctx, threads, port_reps)
    scaled = f"x {HKV} KV heads of one layer's config-1 cache, scaled to {layers} layers per token"
    return {
        "value": t_rate / per_token, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "torch-restatement",
        "sample": f"{torch_passes} sequence passes x {ctx} tokens {scaled} ({t_dt:.2f} s)",
        "cpu": cpu_model(), "host_cores": threads, "torch": torch.__version__,
        "port": {"value": p_rate / per_token, "unit": "tokens/s", "cores": threads, "kind": "port",
                 "sample": f"{threads * port_reps} sequence passes x {ctx} tokens {scaled} ({p_dt:.2f} s)"},
    }


def run_reference(args):
    """The reference's CPU implementation of the path on the box's host cores: its torch calls
    restated (the reference's own modules cannot travel to the GPU box), one full 32768-token
    sequence pass of one layer per step, torch's intra-op threads; the C port beside it."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    ctx = args.ctx
    cache, bt, q, signs = synthetic_host_cache(ctx, 2, seed=1)
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt = torch_decode_rate(cache, bt, q, signs, ctx, 1)
        if i >= args.warmup:
            rates.append((r, dt))
    rate = statistics.median(r for r, _ in rates)
    per_token = ctx * HKV * args.layers
    value = rate / per_token
    threads = os.cpu_count() or 1
    p_rate, p_dt = cpu_decode_rate(cache, bt, q, signs, ctx, threads, 1)
    sample = (f"one sequence pass x {ctx} tokens x {HKV} KV heads of config-1-shaped quantized cache per step "
              f"(one layer), scaled to {args.layers} layers per token")
    line = {
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.median(dt for _, dt in rates), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "global_batch": args.batch * args.gpus,
                   "note": "CPU arm: the reference's torch CPU path (restated call for call), torch intra-op threads"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "torch-restatement",
                         "sample": sample, "cpu": cpu_model(), "host_cores": threads, "torch": torch.__version__,
                         "port": {"value": p_rate / per_token, "unit": "tokens/s", "cores": threads, "kind": "port",
                                  "sample": f"{threads} sequence passes x {ctx} tokens ({p_dt:.2f} s)"}},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(args):
    return (f"config1: Qwen3-8B-shaped decode layer, batch {args.batch}/GPU x ctx {args.ctx}, {HQ}q/{HKV}kv heads, "
            f"head_dim {D}, bf16 q, 16-token pages (seeded random permutation), {args.layers} layers per step")


# ------------------------------------------------------------------------------------------------
# Extra sections of the config-1 line: the other BASELINE configs and the multi-GPU splits
# ------------------------------------------------------------------------------------------------
def _dist_max(ms: float, world: int, dev) -> float:
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def _time_steps(fn, steps: int, world: int, dev) -> float:
    """ms per step: barrier + synchronize on both sides, CUDA events, max over ranks."""
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = _dist_max(e0.elapsed_time(e1), world, dev)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    return ms / steps


def _fill_sequence(attn, cache, block_table_row, n_tokens, gen, dev, chunk=65536, heads=HKV):
    """Quantize seeded N(0,1) K/V for one sequence into its pages with the cache-write kernel."""
    for t0 in range(0, n_tokens, chunk):
        n = min(chunk, n_tokens - t0)
        k = torch.randn(n, heads, D, generator=gen, device=dev).to(torch.bfloat16)
        v = torch.randn(n, heads, D, generator=gen, device=dev).to(torch.bfloat16)
        tok = torch.arange(t0, t0 + n, device=dev)
        slots = block_table_row.long()[tok // PAGE] * PAGE + tok % PAGE
        attn.write(k, v, cache, slots)


def section_mixed(args, rank, world, dev, peak):
    """Config 3: 64 sequences, lengths log-uniform in [512, 131072] (seed 3), one layer, sharded
    over the ranks by sequence (longest first): no collective on the data path.  Every rank
    checks its own shard against the oracle."""
    from oracle import tq_oracle
    from turboquant_b200 import synthetic
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    from turboquant_b200.parallel import shard_sequences
    lens_all = synthetic.mixed_lengths(seed=3, n=64)
    shards = shard_sequences(lens_all, world)
    lens = [lens_all[i] for i in shards[rank]]
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    bt_cpu, _, nb = synthetic.paged_layout(lens, seed=3 + rank)
    bt = bt_cpu.to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3 + 1000 * rank)
    ncache = 2   # alternated so that consecutive launches stream different memory (each far larger than L2)
    caches = [torch.zeros(kv_cache_shape(nb, PAGE, HKV, D), dtype=torch.uint8, device=dev) for _ in range(ncache)]
    for c in caches:
        for b, n in enumerate(lens):
            _fill_sequence(attn, c, bt[b], n, gen, dev)
    q = torch.randn(len(lens), HQ, D, generator=gen, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    state = {"i": 0}

    def step():
        attn.decode(q, caches[state["i"] % ncache], bt, sl, out)
        state["i"] += 1
    for _ in range(4):
        step()
    steps = max(args.steps, 10)
    ms = _time_steps(step, steps, world, dev)
    attn.decode(q, caches[0], bt, sl, out)
    torch.cuda.synchronize()
    status = attn.status(len(lens), dev)
    want = tq_oracle.decode_paged_parallel(q.float().cpu().numpy(), caches[0].cpu().numpy(), bt_cpu.numpy(),
                                           np.asarray(lens, np.int32), attn.signs(dev).cpu().numpy(), 1.0 / math.sqrt(D),
                                           threads=max(1, (os.cpu_count() or 1) // world))
    par = oracle_parity(out.float().cpu().numpy(), want, f"rank {rank}'s shard, all {len(lens)} sequences")
    worst = _dist_max(par["max_abs"], world, dev)
    loads = [sum(lens_all[i] for i in sh) for sh in shards]
    alg = sum(lens_all) * HKV * ALG_BYTES_PER_TOKEN_HEAD
    ach = alg / (ms * 1e-3) / 1e9
    del caches
    torch.cuda.empty_cache()
    return {"workload": "config3: 64 sequences, lengths log-uniform in [512, 131072] (seed 3), one layer, sharded over "
                        "the GPUs by sequence (greedy by length), no collective",
            "total_tokens": sum(lens_all), "ms_per_step": ms, "tokens_per_s": 64 / (ms * 1e-3), "steps": steps,
            "achieved_GBps": ach, "frac_of_n_peak": ach / (peak * world), "algorithmic_bytes": alg,
            "load_imbalance_max_over_mean": max(loads) / (sum(loads) / world), "status": status,
            "parity": dict(par, max_abs_over_ranks=worst), "scaling": "strong",
            "limit": "whole call (decode + merge); bounded by the most loaded rank and the fixed cost of a call"}


def section_short_chunk(args, rank, world, dev, peak):
    """A chunk of 8 new tokens per sequence over batch 8 x 32768 cached tokens (a short continuation
    of a prefill, or the verification step of speculative decoding with 8 draft tokens), one layer,
    the same on every rank: (a) one pass of the causal wide-tile kernel over the quantized cache,
    (b) the same 8 tokens as 8 plain decode rows per sequence (what the reference's decode op would
    need: one query per batch row), (c) the bulk dequantization of the whole context to dense bf16
    K / V alone, which a dense attention kernel would still have to follow.  Parity of (a) against
    the oracle with one batch row per query token, first sequence."""
    from oracle import tq_oracle
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    B, L, NQ = 8, 32768, 8
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    pages = L // PAGE
    nb = B * pages
    bt = torch.randperm(nb, generator=torch.Generator().manual_seed(8)).view(B, pages).to(torch.int32).to(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(8)
    caches = [torch.zeros(kv_cache_shape(nb, PAGE, HKV, D), dtype=torch.uint8, device=dev) for _ in range(2)]
    for c in caches:
        for b in range(B):
            _fill_sequence(attn, c, bt[b], L, gen, dev)
    q = torch.randn(B, NQ, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
    sl = torch.full((B,), L, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    state = {"i": 0}

    def causal():
        attn.decode_causal(q, caches[state["i"] % 2], bt, sl, out)
        state["i"] += 1
    rep_bt = bt.repeat_interleave(NQ, dim=0).contiguous()
    rep_sl = (sl.repeat_interleave(NQ) - torch.arange(NQ - 1, -1, -1, dtype=torch.int32, device=dev).repeat(B)).contiguous()
    q_rows, out_rows = q.view(B * NQ, HQ, D), torch.empty(B * NQ, HQ, D, dtype=q.dtype, device=dev)

    def rows():
        attn.decode(q_rows, caches[state["i"] % 2], rep_bt, rep_sl, out_rows)
        state["i"] += 1
    for _ in range(3):
        causal()
        rows()
    steps = max(args.steps, 10)
    ms_causal = _time_steps(causal, steps, world, dev)
    ms_rows = _time_steps(rows, steps, world, dev)
    cached = torch.full((B,), L - NQ, dtype=torch.int32, device=dev)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev) * (L - NQ)
    for _ in range(2):
        attn.dequant_cached(caches[0], bt, cached, cu, B * (L - NQ))
    ms_dequant = _time_steps(lambda: attn.dequant_cached(caches[state["i"] % 2], bt, cached, cu, B * (L - NQ)), steps, world, dev)
    attn.decode_causal(q, caches[0], bt, sl, out)
    attn.decode(q_rows, caches[0], rep_bt, rep_sl, out_rows)
    torch.cuda.synchronize()
    status = attn.status(B, dev, NQ)
    want = tq_oracle.decode_paged_parallel(q[0].float().cpu().numpy(), caches[0].cpu().numpy(), rep_bt[:NQ].cpu().numpy(),
                                           rep_sl[:NQ].cpu().numpy(), attn.signs(dev).cpu().numpy(), 1.0 / math.sqrt(D),
                                           threads=max(1, (os.cpu_count() or 1) // world))
    par = oracle_parity(out[0].float().cpu().numpy(), want, "the 8 query tokens of sequence 0, 32768 cached tokens")
    same = float((out.view(B * NQ, HQ, D).float() - out_rows.float()).abs().max())
    alg = B * L * HKV * ALG_BYTES_PER_TOKEN_HEAD
    del caches
    torch.cuda.empty_cache()
    return {"workload": "8 new tokens per sequence over batch 8 x 32768 cached tokens, one layer, per GPU",
            "causal_one_pass": {"ms": ms_causal, "new_tokens_per_s": B * NQ / (ms_causal * 1e-3),
                                "achieved_GBps": alg / (ms_causal * 1e-3) / 1e9, "frac": alg / (ms_causal * 1e-3) / 1e9 / peak},
            "as_decode_rows": {"ms": ms_rows, "rows": B * NQ, "new_tokens_per_s": B * NQ / (ms_rows * 1e-3)},
            "bulk_dequant_of_the_context_alone": {"ms": ms_dequant},
            "speedup_over_decode_rows": ms_rows / ms_causal, "max_abs_difference_from_decode_rows": same,
            "status": status, "parity": par, "steps": steps}


def section_kv_split(args, rank, world, dev, peak):
    """Config 4: one sequence of 1,048,576 tokens, 8 decode queries, one layer.  The KV axis is split
    contiguously over the ranks; every rank decodes its range for all queries, the rotated partials
    + LSE are exchanged (kernel-side: peer stores + flags; and through an NCCL all-gather) and merged
    on every rank.  Parity: every rank runs the oracle over its own range for two of the queries,
    the oracle partials are merged on rank 0 and compared with the GPU result."""
    from oracle import tq_oracle
    from turboquant_b200 import _cabi
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    from turboquant_b200.parallel import kv_ranges, kv_split_decode
    total, nq = 1_048_576, 8
    a, b = kv_ranges(total, world)[rank]
    n_local = b - a
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    pages = (n_local + PAGE - 1) // PAGE
    bt_row = torch.randperm(pages, generator=torch.Generator().manual_seed(4 + rank)).to(torch.int32).to(dev)
    cache = torch.zeros(kv_cache_shape(pages, PAGE, HKV, D), dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4 + 1000 * rank)
    _fill_sequence(attn, cache, bt_row, n_local, gen, dev)
    qgen = torch.Generator(device=dev)
    qgen.manual_seed(123457)                              # the same queries on every rank; a stream of their own,
    #                                                       not one of the ranks' K/V streams (seeds 4 + 1000 r)
    share = min(nq, _cabi.decode_max_queries_per_seq(HQ, HKV))   # queries that ride one pass over the KV
    rows = nq // share
    q = torch.randn(rows, share, HQ, D, generator=qgen, device=dev).to(torch.bfloat16)
    bt = bt_row.unsqueeze(0).expand(rows, -1).contiguous()  # every row is the same sequence
    sl = torch.full((rows,), n_local, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    steps = max(args.steps, 10)
    res = {"workload": "config4: one 1,048,576-token sequence, 8 decode queries, one layer, KV axis split contiguously "
                       "over the GPUs, partial (o, lse) exchanged and merged on every GPU",
           "passes_over_the_kv": rows, "queries_per_pass": share, "steps": steps,
           "exchange_bytes_per_rank": nq * HQ * (D + 1) * 4, "scaling": "strong"}
    alg = total * HKV * ALG_BYTES_PER_TOKEN_HEAD

    def rate(ms):
        ach = alg / (ms * 1e-3) / 1e9
        return {"ms_per_step": ms, "tokens_per_s": nq / (ms * 1e-3), "achieved_GBps": ach,
                "frac_of_n_peak": ach / (peak * world)}
    if world > 1:
        from turboquant_b200.parallel import KVSplitExchange
        ex = KVSplitExchange(attn, rows, share, dev)
        for _ in range(4):
            ex.decode(q, cache, bt, sl, out)
        res["kernel_exchange"] = rate(_time_steps(lambda: ex.decode(q, cache, bt, sl, out), steps, world, dev))
        out_nccl = torch.empty_like(q)
        for _ in range(4):
            kv_split_decode(attn, q, cache, bt, sl, out_nccl)
        res["nccl_all_gather"] = rate(_time_steps(lambda: kv_split_decode(attn, q, cache, bt, sl, out_nccl), steps, world, dev))
        ex.decode(q, cache, bt, sl, out)
        torch.cuda.synchronize()
        res["exchange_status"] = int(_dist_max(float(ex.status()), world, dev))
        res["nccl_equals_kernel_exchange"] = bool(torch.equal(out, out_nccl))
        res.update(res["kernel_exchange"])
    else:
        for _ in range(4):
            attn.decode(q, cache, bt, sl, out)
        res.update(rate(_time_steps(lambda: attn.decode(q, cache, bt, sl, out), steps, world, dev)))
        torch.cuda.synchronize()
    res["decode_status"] = int(_dist_max(float(attn.status(rows, dev, share)), world, dev))
    # ---- parity of two of the queries: oracle partial per rank (natural-log LSE), merged on rank 0
    pq = [0, nq - 1]
    qsel = q.view(nq, HQ, D)[pq].float().cpu().numpy()                      # [2, 32, 128]
    qv = qsel.reshape(len(pq), HKV, HQ // HKV, D).transpose(1, 0, 2, 3).reshape(1, len(pq) * HQ, D)
    po, pl = tq_oracle.decode_paged_parallel(qv, cache.cpu().numpy(), bt_row.cpu().numpy()[None],
                                             np.array([n_local], np.int32), attn.signs(dev).cpu().numpy(),
                                             1.0 / math.sqrt(D), threads=max(1, (os.cpu_count() or 1) // world),
                                             chunk_tokens=16384, return_lse=True)
    po_t, pl_t = torch.from_numpy(po).to(dev), torch.from_numpy(pl).to(dev)
    if world > 1:
        import torch.distributed as dist
        go = [torch.empty_like(po_t) for _ in range(world)]
        gl = [torch.empty_like(pl_t) for _ in range(world)]
        dist.all_gather(go, po_t)
        dist.all_gather(gl, pl_t)
        po_all = torch.stack(go).cpu().numpy()
        pl_all = torch.stack(gl).cpu().numpy()
    else:
        po_all, pl_all = po[None], pl[None]
    if rank == 0:
        merged, _ = tq_oracle.merge_partials(po_all, pl_all)
        want = merged.reshape(HKV, len(pq), HQ // HKV, D).transpose(1, 0, 2, 3).reshape(len(pq), HQ, D)
        got = out.view(nq, HQ, D)[pq].float().cpu().numpy()
        res["parity"] = oracle_parity(got, want, f"queries {pq} of 8, all 1,048,576 tokens, oracle partials merged over the ranks")
    # ---- the same sequence whole on one GPU, same run (rank 0), for the speed-up
    if world > 1:
        import torch.distributed as dist
        if rank == 0:
            pages1 = total // PAGE
            bt1 = torch.randperm(pages1, generator=torch.Generator().manual_seed(4)).to(torch.int32).to(dev)
            cache1 = torch.zeros(kv_cache_shape(pages1, PAGE, HKV, D), dtype=torch.uint8, device=dev)
            _fill_sequence(attn, cache1, bt1, total, gen, dev)
            bt1r = bt1.unsqueeze(0).expand(rows, -1).contiguous()
            sl1 = torch.full((rows,), total, dtype=torch.int32, device=dev)
            for _ in range(3):
                attn.decode(q, cache1, bt1r, sl1, out_nccl)
            ms1 = _time_steps(lambda: attn.decode(q, cache1, bt1r, sl1, out_nccl), steps, 1, dev)
            res["one_gpu_same_run"] = rate(ms1)
            res["one_gpu_same_run"]["frac_of_n_peak"] *= world          # one GPU's peak
            res["speedup_over_one_gpu"] = ms1 / res["ms_per_step"]
            del cache1
        dist.barrier()
        res["limit"] = ("per rank: 1/N of the KV (the streaming part scales) + the fixed cost of a call (plan, query rotation, "
                        "first stage, merge: about 20 us) + the exchange: peer stores of 132 KB to every rank, a release flag "
                        "per source, then the flag-gated merge")
    del cache
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    from turboquant_b200 import _cabi
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    B, L, NL = args.batch, args.ctx, args.layers
    pages_per_seq = (L + PAGE - 1) // PAGE
    nb = B * pages_per_seq
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, seed=42, num_ctas=args.num_ctas)

    # ---- inputs: seeded, generated on the device, quantized by the cache-write kernel -----------
    gen = torch.Generator(device=dev)
    gen.manual_seed(1 + 1000 * rank)
    cpu_gen = torch.Generator().manual_seed(1 + 1000 * rank)
    block_table = torch.randperm(nb, generator=cpu_gen).view(B, pages_per_seq).to(torch.int32).to(dev)
    seq_lens = torch.full((B,), L, dtype=torch.int32, device=dev)
    caches = torch.zeros((NL,) + kv_cache_shape(nb, PAGE, HKV, D), dtype=torch.uint8, device=dev)
    tok = torch.arange(L, device=dev)
    for layer in range(NL):
        for b in range(B):
            k = torch.randn(L, HKV, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            v = torch.randn(L, HKV, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            slots = block_table[b].long()[tok // PAGE] * PAGE + tok % PAGE
            attn.write(k, v, caches[layer], slots)
    del k, v
    q_dev = torch.randn(NL, B, HQ, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    out_dev = torch.empty_like(q_dev)
    torch.cuda.synchronize()

    def step_resident():
        for layer in range(NL):
            attn.decode(q_dev[layer], caches[layer], block_table, seq_lens, out_dev[layer])

    # ---- e2e step: host buffers, copies inside the timed region, through the public API ----------
    q_host = q_dev.cpu().pin_memory()
    newk_host = torch.randn(NL, B, HKV, D, generator=cpu_gen).to(torch.bfloat16).pin_memory()
    newv_host = torch.randn(NL, B, HKV, D, generator=cpu_gen).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(NL, B, HQ, D, dtype=torch.bfloat16).pin_memory()
    q_in = torch.empty_like(q_dev)
    newk = torch.empty(NL, B, HKV, D, dtype=torch.bfloat16, device=dev)
    newv = torch.empty_like(newk)
    out_e2e = torch.empty_like(q_dev)
    # the new token of every sequence overwrites its last position (the cache stays full-length)
    last_slots = (block_table[:, (L - 1) // PAGE].long() * PAGE + (L - 1) % PAGE).contiguous()

    # The copies run on two copy streams beside the kernels: the inputs of the next few layers arrive
    # while the current ones compute, and finished outputs leave the same way.  Chunks of a few layers
    # keep the number of cross-stream waits (each one ends the kernels' programmatic overlap) small;
    # the first and last chunk are one layer so that the exposed head and tail copies stay short.
    bounds = sorted(set([0, 1] + list(range(4, NL - 1, 4)) + [NL - 1, NL]))
    chunks = [(a, b) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in chunks]
    ev_done = [torch.cuda.Event() for _ in chunks]

    def step_e2e():
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        with torch.cuda.stream(copy_in):
            for (a, b), ev in zip(chunks, ev_in):
                q_in[a:b].copy_(q_host[a:b], non_blocking=True)
                newk[a:b].copy_(newk_host[a:b], non_blocking=True)
                newv[a:b].copy_(newv_host[a:b], non_blocking=True)
                ev.record(copy_in)
        for (a, b), e_in, e_done in zip(chunks, ev_in, ev_done):
            main.wait_event(e_in)
            for layer in range(a, b):
                attn.write(newk[layer], newv[layer], caches[layer], last_slots)
                attn.decode(q_in[layer], caches[layer], block_table, seq_lens, out_e2e[layer])
            e_done.record(main)
            copy_out.wait_event(e_done)
            with torch.cuda.stream(copy_out):
                out_host[a:b].copy_(out_e2e[a:b], non_blocking=True)
        main.wait_stream(copy_in)
        main.wait_stream(copy_out)

    h2d = q_host.numel() * 2 + newk_host.numel() * 2 + newv_host.numel() * 2
    d2h = out_host.numel() * 2

    # warm-up (also sets kernel attributes and allocates workspaces before any capture)
    for _ in range(max(args.warmup, 3)):
        step_resident()
    torch.cuda.synchronize()
    assert attn.status(B, dev) == 0, "decode kernel reported a failed wait"

    graph = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_resident()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                step_resident()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()

    def timed(fn, steps):
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(graph.replay if graph is not None else step_resident, args.steps)
    ms_step = ms_total / args.steps
    value = world * B / (ms_step * 1e-3)

    for _ in range(3):
        step_e2e()
    e2e_fn = step_e2e
    if not args.no_graph:
        # the same calls (copies from and to pinned host memory included) captured once and replayed,
        # as a serving engine replays its decode step
        torch.cuda.synchronize()
        graph_e2e = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph_e2e, stream=side):
                step_e2e()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(2):
            graph_e2e.replay()
        torch.cuda.synchronize()
        e2e_fn = graph_e2e.replay
    ms_e2e = timed(e2e_fn, args.steps) / args.steps
    e2e_value = world * B / (ms_e2e * 1e-3)

    # ---- roofline of the decode kernel: per-launch device time from events around that kernel ----
    n_ev = NL * min(args.steps, 5)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_ev)]
    for trio in evs:
        for e in trio:
            e.record()
    torch.cuda.synchronize()
    i = 0
    for _ in range(min(args.steps, 5)):
        for layer in range(NL):
            _cabi.set_decode_events(*evs[i])
            attn.decode(q_dev[layer], caches[layer], block_table, seq_lens, out_dev[layer])
            i += 1
    _cabi.set_decode_events(None, None, None)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None   # sampled over the timed, e2e and per-launch passes
    dec_ms = [t[0].elapsed_time(t[1]) for t in evs]
    mrg_ms = [t[1].elapsed_time(t[2]) for t in evs]
    dec_avg = sum(dec_ms) / len(dec_ms)
    alg_bytes = B * L * HKV * ALG_BYTES_PER_TOKEN_HEAD
    peak, peak_src = measured_peak()
    achieved = alg_bytes / (dec_avg * 1e-3) / 1e9
    # DRAM traffic per launch is not measured by this run: it is dram__bytes_read.sum + dram__bytes_write.sum
    # of one ncu capture of this kernel on this very shape (335.7 MB + 3.3 MB at batch 8 x ctx 32768) and is
    # only reported for that shape.  The physical slots are 160 B per 136 algorithmic bytes, so 1.18x the
    # algorithmic bytes is the floor; the rest is the partial outputs.
    traffic = 339.09e6 if (B, L) == (8, 32768) else None
    roofline = {"bound": "hbm", "kernel": "decode_paged_kernel<8>", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                "traffic": traffic, "traffic_source": "ncu capture of this kernel and shape (one launch, --clock-control none), "
                                                      "not measured in this run",
                "expected_min_traffic": alg_bytes * 160.0 / 136.0,
                "algorithmic_bytes_per_launch": alg_bytes, "avg_launch_ms": dec_avg,
                "merge_avg_launch_ms": sum(mrg_ms) / len(mrg_ms),
                "frac_whole_step": (alg_bytes * NL / (ms_step * 1e-3) / 1e9) / peak}
    # The same launch counted on the packed cache bytes it streams (80-byte slots: 68 information bytes + pad), the
    # figure the DRAM counters see; `frac` above counts the 136 information bytes per (token, KV head).
    phys = alg_bytes * 160.0 / 136.0
    roofline["packed_cache_bytes"] = {"bytes_per_launch": phys, "achieved": phys / (dec_avg * 1e-3) / 1e9,
                                      "frac": phys / (dec_avg * 1e-3) / 1e9 / peak}
    # The tcgen05 / tensor-memory variant of the loop on the same launch, for the record: the wide-tile kernel takes
    # any number of query columns through its causal entry point (one query per sequence: the mask is a no-op).
    try:
        ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(2 * min(NL, 6))]
        alt = torch.empty_like(out_dev[0]).unsqueeze(1)
        for layer in range(min(NL, 6) + 2):
            lay = layer % min(NL, 6)
            if layer >= 2:
                ev0[2 * lay].record()
            attn.decode_causal(q_dev[lay].unsqueeze(1), caches[lay], block_table, seq_lens, alt)
            if layer >= 2:
                ev0[2 * lay + 1].record()
        torch.cuda.synchronize()
        wide_ms = sorted(ev0[2 * i].elapsed_time(ev0[2 * i + 1]) for i in range(min(NL, 6)))
        roofline["tcgen05_variant_same_launch"] = {
            "kernel": "decode_mq_kernel + merge (whole call)", "ms": wide_ms[len(wide_ms) // 2],
            "frac": alg_bytes / (wide_ms[len(wide_ms) // 2] * 1e-3) / 1e9 / peak,
            "note": "operands through shared memory into tensor memory; kept for more than 8 query columns only"}
    except Exception as e:  # geometry the wide-tile kernel does not take (odd KV head counts)
        roofline["tcgen05_variant_same_launch"] = {"unavailable": str(e)[:200]}

    # ---- parity of the timed workload: layer 0's output against the oracle over the same bytes ----
    parity = None
    if rank == 0:
        from oracle import tq_oracle
        attn.decode(q_dev[0], caches[0], block_table, seq_lens, out_dev[0])
        torch.cuda.synchronize()
        want0 = tq_oracle.decode_paged_parallel(q_dev[0].float().cpu().numpy(), caches[0].cpu().numpy(),
                                                block_table.cpu().numpy(), seq_lens.cpu().numpy(),
                                                attn.signs(dev).cpu().numpy(), 1.0 / math.sqrt(D))
        parity = oracle_parity(out_dev[0].float().cpu().numpy(), want0,
                               f"layer 0 of the timed step: batch {B} x {L} tokens, bf16 output")
        del want0

    # ---- strong scaling of the stated batch: the same B sequences split over the GPUs ------------
    wanted = {x.strip() for x in args.sections.split(",")} if args.sections not in ("all", "") else {"mixed", "kv_split", "strong", "short_chunk"}
    if args.sections == "none":
        wanted = set()
    strong = None
    if world > 1 and "strong" in wanted and B % world == 0 and HKV % world == 0:
        def graph_ms(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            side2 = torch.cuda.Stream(dev)
            side2.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side2):
                with torch.cuda.graph(g, stream=side2):
                    fn()
            torch.cuda.current_stream().wait_stream(side2)
            g.replay()
            torch.cuda.synchronize()
            return timed(g.replay, args.steps) / args.steps
        # (a) by sequence: this rank decodes B / world of its sequences, all KV heads
        bs = B // world
        bt_s, sl_s = block_table[rank * bs:(rank + 1) * bs].contiguous(), seq_lens[:bs].contiguous()
        q_s, o_s = q_dev[:, rank * bs:(rank + 1) * bs].contiguous(), torch.empty(NL, bs, HQ, D, dtype=torch.bfloat16, device=dev)

        def step_seq():
            for layer in range(NL):
                attn.decode(q_s[layer], caches[layer], bt_s, sl_s, o_s[layer])
        ms_seq = graph_ms(step_seq)
        # (b) by KV head: this rank holds HKV / world heads of every token of all B sequences
        hk, hq = HKV // world, HQ // world
        attn_h = TurboQuantPagedAttention(hq, D, 1.0 / math.sqrt(D), hk, seed=42, num_ctas=args.num_ctas)
        caches_h = torch.zeros((NL,) + kv_cache_shape(nb, PAGE, hk, D), dtype=torch.uint8, device=dev)
        for layer in range(NL):
            for b in range(B):
                _fill_sequence(attn_h, caches_h[layer], block_table[b], L, gen, dev, heads=hk)
        q_h = torch.randn(NL, B, hq, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        o_h = torch.empty_like(q_h)

        def step_head():
            for layer in range(NL):
                attn_h.decode(q_h[layer], caches_h[layer], block_table, seq_lens, o_h[layer])
        ms_head = graph_ms(step_head)
        del caches_h
        torch.cuda.empty_cache()
        strong = {"workload": f"the stated batch of {B} x ctx {L}, {NL} layers per step, split over {world} GPUs (total work fixed)",
                  "one_gpu_ms_per_step_same_run": ms_step, "one_gpu_tokens_per_s": B / (ms_step * 1e-3),
                  "by_sequence": {"sequences_per_gpu": bs, "ms_per_step": ms_seq, "tokens_per_s": B / (ms_seq * 1e-3),
                                  "speedup": ms_step / ms_seq},
                  "by_kv_head": {"kv_heads_per_gpu": hk, "ms_per_step": ms_head, "tokens_per_s": B / (ms_head * 1e-3),
                                 "speedup": ms_step / ms_head},
                  "scaling": "strong",
                  "limit": "no collective on either split; what stays constant as the data per GPU shrinks is the fixed cost of "
                           "a call (two launches, the device-side plan, query rotation, first stage, merge: about 20 us per layer)"}

    # ---- cache-write path (the prefill-quantization config): 32768 tokens x 8 KV heads, bf16 ------
    write = None
    dequant = None
    if rank == 0:
        from turboquant_b200 import synthetic
        wk, wv, wslots, wnb = synthetic.write_case(seed=2, num_tokens=32768)
        wk, wv, wslots = wk.to(dev), wv.to(dev), wslots.to(dev)
        wcaches = [torch.zeros(kv_cache_shape(wnb, PAGE, HKV, D), dtype=torch.uint8, device=dev) for _ in range(4)]
        for c in wcaches:
            attn.write(wk, wv, c, wslots)
        torch.cuda.synchronize()
        wt = []
        for i in range(12):
            out_dev.zero_(); caches[i % NL].add_(0)      # touch > L2 worth of other data between launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); attn.write(wk, wv, wcaches[i % 4], wslots); e1.record()
            torch.cuda.synchronize()
            wt.append(e0.elapsed_time(e1))
        wt.sort()
        w_alg = 2 * 32768 * HKV * D * 2 + 2 * 32768 * HKV * 68 + 32768 * 8
        w_ach = w_alg / (wt[len(wt) // 2] * 1e-3) / 1e9
        write = {"workload": "config2: 32768 tokens x 8 KV heads x 128, bf16, K with an x20 outlier channel, pages permuted",
                 "kernel": "write_kv_cache_mma_kernel<bf16> (tensor-core rotation + guarded codes; exact path for flagged rows)", "ms": wt[len(wt) // 2], "algorithmic_bytes": w_alg,
                 "achieved": w_ach, "peak": peak, "unit": "GB/s", "frac": w_ach / peak,
                 "tokens_per_s": 32768 / (wt[len(wt) // 2] * 1e-3)}
        if not args.no_cpu_baseline:
            nsample, w_reps = 32768, 4
            w_rate, w_dt = cpu_write_rate(wk[:nsample].float().cpu().numpy(), wv[:nsample].float().cpu().numpy(),
                                          wslots[:nsample].cpu().numpy(), attn.signs(dev).cpu().numpy(), wnb,
                                          os.cpu_count() or 1, w_reps)
            t_rate, t_dt = torch_write_rate(wk[:nsample].float().cpu(), wv[:nsample].float().cpu(), wslots[:nsample].cpu(),
                                            attn.signs(dev).cpu(), wnb, 2)
            write["cpu_baseline"] = {"value": t_rate, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                     "kind": "torch-restatement",
                                     "sample": f"2 passes over the {nsample} tokens of the same case ({t_dt:.2f} s)",
                                     "port": {"value": w_rate, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                                              "sample": f"{w_reps} passes over the {nsample} tokens of the same case ({w_dt:.2f} s)"}}
        del wk, wv, wcaches
        # ---- bulk dequantization of cached tokens (continuation of a prefill): layer caches of the
        # decode workload, first ctx_d tokens of every sequence -> dense bf16 K / V
        ctx_d = min(L, 8192)
        cu_d = torch.arange(B + 1, dtype=torch.int32, device=dev) * ctx_d
        sl_d = torch.full((B,), ctx_d, dtype=torch.int32, device=dev)
        dk, dv = attn.dequant_cached(caches[0], block_table, sl_d, cu_d, B * ctx_d)
        torch.cuda.synchronize()
        dt_ = []
        from turboquant_b200 import _cabi as _c
        for i in range(8):
            out_dev.zero_(); caches[(i + 1) % NL].add_(0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _c.dequant_paged(caches[i % NL], block_table, sl_d, cu_d, attn.signs(dev), dk, dv)
            e1.record()
            torch.cuda.synchronize()
            dt_.append(e0.elapsed_time(e1))
        dt_.sort()
        d_alg = B * ctx_d * HKV * (136 + 2 * D * 2)      # 136 B of codes + norms in, 2 x 128 bf16 out
        d_ach = d_alg / (dt_[len(dt_) // 2] * 1e-3) / 1e9
        dequant = {"workload": f"cached tokens -> dense bf16 K/V: {B} sequences x {ctx_d} tokens x {HKV} KV heads",
                   "kernel": "dequant_paged_kernel<bf16>", "ms": dt_[len(dt_) // 2], "algorithmic_bytes": d_alg,
                   "achieved": d_ach, "peak": peak, "unit": "GB/s", "frac": d_ach / peak,
                   "tokens_per_s": B * ctx_d / (dt_[len(dt_) // 2] * 1e-3)}
        del dk, dv

    # ---- host copy of what the CPU baseline needs, then the big caches can go -------------------
    cpu_sample = None
    if rank == 0 and not args.no_cpu_baseline:
        pages_s = (L + PAGE - 1) // PAGE
        # the sample attends all L tokens of every sequence of layer 0: the same bytes as the GPU
        ids = block_table[:, :pages_s].long()
        cpu_sample = (np.ascontiguousarray(caches[0][:, ids.reshape(-1)].cpu().numpy()),
                      np.arange(B * pages_s, dtype=np.int32).reshape(B, pages_s),
                      q_dev[0].float().cpu().numpy(), attn.signs(dev).cpu().numpy())

    # ---- the other configs, each with its own oracle check (all ranks take part) ------------------
    mixed = kv_split = short_chunk = None
    if "mixed" in wanted or "kv_split" in wanted or "short_chunk" in wanted:
        del caches
        torch.cuda.empty_cache()
        if "mixed" in wanted:
            mixed = section_mixed(args, rank, world, dev, peak)
        if "kv_split" in wanted:
            kv_split = section_kv_split(args, rank, world, dev, peak)
        if "short_chunk" in wanted:
            short_chunk = section_short_chunk(args, rank, world, dev, peak)

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return
    cpu = None
    if cpu_sample is not None:
        cpu = cpu_arm(*cpu_sample, ctx=L, layers=NL, torch_passes=min(B, 6), port_reps=3)
    line = {
        "metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(args), "global_batch": B * world, "parallelism": f"dp{world} (by sequence)",
                   "l2": f"inputs larger than L2: {alg_bytes / 1e6:.0f} MB streamed per launch, {NL} distinct layer caches",
                   "cuda_graph": graph is not None, "algorithmic_bytes_per_step": alg_bytes * NL,
                   "arithmetic": "f16 x f16 tensor-core products with f32 accumulation over 4-bit codes; bf16 queries and outputs"},
        "roofline": roofline, "parity": parity, "write": write, "dequant": dequant, "cpu_baseline": cpu,
        "mixed": mixed, "kv_split": kv_split, "strong": strong, "short_chunk": short_chunk,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "api": "TurboQuantPagedAttention.write + .decode per layer, pinned host buffers, copies on two copy streams beside the kernels" + ("" if args.no_graph else ", step captured in a CUDA graph")},
        "gpu_launches": args.steps * NL * 2, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# Secondary workloads (parity-test shapes timed on request; the default line is config 1)
# ------------------------------------------------------------------------------------------------
def _setup_dist():
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _fill_cache(attn, cache, block_table_row, n_tokens, gen, dev, chunk=65536):
    """Quantize seeded N(0,1) K/V for one sequence into its pages with the cache-write kernel."""
    for t0 in range(0, n_tokens, chunk):
        n = min(chunk, n_tokens - t0)
        k = torch.randn(n, HKV, D, generator=gen, device=dev).to(torch.bfloat16)
        v = torch.randn(n, HKV, D, generator=gen, device=dev).to(torch.bfloat16)
        tok = torch.arange(t0, t0 + n, device=dev)
        slots = block_table_row.long()[tok // PAGE] * PAGE + tok % PAGE
        attn.write(k, v, cache, slots)


def _timed_steps(fn, steps, world, dev):
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms / steps


def run_config3(args):
    """64 sequences with log-uniform lengths in [512, 131072] (seed 3), sharded over the ranks by
    sequence (longest first); every rank decodes its shard, no collective on the data path."""
    from turboquant_b200 import synthetic
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    from turboquant_b200.parallel import shard_sequences
    rank, world, dev = _setup_dist()
    lens_all = synthetic.mixed_lengths(seed=3, n=64)
    shards = shard_sequences(lens_all, world)
    lens = [lens_all[i] for i in shards[rank]]
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    bt_cpu, _, nb = synthetic.paged_layout(lens, seed=3 + rank)
    bt = bt_cpu.to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3 + 1000 * rank)
    ncache = 2   # rotated so that consecutive launches stream different memory (each far larger than L2)
    caches = [torch.zeros(kv_cache_shape(nb, PAGE, HKV, D), dtype=torch.uint8, device=dev) for _ in range(ncache)]
    for c in caches:
        for b, n in enumerate(lens):
            _fill_cache(attn, c, bt[b], n, gen, dev)
    q = torch.randn(len(lens), HQ, D, generator=gen, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    state = {"i": 0}

    def step():
        attn.decode(q, caches[state["i"] % ncache], bt, sl, out)
        state["i"] += 1
    for _ in range(max(args.warmup, 3)):
        step()
    ms = _timed_steps(step, args.steps, world, dev)
    loads = [sum(lens_all[i] for i in s) for s in shards]
    alg = sum(lens_all) * HKV * ALG_BYTES_PER_TOKEN_HEAD
    peak, peak_src = measured_peak()
    if rank == 0:
        ach = alg / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode_attn_tokens_per_s", "value": 64 / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "config3: 64 sequences, lengths log-uniform in [512, 131072] (seed 3), one layer, "
                                   "sharded over the GPUs by sequence (greedy by length)",
                       "total_tokens": sum(lens_all), "load_imbalance_max_over_mean": max(loads) / (sum(loads) / world),
                       "l2": "inputs larger than L2, two caches alternated"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak * world, "unit": "GB/s",
                         "frac": ach / (peak * world), "peak_source": peak_src, "algorithmic_bytes_per_launch": alg,
                         "note": "whole call (decode + merge kernels), aggregate over GPUs"},
            "gpu_launches": args.steps * 2}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_config4(args):
    """One 1,048,576-token sequence, 8 decode queries; the KV axis is split contiguously over the
    ranks, each rank computes rotated partials + LSE, the partials are all-gathered over NCCL and
    every rank finishes with the LSE merge and the inverse rotation."""
    from turboquant_b200 import synthetic
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    from turboquant_b200.parallel import kv_ranges, kv_split_decode
    rank, world, dev = _setup_dist()
    total, nq = args.c4_tokens, 8
    a, b = kv_ranges(total, world)[rank]
    n_local = b - a
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    pages = (n_local + PAGE - 1) // PAGE
    cpu_gen = torch.Generator().manual_seed(4 + rank)
    bt_row = torch.randperm(pages, generator=cpu_gen).to(torch.int32).to(dev)
    cache = torch.zeros(kv_cache_shape(pages, PAGE, HKV, D), dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4 + 1000 * rank)
    _fill_cache(attn, cache, bt_row, n_local, gen, dev)
    qgen = torch.Generator(device=dev)
    qgen.manual_seed(4)                                   # the same queries on every rank
    from turboquant_b200 import _cabi
    share = min(nq, _cabi.decode_max_queries_per_seq(HQ, HKV))   # queries that ride one pass over the KV: 8
    rows = nq // share
    q = torch.randn(rows, share, HQ, D, generator=qgen, device=dev).to(torch.bfloat16)
    bt = bt_row.unsqueeze(0).expand(rows, -1).contiguous()  # every row is the same sequence
    sl = torch.full((rows,), n_local, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)

    fused = world > 1 and args.exchange == "fused"
    if fused:
        from turboquant_b200.parallel import KVSplitExchange
        ex = KVSplitExchange(attn, rows, share, dev)

    def step():
        if fused:
            ex.decode(q, cache, bt, sl, out)
        elif world > 1:
            kv_split_decode(attn, q, cache, bt, sl, out)
        else:
            attn.decode(q, cache, bt, sl, out)
    for _ in range(max(args.warmup, 3)):
        step()
    ms = _timed_steps(step, args.steps, world, dev)
    alg = total * HKV * ALG_BYTES_PER_TOKEN_HEAD
    peak, peak_src = measured_peak()
    if rank == 0:
        ach = alg / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode_attn_tokens_per_s", "value": nq / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"config4: one {total:,}-token sequence, 8 decode queries, one layer, KV axis split "
                                   "contiguously over the GPUs, partial (o, lse) exchanged, merged on every GPU",
                       "exchange_bytes_per_rank": nq * HQ * (D + 1) * 4,
                       "exchange": ("none (one GPU)" if world == 1 else
                                    "kernel-side: peer stores into every rank's buffer + flags, flag-gated merge"
                                    if fused else "NCCL all-gather of the partials, then merge"),
                       "note": f"the 8 queries run as {rows} row(s) of {share} queries that share one pass over the KV "
                               "(the wide-tile tcgen05 kernel: 32 query columns per KV head); the algorithmic bytes "
                               "below count the KV once",
                       "l2": f"{total * HKV * 160 / 1e9:.2f} GB of pages per pass, larger than L2"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak * world, "unit": "GB/s",
                         "frac": ach / (peak * world), "peak_source": peak_src, "algorithmic_bytes_per_launch": alg,
                         "physical_kv_bytes_streamed": rows * total * HKV * 160},
            "gpu_launches": args.steps * (3 if world > 1 else 2)}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()



def run_sweep(args):
    """The shapes of the reference's published kernel tables (batch 1, ctx 256 ... 32768; batch
    1/4/16/32 at ctx 4096/16384/32768; measured by its authors on an A100, CUDA-graph replays of the
    decode op): one decode call (decode + merge kernels) per graph replay, p50 over 100 replays, four
    caches rotated.  Context only: other hardware, so no ratio is formed."""
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    rank, world, dev = _setup_dist()
    attn = TurboQuantPagedAttention(HQ, D, 1.0 / math.sqrt(D), HKV, num_ctas=args.num_ctas)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    shapes = [(1, c) for c in (256, 512, 1024, 2048, 4096, 8192, 16384, 32768)]
    shapes += [(b, c) for c in (4096, 16384, 32768) for b in (4, 16, 32)]
    rows = []
    for B, L in shapes:
        pages = (L + PAGE - 1) // PAGE
        nb = B * pages
        ncache = 4 if B * L <= 16 * 32768 else 2
        bt = torch.randperm(nb, generator=torch.Generator().manual_seed(B * 131 + L)).view(B, pages).to(torch.int32).to(dev)
        caches = [torch.zeros(kv_cache_shape(nb, PAGE, HKV, D), dtype=torch.uint8, device=dev) for _ in range(ncache)]
        for c in caches:
            for b in range(B):
                _fill_cache(attn, c, bt[b], L, gen, dev)
        sl = torch.full((B,), L, dtype=torch.int32, device=dev)
        q = torch.randn(B, HQ, D, generator=gen, device=dev).to(torch.float16)
        out = torch.empty_like(q)
        for c in caches:
            attn.decode(q, c, bt, sl, out)
        torch.cuda.synchronize()
        graphs = []
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for c in caches:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    attn.decode(q, c, bt, sl, out)
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        ts = []
        for i in range(104):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphs[i % ncache].replay()
            e1.record()
            torch.cuda.synchronize()
            if i >= 4:
                ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        rows.append({"batch": B, "ctx": L, "p50_us": round(ts[len(ts) // 2], 2),
                     "GBps": round(B * L * HKV * ALG_BYTES_PER_TOKEN_HEAD / ts[len(ts) // 2] / 1e3, 1)})
        del caches
    if rank == 0:
        print(json.dumps({"metric": "decode_call_latency_us", "unit": "us", "n_gpus": 1, "higher_is_better": False,
                          "vs_baseline": None, "data": "synthetic",
                          "config": {"workload": "sweep: 32 q / 8 kv heads, head_dim 128, fp16 q, one decode call per CUDA-graph "
                                                 "replay (decode + merge), p50 of 100"},
                          "rows": rows}), flush=True)


def run_head_sizes(args):
    """Head sizes 64 and 256 (48- and 144-byte slots; the reference declares them, its decode op rejects
    them): cache write of 32768 tokens x 8 KV heads, one decode call over batch 8 x 32768 tokens and the
    bulk dequantization of 8 x 4096 tokens, each against its algorithmic bytes; head size 128 through
    the same calls beside them.  Parity: the written cache byte for byte and the decode output against
    the oracle, on the first sequence cut to 2048 tokens.  One GPU's figures; every rank runs the same."""
    from oracle import tq_oracle
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    rank, world, dev = _setup_dist()
    peak, peak_src = measured_peak()
    steps = args.steps
    T, H, B, L = 32768, 8, 8, 32768
    rows = []
    for d, hq in ((64, 16), (256, 16), (128, 32)):
        attn = TurboQuantPagedAttention(hq, d, 1.0 / math.sqrt(d), H, num_ctas=args.num_ctas)
        dc = max(d, 64) // 64
        gen = torch.Generator(device=dev)
        gen.manual_seed(d)
        # ---- write ----
        k = torch.randn(T, H, d, generator=gen, device=dev).to(torch.bfloat16)
        v = torch.randn(T, H, d, generator=gen, device=dev).to(torch.bfloat16)
        nb_w = T // PAGE
        perm = torch.randperm(nb_w, generator=torch.Generator().manual_seed(d)).to(dev)
        slots = perm.repeat_interleave(PAGE) * PAGE + torch.arange(T, device=dev) % PAGE
        wcaches = [torch.zeros(kv_cache_shape(nb_w, PAGE, H, d), dtype=torch.uint8, device=dev) for _ in range(4)]
        st = {"i": 0}

        def write():
            attn.write(k, v, wcaches[st["i"] % 4], slots)
            st["i"] += 1
        for _ in range(3):
            write()
        ms_w = _time_steps(write, steps, world, dev)
        alg_w = 2 * T * H * d * 2 + 2 * T * H * (d // 2 + 2 * dc) + T * 8
        # parity of the write: the first 2048 tokens, byte for byte
        n_par = 2048
        signs = attn.signs(dev).cpu().numpy()
        want_cache = np.zeros((2, nb_w, PAGE, H, wcaches[0].shape[-1]), np.uint8)
        tq_oracle.write_kv_cache(want_cache, k[:n_par].float().cpu().numpy(), v[:n_par].float().cpu().numpy(), signs,
                                 slots[:n_par].cpu().numpy(), d)
        pages_par = perm[:n_par // PAGE].cpu().numpy()
        write_equal = bool((wcaches[0][:, pages_par].cpu().numpy() == want_cache[:, pages_par]).all())
        if not write_equal:
            raise SystemExit(f"head size {d}: the written cache differs from the oracle's")
        # ---- dequantization of 8 x 4096 of the written tokens ----
        Bq, Lq = 8, 4096
        bt_q = perm.to(torch.int32).view(Bq, Lq // PAGE).contiguous()
        sl_q = torch.full((Bq,), Lq, dtype=torch.int32, device=dev)
        cu_q = torch.arange(Bq + 1, dtype=torch.int32, device=dev) * Lq

        def dequant():
            attn.dequant_cached(wcaches[st["i"] % 4], bt_q, sl_q, cu_q, Bq * Lq)
            st["i"] += 1
        for _ in range(3):
            dequant()
        ms_q = _time_steps(dequant, steps, world, dev)
        alg_q = Bq * Lq * H * (d + 4 * dc + 2 * d * 2)
        del wcaches, k, v
        # ---- decode: batch 8 x 32768, random codes with unit norms (the time does not depend on the values) ----
        nb = B * L // PAGE
        bt = torch.randperm(nb, generator=torch.Generator().manual_seed(d + 1)).view(B, L // PAGE).to(torch.int32).to(dev)
        sl = torch.full((B,), L, dtype=torch.int32, device=dev)
        caches = torch.randint(0, 256, (3,) + kv_cache_shape(nb, PAGE, H, d), dtype=torch.uint8, device=dev, generator=gen)
        caches[..., d // 2:d // 2 + 2 * dc] = torch.tensor([0, 60], dtype=torch.uint8, device=dev).repeat(dc)   # fp16 1.0
        q = torch.randn(B, hq, d, generator=gen, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)

        def decode():
            attn.decode(q, caches[st["i"] % 3], bt, sl, out)
            st["i"] += 1
        for _ in range(3):
            decode()
        ms_d = _time_steps(decode, steps, world, dev)
        alg_d = B * L * H * (d + 4 * dc)
        # parity of the decode: sequence 0 cut to 2048 tokens
        sl_p = torch.tensor([n_par], dtype=torch.int32, device=dev)
        out_p = torch.empty(1, hq, d, dtype=torch.float32, device=dev)
        attn.decode(q[:1], caches[0], bt[:1].contiguous(), sl_p, out_p)
        torch.cuda.synchronize()
        pages_d = bt[0, :n_par // PAGE].long()
        small = caches[0][:, pages_d].cpu().numpy()
        want = tq_oracle.decode_paged(q[:1].float().cpu().numpy(), small, np.arange(n_par // PAGE, dtype=np.int32)[None],
                                      np.array([n_par], np.int32), signs, 1.0 / math.sqrt(d))
        par = oracle_parity(out_p.cpu().numpy(), want, f"head size {d}: sequence 0 cut to {n_par} tokens")
        assert attn.status(B, dev) == 0
        del caches
        torch.cuda.empty_cache()

        def part(ms, alg):
            return {"ms": ms, "algorithmic_bytes": alg, "achieved_GBps": alg / (ms * 1e-3) / 1e9, "frac": alg / (ms * 1e-3) / 1e9 / peak}
        rows.append({"head_size": d, "q_heads": hq, "kv_heads": H, "slot_bytes": int(kv_cache_shape(1, PAGE, H, d)[-1]),
                     "write": dict(part(ms_w, alg_w), tokens=T, equal_to_oracle_first_tokens=n_par),
                     "decode": dict(part(ms_d, alg_d), batch=B, ctx=L, parity=par),
                     "dequant": dict(part(ms_q, alg_q), tokens=Bq * Lq)})
    if rank == 0:
        r64 = rows[0]
        print(json.dumps({"metric": "decode_attn_tokens_per_s", "value": world * B / (r64["decode"]["ms"] * 1e-3), "unit": "tokens/s",
                          "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": r64["decode"]["ms"], "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                          "config": {"workload": "head_sizes: head 64 / 256 / 128 through the same calls; value = one decode call, "
                                                 "batch 8 x 32768, head size 64, 16 q / 8 kv heads; one layer",
                                     "l2": "three caches in rotation, each larger than L2"},
                          "peak": peak, "peak_source": peak_src, "rows": rows}), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "config3":
        run_config3(args)
    elif args.workload == "config4":
        run_config4(args)
    elif args.workload == "sweep":
        run_sweep(args)
    elif args.workload == "head_sizes":
        run_head_sizes(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
