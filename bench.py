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
recorded by the library around that kernel.  `cpu_baseline` / `--impl reference` time the CPU
oracle (a C restatement of the reference's torch CPU path) on a bounded sample of the same data.
"""
from __future__ import annotations

import argparse
import json
import math
import os
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="config4 on several GPUs: partials exchanged by the kernels themselves (peer stores + "
                         "flags) or by an NCCL all-gather")
    ap.add_argument("--workload", default="config1", choices=["config1", "config3", "config4", "sweep"],
                    help="config1 (default, the headline): batch 8 x 32k per GPU; config3: 64 mixed lengths sharded by "
                         "sequence; config4: one 1M-token sequence, KV axis split over the GPUs, NCCL merge")
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


def run_reference(args):
    """The reference's CPU implementation of the path (its torch modules cannot travel to the
    GPU box, so the oracle port stands in), all host threads, bounded sample per step."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    ctx_s = min(8192, args.ctx)
    cache, bt, q, signs = synthetic_host_cache(ctx_s, min(args.batch, 8), seed=1)
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt = cpu_decode_rate(cache, bt, q, signs, ctx_s, threads)
        if i >= args.warmup:
            rates.append((r, dt))
    rate = statistics.median(r for r, _ in rates)
    per_token = args.ctx * HKV * args.layers           # KV token-heads one decode token attends
    value = rate / per_token
    sample = (f"{threads} sequences x {ctx_s} tokens x {HKV} KV heads of config-1-shaped quantized cache per step "
              f"(one layer), scaled to ctx {args.ctx} x {args.layers} layers per token")
    line = {
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.median(dt for _, dt in rates), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "note": "CPU arm: C port of the reference torch CPU path"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(args):
    return (f"config1: Qwen3-8B-shaped decode layer, batch {args.batch}/GPU x ctx {args.ctx}, {HQ}q/{HKV}kv heads, "
            f"head_dim {D}, bf16 q, 16-token pages (seeded random permutation), {args.layers} layers per step")


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
    # DRAM traffic per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this
    # kernel on this workload (profiles/decode_paged_kernel_config1_layer.md: 335.7 MB + 3.3 MB for
    # batch 8 x ctx 32768), scaled by the tokens of the launch.  The physical slots are 160 B per 136
    # algorithmic bytes, so 1.18x is the floor; the rest is the partial outputs.
    traffic = 339.09e6 * (B * L) / (8 * 32768)
    roofline = {"bound": "hbm", "kernel": "decode_paged_kernel<8>", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                "traffic": traffic, "expected_min_traffic": alg_bytes * 160.0 / 136.0,
                "algorithmic_bytes_per_launch": alg_bytes, "avg_launch_ms": dec_avg,
                "merge_avg_launch_ms": sum(mrg_ms) / len(mrg_ms),
                "frac_whole_step": (alg_bytes * NL / (ms_step * 1e-3) / 1e9) / peak}

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
                 "kernel": "write_kv_cache_kernel<bf16>", "ms": wt[len(wt) // 2], "algorithmic_bytes": w_alg,
                 "achieved": w_ach, "peak": peak, "unit": "GB/s", "frac": w_ach / peak,
                 "tokens_per_s": 32768 / (wt[len(wt) // 2] * 1e-3)}
        if not args.no_cpu_baseline:
            nsample, w_reps = 32768, 4
            w_rate, w_dt = cpu_write_rate(wk[:nsample].float().cpu().numpy(), wv[:nsample].float().cpu().numpy(),
                                          wslots[:nsample].cpu().numpy(), attn.signs(dev).cpu().numpy(), wnb,
                                          os.cpu_count() or 1, w_reps)
            write["cpu_baseline"] = {"value": w_rate, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                                     "sample": f"{w_reps} passes over the {nsample} tokens of the same case ({w_dt:.2f} s)"}
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

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return
    cpu = None
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        ctx_s = L
        pages_s = (ctx_s + PAGE - 1) // PAGE
        # the sample attends the first ctx_s tokens of every sequence of layer 0, same bytes as the GPU
        ids = block_table[:, :pages_s].long()
        sub = caches[0][:, ids.reshape(-1)].cpu().numpy()
        bt_s = np.arange(B * pages_s, dtype=np.int32).reshape(B, pages_s)
        signs = attn.signs(dev).cpu().numpy()
        reps = 3
        rate, dt = cpu_decode_rate(np.ascontiguousarray(sub), bt_s, q_dev[0].float().cpu().numpy(), signs, ctx_s, threads,
                                   reps)
        cpu = {"value": rate / (L * HKV * NL), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{threads * reps} sequence passes x {ctx_s} tokens x {HKV} KV heads of layer 0's cache ({dt:.2f} s), "
                         f"scaled to ctx {L} x {NL} layers per token"}
    line = {
        "metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(args), "global_batch": B * world, "parallelism": f"dp{world} (by sequence)",
                   "l2": f"inputs larger than L2: {alg_bytes / 1e6:.0f} MB streamed per launch, {NL} distinct layer caches",
                   "cuda_graph": graph is not None, "algorithmic_bytes_per_step": alg_bytes * NL},
        "roofline": roofline, "write": write, "dequant": dequant, "cpu_baseline": cpu,
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
    total, nq = 1_048_576, 8
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
    share = max(1, 8 // (HQ // HKV))                      # queries that fit one 8-column query tile: 2
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
            "config": {"workload": "config4: one 1,048,576-token sequence, 8 decode queries, one layer, KV axis split "
                                   "contiguously over the GPUs, partial (o, lse) exchanged, merged on every GPU",
                       "exchange_bytes_per_rank": nq * HQ * (D + 1) * 4,
                       "exchange": ("none (one GPU)" if world == 1 else
                                    "kernel-side: peer stores into every rank's buffer + flags, flag-gated merge"
                                    if fused else "NCCL all-gather of the partials, then merge"),
                       "note": "the 8 queries run as 4 rows of 2 queries that share one pass over the KV (8 batch rows, "
                               "each streaming the KV, through the reference's API); the algorithmic bytes below "
                               "count the KV once",
                       "l2": "1.34 GB of pages per pass, far larger than L2"},
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
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
