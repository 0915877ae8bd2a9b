"""Host-side logic of the reference-facing surface (no GPU): presets, packing, sharding helpers,
op schemas, plugin registration, and the KV-axis split + LSE merge across two gloo ranks."""
import math
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_tile_pack_known_answer_and_roundtrip():
    from turboquant_b200.tile import pack_4bit, unpack_4bit
    assert pack_4bit(torch.tensor([0x0A, 0x05], dtype=torch.uint8)).tolist() == [0xA5]
    idx = torch.randint(0, 16, (7, 128), dtype=torch.uint8)
    assert torch.equal(unpack_4bit(pack_4bit(idx), 128), idx)


def test_kernel_config_presets():
    from turboquant_b200.kernel_config import MODEL_PRESETS, ModelConfig, compute_kernel_config
    assert len(MODEL_PRESETS) == 22
    q = MODEL_PRESETS["qwen3-8b"]
    assert (q.num_qo_heads, q.num_kv_heads, q.head_dim, q.gqa_ratio, q.padded_dim) == (32, 8, 128, 4, 128)
    kc = compute_kernel_config(q)
    assert kc.supported and kc.threads_per_block == 640 and kc.pages_per_stage == 2 and kc.stages == 3
    assert kc.stages * kc.stage_bytes + 65536 < 227 * 1024                     # three stages + the table
    assert compute_kernel_config(ModelConfig(64, 8, 128)).stages == 3          # 8 query heads per KV head
    assert compute_kernel_config(ModelConfig(16, 4, 128)).pages_per_stage == 4  # a TP shard with 4 KV heads
    for name in ("gemma-2-9b", "gemma-2-2b", "qwen3-0.6b"):                    # head sizes 256 and 64: second-tier kernels
        kc2 = compute_kernel_config(MODEL_PRESETS[name])
        assert kc2.supported and not kc2.tuned
    assert all(compute_kernel_config(m).supported for m in MODEL_PRESETS.values())
    assert compute_kernel_config(MODEL_PRESETS["llama-2-7b"]).supported        # 32 KV heads: two launches of 16
    assert compute_kernel_config(ModelConfig(16, 16, 128)).pages_per_stage == 1
    assert not compute_kernel_config(ModelConfig(6, 6, 128)).supported


def test_sequence_sharding_is_balanced_and_complete():
    from turboquant_b200 import synthetic
    from turboquant_b200.parallel import kv_ranges, shard_sequences
    lens = synthetic.mixed_lengths(seed=3, n=64)
    assert min(lens) >= 512 and max(lens) <= 131072
    for world in (1, 2, 4, 8):
        shards = shard_sequences(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) / (sum(loads) / world) < 1.25
    r = kv_ranges(1_048_576, 8)
    assert r[0] == (0, 131072) and r[-1][1] == 1_048_576 and all(a % 16 == 0 for a, _ in r)
    r = kv_ranges(1000, 3)
    assert r[0][0] == 0 and r[-1][1] == 1000 and all(r[i][1] == r[i + 1][0] for i in range(2))


def test_ops_are_registered_with_reference_schemas():
    from turboquant_b200 import ops  # noqa: F401
    w = torch.ops.turboquant_write.quantize_write_kv_cache.default._schema
    assert [a.name for a in w.arguments] == ["kv_cache", "key", "value", "signs", "slot_mapping", "head_dim",
                                             "padded_dim"]
    assert w.arguments[0].alias_info is not None and w.arguments[0].alias_info.is_write
    d = torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws.default._schema
    assert len(d.arguments) == 23 and d.arguments[-1].name == "num_splits"
    assert len(torch.ops.turboquant_v5.decode_v5_from_cache_ws.default._schema.arguments) == 20
    with pytest.raises(Exception):      # CUDA-only implementation: CPU tensors are refused by the dispatcher
        torch.ops.turboquant_write.quantize_write_kv_cache(torch.zeros(2, 1, 16, 8, 80, dtype=torch.uint8),
                                                           torch.zeros(1, 8, 128), torch.zeros(1, 8, 128),
                                                           torch.ones(128), torch.zeros(1, dtype=torch.int64), 128, 128)


def test_dispatcher_refuses_non_blackwell(monkeypatch):
    from turboquant_b200 import decoder_dispatch as dd
    dd.pick_decode_op.cache_clear()
    monkeypatch.setattr(dd, "_device_capability", lambda: (8, 0))
    with pytest.raises(RuntimeError, match="sm_100a"):
        dd.pick_decode_op()
    dd.pick_decode_op.cache_clear()
    monkeypatch.setattr(dd, "_device_capability", lambda: (10, 0))
    op, name = dd.pick_decode_op()
    assert name == dd.KERNEL_NAME and op is torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws
    dd.pick_decode_op.cache_clear()
    monkeypatch.setenv("TQ_FORCE_KERNEL", "v5")
    with pytest.raises(ValueError, match="not recognised"):
        dd.pick_decode_op()
    dd.pick_decode_op.cache_clear()


def test_vllm_plugin_registers_custom_backend():
    pytest.importorskip("vllm")
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from turboquant_b200 import vllm_plugin\n"
            "vllm_plugin.register(); vllm_plugin.register()\n"
            "from vllm.v1.attention.backends.registry import AttentionBackendEnum\n"
            "c = AttentionBackendEnum.CUSTOM.get_class()\n"
            "assert c.get_name() == 'CUSTOM' and c.forward_includes_kv_cache_update is False\n"
            "assert c.get_kv_cache_shape(10, 16, 8, 128, 'fp8') == (2, 10, 16, 8, 80)\n"
            "assert c.get_kv_cache_page_size(16, 8, 128, None, 'fp8') == 20480\n"
            "assert c.get_kv_cache_page_size(16, 8, 128, None, 'auto') is None\n"
            "assert c.supports_kv_cache_dtype('fp8') and c.get_impl_cls().__name__ == 'TurboQuantFusedImpl'\n"
            "assert c.get_builder_cls().__name__ == 'TurboQuantMetadataBuilder'\n"
            "print('ok')\n") % str(ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd="/tmp", timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_backend_step_facts_and_causal_kernel_geometries():
    """Host logic of the vLLM backend: the step's row classes from the metadata's CPU copies (both dense-row
    totals: with and without the short rows), and which geometries fuse short chunks."""
    pytest.importorskip("vllm")
    code = ("import sys, types; sys.path.insert(0, %r)\n"
            "import torch\n"
            "from turboquant_b200.vllm_backend_fused import step_shape, causal_chunk_supported\n"
            "cached, chunk = [500, 3, 37, 1200, 0, 64], [1, 6, 3, 12, 2, 8]\n"
            "qsl = torch.tensor([0, 1, 7, 10, 22, 24, 32], dtype=torch.int32)\n"
            "seq = torch.tensor([c + q for c, q in zip(cached, chunk)], dtype=torch.int32)\n"
            "st = step_shape(types.SimpleNamespace(query_start_loc_cpu=qsl, num_reqs=6, seq_lens_cpu=seq))\n"
            "assert st['any_cached'] and st['num_decode_rows'] == 1 and st['num_short_rows'] == 3\n"
            "assert st['dense_rows'] == 1212 + 2 and st['max_prefill_seq'] == 1212\n"
            "assert st['dense_rows_with_short'] == 1214 + 9 + 40 + 72 and st['max_prefill_seq_with_short'] == 1212\n"
            "assert causal_chunk_supported(32, 8, 128) and causal_chunk_supported(24, 8, 96)\n"
            "assert not causal_chunk_supported(64, 8, 128)      # 8 x 8 query columns\n"
            "assert not causal_chunk_supported(16, 8, 64)       # head size without the kernel\n"
            "assert not causal_chunk_supported(8, 1, 128)       # one KV head\n"
            "print('ok')\n") % str(ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd="/tmp", timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


_RANK_SCRIPT = r"""
import math, os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from oracle import tq_oracle
from turboquant_b200 import synthetic
from turboquant_b200.parallel import all_gather_partials, kv_ranges
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=int(sys.argv[1]), world_size=2)
rank = dist.get_rank()
case = synthetic.decode_case(seed=90, seq_lens=[777], dtype=torch.float16, num_q_rows=1)
signs = synthetic.make_signs().numpy()
cache = np.zeros((2, case.num_blocks, 16, 8, 80), np.uint8)
tq_oracle.write_kv_cache(cache, case.k.float().numpy(), case.v.float().numpy(), signs, case.slot_mapping.numpy(), 128)
args = (case.q.float().numpy(), cache, case.block_table.numpy(), case.seq_lens.numpy(), signs, 1 / math.sqrt(128))
a, b = kv_ranges(777, 2)[rank]                      # this rank's contiguous, page-aligned KV range
o, lse = tq_oracle.decode_paged(*args, kv_begin=a, kv_end=b, return_lse=True)
go, gl = all_gather_partials(torch.from_numpy(o), torch.from_numpy(lse))
merged, _ = tq_oracle.merge_partials(go.numpy(), gl.numpy())
full = tq_oracle.decode_paged(*args)
assert np.abs(merged - full).max() < 2e-6, np.abs(merged - full).max()
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_kv_axis_split_across_two_gloo_ranks(oracle, tmp_path):
    """Config-4 logic at small size on CPU ranks: each rank attends its KV range, partials are
    all-gathered, the LSE merge reproduces the unsplit result."""
    port = 29500 + os.getpid() % 400
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT % {"root": str(ROOT), "port": port})
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                              text=True) for r in range(2)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0 and f"rank {r} ok" in out, err[-2000:]
