"""KV-axis split of one long sequence over two GPUs, checked against the single-GPU result and the
oracle: NCCL all-gather of the partials + LSE merge, and the kernel-side exchange (peer stores +
flags).  The two-GPU cases are skipped on a single GPU; the exchange protocol with one rank
(its own buffer as the only peer) runs everywhere."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

_RANK = r"""
import math, os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from oracle import tq_oracle
from turboquant_b200 import synthetic
from turboquant_b200.paged_attention import TurboQuantPagedAttention
from turboquant_b200.parallel import kv_ranges, kv_split_decode, KVSplitExchange
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=dev)
total, nq = 5000, 3
case = synthetic.decode_case(seed=95, seq_lens=[total], dtype=torch.bfloat16, num_q_rows=nq)
signs = synthetic.make_signs().numpy()
full_cache = np.zeros((2, case.num_blocks, 16, 8, 80), np.uint8)
tq_oracle.write_kv_cache(full_cache, case.k.float().numpy(), case.v.float().numpy(), signs, case.slot_mapping.numpy(), 128)
bt_full = np.repeat(case.block_table.numpy(), nq, axis=0)
want = tq_oracle.decode_paged(case.q.float().numpy(), full_cache, bt_full, np.full(nq, total, np.int32), signs, 1 / math.sqrt(128))
# this rank holds only the pages of its token range, written by the CUDA kernel into a local cache
a, b = kv_ranges(total, world)[rank]
n_local = b - a
pages = (n_local + 15) // 16
attn = TurboQuantPagedAttention(32, 128, 1 / math.sqrt(128), 8)
cache = torch.zeros((2, pages, 16, 8, 80), dtype=torch.uint8, device=dev)
perm = torch.randperm(pages, generator=torch.Generator().manual_seed(rank)).to(dev)
tok = torch.arange(n_local, device=dev)
slots = perm[tok // 16] * 16 + tok %% 16
attn.write(case.k[a:b].to(dev), case.v[a:b].to(dev), cache, slots)
bt = perm.to(torch.int32).unsqueeze(0).expand(nq, -1).contiguous()
sl = torch.full((nq,), n_local, dtype=torch.int32, device=dev)
out = torch.empty(nq, 32, 128, dtype=torch.float32, device=dev)
kv_split_decode(attn, case.q.to(dev), cache, bt, sl, out)
torch.cuda.synchronize()
got = out.cpu().numpy()
err = np.abs(got - want)
assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), err.max()
assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-2
gathered = [torch.empty_like(out) for _ in range(world)]
dist.all_gather(gathered, out)
assert all(torch.equal(g, gathered[0]) for g in gathered)      # every rank ends with the same result
# the same through the kernel-side exchange, several steps in a row (both buffer generations), 3 queries = 3 rows
ex = KVSplitExchange(attn, nq, 1, dev)
q4 = case.q.to(dev).view(nq, 1, 32, 128)
for step in range(5):
    out2 = torch.full((nq, 1, 32, 128), float("nan"), dtype=torch.float32, device=dev)
    ex.decode(q4 * (1.0 + step), cache, bt, sl, out2)
    if step == 0:
        torch.cuda.synchronize()
        assert ex.status() == 0
        assert torch.equal(out2.view(nq, 32, 128), out), float((out2.view(nq, 32, 128) - out).abs().max())
torch.cuda.synchronize()
assert ex.status() == 0 and attn.status(nq, dev) == 0
ref = torch.empty(nq, 32, 128, dtype=torch.float32, device=dev)
kv_split_decode(attn, case.q.to(dev) * 5.0, cache, bt, sl, ref)
assert torch.equal(out2.view(nq, 32, 128), ref)
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok", float(err.max()))
"""


def test_kv_split_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(_RANK % {"root": str(ROOT)})
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29600 + os.getpid() % 300), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=600)
        assert p.returncode == 0 and f"rank {r} ok" in out, err[-3000:]


def test_exchange_protocol_single_rank(oracle, golden):
    """tq_decode_paged_exchange with world = 1 (this rank's buffer is the only peer): push, flag,
    wait, merge and the step counter over several calls and a graph replay, against
    tq_decode_paged_multi."""
    import math
    from turboquant_b200 import _cabi, synthetic
    from turboquant_b200.paged_attention import TurboQuantPagedAttention
    from turboquant_b200.parallel import KVSplitExchange
    from tests.gpu_util import DEV, oracle_cache
    lens = [300, 0, 1500]
    B, nq = len(lens), 2
    case = synthetic.decode_case(seed=31, seq_lens=lens, dtype=torch.float16)
    cache = torch.from_numpy(oracle_cache(oracle, case, golden["signs_seed42_d128"])).to(DEV)
    attn = TurboQuantPagedAttention(32, 128, 1 / math.sqrt(128), 8)
    q = torch.randn(B, nq, 32, 128, generator=torch.Generator().manual_seed(3)).to(torch.float16).to(DEV)
    bt, sl = case.block_table.to(DEV), case.seq_lens.to(DEV)
    want = attn.decode_shared(q, cache, bt, sl)
    nbytes = _cabi.exchange_bytes(B * nq * 32, 1)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    ex = KVSplitExchange(attn, B, nq, DEV, buffers=[buf])
    for step in range(3):
        out = torch.full_like(want, float("nan"))
        ex.decode(q, cache, bt, sl, out)
        torch.cuda.synchronize()
        assert ex.status() == 0 and int(buf[:4].view(torch.int32).item()) == step + 1
        assert torch.equal(out, want)
    out = torch.full_like(want, float("nan"))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ex.decode(q, cache, bt, sl, out)
    for _ in range(3):
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    assert ex.status() == 0


def test_exchange_head96_one_rank():
    """The same protocol for a padded head (96 -> 128): the exchanged partials are 128 wide, the output 96."""
    import math
    from turboquant_b200 import _cabi, synthetic
    from turboquant_b200.paged_attention import TurboQuantPagedAttention, kv_cache_shape
    from turboquant_b200.parallel import KVSplitExchange
    from tests.gpu_util import DEV
    lens, d, hq, hkv, nq = [300, 1500], 96, 32, 8, 2
    B = len(lens)
    case = synthetic.decode_case(seed=32, seq_lens=lens, dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    attn = TurboQuantPagedAttention(hq, d, 1 / math.sqrt(d), hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    attn.write(case.k.to(DEV), case.v.to(DEV), cache, case.slot_mapping.to(DEV))
    q = torch.randn(B, nq, hq, d, generator=torch.Generator().manual_seed(4)).to(torch.float16).to(DEV)
    bt, sl = case.block_table.to(DEV), case.seq_lens.to(DEV)
    want = attn.decode_shared(q, cache, bt, sl)
    buf = torch.zeros(_cabi.exchange_bytes(B * nq * hq, 1), dtype=torch.uint8, device=DEV)
    ex = KVSplitExchange(attn, B, nq, DEV, buffers=[buf])
    guard = torch.full((3,) + tuple(want.shape), 7.0, dtype=want.dtype, device=DEV)
    for step in range(2):
        ex.decode(q, cache, bt, sl, guard[1])
        torch.cuda.synchronize()
        assert ex.status() == 0
        assert torch.equal(guard[1], want)
    assert (guard[0] == 7.0).all() and (guard[2] == 7.0).all()
