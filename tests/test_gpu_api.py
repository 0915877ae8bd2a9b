"""The reference-facing Python surface on the GPU: algorithm API against the reference-made
fixtures, the torch ops under the reference's names, the engine-independent attention class and
the vLLM backend implementation class."""
import math
import types

import numpy as np
import pytest
import torch

from turboquant_b200 import synthetic
from tests.gpu_util import DEV, assert_attention_close, oracle_cache

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128)


def test_algorithm_api_matches_reference_fixtures(golden):
    from turboquant_b200 import Codebook, RandomHadamardRotation, TurboQuantMSE, fwht
    tq = TurboQuantMSE(128, 4, device=DEV, seed=42)
    rows = torch.from_numpy(golden["q_rows"]).to(DEV)
    packed, norms = tq.quantize(rows)
    np.testing.assert_array_equal(packed.cpu().numpy(), golden["q_packed_b4"])
    np.testing.assert_array_equal(norms.cpu().numpy().view(np.uint32), golden["q_norms"].view(np.uint32))
    np.testing.assert_allclose(tq.dequantize(packed[:64], norms[:64]).cpu().numpy(), golden["q_dequant_b4"],
                               rtol=1e-5, atol=1e-30)
    # determinism under the same seed, and the MSE bound of the reference's tests (4 bits: 0.009 x 2.5)
    p2, n2 = TurboQuantMSE(128, 4, device=DEV, seed=42).quantize(rows)
    assert torch.equal(p2, packed)
    x = torch.randn(2000, 128, device=DEV)
    x = x / x.norm(dim=-1, keepdim=True)
    xh = tq.dequantize(*tq.quantize(x))
    assert float(((x - xh) ** 2).sum(-1).mean()) < 0.009 * 2.5
    np.testing.assert_array_equal(fwht(torch.from_numpy(golden["fwht_in"]).to(DEV)).cpu().numpy(), golden["fwht_out"])
    assert fwht(torch.tensor([1.0, 0, 0, 0], device=DEV)).tolist() == [0.5, 0.5, 0.5, 0.5]
    rot = RandomHadamardRotation(96, device=DEV, seed=42)
    assert rot.padded_dim == 128 and rot.signs.cpu().tolist() == golden["signs_seed42_d96"].tolist()
    v = torch.randn(5, 96, device=DEV)
    y = rot.rotate(v)
    assert y.shape == (5, 128)
    np.testing.assert_allclose(rot.inverse_rotate(y).cpu().numpy(), v.cpu().numpy(), atol=1e-5)
    np.testing.assert_allclose(y.norm(dim=-1).cpu().numpy(), v.norm(dim=-1).cpu().numpy(), rtol=1e-5)
    cb = Codebook(128, 4, device=DEV)
    np.testing.assert_array_equal(cb.centroids.cpu().numpy(), golden["centroids_d128_b4"])
    idx = cb.quantize(torch.tensor([-1.0, 0.0, 1e-9, 1.0], device=DEV))
    assert idx.tolist() == [0, 7, 8, 15]
    assert torch.equal(cb.dequantize(idx), cb.centroids[idx.long()])


def test_torch_ops_with_reference_schemas(oracle, golden):
    from turboquant_b200 import ops  # noqa: F401
    case = synthetic.decode_case(seed=80, seq_lens=[300, 17, 640], dtype=torch.float16)
    signs = synthetic.make_signs().to(DEV)
    cache = torch.zeros((2, case.num_blocks, 16, 8, 80), dtype=torch.uint8, device=DEV)
    # the reference's call: fp32 K/V and int32 slots (vllm_backend_fused.py:299-304 there)
    torch.ops.turboquant_write.quantize_write_kv_cache(cache, case.k.float().to(DEV), case.v.float().to(DEV), signs,
                                                       case.slot_mapping.to(torch.int32).to(DEV), 128, 128)
    want_cache = oracle_cache(oracle, case, golden["signs_seed42_d128"])
    np.testing.assert_array_equal(cache.cpu().numpy(), want_cache)
    want = oracle.decode_paged(case.q.float().numpy(), want_cache, case.block_table.numpy(), case.seq_lens.numpy(),
                               golden["signs_seed42_d128"], SCALE)
    B, max_pages = 3, case.block_table.shape[1]
    bt, sl = case.block_table.to(DEV), case.seq_lens.to(DEV)
    indptr = torch.arange(B + 1, dtype=torch.int32, device=DEV) * max_pages       # the reference's strided table
    last = sl - ((sl + 15) // 16 - 1) * 16
    o_ws = torch.empty(B, 32, 128, dtype=torch.float16, device=DEV)
    e = torch.empty(0, device=DEV)
    ei = torch.empty(0, dtype=torch.int32, device=DEV)
    out = torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws(
        case.q.to(DEV), cache, bt.reshape(-1), indptr, last, sl, 8, 16, 128, 128, SCALE, signs, 64, 4, o_ws,
        max_pages * 16, e, e, ei, ei, ei, ei, 4)
    assert out.data_ptr() == o_ws.data_ptr()
    assert_attention_close(out.float().cpu().numpy(), want, "paged split op")
    o2 = torch.zeros_like(o_ws)
    torch.ops.turboquant_v5.decode_v5_from_cache_ws(case.q.to(DEV), cache, bt.reshape(-1), indptr, last, sl, 8, 16,
                                                    128, 128, SCALE, signs, 64, 4, e, e, e, e, o2, max_pages * 16)
    assert torch.equal(o2, o_ws)


@pytest.mark.parametrize("d,pd,hq,hkv", [(64, 64, 16, 8), (256, 256, 8, 4), (96, 128, 24, 8)])
def test_torch_ops_take_the_other_head_sizes(oracle, golden, d, pd, hq, hkv):
    """The reference declares these geometries (kernel_config presets) while its decode op takes 128 only; the
    ops here take head sizes 33 ... 256 with the reference's padded size, and refuse a padded size that is not it."""
    from turboquant_b200 import ops, _cabi  # noqa: F401
    from turboquant_b200.paged_attention import kv_cache_shape
    case = synthetic.decode_case(seed=84 + d, seq_lens=[300, 17, 640], dtype=torch.float16, heads=(hq, hkv), head_dim=d)
    signs_np = golden[f"signs_seed42_d{d if d == 96 else pd}"]
    signs = torch.from_numpy(signs_np).to(DEV)
    scale = 1.0 / math.sqrt(d)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    torch.ops.turboquant_write.quantize_write_kv_cache(cache, case.k.float().to(DEV), case.v.float().to(DEV), signs,
                                                       case.slot_mapping.to(torch.int32).to(DEV), d, pd)
    want_cache = np.zeros(tuple(cache.shape), np.uint8)
    oracle.write_kv_cache(want_cache, case.k.float().numpy(), case.v.float().numpy(), signs_np, case.slot_mapping.numpy(), d)
    np.testing.assert_array_equal(cache.cpu().numpy(), want_cache)
    want = oracle.decode_paged(case.q.float().numpy(), want_cache, case.block_table.numpy(), case.seq_lens.numpy(), signs_np, scale)
    B, max_pages = 3, case.block_table.shape[1]
    bt, sl = case.block_table.to(DEV), case.seq_lens.to(DEV)
    indptr = torch.arange(B + 1, dtype=torch.int32, device=DEV) * max_pages
    last = sl - ((sl + 15) // 16 - 1) * 16
    o_ws = torch.empty(B, hq, d, dtype=torch.float16, device=DEV)
    e = torch.empty(0, device=DEV)
    ei = torch.empty(0, dtype=torch.int32, device=DEV)
    out = torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws(
        case.q.to(DEV), cache, bt.reshape(-1), indptr, last, sl, hkv, 16, d, pd, scale, signs, pd // 2, 2 * (pd // 64), o_ws,
        max_pages * 16, e, e, ei, ei, ei, ei, 4)
    assert out.data_ptr() == o_ws.data_ptr()
    assert_attention_close(out.float().cpu().numpy(), want, f"paged split op, head size {d}")
    with pytest.raises(Exception, match="padded"):
        torch.ops.turboquant_write.quantize_write_kv_cache(cache, case.k.float().to(DEV), case.v.float().to(DEV), signs,
                                                           case.slot_mapping.to(torch.int32).to(DEV), d, 2 * pd)


def test_decoder_dispatch_returns_the_single_kernel():
    from turboquant_b200.decoder_dispatch import KERNEL_NAME, pick_decode_op
    pick_decode_op.cache_clear()
    op, name = pick_decode_op()
    assert name == KERNEL_NAME and callable(op)


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (64, 16, 8), (256, 8, 4)])
def test_cuda_graph_capture_of_write_and_decode(oracle, golden, d, hq, hkv):
    """The step a serving engine replays: cache write + decode captured once, replayed on new data."""
    from turboquant_b200 import TurboQuantPagedAttention
    from turboquant_b200.paged_attention import kv_cache_shape
    SCALE = 1.0 / math.sqrt(d)
    case = synthetic.decode_case(seed=81, seq_lens=[400, 90], dtype=torch.bfloat16, heads=(hq, hkv), head_dim=d)
    attn = TurboQuantPagedAttention(hq, d, SCALE, hkv)
    cache = torch.zeros(kv_cache_shape(case.num_blocks, 16, hkv, d), dtype=torch.uint8, device=DEV)
    k, v, slots = case.k.to(DEV), case.v.to(DEV), case.slot_mapping.to(DEV)
    q, bt, sl = case.q.to(DEV), case.block_table.to(DEV), case.seq_lens.to(DEV)
    out = torch.empty_like(q)
    attn.write(k, v, cache, slots)
    attn.decode(q, cache, bt, sl, out)                          # warm-up: workspaces, kernel attributes
    eager = out.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        attn.write(k, v, cache, slots)
        attn.decode(q, cache, bt, sl, out)
    torch.cuda.current_stream().wait_stream(side)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    q.copy_(torch.randn_like(q))                                 # new query, same graph
    graph.replay()
    torch.cuda.synchronize()
    want = oracle.decode_paged(q.float().cpu().numpy(), cache.cpu().numpy(), case.block_table.numpy(),
                               case.seq_lens.numpy(), golden[f"signs_seed42_d{d}"], SCALE)
    assert_attention_close(out.float().cpu().numpy(), want, f"graph replay, head size {d}")
    assert attn.status(2, q.device) == 0


def test_vllm_backend_impl_write_and_decode(oracle, golden):
    pytest.importorskip("vllm")
    from turboquant_b200.vllm_backend_fused import TurboQuantBackend, TurboQuantFusedImpl
    try:
        impl = TurboQuantFusedImpl(32, 128, SCALE, 8, None, None, "fp8")
    except Exception as e:  # the parent constructor may need an engine context in this vLLM version
        pytest.skip(f"FlashAttentionImpl cannot be built outside an engine here: {type(e).__name__}: {e}")
    case = synthetic.decode_case(seed=82, seq_lens=[257, 1000, 31, 64], dtype=torch.bfloat16)
    shape = TurboQuantBackend.get_kv_cache_shape(case.num_blocks, 16, 8, 128, "fp8")
    kv_cache = torch.zeros(shape, dtype=torch.uint8, device=DEV)
    impl.do_kv_cache_update(None, case.k.to(DEV), case.v.to(DEV), kv_cache, case.slot_mapping.to(DEV))
    np.testing.assert_array_equal(kv_cache.cpu().numpy(), oracle_cache(oracle, case, golden["signs_seed42_d128"]))
    md = types.SimpleNamespace(max_query_len=1, num_actual_tokens=4, block_table=case.block_table.to(DEV),
                               seq_lens=case.seq_lens.to(DEV), query_start_loc=None)
    q = case.q.to(DEV).reshape(4, 32 * 128)
    out = torch.zeros_like(q)
    impl.forward(None, q, None, None, kv_cache, md, output=out)
    want = oracle.decode_paged(case.q.float().numpy(), kv_cache.cpu().numpy(), case.block_table.numpy(),
                               case.seq_lens.numpy(), golden["signs_seed42_d128"], SCALE)
    assert_attention_close(out.float().cpu().numpy().reshape(4, 32, 128), want, "vLLM impl decode")


def _backend_step(oracle, golden, cached, chunk, with_builder_facts, heads=(32, 8), d=128):
    """One forward of the vLLM backend on a step with the given cached / new token counts per
    sequence, checked against plain torch attention: rows with one new token and cached context are
    decode rows, rows with up to eight new tokens and cached context are short rows (for both, every
    key, the new ones included, is read from the quantized cache); all other rows attend their
    dequantized cached tokens followed by the chunk's fresh K/V."""
    pytest.importorskip("vllm")
    from turboquant_b200.vllm_backend_fused import (TurboQuantBackend, TurboQuantFusedImpl, causal_chunk_supported,
                                                    step_shape)
    hq, hkv = heads
    grp, scale = hq // hkv, 1.0 / math.sqrt(d)
    fuse_short = causal_chunk_supported(hq, hkv, d)    # else rows of 2 ... 8 new tokens go the dense way
    try:
        impl = TurboQuantFusedImpl(hq, d, scale, hkv, None, None, "fp8")
        from vllm.vllm_flash_attn import flash_attn_varlen_func  # noqa: F401
    except Exception as e:
        pytest.skip(f"vLLM attention pieces not usable here: {type(e).__name__}: {e}")
    B = len(cached)
    total = [c + q for c, q in zip(cached, chunk)]
    case = synthetic.decode_case(seed=83 + B + sum(chunk), seq_lens=total, dtype=torch.bfloat16, heads=heads, head_dim=d)
    shape = TurboQuantBackend.get_kv_cache_shape(case.num_blocks, 16, hkv, d, "fp8")
    kv_cache = torch.zeros(shape, dtype=torch.uint8, device=DEV)
    impl.do_kv_cache_update(None, case.k.to(DEV), case.v.to(DEV), kv_cache, case.slot_mapping.to(DEV))
    # the chunk: the last chunk[b] tokens of every sequence (their K/V are case.k / case.v rows)
    starts = np.concatenate([[0], np.cumsum(total)])
    rows = np.concatenate([np.arange(starts[b] + cached[b], starts[b + 1]) for b in range(B)])
    n = len(rows)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(n, hq, d, generator=g).to(torch.bfloat16)
    key, value = case.k[rows], case.v[rows]
    qsl_cpu = torch.tensor(np.concatenate([[0], np.cumsum(chunk)]), dtype=torch.int32)
    md = types.SimpleNamespace(max_query_len=max(chunk), num_actual_tokens=n, block_table=case.block_table.to(DEV),
                               seq_lens=case.seq_lens.to(DEV), query_start_loc=qsl_cpu.to(DEV), max_seq_len=max(total))
    if with_builder_facts:
        md.tq_step = step_shape(types.SimpleNamespace(query_start_loc_cpu=qsl_cpu, num_reqs=B,
                                                      seq_lens_cpu=case.seq_lens))
    out = torch.zeros(n, hq * d, dtype=torch.bfloat16, device=DEV)
    try:
        impl.forward(None, q.to(DEV).reshape(n, -1), key.to(DEV), value.to(DEV), kv_cache, md, output=out)
    except (RuntimeError, ImportError) as e:
        if "flash" in str(e).lower() or "FA" in str(e):
            pytest.skip(f"vLLM's FlashAttention does not run on this device: {e}")
        raise
    got = out.float().cpu().numpy().reshape(n, hq, d)
    cache_np = kv_cache.cpu().numpy()
    signs = golden[f"signs_seed42_d{max(64, 1 << (d - 1).bit_length())}"]
    want = np.zeros_like(got)
    decode_rows = []
    qi = 0
    for b in range(B):
        is_decode = 1 <= chunk[b] <= (8 if fuse_short else 1) and cached[b] > 0   # decode and short rows: this package's kernels
        if is_decode:
            decode_rows.extend(range(qi, qi + chunk[b]))
        t = np.arange(total[b] if is_decode else cached[b])
        pages = case.block_table.numpy()[b, t // 16]
        kc = oracle.dequant_cache_rows(cache_np[0, pages, t % 16], signs, d).reshape(-1, hkv, d)
        vc = oracle.dequant_cache_rows(cache_np[1, pages, t % 16], signs, d).reshape(-1, hkv, d)
        kc, vc = torch.from_numpy(kc), torch.from_numpy(vc)
        if is_decode:
            ka, va = kc, vc
        else:                                                        # the backend holds them in the query dtype
            ka = torch.cat([kc.to(torch.bfloat16).float(), case.k[starts[b] + cached[b]:starts[b + 1]].float()])
            va = torch.cat([vc.to(torch.bfloat16).float(), case.v[starts[b] + cached[b]:starts[b + 1]].float()])
        for i in range(chunk[b]):
            kk, vv = ka[: cached[b] + i + 1], va[: cached[b] + i + 1]
            qq = q[qi].float().view(hkv, grp, d)
            sc = torch.einsum("hgd,thd->hgt", qq, kk) * scale
            want[qi] = torch.einsum("hgt,thd->hgd", torch.softmax(sc, -1), vv).reshape(hq, d).numpy()
            qi += 1
    # Decode rows come from this package's kernel: the usual bar.  The other rows come out of vLLM's
    # FlashAttention on bf16 K/V with bf16 probabilities (a library kernel, the same one the
    # reference runs on a first chunk): the tensor within 1e-2 relative, every element within 1 % of
    # the largest output.
    dec = np.zeros(n, bool)
    dec[decode_rows] = True
    if dec.any():
        assert_attention_close(got[dec], want[dec], f"decode rows, cached={cached} chunk={chunk}")
    if (~dec).any():
        err = np.abs(got[~dec] - want[~dec])
        assert err.max() <= 2e-3 + 1e-2 * np.abs(want[~dec]).max(), err.max()
        assert np.linalg.norm(got[~dec] - want[~dec]) / np.linalg.norm(want[~dec]) <= 1e-2


@pytest.mark.parametrize("with_builder_facts", [False, True])
def test_vllm_backend_continuation_prefill(oracle, golden, with_builder_facts):
    """Chunks of new tokens over sequences with cached context (and one without)."""
    _backend_step(oracle, golden, [100, 0, 37], [5, 8, 3], with_builder_facts)


@pytest.mark.parametrize("with_builder_facts", [False, True])
def test_vllm_backend_long_first_chunk_beside_a_short_continuation(oracle, golden, with_builder_facts):
    """The longest sequence of the step is a first chunk: max_seq_len == max_query_len although
    another sequence has cached context, which must still be attended."""
    _backend_step(oracle, golden, [0, 1400], [2048, 100], with_builder_facts)


@pytest.mark.parametrize("with_builder_facts", [False, True])
def test_vllm_backend_mixed_decode_and_prefill_rows(oracle, golden, with_builder_facts):
    """vLLM's default mixed batches: decode rows ride the paged decode kernel, the prefill rows the
    dense path, in one step; a one-token prompt (nothing cached) stays on the dense path."""
    _backend_step(oracle, golden, [500, 0, 37, 1200, 0], [1, 8, 3, 1, 1], with_builder_facts)


def test_vllm_backend_pure_first_chunks_use_fresh_kv(oracle, golden):
    _backend_step(oracle, golden, [0, 0], [33, 70], True)


@pytest.mark.parametrize("with_builder_facts", [False, True])
def test_vllm_backend_short_chunks_attend_the_quantized_cache(oracle, golden, with_builder_facts):
    """Rows with two to eight new tokens over cached context (short continuation chunks, speculative
    verification) go through the causal wide-tile kernel, next to decode rows, a longer chunk and a
    first chunk; one of them has fewer cached tokens than pad queries."""
    _backend_step(oracle, golden, [500, 3, 37, 1200, 0, 64], [1, 6, 3, 12, 2, 8], with_builder_facts)


@pytest.mark.parametrize("heads,d", [((64, 8), 128), ((16, 8), 64), ((8, 1), 128)])
@pytest.mark.parametrize("with_builder_facts", [False, True])
def test_vllm_backend_short_chunks_without_the_causal_kernel(oracle, golden, with_builder_facts, heads, d):
    """Geometries the causal wide-tile kernel does not take (eight query heads per KV head, head size 64, one KV
    head): rows with two to eight new tokens go the dense way, decode rows still ride the paged kernel, and the
    dense buffer is sized for them."""
    _backend_step(oracle, golden, [500, 3, 37, 300, 0, 64], [1, 6, 3, 12, 2, 8], with_builder_facts, heads=heads, d=d)
