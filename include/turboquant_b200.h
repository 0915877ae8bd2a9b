/*
 * turboquant_b200 — C ABI of the B200 (sm_100a) TurboQuant KV-cache hot paths.
 *
 * Every entry point takes plain device/host pointers, sizes and a CUDA stream (passed as
 * void*, i.e. a cudaStream_t), returns an int status (0 = TQ_OK), launches asynchronously on
 * that stream, never synchronises and — unless its comment says otherwise — never allocates.
 * On a non-zero return tq_last_error() gives a message for the calling thread.
 *
 * Each declaration names the reference interface it stands in for (path:line within the
 * RRoundTable/turboquant tree).
 */
#ifndef TURBOQUANT_B200_H
#define TURBOQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_ABI_VERSION 1

/* status codes */
enum {
    TQ_OK = 0,
    TQ_ERR_INVALID = 1,     /* bad argument (null pointer, shape, alignment) */
    TQ_ERR_UNSUPPORTED = 2, /* valid but not implemented for this geometry */
    TQ_ERR_CUDA = 3,        /* a CUDA runtime call or launch failed */
    TQ_ERR_WORKSPACE = 4    /* caller-provided workspace too small */
};

/* element types of caller tensors */
enum { TQ_F32 = 0, TQ_F16 = 1, TQ_BF16 = 2 };
/* integer types of index tensors */
enum { TQ_I32 = 0, TQ_I64 = 1 };
/* nibble order of flat packed codes */
enum {
    TQ_PACK_LOW_FIRST = 0, /* TurboQuantMSE._pack_bits: value i at bit offset i*bits (quantizer.py:17-39) */
    TQ_PACK_CACHE = 1      /* paged cache / tile order: even dim in the high nibble (tile.py:37-41) */
};
/* flags of tq_write_kv_cache */
enum {
    TQ_WRITE_DEFAULT = 0,
    TQ_WRITE_ZERO_PAD = 1, /* also store zeros to the pad bytes after the norms (the reference leaves them alone) */
    TQ_WRITE_EXACT_PATH = 2, /* always run the kernel that evaluates the reference's arithmetic for every element
                                (default: large writes of 16-bit rows take the tensor-core kernel, which produces
                                the same bytes and re-derives only the codes next to a boundary that way) */
    TQ_WRITE_TENSOR_PATH = 4 /* always run the tensor-core kernel (fp16 / bf16 rows of 128 elements only) */
};

int tq_abi_version(void);
const char* tq_last_error(void);

/* Lloyd-Max centroids (2^bits) and decision boundaries (2^bits - 1) for a rotated unit vector
 * of dimension dim, rounded to fp32 the way the reference builds its tensors.  Host only.
 * Replaces: Codebook.__init__ (turboquant/codebook.py:72-90). */
int tq_codebook(int dim, int bits, float* centroids, float* boundaries);

/* ---------------------------------------------------------------------------------------
 * Cache write.  Quantizes num_tokens x num_kv_heads K rows and V rows (seeded signs -> FWHT ->
 * L2 norm -> 4-bit Lloyd-Max code -> nibble pack) and scatters them into the paged cache
 *   kv_cache : uint8 [2][num_blocks][block_size][num_kv_heads][slot_bytes]
 * at slot_mapping[t] = block*block_size + entry; a negative slot skips the token, and so does a
 * slot at or beyond num_blocks * block_size (counted, see tq_fault_counts).  Per slot:
 * bytes [0, pd/2) codes (even dim high nibble), then the fp16 norm once per 64 dims, pad
 * untouched.  key/value: [num_tokens][num_kv_heads][head_dim] of in_dtype with
 * k_token_stride / v_token_stride elements between tokens (heads contiguous).  One launch
 * covers K and V.  Codes and norms are bit-identical to TurboQuantMSE.quantize on the CPU.
 * head_dim 128, or 96 (rows of 96 elements, zero-padded to 128 by the rotation; signs has 128
 * entries either way).  Any other head size from 33 to 256 (64 with 48-byte slots, 256 with
 * 144-byte slots: turboquant/vllm_backend_fused.py:64-72, turboquant/kernel_config.py:75-109)
 * goes through plain, untuned kernels with the same arithmetic; signs then has next_pow2(head_dim)
 * entries.  signs is a constant of the context, as in the reference (one seeded
 * vector per process): the kernel reads it ahead of its wait on the preceding kernel, so it must
 * be complete before that kernel is launched.
 * Replaces: torch.ops.turboquant_write.quantize_write_kv_cache
 *   (csrc/src/quantize_write_binding.cu:207-269, kernel csrc/include/turboquant/quantize_write_kernel.cuh:332-431),
 *   called from TurboQuantFusedImpl._write_to_cache (turboquant/vllm_backend_fused.py:293-305). */
int tq_write_kv_cache(void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                      int slot_bytes, const void* key, const void* value, int in_dtype,
                      int64_t num_tokens, int64_t k_token_stride, int64_t v_token_stride,
                      const float* signs, const void* slot_mapping, int slot_dtype, int head_dim,
                      int flags, void* stream);

/* ---------------------------------------------------------------------------------------
 * Flat quantizer API (any leading shape flattened to n rows of dim elements, dim <= 256,
 * padded to the next power of two with zeros).  bits in 1..4.
 * Replaces: TurboQuantMSE.quantize / .dequantize (turboquant/quantizer.py:77-106). */
int tq_quantize_flat(const void* x, int x_dtype, int64_t n, int dim, const float* signs, int bits,
                     int pack_order, uint8_t* packed, float* norms, void* stream);
int tq_dequantize_flat(const uint8_t* packed, const float* norms, int64_t n, int dim,
                       const float* signs, int bits, int pack_order, float* out, void* stream);

/* Normalized fast Walsh-Hadamard transform of n rows of padded_dim (power of two <= 256)
 * fp32 elements: out = FWHT(pre_signs * pad(x)) * post_signs, either sign vector may be NULL.
 * in_dim <= padded_dim elements are read per row, out_dim <= padded_dim written.
 * Replaces: fwht, RandomHadamardRotation.rotate / inverse_rotate (turboquant/hadamard.py:21-78). */
int tq_fwht(const float* x, int64_t n, int in_dim, int padded_dim, int out_dim,
            const float* pre_signs, const float* post_signs, float* out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Paged decode attention over the quantized cache: one query token per sequence,
 *   out[b, hq, :] = softmax(q[b, hq] . K^[b]^T * sm_scale) V^[b]
 * evaluated in the rotated domain (Q is rotated once, the output is rotated back after the
 * split-KV merge).  The KV range of every sequence is cut into page-aligned pieces that are
 * balanced over num_ctas thread blocks on the device (no host planning, no host sync); the
 * pieces' normalized partial outputs and base-2 log-sum-exps go to the workspace and a second
 * kernel merges them, applies the inverse rotation and stores out.
 *
 *   q            [batch][num_q_heads][head_dim]            q_dtype (f16 | bf16 | f32)
 *   kv_cache     uint8 [2][num_blocks][block_size][num_kv_heads][slot_bytes]
 *   page_indices int32; sequence b's pages are page_indices[page_indptr[b] + i];
 *                page_indptr == NULL means a dense block table with row stride max_pages
 *   seq_lens     int32 [batch] (device)
 *   out          [batch][num_q_heads][head_dim]            out_dtype
 *   out_lse      optional fp32 [batch][num_q_heads], natural-log LSE of the scaled scores
 *   workspace    at least tq_decode_workspace_bytes(...) bytes, 256-byte aligned.  Its first int32 is a
 *                sticky status word (0 ok, 1 a bounded wait ran out, 2 too many sequences per block,
 *                3 shared-memory map did not fit, 4 a sequence is longer than its page table: nothing
 *                is read and out is zero, 5 a page id outside [0, num_blocks): that page is replaced
 *                by page 0, out is wrong but no address is formed from the id): zero the workspace
 *                once if you want to read it; no call clears it and nothing else in the workspace
 *                needs initialising
 *   num_ctas     thread blocks to balance over; 0 = one per SM of the current device
 *
 * Other head sizes (33..256; 64 and 256 are the reference's other presets) run a second tier of
 * kernels behind the same entry points (a quarter to two fifths of the HBM peak against the tuned
 * kernels' three fifths): block_size 16, slot_bytes >= the slot of that head size (a multiple of 16
 * for the tensor-core decode, anything else takes a plain one), any number of KV heads, up to 8
 * query columns per KV head (query heads per KV head x queries sharing a sequence), KV windows and
 * tq_merge_rotated, no causal queries and no kernel-side exchange; pass head_dim to
 * tq_decode_workspace_bytes.  The rest of this paragraph is the tuned path.
 * Supported geometry: head_dim 128, or 96 (q and out rows of 96 elements; the rotation pads them
 * with zeros to 128 and the slot is the same 80 bytes); block_size 16, slot_bytes 80,
 * num_q_heads/num_kv_heads <= 8, num_kv_heads in {1, 2, 4, 8, 16} (one launch) or a larger
 * multiple of 4 (several launches of 16 / 8 / 4 heads; the workspace is sized for the largest).
 * Replaces: torch.ops.turboquant_v5.decode_v5_from_cache_paged_splitkv_ws and
 *   decode_v5_from_cache_ws (csrc/src/decode_v5_tc_binding.cu:754-874, 440-551), kernels
 *   csrc/include/flashinfer_decode_turboquant_v5_tc.cuh:112-795 and
 *   csrc/include/flashinfer_decode_turboquant_combine.cuh:18-79; the split planning replaces
 *   TurboQuantFusedImpl._choose_num_splits/_get_v5_ws (turboquant/vllm_backend_fused.py:129-215). */
size_t tq_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                 int num_ctas);
/* Widest query tile of the decode kernels: queries_per_seq x (num_q_heads / num_kv_heads) of
 * tq_decode_paged_multi may not exceed it.  The reference's kernel has a fixed tile of 4 query
 * heads per KV head (csrc/src/decode_v5_tc_binding.cu:779-785). */
int tq_decode_max_query_columns(void);
int tq_decode_paged(const void* q, int q_dtype, int batch, int num_q_heads, int num_kv_heads,
                    int head_dim, const void* kv_cache, int64_t num_blocks, int block_size,
                    int slot_bytes, const int32_t* page_indices, const int32_t* page_indptr,
                    int max_pages, const int32_t* seq_lens, const float* signs, float sm_scale,
                    void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                    float* out_lse, int num_ctas, void* stream);

/* tq_decode_paged for sequences that carry several decode queries sharing one KV (the 8 queries
 * of the 1M-token configuration, or any caller that would otherwise repeat a sequence as batch
 * rows): q and out are [batch][queries_per_seq][num_q_heads][head_dim], out_lse
 * [batch][queries_per_seq][num_q_heads]; seq_lens and the page table are per sequence.  The
 * queries ride in the columns of one query tile, so the KV is streamed and dequantized once for
 * all of them.  queries_per_seq x (num_q_heads / num_kv_heads) <= 8 takes the 8-wide tile of the
 * mma.sync kernel; 9 ... 32 columns take the wide-tile kernel (tcgen05.mma, accumulators in tensor
 * memory), which needs head_dim 128 or 96 and 2, 4, 8 or 16 KV heads and ignores num_ctas below the
 * number of KV-head pairs.  Other head sizes (33 ... 256) take up to 8 columns.
 * The workspace is sized with tq_decode_workspace_bytes(batch, queries_per_seq * num_q_heads, ...).
 * kv_begin / kv_end restrict the tokens as in tq_decode_paged_partial (0, -1: all of them);
 * rotated_partial != 0 makes out (fp32) and out_lse (required) the rotated-domain partial and
 * base-2 LSE that tq_merge_rotated takes, rows ordered [batch][queries_per_seq][num_q_heads].
 * The reference's ops have no such mode: there each query is a batch row that re-reads the KV
 * (csrc/src/decode_v5_tc_binding.cu:783-785). */
int tq_decode_paged_multi(const void* q, int q_dtype, int batch, int queries_per_seq, int num_q_heads,
                          int num_kv_heads, int head_dim, const void* kv_cache, int64_t num_blocks,
                          int block_size, int slot_bytes, const int32_t* page_indices,
                          const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                          int64_t kv_begin, int64_t kv_end, const float* signs, float sm_scale,
                          void* workspace, size_t workspace_bytes, void* out, int out_dtype, float* out_lse,
                          int rotated_partial, int num_ctas, void* stream);

/* tq_decode_paged_multi with a causal mask among the queries of a sequence: the queries_per_seq
 * queries of a row are the LAST queries_per_seq tokens of that sequence, in order, their K / V already
 * written to the cache (seq_lens counts them); query i attends to the first
 * seq_len - (queries_per_seq - 1 - i) tokens.  This is a chunk of a prefill that continues over the
 * quantized cache, or the verification step of speculative decoding, in one pass over the KV for
 * up to 32 / (num_q_heads / num_kv_heads) query tokens; a longer chunk is several batch rows that
 * share the page table and differ in seq_lens.  Always the wide-tile kernel: head_dim 128 or 96,
 * 2, 4, 8 or 16 KV heads, whole sequences.  A query without a visible token gets zeros and LSE -inf.
 * The reference's prefill does not read the cache at all (turboquant/vllm_backend_fused.py:336-369:
 * FlashAttention over the fresh K / V only), so a chunk after the first one is wrong there; its
 * upstream successor dequantizes the whole context to dense K / V first
 * (docs/reference/vllm-upstream-turboquant-architecture.md:241-270). */
int tq_decode_paged_causal(const void* q, int q_dtype, int batch, int queries_per_seq, int num_q_heads,
                           int num_kv_heads, int head_dim, const void* kv_cache, int64_t num_blocks,
                           int block_size, int slot_bytes, const int32_t* page_indices,
                           const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                           const float* signs, float sm_scale, void* workspace, size_t workspace_bytes,
                           void* out, int out_dtype, float* out_lse, int num_ctas, void* stream);

/* Bulk dequantization of the cached tokens of `batch` sequences into dense, varlen-packed K and V
 * ([total_tokens][num_kv_heads][head_dim], row cu_seqlens[b] + t for token t of sequence b,
 * out_token_stride elements between tokens): what a chunk of new query tokens needs in order to
 * attend to KV that already sits quantized in the cache (continuation of a prefill) through a
 * dense varlen attention kernel.  Per row: centroid lookup, inverse rotation (butterflies h = 1..64,
 * 1/sqrt(128), signs), times the slot's fp16 norm — TurboQuantMSE.dequantize (quantizer.py:93-106)
 * on cache slots, as in the reference's dequant-attention check (tests/test_fused_integration.py:
 * 127-159).  The reference backend itself never reads the cache during prefill
 * (vllm_backend_fused.py:336-369).  fp32 output is bit-identical to that arithmetic; fp16/bf16
 * output is its rounding.  seq_lens, cu_seqlens [batch + 1] and the page table are device int32. */
int tq_dequant_paged(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                     int slot_bytes, const int32_t* page_indices, const int32_t* page_indptr,
                     int max_pages, const int32_t* seq_lens, const int32_t* cu_seqlens, int batch,
                     const float* signs, int head_dim, void* k_out, void* v_out, int out_dtype,
                     int64_t out_token_stride, void* stream);

/* Offload / restore of packed cache pages: the K and V halves of the pages listed in page_ids
 * (device int32) are gathered into / scattered from one contiguous buffer
 *   packed[n_pages][2][block_size][num_kv_heads][68]   (64 code bytes + the fp16 norm twice);
 * the 12 pad bytes of a slot are not moved and stay as they are on restore.  `packed` is device
 * memory, sized by tq_pages_packed_bytes; copy it to and from pinned host memory on the same
 * stream.  The reference measures this trade (restore over PCIe against re-running the prefill)
 * with a raw copy of a whole slab, pad bytes included (tests/bench_kv_offload.py:23-62). */
size_t tq_pages_packed_bytes(int n_pages, int block_size, int num_kv_heads);
/* The same for other slot sizes: 48-byte slots (head size 64) move 36 bytes, 144-byte slots (head
 * size 256) 136, any other size is moved whole; tq_pages_gather / _scatter pick the payload from
 * slot_bytes the same way. */
size_t tq_pages_packed_bytes_for_slot(int n_pages, int block_size, int num_kv_heads, int slot_bytes);
int tq_pages_gather(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                    int slot_bytes, const int32_t* page_ids, int n_pages, void* packed,
                    size_t packed_bytes, void* stream);
int tq_pages_scatter(void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                     int slot_bytes, const int32_t* page_ids, int n_pages, const void* packed,
                     size_t packed_bytes, void* stream);

/* One long sequence whose KV axis is split over `world` GPUs (one process per GPU): decode this
 * rank's token range, push the rotated partial + LSE into EVERY rank's exchange buffer with plain
 * peer stores (NVLink), release a per-source flag, then wait (bounded, about a second) until all
 * ranks' partials of this step have arrived in this rank's buffer, merge them and rotate back.
 * Every rank ends with the same full `out`.  Arguments as tq_decode_paged_multi, plus:
 *   exchange_bufs  host array [world] of device pointers: rank r's exchange buffer as mapped in
 *                  THIS process (symmetric memory / IPC); exchange_bufs[rank] is this rank's own.
 *                  Each is tq_exchange_bytes(batch * queries_per_seq * num_q_heads, world) bytes,
 *                  256-byte aligned, zeroed once on every rank before any rank's first call.
 * The step counter lives in the buffer, so the call can be captured in a CUDA graph and replayed.
 * Word 1 of the buffer is a sticky status: 1 = a wait for a peer ran out (out is then not written).
 * tq_set_exchange_wait_limit sets, for the calls this process makes afterwards, how many polls
 * (256 ns apart) that wait may take before it gives up; 0 restores the default (2^22, about a
 * second).  All ranks must make the same sequence of calls.  Replaces the reference-side plan of an
 * all-gather of split partials followed by SplitKVCombineKernel (combine.cuh:18-79) across GPUs;
 * the reference itself has no multi-GPU decode. */
size_t tq_exchange_bytes(int64_t rows, int world);
int tq_set_exchange_wait_limit(int polls);
int tq_decode_paged_exchange(const void* q, int q_dtype, int batch, int queries_per_seq, int num_q_heads,
                             int num_kv_heads, int head_dim, const void* kv_cache, int64_t num_blocks,
                             int block_size, int slot_bytes, const int32_t* page_indices,
                             const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                             int64_t kv_begin, int64_t kv_end, const float* signs, float sm_scale,
                             void* workspace, size_t workspace_bytes, int rank, int world,
                             void* const* exchange_bufs, size_t exchange_bytes, void* out, int out_dtype,
                             float* out_lse, int num_ctas, void* stream);

/* As tq_decode_paged, but stops before the inverse rotation: writes the merged, normalized,
 * still-rotated output (fp32 [batch][num_q_heads][padded width: 128, or 64 / 256 for those head sizes]) and its base-2 LSE, restricted to
 * tokens [kv_begin, kv_end) of every sequence (kv_end < 0: to the end).  This is the per-GPU
 * half of a KV-axis split across GPUs; the halves are exchanged and finished with
 * tq_merge_rotated.  No reference counterpart (the reference has no multi-GPU path); it
 * extends the partial/LSE contract of combine.cuh:18-79. */
int tq_decode_paged_partial(const void* q, int q_dtype, int batch, int num_q_heads,
                            int num_kv_heads, int head_dim, const void* kv_cache,
                            int64_t num_blocks, int block_size, int slot_bytes,
                            const int32_t* page_indices, const int32_t* page_indptr, int max_pages,
                            const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                            const float* signs, float sm_scale, void* workspace,
                            size_t workspace_bytes, float* out_rot, float* out_lse2, int num_ctas,
                            void* stream);

/* Log-sum-exp merge of num_parts rotated partial outputs, then inverse rotation:
 *   partial_o    fp32 [num_parts][rows][padded]     (normalized, rotated domain: the padded width,
 *                                                     128 for head_dim 128 / 96, else 64, 128 or 256)
 *   partial_lse2 fp32 [num_parts][rows]             (base-2 LSE; -inf marks an empty part)
 *   out          [rows][head_dim] out_dtype (head_dim 33 ... 256); out_lse optional natural-log LSE [rows]
 * Replaces: SplitKVCombineKernel (csrc/include/flashinfer_decode_turboquant_combine.cuh:18-79)
 * plus the inverse rotation at flashinfer_decode_turboquant_v5_tc.cuh:709-765. */
int tq_merge_rotated(const float* partial_o, const float* partial_lse2, int num_parts,
                     int64_t rows, int head_dim, const float* signs, void* out, int out_dtype,
                     float* out_lse, void* stream);

/* tq_decode_paged for callers that cannot hand over (or create) a workspace: an engine plugin
 * whose device memory pool is already fully assigned, or a caller on a path where cudaMalloc is
 * not allowed.  It has no counterpart in the reference (there the caller always allocates the
 * split-KV workspaces, turboquant/vllm_backend_fused.py:158-215).  The split-KV scratch is a
 * fixed array of TQ_STATIC_SCRATCH_BYTES (8 MiB) inside the library image; every GPU
 * that loads the library holds it until the process exits.  Arguments and results are those of
 * tq_decode_paged without the workspace pair, with num_kv_heads restricted to 1, 2, 4, 8 or 16.
 *   - Calls whose scratch need (tq_decode_workspace_bytes: it grows with batch, num_q_heads and
 *     num_ctas) exceeds the array fail with TQ_ERR_WORKSPACE and a message.  With one block per
 *     SM on a 148-SM part: 32 query / 8 KV heads fit up to batch 105; a tensor-parallel shard
 *     with 32 query heads over 4 KV heads needs 9.8 MB already at batch 1 and never fits (pass a
 *     smaller num_ctas, or use tq_decode_paged with your own workspace).
 *   - The first call on each device looks up the array's device address; make that call before
 *     starting any stream capture.  No call allocates or frees device memory.
 *   - All calls on one device share the array and find the previous call's contents in it: every
 *     part that a call reads is overwritten by that call first, and the only word that has to
 *     start at zero, the sticky status word, does so because the array is zero-initialised at
 *     load.  Two calls that can overlap on the GPU (different streams) race on the array; keep
 *     them on one stream or order them.
 *   - tq_decode_static_status copies that status word (same codes as the workspace's first word
 *     in tq_decode_paged) to status_out, device or pinned host memory, asynchronously on
 *     `stream`: a non-zero value after a call means that call (or an earlier one) left partials
 *     unwritten and out must not be trusted. */
#define TQ_STATIC_SCRATCH_BYTES (8u << 20)
int tq_decode_paged_static(const void* q, int q_dtype, int batch, int num_q_heads, int num_kv_heads,
                           int head_dim, const void* kv_cache, int64_t num_blocks, int block_size,
                           int slot_bytes, const int32_t* page_indices, const int32_t* page_indptr,
                           int max_pages, const int32_t* seq_lens, const float* signs, float sm_scale,
                           void* out, int out_dtype, float* out_lse, int num_ctas, void* stream);
int tq_decode_static_status(int32_t* status_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Diagnostics.  Not part of the data path and without a reference counterpart: an integration
 * does not need to bind these.
 * --------------------------------------------------------------------------------------- */

/* Index faults that the kernels without a workspace caught instead of dereferencing, since the
 * library was loaded on the current device: counts3[0] tokens whose slot was at or beyond
 * num_blocks * block_size in tq_write_kv_cache (dropped like a negative slot), counts3[1] page
 * halves tq_dequant_paged skipped (page id outside the cache, or a sequence longer than its page
 * list; their output rows stay unwritten), counts3[2] pages tq_pages_gather / _scatter skipped.
 * Host array of three; synchronises the device.  The reference only checks shapes
 * (csrc/src/quantize_write_binding.cu:216-227). */
int tq_fault_counts(int32_t* counts3);

/* Rows (K and V rows of every token and head, tile padding included) the tensor-core write kernel
 * has processed on the current device since the library was loaded, and how many of them it
 * re-derived with the exact path because a value lay within 2^-18 of a code boundary or the
 * row's norm was zero, huge or not finite.  Synchronises the device. */
int tq_write_guard_stats(int64_t* rows_total, int64_t* rows_exact);

/* Measurement hook.  While three CUDA events are set for the calling thread, the decode entry
 * points record them on the call's stream: ev_start before the decode kernel, ev_mid between
 * the decode kernel and the merge kernel, ev_end after the merge kernel.  Pass NULLs to switch
 * it off.  Not for use inside a stream capture. */
int tq_debug_set_decode_events(void* ev_start, void* ev_mid, void* ev_end);

/* ---- The slot format of vLLM's native TurboQuant backend ("turboquant_4bit_nc") --------------
 * A second wire format behind the same library, as the reference documents it
 * (docs/reference/vllm-upstream-turboquant-architecture.md:33-94 layout, :100-175 store, :178-240
 * decode): ONE cache tensor uint8 [num_blocks][block_size][num_kv_heads][slot_bytes], slot =
 * [K codes d/2 | ||k|| fp16 | V codes d/2 | V scale fp16 | V zero fp16] (134 bytes at d = 128), the
 * even dim in the LOW nibble.  K: x / (||x|| + 1e-8), Hadamard / sqrt(d) WITHOUT the sign vector,
 * 4-bit Lloyd-Max of N(0, 1/d); V: uniform 4 bits between the row's minimum and maximum
 * (scale = (max - min) / 15, code = clamp(trunc((v - min) / scale + 1/2), 0, 15), zero = min; a
 * constant row gets code 0), dequantized as code * scale + zero in the original domain.
 * head_dim 64, 128 or 256; 16-token pages for the decode; up to 8 query heads per KV head.
 * The store takes a warp per row; the decode runs on the tensor cores over shared-memory tiles (a block per
 * (split, sequence, KV head)), without the staged copy pipelines of the tuned kernels.
 * tq_nc_write_kv_cache stands in for upstream's do_kv_cache_update / _tq_fused_store_mse,
 * tq_nc_decode_paged for _tq_decode_stage1 + the stage-2 merge.  A slot id outside the cache is
 * skipped and counted (tq_nc_write_dropped); the decode's workspace starts with the sticky status
 * word of the other decode kernels (4: sequence longer than its page table, 5: page id outside the
 * cache; both skip the access). */
int tq_nc_slot_bytes(int head_dim);
int tq_nc_write_kv_cache(const void* key, const void* value, int in_dtype, int64_t num_tokens, int num_kv_heads,
                         int head_dim, int64_t k_token_stride, int64_t v_token_stride, void* kv_cache,
                         int64_t num_blocks, int block_size, int slot_bytes, const void* slot_mapping,
                         int slot_dtype, void* stream);
size_t tq_nc_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim, int num_ctas);
int tq_nc_decode_paged(const void* q, int q_dtype, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                       const void* kv_cache, int64_t num_blocks, int block_size, int slot_bytes,
                       const int32_t* page_indices, const int32_t* page_indptr, int max_pages,
                       const int32_t* seq_lens, float sm_scale, void* workspace, size_t workspace_bytes,
                       void* out, int out_dtype, float* out_lse, int num_ctas, void* stream);
int tq_nc_write_dropped(int32_t* count);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_B200_H */
