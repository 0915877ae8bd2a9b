// Bulk dequantization of paged cache contents into dense K / V tensors.
//
// Used when a chunk of new query tokens has to attend to KV that already sits quantized in the
// cache (continuation of a prefill): the cached tokens of every sequence are gathered through the
// block table, dequantized (centroid lookup, inverse rotation, times the stored fp16 norm) and
// written as varlen-packed [total_tokens][num_kv_heads][128] K and V, the layout a varlen
// attention kernel takes.  The reference's backend ignores the cache during prefill
// (turboquant/vllm_backend_fused.py:336-369); its per-row arithmetic for this is
// TurboQuantMSE.dequantize (turboquant/quantizer.py:93-106) with the fp16 norm of the cache slot,
// as in its dequant-attention check (tests/test_fused_integration.py:127-159).
//
// Arithmetic, in this order, each step rounded to fp32: y[d] = (float)(C[idx[d]] / sqrt(128));
// butterflies h = 1..64; times (float)(1/sqrt(128)); times signs[d]; times float(fp16 norm).
// With fp32 output the result equals the CPU restatement bit for bit; fp16/bf16 outputs are its
// correctly rounded values.
//
// Mapping: two lanes own one row (lane m: dims 64m .. 64m+63, i.e. code bytes 32m .. 32m+31), a
// warp works on 16 rows; stages h = 1..32 are register-local (packed f32x2 arithmetic from h = 2
// on), h = 64 is one shuffle per element.  Persistent blocks walk the (sequence, page, K / V) items
// and fetch each item's codes one item ahead.
#include <cmath>

#include "tq_common.cuh"

namespace tq {

constexpr int kDqThreads = 256;
constexpr int kDqDim = 128;
constexpr int kDqSlotCodes = 64;

struct DequantParams {
    const uint8_t* kv_cache;
    int64_t slab_bytes;
    int64_t num_blocks;           // page ids outside [0, num_blocks) are skipped and counted
    const int32_t* page_indices;
    const int32_t* page_indptr;   // null: dense block table [batch][max_pages]
    const int32_t* seq_lens;
    const int32_t* cu_seqlens;    // [batch + 1]: first output row of every sequence
    const float* signs;
    void* out[2];                 // K, V: [total_tokens][H][128]
    int64_t out_token_stride;     // elements between tokens
    int max_pages, H, head_shift, block_size, slot_bytes, out_dtype, batch;  // head_shift: log2(H) or -1
    int head_dim;                 // elements per output row: 128, or 96 (the padded dims are dropped)
    float cen[16];                // (float)(C[i] / sqrt(128))
    float scale;                  // (float)(1 / sqrt(128))
};

struct Q2 { unsigned long long v; };
__device__ __forceinline__ Q2 qpk(float lo, float hi) {
    Q2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void qup(Q2 a, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v)); }
__device__ __forceinline__ Q2 qadd(Q2 a, Q2 b) { Q2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ Q2 qsub(Q2 a, Q2 b) { Q2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ Q2 qmul(Q2 a, Q2 b) { Q2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ Q2 qfma(Q2 a, Q2 b, Q2 c) {
    Q2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
    return r;
}

// 16-byte piece i of a lane's 64 output elements in the output type.
template <int DT>
__device__ __forceinline__ uint4 out_piece(const Q2 (&x)[32], int i);

template <>
__device__ __forceinline__ uint4 out_piece<TQ_F32>(const Q2 (&x)[32], int i) {  // 16 pieces of 4 floats
    float a, b, c, e;
    qup(x[2 * i], a, b);
    qup(x[2 * i + 1], c, e);
    return make_uint4(__float_as_uint(a), __float_as_uint(b), __float_as_uint(c), __float_as_uint(e));
}
template <>
__device__ __forceinline__ uint4 out_piece<TQ_F16>(const Q2 (&x)[32], int i) {  // 8 pieces of 8 halves
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float a, b;
        qup(x[4 * i + k], a, b);
        const __half2 h = __floats2half2_rn(a, b);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 out_piece<TQ_BF16>(const Q2 (&x)[32], int i) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float a, b;
        qup(x[4 * i + k], a, b);
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Output staging of one warp pass: 16 rows in the output type, 16-byte pieces.  Piece j of the half
// row (row, m) sits at position j ^ ((2 row + m) & 7) of that half row: the eight lanes served
// together hit eight different bank groups both when the lanes write their own half rows and when
// they read the pass back in linear order for the global stores.
template <int DT>
struct DqStage {
    static constexpr int kEsz = DT == TQ_F32 ? 4 : 2;
    static constexpr int kRowBytes = kDqDim * kEsz;
    static constexpr int kHalfPieces = kRowBytes / 32;     // 16-byte pieces per lane: 8 or 16
    static constexpr int kRowPieces = 2 * kHalfPieces;
    static constexpr int kWarpBytes = 16 * kRowBytes;      // 4 KB or 8 KB
    static constexpr int kTableBytes = 256 * 16 * 8;
    static constexpr int kSmem = kTableBytes + (kDqThreads / 32) * kWarpBytes;
};

// What one warp needs of one work item (the K or V half of one page): its rows' codes and norm
// are fetched one item ahead, so that the loads of the next page are in flight during the
// arithmetic of the current one.
// Page halves skipped because the page id lay outside the cache or the sequence was longer than
// its page list; read back by tq_fault_counts.
static __device__ int32_t g_dequant_skipped = 0;

struct DqItem {
    uint4 c0, c1;
    float norm;
    int64_t out_row0;  // first output row (token) of the page
    int rows;          // (token, head) rows in the page half; 0: nothing to do
    int which;
};

template <int DT>
__device__ __forceinline__ void fetch_item(const DequantParams& p, int64_t item, int64_t num_items, int warp, int lane,
                                           DqItem& it) {
    it.rows = 0;
    it.which = 0;
    it.out_row0 = 0;
    if (item >= num_items) return;
    const int which = (int)(item & 1);
    const int64_t pb = item >> 1;
    const int b = (int)(pb / p.max_pages), page_in_seq = (int)(pb - (int64_t)b * p.max_pages);
    const int len = p.seq_lens[b];
    const int tok0 = page_in_seq * p.block_size;
    if (tok0 >= len) return;
    const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
    const bool listed = !p.page_indptr || tbl + page_in_seq < (int64_t)p.page_indptr[b + 1];
    const int64_t page = listed ? (int64_t)p.page_indices[tbl + page_in_seq] : -1;
    if ((uint64_t)page >= (uint64_t)p.num_blocks) {  // never form an address from it: the rows stay unwritten
        if (warp == 0 && lane == 0 && which == 0) atomicAdd(&g_dequant_skipped, 1);
        return;
    }
    const int ntok = len - tok0 < p.block_size ? len - tok0 : p.block_size;
    it.rows = ntok * p.H;
    it.which = which;
    it.out_row0 = (int64_t)p.cu_seqlens[b] + tok0;
    // rows beyond a warp's first pass (more than 128 rows per page half) are fetched in place
    const int r = warp * 16 + (lane >> 1);
    const uint8_t* slot = p.kv_cache + (size_t)which * p.slab_bytes +
                          ((size_t)page * p.block_size * p.H + (size_t)(r < it.rows ? r : 0)) * p.slot_bytes;
    it.c0 = *reinterpret_cast<const uint4*>(slot + 32 * (lane & 1));
    it.c1 = *reinterpret_cast<const uint4*>(slot + 32 * (lane & 1) + 16);
    it.norm = __half2float(*reinterpret_cast<const __half*>(slot + kDqSlotCodes));
}

// Persistent blocks over the work items (sequence, page, K / V), item = 2 * (b * max_pages + page) + which.
template <int DT>
__global__ void __launch_bounds__(kDqThreads) dequant_paged_kernel(const __grid_constant__ DequantParams p) {
    // byte -> {centroid(high nibble), centroid(low nibble)}, 16 columns: an 8-byte load is served
    // half a warp at a time, so the lookups of a warp never conflict
    extern __shared__ __align__(128) uint8_t dq_smem[];
    float2* table_s = reinterpret_cast<float2*>(dq_smem);
    // scale * sign of dims 0..63 and 64..127 in different banks: a half warp reads both halves
    __shared__ __align__(16) float sgn_s[2][kDqDim / 2 + 2];
    using St = DqStage<DT>;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_launch_dependents();
    for (int i = tid; i < 256 * 16; i += kDqThreads) {
        const int v = i >> 4;
        table_s[i] = make_float2(p.cen[v >> 4], p.cen[v & 15]);
    }
    grid_dependency_wait();  // the cache, the page table and the lengths belong to earlier kernels
    if (tid < kDqDim) sgn_s[tid >> 6][tid & 63] = __fmul_rn(p.signs[tid], p.scale);  // exact: the sign is +-1
    __syncthreads();

    constexpr int kEsz = St::kEsz;
    uint8_t* stage = dq_smem + St::kTableBytes + (size_t)warp * St::kWarpBytes;
    // Linear read-back of a staged pass: iteration i of lane l takes piece lin_pin of row
    // lin_row + i * kLinRows, stored at position piece ^ ((2 row + half) & 7) of its half row.
    constexpr int kLinRows = 32 / St::kRowPieces;            // rows covered by one warp-wide access: 2 or 1
    constexpr int kLinIters = 16 / kLinRows;
    const int lin_row = lane / St::kRowPieces, lin_pin = lane % St::kRowPieces;
    const int lin_half = lin_pin / St::kHalfPieces, lin_pp = lin_pin % St::kHalfPieces;
    const int lin_key = 2 * lin_row + lin_half;
    const int lin_base = lin_row * St::kRowBytes + lin_half * (St::kRowBytes / 2);
    const bool dense = p.head_dim == kDqDim && p.out_token_stride == (int64_t)p.H * kDqDim;
    const int m = lane & 1;
    const uint32_t table_lane = smem_u32(table_s) + 8u * (lane & 15);
    const float hsgn = m ? -1.0f : 1.0f;
    const int64_t num_items = 2 * (int64_t)p.batch * p.max_pages;

    DqItem cur, nxt;
    fetch_item<DT>(p, blockIdx.x, num_items, warp, lane, cur);
    for (int64_t item = blockIdx.x; item < num_items; item += gridDim.x) {
        fetch_item<DT>(p, item + gridDim.x, num_items, warp, lane, nxt);
        uint8_t* out_base = static_cast<uint8_t*>(p.out[cur.which]);
        for (int r0 = warp * 16; r0 < cur.rows; r0 += (kDqThreads / 32) * 16) {
            const int r = r0 + (lane >> 1);
            const bool ok = r < cur.rows;
            uint4 c0 = cur.c0, c1 = cur.c1;
            float norm = cur.norm;
            if (r0 != warp * 16) {  // later passes of a page half with more than 128 rows: fetch now
                const int64_t pb = item >> 1;
                const int b = (int)(pb / p.max_pages), page_in_seq = (int)(pb - (int64_t)b * p.max_pages);
                const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
                const int64_t page = p.page_indices[tbl + page_in_seq];
                const uint8_t* slot = p.kv_cache + (size_t)cur.which * p.slab_bytes +
                                      ((size_t)page * p.block_size * p.H + (size_t)(ok ? r : 0)) * p.slot_bytes;
                c0 = *reinterpret_cast<const uint4*>(slot + 32 * m);
                c1 = *reinterpret_cast<const uint4*>(slot + 32 * m + 16);
                norm = __half2float(*reinterpret_cast<const __half*>(slot + kDqSlotCodes));
            }
            const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            Q2 x[32];  // x[i] = dims (64m + 2i, 64m + 2i + 1) = code byte 32m + i
#pragma unroll
            for (int i = 0; i < 32; i++) {
                uint32_t byte;  // byte i & 3 of the word, zero extended, by one byte permute
                asm("prmt.b32 %0, %1, 0, %2;" : "=r"(byte) : "r"(w[i >> 2]), "r"(0x4440u | (uint32_t)(i & 3)));
                float hi, lo;
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(hi), "=f"(lo) : "r"(byte * 128u + table_lane));
                // stage h = 1 inside the pair
                x[i] = qpk(__fadd_rn(hi, lo), __fsub_rn(hi, lo));
            }
            // stages h = 2 .. 32: pairs i and i + h/2
#pragma unroll
            for (int hp = 1; hp < 32; hp <<= 1)
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (!(i & hp)) {
                        const Q2 a = x[i], c = x[i + hp];
                        x[i] = qadd(a, c);
                        x[i + hp] = qsub(a, c);
                    }
            // stage h = 64 between the two lanes: lower half mine + other, upper half other - mine
            {
                const Q2 s2 = qpk(hsgn, hsgn);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float a, c;
                    qup(x[i], a, c);
                    const float oa = __shfl_xor_sync(0xffffffffu, a, 1), oc = __shfl_xor_sync(0xffffffffu, c, 1);
                    x[i] = qfma(x[i], s2, qpk(oa, oc));
                }
            }
            // (w * scale) * sign == w * (scale * sign) exactly; then the norm
            const Q2 n2 = qpk(norm, norm);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const float2 sg = *reinterpret_cast<const float2*>(&sgn_s[m][2 * i]);
                x[i] = qmul(qmul(x[i], qpk(sg.x, sg.y)), n2);
            }
            // stage the 16 rows, then store them in linear order: every store instruction of the warp
            // covers whole rows (512 contiguous bytes when the heads of a token are contiguous)
            {
                uint8_t* half_row = stage + (lane >> 1) * St::kRowBytes + m * (St::kRowBytes / 2);
                const int key = lane & 7;  // (2 row + m) & 7
#pragma unroll
                for (int i = 0; i < St::kHalfPieces; i++)
                    *reinterpret_cast<uint4*>(half_row + ((i ^ key) << 4)) = out_piece<DT>(x, i);
            }
            __syncwarp();
            if (dense) {
                // heads of a token contiguous: the rows of the page half are one contiguous range
                uint8_t* dst = out_base + ((cur.out_row0 * p.H + r0 + lin_row) * (int64_t)St::kRowBytes) + lin_pin * 16;
#pragma unroll
                for (int i = 0; i < kLinIters; i++) {
                    const uint4 piece = *reinterpret_cast<const uint4*>(stage + lin_base + i * kLinRows * St::kRowBytes +
                                                                        ((lin_pp ^ ((lin_key + 2 * i * kLinRows) & 7)) << 4));
                    if (r0 + lin_row + i * kLinRows < cur.rows)
                        *reinterpret_cast<uint4*>(dst + (size_t)i * kLinRows * St::kRowBytes) = piece;
                }
            } else {
#pragma unroll
                for (int i = 0; i < kLinIters; i++) {
                    const uint4 piece = *reinterpret_cast<const uint4*>(stage + lin_base + i * kLinRows * St::kRowBytes +
                                                                        ((lin_pp ^ ((lin_key + 2 * i * kLinRows) & 7)) << 4));
                    const int rr = r0 + lin_row + i * kLinRows;
                    if (rr < cur.rows && lin_pin * 16 < p.head_dim * kEsz) {
                        int t, h;
                        if (p.head_shift >= 0) { t = rr >> p.head_shift; h = rr & (p.H - 1); }
                        else { t = rr / p.H; h = rr - t * p.H; }
                        uint8_t* dst = out_base + ((cur.out_row0 + t) * p.out_token_stride + (int64_t)h * p.head_dim) * kEsz;
                        *reinterpret_cast<uint4*>(dst + lin_pin * 16) = piece;
                    }
                }
            }
            __syncwarp();
        }
        cur = nxt;
    }
}

int device_sm_count(int* out);

template <int DT>
static int launch_dequant(const DequantParams& p, dim3 grid, cudaStream_t stream) {
    static bool configured[64] = {};  // per template instance and device
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(dequant_paged_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     DqStage<DT>::kSmem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    TQ_CUDA(launch_serialized(dequant_paged_kernel<DT>, grid, dim3(kDqThreads), DqStage<DT>::kSmem, stream, p));
    return TQ_OK;
}
void host_codebook(int dim, int bits, float* centroids, float* boundaries);

int generic_dequant(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads, int slot_bytes,
                    const int32_t* page_indices, const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                    const int32_t* cu_seqlens, int batch, const float* signs, int head_dim, void* k_out, void* v_out,
                    int out_dtype, int64_t out_token_stride, void* stream);
int generic_fault_counts(int32_t* write_dropped, int32_t* dequant_skipped);

int dequant_fault_count(int32_t* out) {
    int32_t a = 0, b = 0, c = 0;
    TQ_CUDA(cudaMemcpyFromSymbol(&a, g_dequant_skipped, sizeof(int32_t)));
    int rc = generic_fault_counts(&b, &c);
    if (rc != TQ_OK) return rc;
    *out = a + c;
    return TQ_OK;
}

}  // namespace tq

extern "C" int tq_dequant_paged(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                                int slot_bytes, const int32_t* page_indices, const int32_t* page_indptr,
                                int max_pages, const int32_t* seq_lens, const int32_t* cu_seqlens, int batch,
                                const float* signs, int head_dim, void* k_out, void* v_out, int out_dtype,
                                int64_t out_token_stride, void* stream) {
    using namespace tq;
    TQ_REQUIRE(batch >= 0 && num_blocks >= 0, TQ_ERR_INVALID, "negative size");
    if (batch == 0 || max_pages == 0) return TQ_OK;
    TQ_REQUIRE(kv_cache && page_indices && seq_lens && cu_seqlens && signs && k_out && v_out, TQ_ERR_INVALID, "null pointer");
    if (head_dim != kDqDim && head_dim != 96) {  // other head sizes (64, 256, ...): the plain kernel
        TQ_REQUIRE(num_kv_heads >= 1 && out_dtype >= TQ_F32 && out_dtype <= TQ_BF16 &&
                       out_token_stride >= (int64_t)num_kv_heads * head_dim, TQ_ERR_INVALID, "bad geometry");
        return generic_dequant(kv_cache, num_blocks, block_size, num_kv_heads, slot_bytes, page_indices, page_indptr, max_pages,
                               seq_lens, cu_seqlens, batch, signs, head_dim, k_out, v_out, out_dtype, out_token_stride, stream);
    }
    TQ_REQUIRE(slot_bytes >= 80 && slot_bytes % 16 == 0, TQ_ERR_INVALID, "slot_bytes must be a multiple of 16 and >= 80");
    TQ_REQUIRE(block_size >= 1 && num_kv_heads >= 1 && max_pages >= 1 && batch >= 1, TQ_ERR_INVALID, "bad geometry");
    TQ_REQUIRE(out_dtype >= TQ_F32 && out_dtype <= TQ_BF16, TQ_ERR_INVALID, "bad out_dtype");
    TQ_REQUIRE(out_token_stride >= (int64_t)num_kv_heads * head_dim && out_token_stride % 8 == 0, TQ_ERR_INVALID,
               "out_token_stride must cover one token and keep rows 16-byte aligned");
    TQ_REQUIRE(((uintptr_t)kv_cache % 16) == 0 && ((uintptr_t)k_out % 16) == 0 && ((uintptr_t)v_out % 16) == 0,
               TQ_ERR_INVALID, "kv_cache, k_out and v_out must be 16-byte aligned");
    DequantParams p{};
    p.kv_cache = static_cast<const uint8_t*>(kv_cache);
    p.slab_bytes = num_blocks * block_size * (int64_t)num_kv_heads * slot_bytes;
    p.num_blocks = num_blocks;
    p.page_indices = page_indices;
    p.page_indptr = page_indptr;
    p.seq_lens = seq_lens;
    p.cu_seqlens = cu_seqlens;
    p.signs = signs;
    p.out[0] = k_out;
    p.out[1] = v_out;
    p.out_token_stride = out_token_stride;
    p.max_pages = max_pages;
    p.H = num_kv_heads;
    p.head_shift = -1;
    for (int sft = 0; sft < 16; sft++)
        if ((1 << sft) == num_kv_heads) p.head_shift = sft;
    p.block_size = block_size;
    p.slot_bytes = slot_bytes;
    p.out_dtype = out_dtype;
    p.batch = batch;
    p.head_dim = head_dim;
    float bnd[15];
    host_codebook(kDqDim, 4, p.cen, bnd);
    p.scale = (float)(1.0 / std::sqrt((double)kDqDim));
    int sms = 0;
    int rc = device_sm_count(&sms);
    if (rc != TQ_OK) return rc;
    const int64_t items = 2 * (int64_t)batch * max_pages;
    const dim3 grid((unsigned)(items < 2 * (int64_t)sms ? items : 2 * (int64_t)sms));  // two resident blocks per SM
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case TQ_F32: return launch_dequant<TQ_F32>(p, grid, s);
        case TQ_F16: return launch_dequant<TQ_F16>(p, grid, s);
        default: return launch_dequant<TQ_BF16>(p, grid, s);
    }
}
