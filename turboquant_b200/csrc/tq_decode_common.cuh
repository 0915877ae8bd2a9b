// Pieces shared by the decode kernels (the mma.sync kernel for up to 8 query columns per KV head
// and the tcgen05 kernel for wider query tiles): geometry constants, the launch parameters, the
// device-side helpers for the page window of a sequence and for the lookup-table dequantizer.
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr int kHeadDim = 128;
constexpr int kPageTokens = 16;
constexpr int kSlotBytes = 80;
constexpr int kConsumerWarps = 16;
// Four consumer warpgroups and a producer warpgroup: the producer warp plus three warps that only
// hand their registers back.  Twenty warps launch with 96 registers each (five per scheduler);
// the producer group shrinks to 24 and every consumer grows to 112 (setmaxnreg), which is what
// the consumer loop needs to stay out of local memory and keep its lookups in flight
// (measured: 86.5 -> 78.3 us per launch against 17 warps at 96 registers).
constexpr int kDecodeThreads = (kConsumerWarps + 4) * 32;
constexpr int kStages = 3;  // ring depth: one stage below the lookup table, two above it
constexpr int kMaxExchangeRanks = 16;
constexpr int kExchangeSpinLimit = 1 << 22;  // default, x 256 ns sleeps: a second or so, then status 1
// status words (workspace header word 0, sticky): 1 a bounded wait ran out, 2 more sequences inside
// one block's page range than its list holds, 3 the shared-memory map did not fit, 4 a sequence is
// longer than its page table (nothing is read, the output is zero), 5 a page id outside
// [0, num_blocks) (the page is replaced by page 0, the output is wrong but nothing faults)
constexpr int kStatusSeqTooLong = 4, kStatusBadPage = 5;
constexpr int kMaxSegments = 96;
constexpr int kMinPagesPerCta = 4;
// Starting a sequence inside a block (rotate its queries, later write its partial) costs about as
// much as three stages of streaming.  The page list is therefore split in a virtual space where
// every non-empty sequence is preceded by kSegCostStages x pages-per-stage virtual pages: a block
// that takes on an additional sequence gets correspondingly fewer real pages.
constexpr int kSegCostStages = 3;
constexpr int kSegCostMinStages = 16;  // ... and only when a block streams at least this many stages
constexpr float kRaiseThreshold = 6.0f;  // log2 units

struct DecodeParams {
    const void* q;
    const uint8_t* kv_cache;
    const int32_t* page_indices;
    const int32_t* page_indptr;  // may be null: dense block table with row stride max_pages
    const int32_t* seq_lens;
    const float* signs;
    int32_t* header;        // workspace: [0] status, [1] effective block count, [2] total (virtual) pages, [3] pages charged per sequence start
    int32_t* page_prefix;   // workspace: [batch + 1]
    float* partial_lse;     // workspace: [slots][num_q_heads]
    float* partial_o;       // workspace: [slots][num_q_heads][128]
    int64_t slab_bytes;
    int64_t num_blocks;        // pages in the cache: page ids outside [0, num_blocks) are never dereferenced
    int64_t kv_begin, kv_end;  // token window applied to every sequence (kv_end < 0: none)
    // A sequence may carry several decode queries that share its KV (queries_per_seq).  Inside the
    // kernels they are extra columns of the query tile: num_q_heads and group below are the VIRTUAL
    // counts (queries_per_seq x the real ones), column c of a KV head being query c / real_group,
    // head c % real_group.  real_heads / real_group / nq give the layout of q and out.
    int batch, num_q_heads, group, max_pages, q_dtype;
    int nq, real_heads, real_group;
    int head_dim;  // elements per q / out row: 128, or 96 (the rotation pads it with zeros to 128)
    // the KV heads of this launch inside the cache's token rows, and its query heads inside q / out
    int64_t kv_row_bytes;  // bytes between tokens in the cache (all KV heads of the cache)
    int kv_head_off;       // byte offset of this launch's first KV head inside a token row
    int q_head_base;       // first real query head of this launch
    float k_scale;  // (1/sqrt(128)) * sm_scale * log2(e): multiplies raw code-domain scores
    float v_scale;  // 1/sqrt(128): centroid scale folded into P
    uint16_t centroid_h[16];  // fp16 bit patterns of the N(0,1) centroids
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}
// The same with a compile-time byte offset folded into the instruction's address field.
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64_at(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ float lds_half_at(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Eight packed 4-bit codes (one 32-bit word) -> four half2 registers, one per byte:
// r[j] = { low half: centroid(low nibble of byte j), high half: centroid(high nibble) } in units
// of the N(0,1) codebook.  The table has one 4-byte column per lane and 256 bytes between entries,
// and starts at a 64 KB boundary of the shared window: lut_lane = table address + 4 * lane has a
// zero second byte, and one byte permute drops the code byte into it, so address and lookup are
// two instructions per code byte.
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t lut_lane, uint32_t (&r)[4]) {
#pragma unroll
    for (int j = 0; j < 4; j++) r[j] = lds32(prmt(w, lut_lane, 0x7604u | (j << 4)));
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// 2^x, hardware approximation (2 ulp), flushes denormals; exp2(-inf) = 0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float load_q(const void* q, int dtype, int64_t i) {
    if (dtype == TQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]);
    if (dtype == TQ_F16) return __half2float(reinterpret_cast<const __half*>(q)[i]);
    return reinterpret_cast<const float*>(q)[i];
}

// Pages of sequence b inside the token window, and the first page index.
__device__ __forceinline__ void seq_pages(const DecodeParams& p, int b, int& first_page, int& npages,
                                          int& len_eff) {
    int64_t len = p.seq_lens[b];
    if (p.kv_end >= 0 && p.kv_end < len) len = p.kv_end;
    const int64_t begin = p.kv_begin > 0 ? p.kv_begin : 0;
    first_page = (int)(begin / kPageTokens);
    const int64_t last = (len + kPageTokens - 1) / kPageTokens;
    npages = last > first_page ? (int)(last - first_page) : 0;
    len_eff = (int)len;
}

// Shared-memory map.  The lookup table must start at offset 64 KB of the block's shared window
// (one byte permute then builds a lookup address); what the kernels put below and above it is
// theirs.
constexpr uint32_t kLutAddr = 65536, kLutSpan = 65536;

}  // namespace tq
