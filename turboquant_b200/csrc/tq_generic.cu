// Paged cache write, decode attention, merge and bulk dequantization for head sizes whose padded
// size is not 128 (64: 48-byte slots, 256: 144-byte slots; any head size up to 256).
//
// The reference declares these geometries (turboquant/kernel_config.py:75-109: qwen3-0.6b with
// head size 64, gemma-2 with 256; slot size turboquant/vllm_backend_fused.py:64-72: 32 code bytes
// and one fp16 norm per 64 padded dims, rounded up to 16 bytes) but its decode op rejects
// everything except 128 (csrc/src/decode_v5_tc_binding.cu:779).  These kernels are the plain
// formulation of the same arithmetic -- eight lanes (write, dequantization) or a warp (decode) per row, fp32 math --
// with the interfaces, the split-KV workspace contract and the parity bars of the tuned 128-wide
// kernels; they are not tuned to the HBM roofline.  Quantizer arithmetic as in tq_flat.cu (the torch
// evaluation order), compiled with -fmad=false.
#include <cmath>
#include <cstring>

#include "tq_common.cuh"

namespace tq {

constexpr int kGenMaxDim = 256;
constexpr int kGenWarps = 4;
constexpr int kGenMaxGroup = 8;
constexpr int kGenPage = 16;
constexpr int kGenStatusSeqTooLong = 4, kGenStatusBadPage = 5;

struct GenGeom {
    int head_dim, padded, qbytes, dc, slot_bytes;
};

__host__ __device__ inline int gen_next_pow2(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

static GenGeom make_geom(int head_dim, int slot_bytes) {
    GenGeom g;
    g.head_dim = head_dim;
    g.padded = gen_next_pow2(head_dim);  // 64, 128 or 256: callers admit head sizes 33..256 only
    g.dc = g.padded / 64;
    g.qbytes = g.padded / 2;
    g.slot_bytes = slot_bytes;
    return g;
}

// butterflies h = 1 .. padded/2 on a shared-memory row, by one warp: lane l takes elements l E .. l E + E - 1
// (E = padded / 32) into registers, runs the stages h < E there and the stages h >= E as one shuffle per
// element, and puts the row back.  Every stage forms the same a + b and a - b as the in-place loop would,
// so the result is bit-identical to it.
template <int E>
__device__ __forceinline__ void gen_warp_fwht_regs(float* buf, int lane) {
    float v[E];
#pragma unroll
    for (int i = 0; i < E; i++) v[i] = buf[lane * E + i];
#pragma unroll
    for (int h = 1; h < E; h <<= 1) {
#pragma unroll
        for (int i = 0; i < E; i++) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = __fadd_rn(a, b);
                v[i + h] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {   // element stride h = m E: the partner sits in lane ^ m
#pragma unroll
        for (int i = 0; i < E; i++) {
            const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
            v[i] = (lane & m) ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
        }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < E; i++) buf[lane * E + i] = v[i];
    __syncwarp();
}
__device__ __forceinline__ void gen_warp_fwht(float* buf, int padded, int lane) {
    if (padded == 64) gen_warp_fwht_regs<2>(buf, lane);
    else if (padded == 128) gen_warp_fwht_regs<4>(buf, lane);
    else gen_warp_fwht_regs<8>(buf, lane);
}

// ---------------------------------------------------------------------------------------------
// cache write
// ---------------------------------------------------------------------------------------------
struct GenWriteParams {
    uint8_t* kv_cache;
    const void* src[2];
    int64_t token_stride[2];
    const void* slot_mapping;
    const float* signs;
    int64_t num_tokens, slab_bytes, total_slots;
    int num_kv_heads, slot_is_i64, zero_pad;
    int walk;   // rows a lane group takes of its token: all 2 H (large jobs) or 1 (a decode step's few tokens: more groups in flight)
    GenGeom g;
    float scale;
    float boundaries[15];
};

static __device__ int32_t g_gen_write_dropped = 0;

// Eight lanes own one row and a warp works on four rows at a time.  Lane q of a row holds elements
// q, q + 8, q + 16, ... (E = padded / 8 registers), which is the torch evaluation order of the norm laid out
// across lanes: accumulator k of the eight interleaved ones is lane k's running sum over its registers.  Butterfly
// stages h = 1, 2, 4 are one shuffle per element, stages h >= 8 are register-local.  The quotient x / norm is
// q = x r, e = fma(-q, norm, x), q' = fma(e, r, q) with r the correctly rounded reciprocal, which equals the IEEE
// quotient when every square of the row is a normal number, the norm is moderate and its significand is not all
// ones (checked per row; the row takes the division instruction otherwise).  The codes of a row are assembled
// in shared memory and leave as 16-byte stores when the slots are 16-byte aligned.
template <int E>
struct GenRows8 {
    static constexpr int kPd = 8 * E, kQb = kPd / 2, kDc = kPd / 64;
    static constexpr int kRowStride = kQb + 16;   // rows of a pass in different banks
};

template <typename T, int E, bool WALK>
__global__ void __launch_bounds__(kGenWarps * 32, 8) write_rows8_kernel(const __grid_constant__ GenWriteParams p) {
    using G = GenRows8<E>;
    __shared__ float bnd_s[16];
    __shared__ __align__(16) uint8_t code_s[kGenWarps][4][G::kRowStride];
    __shared__ float sg_s[G::kPd];
    if (threadIdx.x < 15) bnd_s[threadIdx.x] = p.boundaries[threadIdx.x];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = lane & 7, rg = lane >> 3;
    const int H = p.num_kv_heads, hd = p.g.head_dim;
    const int full = hd & ~7, ntail = hd - full;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.kv_cache) | (uintptr_t)p.slab_bytes | (uintptr_t)p.g.slot_bytes) & 15) == 0;
    uint8_t* stage = code_s[warp][rg];

    // signs in shared memory (1 for the padding, which stays +0): E registers less than holding them
    for (int j = threadIdx.x; j < G::kPd; j += kGenWarps * 32) sg_s[j] = j < hd ? p.signs[j] : 1.0f;
    __syncthreads();
    const float* sg = sg_s + q;

    // a group of eight lanes takes one token and `walk` of its 2 H rows (K and V of head 0, of head 1, ...; the two
    // tensors alternating measured 3 % faster at head 256 than all K rows first): the slot lookup and
    // the index arithmetic are done once per token
    const int walk = WALK ? p.walk : 1;   // WALK = false: p.walk is 1 and the row loop below is straight code
    const int parts = 2 * H / walk;
    const int64_t items = p.num_tokens * parts;
    for (int64_t base = ((int64_t)blockIdx.x * kGenWarps + warp) * 4; base < items; base += (int64_t)gridDim.x * kGenWarps * 4) {
        // a group past the end works on the last item again and stores nothing: the shuffles below take every lane
        const bool live = base + rg < items;
        const int64_t it = live ? base + rg : items - 1;
        int64_t t;
        int r0;
        if (it < 0x7fffffff) {
            const uint32_t t32 = (uint32_t)it / (uint32_t)parts;
            t = t32;
            r0 = (int)((uint32_t)it - t32 * (uint32_t)parts) * walk;
        } else {
            t = it / parts;
            r0 = (int)(it - t * parts) * walk;
        }
        int64_t slot = p.slot_is_i64 ? reinterpret_cast<const int64_t*>(p.slot_mapping)[t]
                                     : (int64_t) reinterpret_cast<const int32_t*>(p.slot_mapping)[t];
        if (slot >= p.total_slots) {
            if (live && q == 0 && r0 == 0) atomicAdd(&g_gen_write_dropped, 1);
            slot = -1;
        }
        const bool store = live && slot >= 0;
        if (!__any_sync(0xffffffffu, store)) continue;   // four skipped tokens
        for (int rr = r0; rr < r0 + walk; rr++) {
        const int which = rr & 1, h = rr >> 1;   // K and V rows of a head alternate
        const T* row = reinterpret_cast<const T*>(p.src[which]) + t * p.token_stride[which] + (int64_t)h * hd;
        float x[E];
#pragma unroll
        for (int r = 0; r < E; r++) x[r] = q + 8 * r < hd ? to_f32(row[q + 8 * r]) : 0.0f;

        // norm in the reference order: eight interleaved accumulators (one per lane), combined left to right,
        // then the elements past the last multiple of eight
        float acc = 0.0f, minsq = 3.0e38f, tail_sq = 0.0f;
#pragma unroll
        for (int r = 0; r < E; r++) {
            const float sq = __fmul_rn(x[r], x[r]);
            if (8 * r < full) {
                acc = __fadd_rn(acc, sq);
                minsq = fminf(minsq, sq);
            } else if (8 * r == full) {
                tail_sq = sq;
                if (q < ntail) minsq = fminf(minsq, sq);
            }
        }
        float s = __shfl_sync(0xffffffffu, acc, 0, 8);
#pragma unroll
        for (int k = 1; k < 8; k++) s = __fadd_rn(s, __shfl_sync(0xffffffffu, acc, k, 8));
        for (int k = 0; k < ntail; k++) s = __fadd_rn(s, __shfl_sync(0xffffffffu, tail_sq, k, 8));
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) minsq = fminf(minsq, __shfl_xor_sync(0xffffffffu, minsq, m));
        float norm = __fsqrt_rn(s);
        if (!(norm >= 1e-8f)) norm = (norm != norm) ? __uint_as_float(0x7fc00000u) : 1e-8f;

        const bool fast = minsq >= 1.1754944e-38f && norm >= 9.0949470e-13f && norm <= 1.0995116e12f &&
                          (__float_as_uint(norm) & 0x7fffffu) != 0x7fffffu;
        if (fast) {
            const float rcp = __frcp_rn(norm), nneg = -norm;
#pragma unroll
            for (int r = 0; r < E; r++) {
                const float qv = __fmul_rn(x[r], rcp);
                const float err = __fmaf_rn(qv, nneg, x[r]);   // x - q norm, exact
                x[r] = __fmul_rn(__fmaf_rn(err, rcp, qv), sg[8 * r]);
            }
        } else {
#pragma unroll
            for (int r = 0; r < E; r++) x[r] = q + 8 * r < hd ? __fmul_rn(__fdiv_rn(x[r], norm), sg[8 * r]) : 0.0f;
        }

        // butterflies in stage order: h = 1, 2, 4 between the lanes of the row, h = 8 ... between registers
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
            for (int r = 0; r < E; r++) {
                const float o = __shfl_xor_sync(0xffffffffu, x[r], m);
                x[r] = (q & m) ? __fsub_rn(o, x[r]) : __fadd_rn(x[r], o);
            }
        }
#pragma unroll
        for (int hr = 1; hr < E; hr <<= 1) {
#pragma unroll
            for (int r = 0; r < E; r++) {
                if ((r & hr) == 0) {
                    const float a = x[r], b = x[r + hr];
                    x[r] = __fadd_rn(a, b);
                    x[r + hr] = __fsub_rn(a, b);
                }
            }
        }

        // codes: element q + 8 r is the high (q even) or low (q odd) nibble of byte q / 2 + 4 r
        uint32_t word[E / 4];
        const int nib = (q & 1) ? 0 : 4;
#pragma unroll
        for (int w = 0; w < E / 4; w++) {
            uint32_t acc_w = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float y = __fmul_rn(x[4 * w + i], p.scale);
                // boundaries strictly below y (they ascend): a binary search over the shared copy
                int c = (bnd_s[7] < y) ? 8 : 0;
                c += (bnd_s[c + 3] < y) ? 4 : 0;
                c += (bnd_s[c + 1] < y) ? 2 : 0;
                c += (bnd_s[c] < y) ? 1 : 0;
                if (y != y) c = 15;
                acc_w |= (uint32_t)c << (8 * i + nib);
            }
            word[w] = acc_w | __shfl_xor_sync(0xffffffffu, acc_w, 1);
        }
        __syncwarp();   // the previous pass has read its rows out of the staging buffer
        if ((q & 1) == 0) {
#pragma unroll
            for (int w = 0; w < E / 4; w++)
#pragma unroll
                for (int i = 0; i < 4; i++) stage[(q >> 1) + 16 * w + 4 * i] = (uint8_t)(word[w] >> (8 * i));
        }
        __syncwarp();
        if (store) {
            uint8_t* dst = p.kv_cache + (size_t)which * p.slab_bytes + ((size_t)slot * H + h) * p.g.slot_bytes;
            if (vec_ok) {
                for (int v = q; v < G::kQb / 16; v += 8)
                    reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(stage)[v];
            } else {
                for (int b = q; b < G::kQb; b += 8) dst[b] = stage[b];
            }
            const uint16_t nh = (norm != norm) ? (uint16_t)0x7e00u : __half_as_ushort(__float2half_rn(norm));
            if (q < G::kDc) *reinterpret_cast<uint16_t*>(dst + G::kQb + 2 * q) = nh;
            if (p.zero_pad)
                for (int b = G::kQb + 2 * G::kDc + q; b < p.g.slot_bytes; b += 8) dst[b] = 0;
        }
        }   // rows of the token
    }
}

template <typename T>
static void launch_write_rows8(const GenWriteParams& p, unsigned grid, cudaStream_t s) {
    switch (p.g.padded) {
        case 64:
            if (p.walk > 1) write_rows8_kernel<T, 8, true><<<grid, kGenWarps * 32, 0, s>>>(p);
            else write_rows8_kernel<T, 8, false><<<grid, kGenWarps * 32, 0, s>>>(p);
            break;
        case 128: write_rows8_kernel<T, 16, false><<<grid, kGenWarps * 32, 0, s>>>(p); break;
        default: write_rows8_kernel<T, 32, false><<<grid, kGenWarps * 32, 0, s>>>(p); break;
    }
}

// ---------------------------------------------------------------------------------------------
// decode: one block per (split, sequence, KV head), four warps striding over the split's tokens
// ---------------------------------------------------------------------------------------------
struct GenDecodeParams {
    const void* q;
    const uint8_t* kv_cache;
    const int32_t* page_indices;
    const int32_t* page_indptr;
    const int32_t* seq_lens;
    const float* signs;
    int32_t* header;       // workspace word 0: sticky status
    float* partial_lse;    // [batch][splits][num_q_heads], base 2
    float* partial_o;      // [batch][splits][num_q_heads][padded], normalized, rotated domain
    int64_t slab_bytes, num_blocks, kv_begin, kv_end;
    int batch, num_q_heads, num_kv_heads, group, max_pages, q_dtype, splits;   // num_q_heads, group: virtual (x nq)
    int nq, real_heads, real_group;   // queries that share a sequence's KV: column c of a KV head is (query c / real_group, head c % real_group)
    GenGeom g;
    float score_scale;     // sm_scale * log2(e)
    float scale;           // 1 / sqrt(padded)
    float centroids[16];   // already divided by sqrt(padded)
};

// 2^x, hardware approximation (2 ulp), exp2(-inf) = 0
__device__ __forceinline__ float gen_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float gen_load(const void* q, int dtype, int64_t i) {
    if (dtype == TQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]);
    if (dtype == TQ_F16) return __half2float(reinterpret_cast<const __half*>(q)[i]);
    return reinterpret_cast<const float*>(q)[i];
}

// row of q [batch][nq][real_heads] that column c of KV head h of sequence b stands for
__device__ __forceinline__ int64_t gen_q_row(const GenDecodeParams& p, int b, int h, int c) {
    const int qi = c / p.real_group, hh = c - qi * p.real_group;
    return ((int64_t)b * p.nq + qi) * p.real_heads + h * p.real_group + hh;
}

// BPL = code bytes per lane and token: 1, 2 or 4 for padded head sizes 64, 128, 256.  (This file is compiled without
// FMA contraction for the quantizer's sake; the attention arithmetic asks for its FMAs explicitly.)
template <int BPL>
__global__ void __launch_bounds__(kGenWarps * 32, 4) decode_generic_kernel(const __grid_constant__ GenDecodeParams p) {
    extern __shared__ float gsm[];
    const int pd = p.g.padded, G = p.group;
    float* q_s = gsm;                               // [G][pd] rotated queries
    float* o_s = gsm + kGenMaxGroup * kGenMaxDim;   // [warps][G][pd]
    __shared__ float m_s[kGenWarps][kGenMaxGroup], l_s[kGenWarps][kGenMaxGroup];
    __shared__ float cent_s[16];   // a lookup indexed per lane: shared memory, not the parameter bank
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    if (tid < 16) cent_s[tid] = p.centroids[tid];

    // window of this split, in pages
    int64_t len = p.seq_lens[b];
    if (p.kv_end >= 0 && p.kv_end < len) len = p.kv_end;
    const int64_t begin = p.kv_begin > 0 ? p.kv_begin : 0;
    const int first_page = (int)(begin / kGenPage);
    const int last_page = (int)((len + kGenPage - 1) / kGenPage);
    int npages = last_page > first_page ? last_page - first_page : 0;
    const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
    const int have = p.page_indptr ? p.page_indptr[b + 1] - p.page_indptr[b] : p.max_pages;
    if (npages > 0 && first_page + npages > have) {  // the table cannot back this length: read nothing
        if (tid == 0) atomicExch(&p.header[0], kGenStatusSeqTooLong);
        npages = 0;
    }
    const int per = (npages + p.splits - 1) / p.splits;
    const int pg0 = first_page + split * per;
    const int pg1 = min(first_page + npages, pg0 + per);

    // rotate the group's queries: signs, butterflies, 1/sqrt(pd)
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int g = i / pd, d = i - g * pd;
        q_s[i] = d < p.g.head_dim
                     ? gen_load(p.q, p.q_dtype, gen_q_row(p, b, h, g) * p.g.head_dim + d) * p.signs[d]
                     : 0.0f;
    }
    __syncthreads();
    for (int hh = 1; hh < pd; hh <<= 1) {
        for (int i = tid; i < G * pd / 2; i += blockDim.x) {
            const int g = i / (pd / 2), idx = i - g * (pd / 2);
            const int j = (idx / hh) * 2 * hh + (idx % hh);
            float* row = q_s + g * pd;
            const float a = row[j], c = row[j + hh];
            row[j] = a + c;
            row[j + hh] = a - c;
        }
        __syncthreads();
    }
    for (int i = tid; i < G * pd; i += blockDim.x) q_s[i] *= p.scale;
    __syncthreads();

    float m[kGenMaxGroup], l[kGenMaxGroup], o[kGenMaxGroup][2 * BPL];
#pragma unroll
    for (int g = 0; g < kGenMaxGroup; g++) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < 2 * BPL; e++) o[g][e] = 0.0f;
    }
    bool bad_page = false;
    int64_t page_next = pg0 < pg1 ? (int64_t)p.page_indices[tbl + pg0] : 0;
    for (int pg = pg0; pg < pg1; pg++) {
        const int64_t page = page_next;
        if (pg + 1 < pg1) page_next = p.page_indices[tbl + pg + 1];
        if ((uint64_t)page >= (uint64_t)p.num_blocks) {  // never form an address from it
            bad_page = true;
            continue;
        }
        // A warp takes tokens warp, warp + 4, warp + 8, warp + 12 of the page: all their loads are issued
        // before the arithmetic of the first one, so four tokens' latencies overlap.
        uint8_t kb[4][BPL], vb[4][BPL];
        float kn[4], vn[4];
        bool tv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = warp + kGenWarps * i;
            const int64_t t = (int64_t)pg * kGenPage + e;
            tv[i] = t >= begin && t < len;
            kn[i] = vn[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < BPL; j++) kb[i][j] = vb[i][j] = 0;
            if (tv[i]) {
                const uint8_t* ks = p.kv_cache + ((size_t)(page * kGenPage + e) * p.num_kv_heads + h) * p.g.slot_bytes;
                const uint8_t* vs = ks + p.slab_bytes;
#pragma unroll
                for (int j = 0; j < BPL; j++) {
                    kb[i][j] = ks[lane + 32 * j];
                    vb[i][j] = vs[lane + 32 * j];
                }
                kn[i] = __half2float(*reinterpret_cast<const __half*>(ks + p.g.qbytes));
                vn[i] = __half2float(*reinterpret_cast<const __half*>(vs + p.g.qbytes));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (!tv[i]) continue;
            float kd[2 * BPL], vd[2 * BPL];
#pragma unroll
            for (int j = 0; j < BPL; j++) {
                kd[2 * j] = cent_s[kb[i][j] >> 4] * kn[i];
                kd[2 * j + 1] = cent_s[kb[i][j] & 15] * kn[i];
                vd[2 * j] = cent_s[vb[i][j] >> 4] * vn[i];
                vd[2 * j + 1] = cent_s[vb[i][j] & 15] * vn[i];
            }
#pragma unroll
            for (int g = 0; g < kGenMaxGroup; g++) {
                if (g >= G) break;
                const float* qr = q_s + g * pd;
                float sc = 0.0f;
#pragma unroll
                for (int j = 0; j < BPL; j++) {
                    const float2 q2 = *reinterpret_cast<const float2*>(qr + 2 * (lane + 32 * j));
                    sc = __fmaf_rn(q2.x, kd[2 * j], __fmaf_rn(q2.y, kd[2 * j + 1], sc));
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, off);
                sc *= p.score_scale;
                const float m_new = fmaxf(m[g], sc);
                const float corr = gen_exp2(m[g] - m_new), w = gen_exp2(sc - m_new);
                m[g] = m_new;
                l[g] = __fmaf_rn(l[g], corr, w);
#pragma unroll
                for (int e2 = 0; e2 < 2 * BPL; e2++) o[g][e2] = __fmaf_rn(w, vd[e2], o[g][e2] * corr);
            }
        }
    }
    if (bad_page && lane == 0) atomicExch(&p.header[0], kGenStatusBadPage);
    // combine the four warps
#pragma unroll
    for (int g = 0; g < kGenMaxGroup; g++) {
        if (g >= G) break;
        if (lane == 0) {
            m_s[warp][g] = m[g];
            l_s[warp][g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < BPL; j++) {
            const int d = 2 * (lane + 32 * j);
            o_s[(warp * G + g) * pd + d] = o[g][2 * j];
            o_s[(warp * G + g) * pd + d + 1] = o[g][2 * j + 1];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int g = i / pd, d = i - g * pd;
        float mm = -INFINITY;
        for (int w = 0; w < kGenWarps; w++) mm = fmaxf(mm, m_s[w][g]);
        float ll = 0.0f, acc = 0.0f;
        if (mm > -INFINITY) {
            for (int w = 0; w < kGenWarps; w++) {
                const float sc = exp2f(m_s[w][g] - mm);
                if (sc > 0.0f) {
                    ll += sc * l_s[w][g];
                    acc += sc * o_s[(w * G + g) * pd + d];
                }
            }
        }
        const int64_t row = ((int64_t)b * p.splits + split) * p.num_q_heads + h * G + g;
        p.partial_o[row * pd + d] = ll > 0.0f ? acc / ll : 0.0f;
        if (d == 0) p.partial_lse[row] = ll > 0.0f ? mm + log2f(ll) : -INFINITY;
    }
}

// ---------------------------------------------------------------------------------------------
// decode on the tensor cores for the same head sizes: a warp takes whole pages, stages their slots in
// shared memory with 16-byte asynchronous copies (its own ring of stages, no block-wide barrier in the
// loop) and dequantizes the codes straight into mma.sync.m16n8k16 fragments.
//   S = K^ Q^T (16 tokens x 8 query columns): lane (g, tg) reads bytes tg PD/8 ... of the code rows
//   of tokens g and g + 8; a code byte looked up in a table of fp16 centroid pairs IS one A-fragment
//   register (two neighbouring contraction slots of one token), so the contraction runs over the dims
//   in the order the bytes come, and the Q^T fragments are built in that order once per block.
//   O^T += V^^T P (PD dims x 8 columns): the contraction runs over tokens, so a fragment register
//   pairs two tokens' values of one dim: lane (g, tg) reads bytes g PD/16 ... of tokens 2tg, 2tg + 1,
//   2tg + 8, 2tg + 9 and zips the nibbles of a token pair into bytes before the lookup (low nibbles
//   = odd dims -> accumulator row g, high nibbles = even dims -> row g + 8).
// The table entry of byte v is {low half: centroid of the low nibble, high half: of the high nibble},
// one copy per lane side by side (32 KB).  Online softmax in base 2 per page; the
// K norm is folded into the scores, the V norm into P (moved into place with movmatrix).  Same grid,
// workspace and merge as the plain kernel above, which stays as the fallback for caches that are not
// 16-byte aligned.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t gen_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gen_mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t gen_movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t gen_pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// table entry of byte j of word w (the table's column of this lane is folded into lut_lane; COLS copies per byte value)
template <int COLS>
__device__ __forceinline__ uint32_t gen_lookup(uint32_t w, int j, uint32_t lut_lane) {
    uint32_t r;
    uint32_t v;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(v) : "r"(w), "r"(0x4440u | (uint32_t)j));   // byte j of w
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(v * (4u * COLS) + lut_lane));
    return r;
}
// BYTES (4, 8, 16 or 32) of a staged code row into words
template <int BYTES>
__device__ __forceinline__ void gen_lds_words(uint32_t addr, uint32_t (&w)[BYTES / 4]) {
    if constexpr (BYTES == 4) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(addr));
    } else if constexpr (BYTES == 8) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
    } else {
#pragma unroll
        for (int i = 0; i < BYTES / 16; i++)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3]) : "r"(addr + 16 * i));
    }
}
__device__ __forceinline__ float gen_lds_half(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void gen_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void gen_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void gen_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int PD>
struct FragShape {
    static constexpr int kKBytes = PD / 8, kVBytes = PD / 16;   // code bytes per lane and token, K and V
    static constexpr int kVWords = kVBytes / 4;
    static constexpr int kRow = ((PD / 2 + 2 * (PD / 64)) + 15) & ~15;   // staged bytes of a slot: codes + norms, 48 / 80 / 144
    static constexpr int kChunks = 2 * 16 * kRow / 16;          // 16-byte copies per page and head (K and V): 96 / 160 / 288
    static constexpr int kStageBytes = 2 * 16 * kRow;
    static constexpr int kStages = PD == 256 ? 2 : 3;
    static constexpr int kLutCols = 32;   // copies of the lookup table side by side: one per lane, no two lanes of a lookup share a bank
    static constexpr size_t kRing = (size_t)kGenWarps * kStages * kStageBytes;
    static constexpr size_t kCombine = (size_t)kGenWarps * kGenMaxGroup * PD * 4;   // also covers the rotated queries
    static constexpr size_t kSmem = kRing > kCombine ? kRing : kCombine;
    static_assert(kChunks % 32 == 0, "a page's copies divide evenly over the lanes");
};

template <int PD>
__global__ void __launch_bounds__(kGenWarps * 32, PD == 64 ? 4 : PD == 128 ? 4 : 3) decode_frags_kernel(const __grid_constant__ GenDecodeParams p) {
    using F = FragShape<PD>;
    extern __shared__ __align__(16) uint8_t tsm[];
    __shared__ float m_s[kGenWarps][kGenMaxGroup], l_s[kGenWarps][kGenMaxGroup];
    __shared__ float cent_s[16];
    __shared__ __align__(16) uint32_t lut_s[256 * F::kLutCols];
    constexpr int pd = PD;
    const int G = p.group;
    float* q_s = reinterpret_cast<float*>(tsm);   // [G][pd] rotated queries, before the loop
    float* o_s = reinterpret_cast<float*>(tsm);   // [warps][G][pd], after the loop
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int split = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    if (tid < 16) cent_s[tid] = p.centroids[tid];

    // window of this split, in pages
    int64_t len = p.seq_lens[b];
    if (p.kv_end >= 0 && p.kv_end < len) len = p.kv_end;
    const int64_t begin = p.kv_begin > 0 ? p.kv_begin : 0;
    const int first_page = (int)(begin / kGenPage);
    const int last_page = (int)((len + kGenPage - 1) / kGenPage);
    int npages = last_page > first_page ? last_page - first_page : 0;
    const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
    const int have = p.page_indptr ? p.page_indptr[b + 1] - p.page_indptr[b] : p.max_pages;
    if (npages > 0 && first_page + npages > have) {  // the table cannot back this length: read nothing
        if (tid == 0) atomicExch(&p.header[0], kGenStatusSeqTooLong);
        npages = 0;
    }
    const int per = (npages + p.splits - 1) / p.splits;
    const int pg0 = first_page + split * per;
    const int pg1 = min(first_page + npages, pg0 + per);

    // rotate the group's queries: signs, butterflies, 1/sqrt(pd)
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int gg = i / pd, d = i - gg * pd;
        q_s[i] = d < p.g.head_dim
                     ? gen_load(p.q, p.q_dtype, gen_q_row(p, b, h, gg) * p.g.head_dim + d) * p.signs[d]
                     : 0.0f;
    }
    __syncthreads();
    for (int v = tid; v < 256; v += blockDim.x) {   // a row of copies per byte value
        const uint32_t e = gen_pack_half2(cent_s[v & 15], cent_s[v >> 4]);
        uint4* row = reinterpret_cast<uint4*>(lut_s + v * F::kLutCols);
#pragma unroll
        for (int i = 0; i < F::kLutCols / 4; i++) row[i] = make_uint4(e, e, e, e);
    }
    for (int hh = 1; hh < pd; hh <<= 1) {
        for (int i = tid; i < G * pd / 2; i += blockDim.x) {
            const int gg = i / (pd / 2), idx = i - gg * (pd / 2);
            const int j = (idx / hh) * 2 * hh + (idx % hh);
            float* row = q_s + gg * pd;
            const float a = row[j], c = row[j + hh];
            row[j] = a + c;
            row[j + hh] = a - c;
        }
        __syncthreads();
    }
    // B fragments of Q^T: column g of the query tile (zero beyond the group).  Step s contracts over the dims of
    // this lane's code bytes 2s and 2s + 1 (dims 4 (tg PD/16 + s) ...), each byte's odd dim in the lower slot.
    uint32_t qf[PD / 8];
#pragma unroll
    for (int s = 0; s < PD / 16; s++) {
        const float* row = q_s + g * pd + tg * (PD / 4) + 4 * s;
        const bool on = g < G;
        qf[2 * s] = on ? gen_pack_half2(row[1] * p.scale, row[0] * p.scale) : 0u;
        qf[2 * s + 1] = on ? gen_pack_half2(row[3] * p.scale, row[2] * p.scale) : 0u;
    }
    __syncthreads();   // the queries are in registers: their shared memory becomes the warps' stage rings

    float o_acc[PD / 16][4];
#pragma unroll
    for (int i = 0; i < PD / 16; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o_acc[i][j] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const uint32_t lut_lane = gen_smem_u32(lut_s) + 4u * (lane & (F::kLutCols - 1));
    const uint32_t ring = gen_smem_u32(tsm) + (uint32_t)warp * F::kStages * F::kStageBytes;
    const size_t tok_stride = (size_t)p.num_kv_heads * p.g.slot_bytes;
    const int my_pages = pg1 > pg0 + warp ? (pg1 - pg0 - warp + kGenWarps - 1) / kGenWarps : 0;
    auto page_at = [&](int i) -> int64_t { return i < my_pages ? (int64_t)p.page_indices[tbl + pg0 + warp + i * kGenWarps] : -1; };
    uint32_t staged = 0;   // bit s: stage s holds a page (its id was inside the cache)
    // copies of one page into a stage: the 16-byte pieces of the 16 K rows, then of the 16 V rows, dealt over
    // the lanes; source and destination offsets of this lane's pieces are fixed
    constexpr int kPieces = 16 * F::kRow / 16, kRounds = (kPieces + 31) / 32;
    uint32_t src_off[kRounds], dst_off[kRounds];
#pragma unroll
    for (int i = 0; i < kRounds; i++) {
        const int c = lane + 32 * i, tok = c / (F::kRow / 16), piece = c % (F::kRow / 16);
        src_off[i] = (uint32_t)(tok * tok_stride) + piece * 16;
        dst_off[i] = tok * F::kRow + piece * 16;
    }
    auto issue = [&](int stage, int64_t page) {
        if ((uint64_t)page < (uint64_t)p.num_blocks) {
            const uint8_t* base_k = p.kv_cache + (size_t)(page * kGenPage) * tok_stride + (size_t)h * p.g.slot_bytes;
            const uint8_t* base_v = base_k + p.slab_bytes;
            const uint32_t dst_k = ring + stage * F::kStageBytes, dst_v = dst_k + 16 * F::kRow;
#pragma unroll
            for (int i = 0; i < kRounds; i++) {
                if (kPieces % 32 == 0 || i + 1 < kRounds || lane + 32 * i < kPieces) {
                    gen_cp_async16(dst_k + dst_off[i], base_k + src_off[i]);
                    gen_cp_async16(dst_v + dst_off[i], base_v + src_off[i]);
                }
            }
            staged |= 1u << stage;
        } else {
            staged &= ~(1u << stage);
        }
        gen_cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < F::kStages - 1; i++) issue(i, page_at(i));
    int64_t page_issue = page_at(F::kStages - 1);
    int st = 0, st_issue = F::kStages - 1;
    bool bad_page = false;
    for (int it = 0; it < my_pages; it++) {
        const int64_t page_after = page_at(it + F::kStages);   // its id arrives while this page is worked on
        issue(st_issue, page_issue);                            // into the stage the previous iteration has left
        gen_cp_async_wait<F::kStages - 1>();
        __syncwarp();
        if (!((staged >> st) & 1u)) {
            bad_page = true;   // no address was formed from the id
        } else {
            const uint32_t sk = ring + st * F::kStageBytes, sv = sk + 16 * F::kRow;
            // ---- S = K^ Q^T -------------------------------------------------------------------------------
            uint32_t ka[F::kKBytes / 4], kb[F::kKBytes / 4];
            gen_lds_words<F::kKBytes>(sk + g * F::kRow + tg * F::kKBytes, ka);
            gen_lds_words<F::kKBytes>(sk + (g + 8) * F::kRow + tg * F::kKBytes, kb);
            float s_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s_acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < PD / 16; s++) {
                const uint32_t wa = ka[s >> 1], wb = kb[s >> 1];
                const int j = 2 * (s & 1);
                const uint32_t a0 = gen_lookup<F::kLutCols>(wa, j, lut_lane), a2 = gen_lookup<F::kLutCols>(wa, j + 1, lut_lane);
                const uint32_t a1 = gen_lookup<F::kLutCols>(wb, j, lut_lane), a3 = gen_lookup<F::kLutCols>(wb, j + 1, lut_lane);
                gen_mma16816((s & 1) ? s_acc2 : s_acc, a0, a1, a2, a3, qf[2 * s], qf[2 * s + 1]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) s_acc[i] += s_acc2[i];
            // ---- online softmax (base 2); rows g and g + 8 are tokens, columns 2tg and 2tg + 1 query heads --
            // The window starts on a page boundary, so only the last page of a sequence can hold tokens outside it:
            // their norms are zeroed (whatever the unwritten slots contain) and their scores biased to -inf.  Row 0 of
            // every page is inside, so every column's maximum is finite from the first page on.
            float kfa = gen_lds_half(sk + g * F::kRow + PD / 2) * p.score_scale, kfb = gen_lds_half(sk + (g + 8) * F::kRow + PD / 2) * p.score_scale;
            float vfa = gen_lds_half(sv + g * F::kRow + PD / 2), vfb = gen_lds_half(sv + (g + 8) * F::kRow + PD / 2);
            float bias_a = 0.0f, bias_b = 0.0f;
            const int64_t t0 = (int64_t)(pg0 + warp + it * kGenWarps) * kGenPage;
            if (t0 + kGenPage > len) {
                if (t0 + g >= len) { kfa = 0.0f; vfa = 0.0f; bias_a = -INFINITY; }
                if (t0 + g + 8 >= len) { kfb = 0.0f; vfb = 0.0f; bias_b = -INFINITY; }
            }
            const float x0 = __fmaf_rn(s_acc[0], kfa, bias_a), x1 = __fmaf_rn(s_acc[1], kfa, bias_a);
            const float x2 = __fmaf_rn(s_acc[2], kfb, bias_b), x3 = __fmaf_rn(s_acc[3], kfb, bias_b);
            // The running maximum of a column is raised only when a score of the page exceeds it by more than 2^6
            // (the weights stay within fp16): one vote decides, and only then is the page's maximum reduced across
            // the lanes and the accumulators rescaled.
            float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
            if (__any_sync(0xffffffffu, mx0 > m0 + 6.0f || mx1 > m1 + 6.0f)) {
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
                }
                const bool r0 = mx0 > m0 + 6.0f, r1 = mx1 > m1 + 6.0f;
                const float c0 = r0 ? gen_exp2(m0 - mx0) : 1.0f, c1 = r1 ? gen_exp2(m1 - mx1) : 1.0f;
                if (r0) m0 = mx0;
                if (r1) m1 = mx1;
                l0 *= c0;
                l1 *= c1;
#pragma unroll
                for (int mt = 0; mt < PD / 16; mt++) {
                    o_acc[mt][0] *= c0; o_acc[mt][1] *= c1; o_acc[mt][2] *= c0; o_acc[mt][3] *= c1;
                }
            }
            const float e0 = gen_exp2(x0 - m0), e1 = gen_exp2(x1 - m1), e2 = gen_exp2(x2 - m0), e3 = gen_exp2(x3 - m1);
            l0 += e0 + e2;
            l1 += e1 + e3;
            const uint32_t pb0 = gen_movmatrix_trans(gen_pack_half2(e0 * vfa, e1 * vfa));
            const uint32_t pb1 = gen_movmatrix_trans(gen_pack_half2(e2 * vfb, e3 * vfb));
            // ---- O^T += V^^T P: zip the nibbles of a token pair into bytes, look the pairs up ----------------
            uint32_t v0[F::kVWords], v1[F::kVWords], v2[F::kVWords], v3[F::kVWords];
            const uint32_t vrow = sv + (2 * tg) * F::kRow + g * F::kVBytes;
            gen_lds_words<F::kVBytes>(vrow, v0);
            gen_lds_words<F::kVBytes>(vrow + F::kRow, v1);
            gen_lds_words<F::kVBytes>(vrow + 8 * F::kRow, v2);
            gen_lds_words<F::kVBytes>(vrow + 9 * F::kRow, v3);
#pragma unroll
            for (int w = 0; w < F::kVWords; w++) {
                const uint32_t lo01 = (v0[w] & 0x0F0F0F0Fu) | ((v1[w] << 4) & 0xF0F0F0F0u);
                const uint32_t hi01 = ((v0[w] >> 4) & 0x0F0F0F0Fu) | (v1[w] & 0xF0F0F0F0u);
                const uint32_t lo23 = (v2[w] & 0x0F0F0F0Fu) | ((v3[w] << 4) & 0xF0F0F0F0u);
                const uint32_t hi23 = ((v2[w] >> 4) & 0x0F0F0F0Fu) | (v3[w] & 0xF0F0F0F0u);
#pragma unroll
                for (int j = 0; j < 4; j++)   // rows: g <- odd dim, g + 8 <- even dim of this lane's code byte 4w + j
                    gen_mma16816(o_acc[4 * w + j], gen_lookup<F::kLutCols>(lo01, j, lut_lane), gen_lookup<F::kLutCols>(hi01, j, lut_lane),
                                 gen_lookup<F::kLutCols>(lo23, j, lut_lane), gen_lookup<F::kLutCols>(hi23, j, lut_lane), pb0, pb1);
            }
        }
        __syncwarp();   // every lane has read the stage before the next iteration copies into it
        page_issue = page_after;
        st_issue = st;
        st = st + 1 == F::kStages ? 0 : st + 1;
    }
    gen_cp_async_wait<0>();
    if (bad_page && lane == 0) atomicExch(&p.header[0], kGenStatusBadPage);
    // this warp's sums over its token lanes, then everything to shared memory for the block's combine
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    __syncthreads();   // every warp has left its ring: the region becomes o_s
    if (g == 0) {
        if (2 * tg < G) { m_s[warp][2 * tg] = m0; l_s[warp][2 * tg] = l0; }
        if (2 * tg + 1 < G) { m_s[warp][2 * tg + 1] = m1; l_s[warp][2 * tg + 1] = l1; }
    }
#pragma unroll
    for (int mt = 0; mt < PD / 16; mt++) {
        const int d_even = 2 * (g * (PD / 16) + mt);   // accumulator rows g / g + 8 hold the odd / even dim of byte g PD/16 + mt
        if (2 * tg < G) {
            o_s[(warp * G + 2 * tg) * pd + d_even + 1] = o_acc[mt][0];
            o_s[(warp * G + 2 * tg) * pd + d_even] = o_acc[mt][2];
        }
        if (2 * tg + 1 < G) {
            o_s[(warp * G + 2 * tg + 1) * pd + d_even + 1] = o_acc[mt][1];
            o_s[(warp * G + 2 * tg + 1) * pd + d_even] = o_acc[mt][3];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int gg = i / pd, d = i - gg * pd;
        float mm = -INFINITY;
        for (int w = 0; w < kGenWarps; w++) mm = fmaxf(mm, m_s[w][gg]);
        float ll = 0.0f, acc = 0.0f;
        if (mm > -INFINITY) {
            for (int w = 0; w < kGenWarps; w++) {
                const float sc = gen_exp2(m_s[w][gg] - mm);
                if (sc > 0.0f) {
                    ll += sc * l_s[w][gg];
                    acc += sc * o_s[(w * G + gg) * pd + d];
                }
            }
        }
        const int64_t row = ((int64_t)b * p.splits + split) * p.num_q_heads + h * G + gg;
        p.partial_o[row * pd + d] = ll > 0.0f ? acc / ll : 0.0f;
        if (d == 0) p.partial_lse[row] = ll > 0.0f ? mm + log2f(ll) : -INFINITY;
    }
}

struct GenMergeParams {
    const float* partial_o;
    const float* partial_lse;
    const float* signs;
    void* out;
    float* out_lse;
    int num_q_heads, splits, out_dtype, emit_rotated;   // num_q_heads: virtual (x nq)
    int nq, real_heads, real_group, group;   // virtual head -> (query, real head) of the output row; nq = 1: identity
    GenGeom g;
    float scale;
};

// one block of `padded` threads per (sequence, query head)
__global__ void __launch_bounds__(kGenMaxDim) merge_generic_kernel(const __grid_constant__ GenMergeParams p) {
    __shared__ float buf[kGenMaxDim];
    const int d = threadIdx.x, pd = p.g.padded;
    const int64_t b = blockIdx.x / p.num_q_heads;
    const int hq = (int)(blockIdx.x - b * p.num_q_heads);
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; s++) mm = fmaxf(mm, p.partial_lse[(b * p.splits + s) * p.num_q_heads + hq]);
    float wsum = 0.0f, acc = 0.0f;
    if (mm > -INFINITY) {
        for (int s = 0; s < p.splits; s++) {
            const int64_t row = (b * p.splits + s) * p.num_q_heads + hq;
            const float w = exp2f(p.partial_lse[row] - mm);
            if (w > 0.0f) {
                wsum += w;
                acc += w * p.partial_o[row * pd + d];
            }
        }
    }
    float o = wsum > 0.0f ? acc / wsum : 0.0f;
    const float lse2 = wsum > 0.0f ? mm + log2f(wsum) : -INFINITY;
    // virtual head hq = (KV head, column); column = (query, head of the group): rows of the output are [batch][nq][real heads]
    const int kvh = hq / p.group, col = hq - kvh * p.group, qi = col / p.real_group;
    const int64_t orow = (b * p.nq + qi) * p.real_heads + kvh * p.real_group + (col - qi * p.real_group);
    if (p.emit_rotated) {
        reinterpret_cast<float*>(p.out)[orow * pd + d] = o;
        if (p.out_lse && d == 0) p.out_lse[orow] = lse2;
        return;
    }
    buf[d] = o;
    __syncthreads();
    for (int h = 1; h < pd; h <<= 1) {
        const float a = buf[d & ~h], c = buf[d | h];
        __syncthreads();
        buf[d] = (d & h) ? a - c : a + c;
        __syncthreads();
    }
    o = buf[d] * p.scale * p.signs[d];
    if (d < p.g.head_dim) {
        const int64_t at = orow * p.g.head_dim + d;
        if (p.out_dtype == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(o);
        else if (p.out_dtype == TQ_F16) reinterpret_cast<__half*>(p.out)[at] = __float2half_rn(o);
        else reinterpret_cast<float*>(p.out)[at] = o;
    }
    if (p.out_lse && d == 0) p.out_lse[orow] = lse2 * 0.6931471805599453f;
}

// ---------------------------------------------------------------------------------------------
// bulk dequantization: eight lanes per (sequence, token), walking its heads' K and V rows
// ---------------------------------------------------------------------------------------------
struct GenDequantParams {
    const uint8_t* kv_cache;
    const int32_t* page_indices;
    const int32_t* page_indptr;
    const int32_t* seq_lens;
    const int32_t* cu_seqlens;
    const float* signs;
    void* out[2];
    int64_t slab_bytes, num_blocks, out_token_stride;
    int batch, max_pages, num_kv_heads, out_dtype;
    int walk;   // rows a lane group takes of its token: all 2 H (large jobs) or 1 (small ones: more groups in flight)
    GenGeom g;
    float scale;
    float centroids[16];
};

static __device__ int32_t g_gen_dequant_skipped = 0;

// Eight lanes own one row and a warp works on four rows at a time.  The row is cut into chunks of 64 elements
// (32 code bytes); lane q holds elements 8 q ... 8 q + 7 of every chunk, register r = 8 c + i being element
// 64 c + 8 q + i.  So a chunk's code bytes are one 4-byte load per lane (32 contiguous bytes per row) and its
// output one 16-byte store per lane (128 contiguous bytes per row); butterfly stages 1, 2, 4 and 64, 128 are
// register-local and stages 8, 16, 32 one shuffle per element, in the same stage order as everywhere else.
template <int E>
__global__ void __launch_bounds__(kGenWarps * 32, 8) dequant_rows8_kernel(const __grid_constant__ GenDequantParams p) {
    constexpr int kPd = 8 * E, kQb = kPd / 2, kChunks = E / 8;
    __shared__ float cent_s[16];   // a lookup indexed per lane: shared memory, not the parameter bank
    __shared__ float sg_s[kPd];
    if (threadIdx.x < 16) cent_s[threadIdx.x] = p.centroids[threadIdx.x];
    // sign of element j = 64 c + 8 q + i at [8 c + i][q]: the eight lanes of a row read eight neighbouring words
    for (int j = threadIdx.x; j < kPd; j += kGenWarps * 32)
        sg_s[((j >> 6) * 8 + (j & 7)) * 8 + ((j >> 3) & 7)] = j < p.g.head_dim ? p.signs[j] : 0.0f;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = lane & 7, rg = lane >> 3;
    const int H = p.num_kv_heads, hd = p.g.head_dim;
    const int parts = 2 * H / p.walk;                                   // lane groups per token
    const int64_t per_seq = (int64_t)p.max_pages * kGenPage * parts;   // items of a sequence's table
    const int64_t items = per_seq * p.batch;
    const bool small = items < 0x7fffffff;
    const int esize = p.out_dtype == TQ_F32 ? 4 : 2;
    const bool in_vec = ((reinterpret_cast<uintptr_t>(p.kv_cache) | (uintptr_t)p.slab_bytes | (uintptr_t)p.g.slot_bytes) & 3) == 0;
    const bool out_vec = ((reinterpret_cast<uintptr_t>(p.out[0]) | reinterpret_cast<uintptr_t>(p.out[1])) & 15) == 0 &&
                         ((p.out_token_stride * esize) & 15) == 0 && ((hd * esize) & 15) == 0;
    const float* sg = sg_s + q;
    // code bytes 4 q ... 4 q + 3 of every chunk of a slot, and its norm
    auto fetch = [&](const uint8_t* slot, uint32_t (&cw)[kChunks], float& norm) {
#pragma unroll
        for (int c = 0; c < kChunks; c++) {
            const uint8_t* src = slot + 32 * c + 4 * q;
            if (in_vec) {
                cw[c] = *reinterpret_cast<const uint32_t*>(src);
            } else {
                cw[c] = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) cw[c] |= (uint32_t)src[i] << (8 * i);
            }
        }
        norm = __half2float(*reinterpret_cast<const __half*>(slot + kQb));
    };

    // a group of eight lanes takes one token and walks `walk` of its 2 H rows (K and V of head 0, of head 1, ...): the token's
    // page lookup and output row are worked out once, and the next row's codes are fetched while this one is worked on
    for (int64_t base = ((int64_t)blockIdx.x * kGenWarps + warp) * 4; base < items; base += (int64_t)gridDim.x * kGenWarps * 4) {
        // a group without a token (past the end, past its sequence, an unlisted page) runs the shuffles on zeros
        const int64_t it = base + rg;
        bool live = it < items;
        int b = 0, r0 = 0;
        int64_t t = 0;
        if (live) {
            if (small) {
                const uint32_t bb = (uint32_t)it / (uint32_t)per_seq;
                const uint32_t rem = (uint32_t)it - bb * (uint32_t)per_seq, tt = rem / (uint32_t)parts;
                b = (int)bb;
                t = tt;
                r0 = (int)(rem - tt * (uint32_t)parts) * p.walk;
            } else {
                b = (int)(it / per_seq);
                const int64_t rem = it - (int64_t)b * per_seq;
                t = rem / parts;
                r0 = (int)(rem - t * parts) * p.walk;
            }
            live = t < p.seq_lens[b];
        }
        const uint8_t* slot0 = nullptr;
        if (live) {
            const int pg = (int)(t / kGenPage), e = (int)(t % kGenPage);
            const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
            const bool listed = !p.page_indptr || tbl + pg < (int64_t)p.page_indptr[b + 1];
            const int64_t page = listed ? (int64_t)p.page_indices[tbl + pg] : -1;
            if ((uint64_t)page >= (uint64_t)p.num_blocks) {
                if (q == 0 && e == 0 && r0 == 0) atomicAdd(&g_gen_dequant_skipped, 1);
                live = false;
            } else {
                slot0 = p.kv_cache + (size_t)(page * kGenPage + e) * H * p.g.slot_bytes;
            }
        }
        if (!__any_sync(0xffffffffu, live)) continue;
        const int64_t orow0 = live ? ((int64_t)p.cu_seqlens[b] + t) * p.out_token_stride : 0;
        uint32_t cw_next[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; c++) cw_next[c] = 0;
        float norm_next = 0.0f;
        if (live) fetch(slot0 + ((r0 & 1) ? (size_t)p.slab_bytes : 0) + (size_t)(r0 >> 1) * p.g.slot_bytes, cw_next, norm_next);
        for (int r = r0; r < r0 + p.walk; r++) {
        const int which = r & 1, h = r >> 1;   // K and V rows of a head alternate
        uint32_t cw[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; c++) cw[c] = cw_next[c];
        const float norm = norm_next;
        if (live && r + 1 < r0 + p.walk) {
            const int wn = (r + 1) & 1, hn = (r + 1) >> 1;
            fetch(slot0 + (size_t)wn * p.slab_bytes + (size_t)hn * p.g.slot_bytes, cw_next, norm_next);
        }
        float x[E];
#pragma unroll
        for (int c = 0; c < kChunks; c++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t code = (cw[c] >> (8 * i)) & 0xffu;
                x[8 * c + 2 * i] = cent_s[code >> 4];
                x[8 * c + 2 * i + 1] = cent_s[code & 15];
            }
        }
        // stages 1, 2, 4 (inside a lane's eight), 8, 16, 32 (between the lanes), 64, 128 (between the chunks)
#pragma unroll
        for (int hr = 1; hr < 8; hr <<= 1) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                if ((k & hr) == 0) {
                    const float a = x[k], c = x[k + hr];
                    x[k] = __fadd_rn(a, c);
                    x[k + hr] = __fsub_rn(a, c);
                }
            }
        }
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                const float o = __shfl_xor_sync(0xffffffffu, x[k], m);
                x[k] = (q & m) ? __fsub_rn(o, x[k]) : __fadd_rn(x[k], o);
            }
        }
#pragma unroll
        for (int hr = 8; hr < E; hr <<= 1) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                if ((k & hr) == 0) {
                    const float a = x[k], c = x[k + hr];
                    x[k] = __fadd_rn(a, c);
                    x[k + hr] = __fsub_rn(a, c);
                }
            }
        }
        if (!live) continue;
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = __fmul_rn(__fmul_rn(__fmul_rn(x[i], p.scale), sg[8 * i]), norm);
        const int64_t orow = orow0 + (int64_t)h * hd;
        if (p.out_dtype == TQ_F32) {
            float* out = reinterpret_cast<float*>(p.out[which]) + orow;
#pragma unroll
            for (int c = 0; c < E / 4; c++) {
                const int d0 = 64 * (c >> 1) + 8 * q + 4 * (c & 1);   // registers 4 c ... 4 c + 3
                if (out_vec && d0 + 4 <= hd) {
                    *reinterpret_cast<float4*>(out + d0) = make_float4(x[4 * c], x[4 * c + 1], x[4 * c + 2], x[4 * c + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        if (d0 + i < hd) out[d0 + i] = x[4 * c + i];
                }
            }
        } else {
            uint16_t* out = reinterpret_cast<uint16_t*>(p.out[which]) + orow;
            const bool bf = p.out_dtype == TQ_BF16;
#pragma unroll
            for (int c = 0; c < kChunks; c++) {
                const int d0 = 64 * c + 8 * q;
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float lo = x[8 * c + 2 * i], hi = x[8 * c + 2 * i + 1];
                    if (bf) {
                        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                        w[i] = *reinterpret_cast<const uint32_t*>(&v);
                    } else {
                        const __half2 v = __floats2half2_rn(lo, hi);
                        w[i] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                }
                if (out_vec && d0 + 8 <= hd) {
                    *reinterpret_cast<uint4*>(out + d0) = make_uint4(w[0], w[1], w[2], w[3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        if (d0 + i < hd) out[d0 + i] = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
                }
            }
        }
        }   // rows of the token
    }
}

// ---------------------------------------------------------------------------------------------
// host side (called from the C-ABI entry points when the geometry is not the 128-wide one)
// ---------------------------------------------------------------------------------------------
int device_sm_count(int* out);

int generic_slot_bytes(int head_dim) {
    const int pd = gen_next_pow2(head_dim);
    const int dc = pd / 64;
    return (dc * 32 + dc * 2 + 15) & ~15;
}

int generic_write(void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads, int slot_bytes, const void* key,
                  const void* value, int in_dtype, int64_t num_tokens, int64_t k_token_stride, int64_t v_token_stride,
                  const float* signs, const void* slot_mapping, int slot_dtype, int head_dim, int flags, void* stream) {
    TQ_REQUIRE(head_dim > 32 && head_dim <= kGenMaxDim, TQ_ERR_UNSUPPORTED, "head_dim must be 33..%d, got %d", kGenMaxDim, head_dim);
    TQ_REQUIRE(slot_bytes >= generic_slot_bytes(head_dim), TQ_ERR_INVALID, "slot_bytes %d is smaller than head size %d needs (%d)",
               slot_bytes, head_dim, generic_slot_bytes(head_dim));
    GenWriteParams p{};
    p.kv_cache = static_cast<uint8_t*>(kv_cache);
    p.src[0] = key;
    p.src[1] = value;
    p.token_stride[0] = k_token_stride;
    p.token_stride[1] = v_token_stride;
    p.slot_mapping = slot_mapping;
    p.signs = signs;
    p.num_tokens = num_tokens;
    p.slab_bytes = num_blocks * block_size * (int64_t)num_kv_heads * slot_bytes;
    p.total_slots = num_blocks * (int64_t)block_size;
    p.num_kv_heads = num_kv_heads;
    p.slot_is_i64 = slot_dtype == TQ_I64;
    p.zero_pad = (flags & TQ_WRITE_ZERO_PAD) != 0;
    p.g = make_geom(head_dim, slot_bytes);
    p.scale = (float)(1.0 / std::sqrt((double)p.g.padded));
    float cen[16];
    host_codebook(p.g.padded, 4, cen, p.boundaries);
    // large jobs of the smallest head: a lane group walks all rows of its token (96 us against 101 for 32768 tokens x
    // 8 heads); small jobs (a decode step's new tokens) and the larger heads, where the index arithmetic is a smaller
    // share and fewer groups in flight cost more than it saves (347 us against 337 at head 256): a row per group
    p.walk = num_tokens >= 8192 && p.g.padded == 64 ? 2 * num_kv_heads : 1;
    const int64_t items = num_tokens * (2 * num_kv_heads / p.walk);
    const int64_t blocks = (items + 4 * kGenWarps - 1) / (4 * kGenWarps);   // four lane groups per warp and pass
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case TQ_F32: launch_write_rows8<float>(p, grid, s); break;
        case TQ_F16: launch_write_rows8<__half>(p, grid, s); break;
        default: launch_write_rows8<__nv_bfloat16>(p, grid, s); break;
    }
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

// blocks per SM the decode grid is sized to: one wave of resident blocks for head sizes up to 128 (four fit beside
// their 32 KB tables; more, smaller blocks cost more prologues than they balance), two waves for 256 (three fit;
// 221 us against 229 for batch 8 x 32768)
static int generic_blocks_per_sm(int padded) { return padded == 64 ? 4 : padded == 128 ? 4 : 6; }

static int generic_splits(int batch, int num_kv_heads, int num_ctas, int padded) {
    int ctas = num_ctas;
    if (ctas <= 0 && device_sm_count(&ctas) != TQ_OK) ctas = 148;
    int s = (generic_blocks_per_sm(padded) * ctas) / (batch * num_kv_heads > 0 ? batch * num_kv_heads : 1);
    return s < 1 ? 1 : (s > 64 ? 64 : s);
}

size_t generic_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim, int num_ctas) {
    const int pd = make_geom(head_dim, 0).padded;
    const size_t rows = (size_t)batch * generic_splits(batch, num_kv_heads, num_ctas, pd) * num_q_heads;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    return 256 + up(rows * sizeof(float)) + up(rows * pd * sizeof(float));
}

int generic_decode(const void* q, int q_dtype, int batch, int nq, int real_q_heads, int num_kv_heads, int head_dim,
                   const void* kv_cache, int64_t num_blocks, int block_size, int slot_bytes, const int32_t* page_indices,
                   const int32_t* page_indptr, int max_pages, const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                   const float* signs, float sm_scale, void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                   float* out_lse, int emit_rotated, int num_ctas, void* stream) {
    TQ_REQUIRE(head_dim > 32 && head_dim <= kGenMaxDim, TQ_ERR_UNSUPPORTED, "head_dim must be 33..%d, got %d", kGenMaxDim, head_dim);
    TQ_REQUIRE(block_size == kGenPage, TQ_ERR_UNSUPPORTED, "decode supports 16-token pages, got %d", block_size);
    TQ_REQUIRE(slot_bytes >= generic_slot_bytes(head_dim), TQ_ERR_INVALID, "slot_bytes %d is smaller than head size %d needs (%d)",
               slot_bytes, head_dim, generic_slot_bytes(head_dim));
    TQ_REQUIRE(nq >= 1 && num_kv_heads >= 1 && real_q_heads >= 1 && real_q_heads % num_kv_heads == 0, TQ_ERR_INVALID,
               "query heads must be a positive multiple of the KV heads, queries_per_seq >= 1");
    // the queries that share a sequence ride as extra columns of its KV heads
    const int num_q_heads = nq * real_q_heads;
    TQ_REQUIRE(num_q_heads / num_kv_heads <= kGenMaxGroup, TQ_ERR_UNSUPPORTED,
               "head size %d: queries_per_seq x query heads per KV head must be 1..%d, got %d x %d", head_dim, kGenMaxGroup, nq,
               real_q_heads / num_kv_heads);
    TQ_REQUIRE(kv_begin >= 0 && kv_begin % kGenPage == 0, TQ_ERR_INVALID, "kv_begin must be a multiple of 16");
    TQ_REQUIRE(page_indptr || max_pages > 0, TQ_ERR_INVALID, "max_pages must be positive for a dense block table");
    TQ_REQUIRE(num_blocks >= 1, TQ_ERR_INVALID, "the cache has no pages");
    TQ_REQUIRE(workspace_bytes >= generic_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, num_ctas), TQ_ERR_WORKSPACE,
               "workspace too small: %zu < %zu", workspace_bytes,
               generic_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, num_ctas));
    GenDecodeParams p{};
    p.g = make_geom(head_dim, slot_bytes);
    p.splits = generic_splits(batch, num_kv_heads, num_ctas, p.g.padded);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const size_t rows = (size_t)batch * p.splits * num_q_heads;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    p.header = reinterpret_cast<int32_t*>(ws);
    p.partial_lse = reinterpret_cast<float*>(ws + 256);
    p.partial_o = reinterpret_cast<float*>(ws + 256 + up(rows * sizeof(float)));
    p.q = q;
    p.kv_cache = static_cast<const uint8_t*>(kv_cache);
    p.page_indices = page_indices;
    p.page_indptr = page_indptr;
    p.seq_lens = seq_lens;
    p.signs = signs;
    p.slab_bytes = num_blocks * (int64_t)block_size * num_kv_heads * slot_bytes;
    p.num_blocks = num_blocks;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.batch = batch;
    p.num_q_heads = num_q_heads;
    p.num_kv_heads = num_kv_heads;
    p.group = num_q_heads / num_kv_heads;
    p.nq = nq;
    p.real_heads = real_q_heads;
    p.real_group = real_q_heads / num_kv_heads;
    p.max_pages = max_pages;
    p.q_dtype = q_dtype;
    p.score_scale = (float)((double)sm_scale * 1.4426950408889634);
    p.scale = (float)(1.0 / std::sqrt((double)p.g.padded));
    float bnd[15];
    host_codebook(p.g.padded, 4, p.centroids, bnd);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)(kGenMaxGroup * kGenMaxDim + kGenWarps * kGenMaxGroup * kGenMaxDim) * sizeof(float);
    static bool configured[64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(decode_generic_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TQ_CUDA(cudaFuncSetAttribute(decode_generic_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TQ_CUDA(cudaFuncSetAttribute(decode_generic_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const dim3 grid((unsigned)p.splits, (unsigned)batch, (unsigned)num_kv_heads);
    // the tensor-core kernel reads the codes with 16-byte loads; anything else keeps the plain one
    const bool aligned = slot_bytes % 16 == 0 && ((uintptr_t)kv_cache % 16) == 0 && p.slab_bytes % 16 == 0;
    if (aligned) {
        static bool frags_configured[64] = {};
        if (dev < 0 || dev >= 64 || !frags_configured[dev]) {
            TQ_CUDA(cudaFuncSetAttribute(decode_frags_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FragShape<64>::kSmem));
            TQ_CUDA(cudaFuncSetAttribute(decode_frags_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FragShape<128>::kSmem));
            TQ_CUDA(cudaFuncSetAttribute(decode_frags_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FragShape<256>::kSmem));
            if (dev >= 0 && dev < 64) frags_configured[dev] = true;
        }
        switch (p.g.padded) {
            case 64: decode_frags_kernel<64><<<grid, kGenWarps * 32, FragShape<64>::kSmem, s>>>(p); break;
            case 128: decode_frags_kernel<128><<<grid, kGenWarps * 32, FragShape<128>::kSmem, s>>>(p); break;
            default: decode_frags_kernel<256><<<grid, kGenWarps * 32, FragShape<256>::kSmem, s>>>(p); break;
        }
    } else {
        switch (p.g.qbytes / 32) {
            case 1: decode_generic_kernel<1><<<grid, kGenWarps * 32, smem, s>>>(p); break;
            case 2: decode_generic_kernel<2><<<grid, kGenWarps * 32, smem, s>>>(p); break;
            default: decode_generic_kernel<4><<<grid, kGenWarps * 32, smem, s>>>(p); break;
        }
    }
    TQ_CUDA(cudaGetLastError());
    GenMergeParams m{};
    m.partial_o = p.partial_o;
    m.partial_lse = p.partial_lse;
    m.signs = signs;
    m.out = out;
    m.out_lse = out_lse;
    m.num_q_heads = num_q_heads;
    m.nq = nq;
    m.real_heads = real_q_heads;
    m.real_group = p.real_group;
    m.group = p.group;
    m.splits = p.splits;
    m.out_dtype = out_dtype;
    m.emit_rotated = emit_rotated;
    m.g = p.g;
    m.scale = p.scale;
    merge_generic_kernel<<<(unsigned)batch * (unsigned)num_q_heads, p.g.padded, 0, s>>>(m);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

// partials of several KV windows, [parts][rows][padded] rotated + base-2 LSEs [parts][rows] -> out [rows][head_dim]
int generic_merge_rotated(const float* partial_o, const float* partial_lse2, int num_parts, int64_t rows, int head_dim,
                          const float* signs, void* out, int out_dtype, float* out_lse, void* stream) {
    TQ_REQUIRE(head_dim > 32 && head_dim <= kGenMaxDim, TQ_ERR_UNSUPPORTED, "head_dim must be 33..%d, got %d", kGenMaxDim, head_dim);
    TQ_REQUIRE(rows < (int64_t)1 << 31, TQ_ERR_UNSUPPORTED, "too many rows for one launch");
    GenMergeParams m{};
    m.partial_o = partial_o;
    m.partial_lse = partial_lse2;
    m.signs = signs;
    m.out = out;
    m.out_lse = out_lse;
    m.num_q_heads = (int)rows;   // one "sequence" whose parts are the windows: row (part, r) at part * rows + r
    m.nq = 1;
    m.real_heads = (int)rows;
    m.real_group = m.group = 1;
    m.splits = num_parts;
    m.out_dtype = out_dtype;
    m.emit_rotated = 0;
    m.g = make_geom(head_dim, 0);
    m.scale = (float)(1.0 / std::sqrt((double)m.g.padded));
    merge_generic_kernel<<<(unsigned)rows, m.g.padded, 0, static_cast<cudaStream_t>(stream)>>>(m);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

int generic_dequant(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads, int slot_bytes,
                    const int32_t* page_indices, const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                    const int32_t* cu_seqlens, int batch, const float* signs, int head_dim, void* k_out, void* v_out,
                    int out_dtype, int64_t out_token_stride, void* stream) {
    TQ_REQUIRE(head_dim > 32 && head_dim <= kGenMaxDim, TQ_ERR_UNSUPPORTED, "head_dim must be 33..%d, got %d", kGenMaxDim, head_dim);
    TQ_REQUIRE(block_size == kGenPage, TQ_ERR_UNSUPPORTED, "bulk dequantization supports 16-token pages, got %d", block_size);
    TQ_REQUIRE(slot_bytes >= generic_slot_bytes(head_dim), TQ_ERR_INVALID, "slot_bytes %d is smaller than head size %d needs", slot_bytes,
               head_dim);
    GenDequantParams p{};
    p.kv_cache = static_cast<const uint8_t*>(kv_cache);
    p.page_indices = page_indices;
    p.page_indptr = page_indptr;
    p.seq_lens = seq_lens;
    p.cu_seqlens = cu_seqlens;
    p.signs = signs;
    p.out[0] = k_out;
    p.out[1] = v_out;
    p.slab_bytes = num_blocks * (int64_t)block_size * num_kv_heads * slot_bytes;
    p.num_blocks = num_blocks;
    p.out_token_stride = out_token_stride;
    p.batch = batch;
    p.max_pages = max_pages;
    p.num_kv_heads = num_kv_heads;
    p.out_dtype = out_dtype;
    p.g = make_geom(head_dim, slot_bytes);
    p.scale = (float)(1.0 / std::sqrt((double)p.g.padded));
    float bnd[15];
    host_codebook(p.g.padded, 4, p.centroids, bnd);
    // large jobs: a lane group walks all rows of its token; small ones: a row per group, so that the few tokens
    // there are spread over many warps
    p.walk = (int64_t)batch * max_pages * kGenPage >= 16384 ? 2 * num_kv_heads : 1;
    const int64_t items = (int64_t)batch * max_pages * kGenPage * (2 * num_kv_heads / p.walk);
    const int64_t blocks = (items + 4 * kGenWarps - 1) / (4 * kGenWarps);   // four lane groups per warp and pass
    const unsigned grid = (unsigned)(blocks < 148 * 32 ? (blocks > 0 ? blocks : 1) : 148 * 32);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (p.g.padded) {
        case 64: dequant_rows8_kernel<8><<<grid, kGenWarps * 32, 0, s>>>(p); break;
        case 128: dequant_rows8_kernel<16><<<grid, kGenWarps * 32, 0, s>>>(p); break;
        default: dequant_rows8_kernel<32><<<grid, kGenWarps * 32, 0, s>>>(p); break;
    }
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

int generic_fault_counts(int32_t* write_dropped, int32_t* dequant_skipped) {
    TQ_CUDA(cudaMemcpyFromSymbol(write_dropped, g_gen_write_dropped, sizeof(int32_t)));
    TQ_CUDA(cudaMemcpyFromSymbol(dequant_skipped, g_gen_dequant_skipped, sizeof(int32_t)));
    return TQ_OK;
}

}  // namespace tq
