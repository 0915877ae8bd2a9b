// The slot format of vLLM's native TurboQuant backend ("turboquant_4bit_nc"), as the reference
// documents it (docs/reference/vllm-upstream-turboquant-architecture.md:33-94 layout, :100-175
// store, :178-240 decode): ONE cache tensor [num_blocks][block_size][kv_heads][slot], and per slot
//
//     [ K codes: d/2 bytes | ||k|| fp16 | V codes: d/2 bytes | V scale fp16 | V zero fp16 ]
//
// (134 bytes for d = 128; no 16-byte alignment, so no bulk copies here).  K is quantized as in this
// project's own format but WITHOUT the sign vector, with x / (||x|| + 1e-8) instead of a clamped
// norm, and with the EVEN dim in the LOW nibble; V is a uniform 4-bit quantizer on the raw values:
// scale = (max - min) / 15, code = clamp(trunc((v - min) / scale + 1/2), 0, 15), zero = min, and
// dequantizes to code * scale + zero in the original domain (no rotation on the V side).
//
// The reference repository holds no code for this format (upstream's kernels are Triton inside
// vLLM), only the description above; these kernels follow that description with plain CUDA: one
// warp per row for the store, one block per (split, sequence, KV head) for the decode, the split-KV
// partial / LSE contract of the other decode kernels.  They are a second wire format behind the
// same C ABI, not tuned for bandwidth.  Compiled with -fmad=false (quantizer arithmetic).
#include <cmath>
#include <cstring>

#include "tq_common.cuh"

namespace tq {

constexpr int kNcMaxDim = 256;
constexpr int kNcWarps = 4;
constexpr int kNcMaxGroup = 8;
constexpr int kNcPage = 16;

struct NcGeom {
    int d, qbytes, kps, slot_bytes;   // head size (64, 128, 256), code bytes, offset of the V part
};

static NcGeom nc_geom(int head_dim, int slot_bytes) {
    NcGeom g;
    g.d = head_dim;
    g.qbytes = head_dim / 2;
    g.kps = g.qbytes + 2;
    g.slot_bytes = slot_bytes;
    return g;
}

int nc_slot_bytes(int head_dim) { return ((head_dim / 2 + 2) + (head_dim / 2 + 4) + 1) & ~1; }

static __device__ int32_t g_nc_write_dropped = 0;

struct NcWriteParams {
    uint8_t* kv_cache;
    const void* src[2];
    int64_t token_stride[2];
    const void* slot_mapping;
    int64_t num_tokens, total_slots;
    int num_kv_heads, slot_is_i64;
    NcGeom g;
    float scale;            // 1 / sqrt(d)
    float boundaries[15];   // Lloyd-Max boundaries of N(0, 1/d)
};

__device__ __forceinline__ void nc_warp_fwht(float* buf, int d, int lane) {
    for (int h = 1; h < d; h <<= 1) {
        for (int idx = lane; idx < d / 2; idx += 32) {
            const int i = (idx / h) * 2 * h + (idx % h);
            const float a = buf[i], b = buf[i + h];
            buf[i] = __fadd_rn(a, b);
            buf[i + h] = __fsub_rn(a, b);
        }
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(kNcWarps * 32) write_nc_kernel(const __grid_constant__ NcWriteParams p) {
    __shared__ float buf_s[kNcWarps][kNcMaxDim];
    __shared__ uint8_t idx_s[kNcWarps][kNcMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = buf_s[warp];
    uint8_t* idx = idx_s[warp];
    const int H = p.num_kv_heads, d = p.g.d;
    const int64_t rows = p.num_tokens * H;
    for (int64_t r = (int64_t)blockIdx.x * kNcWarps + warp; r < rows; r += (int64_t)gridDim.x * kNcWarps) {
        const int64_t t = r / H;
        const int h = (int)(r - t * H);
        int64_t slot = p.slot_is_i64 ? reinterpret_cast<const int64_t*>(p.slot_mapping)[t]
                                     : (int64_t) reinterpret_cast<const int32_t*>(p.slot_mapping)[t];
        if (slot >= p.total_slots) {   // never store through an id outside the cache
            if (lane == 0 && h == 0) atomicAdd(&g_nc_write_dropped, 1);
            slot = -1;
        }
        if (slot < 0) continue;
        uint8_t* dst = p.kv_cache + ((size_t)slot * H + h) * p.g.slot_bytes;
        // ---- K: norm, x / (norm + 1e-8), Hadamard / sqrt(d), nearest centroid ----------------------
        const T* krow = reinterpret_cast<const T*>(p.src[0]) + t * p.token_stride[0] + (int64_t)h * d;
        for (int i = lane; i < d; i += 32) buf[i] = to_f32(krow[i]);
        __syncwarp();
        float acc = 0.0f;   // eight interleaved accumulators, combined left to right (the order of the other formats)
        if (lane < 8)
            for (int j = lane; j < d; j += 8) acc = __fadd_rn(acc, __fmul_rn(buf[j], buf[j]));
        float s = 0.0f;
        for (int k = 0; k < 8; k++) {
            const float a = __shfl_sync(0xffffffffu, acc, k);
            s = k == 0 ? a : __fadd_rn(s, a);
        }
        const float norm = __fsqrt_rn(s);
        const float den = __fadd_rn(norm, 1e-8f);
        for (int i = lane; i < d; i += 32) buf[i] = __fdiv_rn(buf[i], den);
        __syncwarp();
        nc_warp_fwht(buf, d, lane);
        for (int i = lane; i < d; i += 32) {
            const float y = __fmul_rn(buf[i], p.scale);
            int c = 0;
            for (int k = 0; k < 15; k++) c += (p.boundaries[k] < y) ? 1 : 0;
            if (y != y) c = 15;
            idx[i] = (uint8_t)c;
        }
        __syncwarp();
        for (int b = lane; b < p.g.qbytes; b += 32) dst[b] = (uint8_t)(idx[2 * b] | (idx[2 * b + 1] << 4));
        // (slot sizes are even and the cache is 2-byte aligned: the fp16 fields take 16-bit stores)
        if (lane == 0) *reinterpret_cast<__half*>(dst + p.g.qbytes) = __float2half_rn(norm);
        __syncwarp();
        // ---- V: uniform 4-bit between the row's minimum and maximum --------------------------------
        const T* vrow = reinterpret_cast<const T*>(p.src[1]) + t * p.token_stride[1] + (int64_t)h * d;
        float mn = INFINITY, mx = -INFINITY;
        for (int i = lane; i < d; i += 32) {
            const float v = to_f32(vrow[i]);
            buf[i] = v;
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        __syncwarp();
        const float vs = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        for (int i = lane; i < d; i += 32) {
            float qv = vs > 0.0f ? __fadd_rn(__fdiv_rn(__fsub_rn(buf[i], mn), vs), 0.5f) : 0.0f;   // a constant row: code 0
            qv = fminf(fmaxf(qv, 0.0f), 15.0f);
            idx[i] = (uint8_t)(int)qv;   // truncation, as the store kernel of the description does
        }
        __syncwarp();
        uint8_t* vdst = dst + p.g.kps;
        for (int b = lane; b < p.g.qbytes; b += 32) vdst[b] = (uint8_t)(idx[2 * b] | (idx[2 * b + 1] << 4));
        if (lane == 0) {
            *reinterpret_cast<__half*>(vdst + p.g.qbytes) = __float2half_rn(vs);
            *reinterpret_cast<__half*>(vdst + p.g.qbytes + 2) = __float2half_rn(mn);
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
// decode: one block per (split, sequence, KV head), four warps striding over the split's tokens
// ---------------------------------------------------------------------------------------------
struct NcDecodeParams {
    const void* q;
    const uint8_t* kv_cache;
    const int32_t* page_indices;
    const int32_t* page_indptr;
    const int32_t* seq_lens;
    int32_t* header;       // workspace word 0: sticky status (4: sequence longer than its table, 5: bad page id)
    float* partial_lse;    // [batch][splits][num_q_heads], base 2
    float* partial_o;      // [batch][splits][num_q_heads][d], normalized, ORIGINAL domain
    int64_t num_blocks;
    int batch, num_q_heads, num_kv_heads, group, max_pages, q_dtype, splits;
    NcGeom g;
    float score_scale;     // sm_scale * log2(e)
    float scale;           // 1 / sqrt(d)
    float centroids[16];   // of N(0, 1/d)
};

__device__ __forceinline__ float nc_load(const void* q, int dtype, int64_t i) {
    if (dtype == TQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]);
    if (dtype == TQ_F16) return __half2float(reinterpret_cast<const __half*>(q)[i]);
    return reinterpret_cast<const float*>(q)[i];
}
// 2^x, hardware approximation (2 ulp), exp2(-inf) = 0
__device__ __forceinline__ float nc_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float nc_half_at(const uint8_t* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

// BPL = code bytes per lane and token: 1, 2 or 4 for head sizes 64, 128, 256.  (This file is compiled without FMA
// contraction for the quantizer's sake; the attention arithmetic asks for its FMAs explicitly.)
template <int BPL>
__global__ void __launch_bounds__(kNcWarps * 32, 4) decode_nc_kernel(const __grid_constant__ NcDecodeParams p) {
    extern __shared__ float ncsm[];
    const int d = p.g.d, G = p.group;
    float* q_s = ncsm;                             // [G][d] rotated queries
    float* o_s = ncsm + kNcMaxGroup * kNcMaxDim;   // [warps][G][d]
    __shared__ float m_s[kNcWarps][kNcMaxGroup], l_s[kNcWarps][kNcMaxGroup];
    __shared__ float cent_s[16];   // a lookup indexed per lane: shared memory, not the parameter bank
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    if (tid < 16) cent_s[tid] = p.centroids[tid];

    const int64_t len = p.seq_lens[b];
    int npages = (int)((len + kNcPage - 1) / kNcPage);
    const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
    const int have = p.page_indptr ? p.page_indptr[b + 1] - p.page_indptr[b] : p.max_pages;
    if (npages > have) {   // the table cannot back this length: read nothing
        if (tid == 0) atomicExch(&p.header[0], 4);
        npages = 0;
    }
    const int per = (npages + p.splits - 1) / p.splits;
    const int pg0 = split * per;
    const int pg1 = min(npages, pg0 + per);

    // rotate the group's queries: q H / sqrt(d), no signs in this format
    for (int i = tid; i < G * d; i += blockDim.x) {
        const int g = i / d, e = i - g * d;
        q_s[i] = nc_load(p.q, p.q_dtype, ((int64_t)b * p.num_q_heads + h * G + g) * d + e);
    }
    __syncthreads();
    for (int hh = 1; hh < d; hh <<= 1) {
        for (int i = tid; i < G * d / 2; i += blockDim.x) {
            const int g = i / (d / 2), idx = i - g * (d / 2);
            const int j = (idx / hh) * 2 * hh + (idx % hh);
            float* row = q_s + g * d;
            const float a = row[j], c = row[j + hh];
            row[j] = a + c;
            row[j + hh] = a - c;
        }
        __syncthreads();
    }
    for (int i = tid; i < G * d; i += blockDim.x) q_s[i] *= p.scale;
    __syncthreads();

    float m[kNcMaxGroup], l[kNcMaxGroup], o[kNcMaxGroup][2 * BPL];
#pragma unroll
    for (int g = 0; g < kNcMaxGroup; g++) {
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
        float kn[4], vsc[4], vz[4];
        bool tv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = warp + kNcWarps * i;
            const int64_t t = (int64_t)pg * kNcPage + e;
            tv[i] = t < len;
            kn[i] = vsc[i] = vz[i] = 0.0f;
#pragma unroll
            for (int j = 0; j < BPL; j++) kb[i][j] = vb[i][j] = 0;
            if (tv[i]) {
                const uint8_t* ks = p.kv_cache + ((size_t)(page * kNcPage + e) * p.num_kv_heads + h) * p.g.slot_bytes;
                const uint8_t* vs = ks + p.g.kps;
#pragma unroll
                for (int j = 0; j < BPL; j++) {
                    kb[i][j] = ks[lane + 32 * j];
                    vb[i][j] = vs[lane + 32 * j];
                }
                kn[i] = nc_half_at(ks + p.g.qbytes);
                vsc[i] = nc_half_at(vs + p.g.qbytes);
                vz[i] = nc_half_at(vs + p.g.qbytes + 2);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (!tv[i]) continue;
            float kd[2 * BPL], vd[2 * BPL];
#pragma unroll
            for (int j = 0; j < BPL; j++) {   // the even dim sits in the low nibble
                kd[2 * j] = cent_s[kb[i][j] & 15] * kn[i];
                kd[2 * j + 1] = cent_s[kb[i][j] >> 4] * kn[i];
                vd[2 * j] = __fmaf_rn((float)(vb[i][j] & 15), vsc[i], vz[i]);
                vd[2 * j + 1] = __fmaf_rn((float)(vb[i][j] >> 4), vsc[i], vz[i]);
            }
#pragma unroll
            for (int g = 0; g < kNcMaxGroup; g++) {
                if (g >= G) break;
                const float* qr = q_s + g * d;
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
                const float corr = nc_exp2(m[g] - m_new), w = nc_exp2(sc - m_new);
                m[g] = m_new;
                l[g] = __fmaf_rn(l[g], corr, w);
#pragma unroll
                for (int e2 = 0; e2 < 2 * BPL; e2++) o[g][e2] = __fmaf_rn(w, vd[e2], o[g][e2] * corr);
            }
        }
    }
    if (bad_page && lane == 0) atomicExch(&p.header[0], 5);
#pragma unroll
    for (int g = 0; g < kNcMaxGroup; g++) {
        if (g >= G) break;
        if (lane == 0) {
            m_s[warp][g] = m[g];
            l_s[warp][g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < BPL; j++) {
            const int e2 = 2 * (lane + 32 * j);
            o_s[(warp * G + g) * d + e2] = o[g][2 * j];
            o_s[(warp * G + g) * d + e2 + 1] = o[g][2 * j + 1];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * d; i += blockDim.x) {
        const int g = i / d, e = i - g * d;
        float mm = -INFINITY;
        for (int w = 0; w < kNcWarps; w++) mm = fmaxf(mm, m_s[w][g]);
        float ll = 0.0f, acc = 0.0f;
        if (mm > -INFINITY) {
            for (int w = 0; w < kNcWarps; w++) {
                const float sc = exp2f(m_s[w][g] - mm);
                if (sc > 0.0f) {
                    ll += sc * l_s[w][g];
                    acc += sc * o_s[(w * G + g) * d + e];
                }
            }
        }
        const int64_t row = ((int64_t)b * p.splits + split) * p.num_q_heads + h * G + g;
        p.partial_o[row * d + e] = ll > 0.0f ? acc / ll : 0.0f;
        if (e == 0) p.partial_lse[row] = ll > 0.0f ? mm + log2f(ll) : -INFINITY;
    }
}

struct NcMergeParams {
    const float* partial_o;
    const float* partial_lse;
    void* out;
    float* out_lse;
    int num_q_heads, splits, out_dtype, d;
};

// one block of d threads per (sequence, query head); V was never rotated, so there is nothing to undo
__global__ void __launch_bounds__(kNcMaxDim) merge_nc_kernel(const __grid_constant__ NcMergeParams p) {
    const int e = threadIdx.x, d = p.d;
    const int64_t b = blockIdx.x;
    const int hq = blockIdx.y;
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; s++) mm = fmaxf(mm, p.partial_lse[(b * p.splits + s) * p.num_q_heads + hq]);
    float wsum = 0.0f, acc = 0.0f;
    if (mm > -INFINITY) {
        for (int s = 0; s < p.splits; s++) {
            const int64_t row = (b * p.splits + s) * p.num_q_heads + hq;
            const float w = exp2f(p.partial_lse[row] - mm);
            if (w > 0.0f) {
                wsum += w;
                acc += w * p.partial_o[row * d + e];
            }
        }
    }
    const float o = wsum > 0.0f ? acc / wsum : 0.0f;
    const int64_t at = (b * p.num_q_heads + hq) * d + e;
    if (p.out_dtype == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(o);
    else if (p.out_dtype == TQ_F16) reinterpret_cast<__half*>(p.out)[at] = __float2half_rn(o);
    else reinterpret_cast<float*>(p.out)[at] = o;
    if (p.out_lse && e == 0) p.out_lse[b * p.num_q_heads + hq] = wsum > 0.0f ? (mm + log2f(wsum)) * 0.6931471805599453f : -INFINITY;
}

int device_sm_count(int* out);   // tq_api.cu

static int nc_splits(int batch, int num_kv_heads, int num_ctas) {
    int ctas = num_ctas;
    if (ctas <= 0 && device_sm_count(&ctas) != TQ_OK) ctas = 148;
    const int s = (4 * ctas) / (batch * num_kv_heads > 0 ? batch * num_kv_heads : 1);
    return s < 1 ? 1 : (s > 64 ? 64 : s);
}

static bool nc_head_dim_ok(int head_dim) { return head_dim == 64 || head_dim == 128 || head_dim == 256; }

}  // namespace tq

using namespace tq;

extern "C" int tq_nc_slot_bytes(int head_dim) { return nc_head_dim_ok(head_dim) ? nc_slot_bytes(head_dim) : 0; }

extern "C" int tq_nc_write_kv_cache(const void* key, const void* value, int in_dtype, int64_t num_tokens, int num_kv_heads,
                                    int head_dim, int64_t k_token_stride, int64_t v_token_stride, void* kv_cache,
                                    int64_t num_blocks, int block_size, int slot_bytes, const void* slot_mapping,
                                    int slot_dtype, void* stream) {
    TQ_REQUIRE(num_tokens >= 0, TQ_ERR_INVALID, "negative num_tokens");
    if (num_tokens == 0) return TQ_OK;
    TQ_REQUIRE(key && value && kv_cache && slot_mapping, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(nc_head_dim_ok(head_dim), TQ_ERR_UNSUPPORTED, "head_dim must be 64, 128 or 256 (a Hadamard size), got %d", head_dim);
    TQ_REQUIRE(in_dtype >= TQ_F32 && in_dtype <= TQ_BF16, TQ_ERR_INVALID, "bad input dtype");
    TQ_REQUIRE(slot_dtype == TQ_I32 || slot_dtype == TQ_I64, TQ_ERR_INVALID, "slot_mapping must be int32 or int64");
    TQ_REQUIRE(num_kv_heads >= 1 && num_blocks >= 1 && block_size >= 1, TQ_ERR_INVALID, "bad cache geometry");
    TQ_REQUIRE(slot_bytes >= nc_slot_bytes(head_dim) && slot_bytes % 2 == 0 && ((uintptr_t)kv_cache % 2) == 0, TQ_ERR_INVALID,
               "slot_bytes %d must be even and at least %d for head size %d; the cache 2-byte aligned", slot_bytes,
               nc_slot_bytes(head_dim), head_dim);
    NcWriteParams p{};
    p.kv_cache = static_cast<uint8_t*>(kv_cache);
    p.src[0] = key;
    p.src[1] = value;
    p.token_stride[0] = k_token_stride;
    p.token_stride[1] = v_token_stride;
    p.slot_mapping = slot_mapping;
    p.num_tokens = num_tokens;
    p.total_slots = num_blocks * (int64_t)block_size;
    p.num_kv_heads = num_kv_heads;
    p.slot_is_i64 = slot_dtype == TQ_I64;
    p.g = nc_geom(head_dim, slot_bytes);
    p.scale = (float)(1.0 / std::sqrt((double)head_dim));
    float cen[16];
    host_codebook(head_dim, 4, cen, p.boundaries);
    const int64_t rows = num_tokens * num_kv_heads;
    const int64_t blocks = (rows + kNcWarps - 1) / kNcWarps;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case TQ_F32: write_nc_kernel<float><<<grid, kNcWarps * 32, 0, s>>>(p); break;
        case TQ_F16: write_nc_kernel<__half><<<grid, kNcWarps * 32, 0, s>>>(p); break;
        default: write_nc_kernel<__nv_bfloat16><<<grid, kNcWarps * 32, 0, s>>>(p); break;
    }
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

extern "C" size_t tq_nc_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim, int num_ctas) {
    if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || !nc_head_dim_ok(head_dim)) return 0;
    const size_t rows = (size_t)batch * nc_splits(batch, num_kv_heads, num_ctas) * num_q_heads;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    return 256 + up(rows * sizeof(float)) + up(rows * head_dim * sizeof(float));
}

extern "C" int tq_nc_decode_paged(const void* q, int q_dtype, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                  const void* kv_cache, int64_t num_blocks, int block_size, int slot_bytes,
                                  const int32_t* page_indices, const int32_t* page_indptr, int max_pages,
                                  const int32_t* seq_lens, float sm_scale, void* workspace, size_t workspace_bytes,
                                  void* out, int out_dtype, float* out_lse, int num_ctas, void* stream) {
    TQ_REQUIRE(batch >= 0, TQ_ERR_INVALID, "negative batch");
    if (batch == 0) return TQ_OK;
    TQ_REQUIRE(q && kv_cache && page_indices && seq_lens && workspace && out, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(nc_head_dim_ok(head_dim), TQ_ERR_UNSUPPORTED, "head_dim must be 64, 128 or 256 (a Hadamard size), got %d", head_dim);
    TQ_REQUIRE(block_size == kNcPage, TQ_ERR_UNSUPPORTED, "decode supports 16-token pages, got %d", block_size);
    TQ_REQUIRE(slot_bytes >= nc_slot_bytes(head_dim) && slot_bytes % 2 == 0 && ((uintptr_t)kv_cache % 2) == 0, TQ_ERR_INVALID,
               "slot_bytes %d must be even and at least %d for head size %d; the cache 2-byte aligned", slot_bytes,
               nc_slot_bytes(head_dim), head_dim);
    TQ_REQUIRE(num_kv_heads >= 1 && num_q_heads % num_kv_heads == 0 && num_q_heads / num_kv_heads <= kNcMaxGroup,
               TQ_ERR_UNSUPPORTED, "query heads per KV head must be 1..%d", kNcMaxGroup);
    TQ_REQUIRE(q_dtype >= TQ_F32 && q_dtype <= TQ_BF16 && out_dtype >= TQ_F32 && out_dtype <= TQ_BF16, TQ_ERR_INVALID, "bad dtype");
    TQ_REQUIRE(page_indptr || max_pages > 0, TQ_ERR_INVALID, "max_pages must be positive for a dense block table");
    TQ_REQUIRE(num_blocks >= 1, TQ_ERR_INVALID, "the cache has no pages");
    TQ_REQUIRE(((uintptr_t)workspace % 256) == 0, TQ_ERR_INVALID, "workspace must be 256-byte aligned");
    const size_t need = tq_nc_decode_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, num_ctas);
    TQ_REQUIRE(workspace_bytes >= need, TQ_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, need);
    NcDecodeParams p{};
    p.g = nc_geom(head_dim, slot_bytes);
    p.splits = nc_splits(batch, num_kv_heads, num_ctas);
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
    p.num_blocks = num_blocks;
    p.batch = batch;
    p.num_q_heads = num_q_heads;
    p.num_kv_heads = num_kv_heads;
    p.group = num_q_heads / num_kv_heads;
    p.max_pages = max_pages;
    p.q_dtype = q_dtype;
    p.score_scale = (float)((double)sm_scale * 1.4426950408889634);
    p.scale = (float)(1.0 / std::sqrt((double)head_dim));
    float bnd[15];
    host_codebook(head_dim, 4, p.centroids, bnd);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)(kNcMaxGroup * kNcMaxDim + kNcWarps * kNcMaxGroup * kNcMaxDim) * sizeof(float);
    static bool configured[64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const dim3 grid((unsigned)p.splits, (unsigned)batch, (unsigned)num_kv_heads);
    switch (head_dim / 64) {
        case 1: decode_nc_kernel<1><<<grid, kNcWarps * 32, smem, s>>>(p); break;
        case 2: decode_nc_kernel<2><<<grid, kNcWarps * 32, smem, s>>>(p); break;
        default: decode_nc_kernel<4><<<grid, kNcWarps * 32, smem, s>>>(p); break;
    }
    TQ_CUDA(cudaGetLastError());
    NcMergeParams m{};
    m.partial_o = p.partial_o;
    m.partial_lse = p.partial_lse;
    m.out = out;
    m.out_lse = out_lse;
    m.num_q_heads = num_q_heads;
    m.splits = p.splits;
    m.out_dtype = out_dtype;
    m.d = head_dim;
    merge_nc_kernel<<<dim3((unsigned)batch, (unsigned)num_q_heads), head_dim, 0, s>>>(m);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

extern "C" int tq_nc_write_dropped(int32_t* count) {
    TQ_REQUIRE(count, TQ_ERR_INVALID, "null pointer");
    TQ_CUDA(cudaMemcpyFromSymbol(count, g_nc_write_dropped, sizeof(int32_t)));
    return TQ_OK;
}
