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
// vLLM), only the description above; these kernels follow that description: one warp per row for the
// store, a tensor-core decode on shared-memory tiles (one block per (split, sequence, KV head)), the
// split-KV partial / LSE contract of the other decode kernels.  They are a second wire format behind
// the same C ABI, without the staged copy pipelines of the tuned kernels.  Compiled with -fmad=false
// (quantizer arithmetic).
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

// butterflies h = 1 .. d/2 on a shared-memory row, by one warp: lane l takes elements l E .. l E + E - 1 (E = d / 32)
// into registers, runs the stages h < E there and the stages h >= E as one shuffle per element
template <int E>
__device__ __forceinline__ void nc_warp_fwht_regs(float* buf, int lane) {
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
    for (int m = 1; m < 32; m <<= 1) {
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
__device__ __forceinline__ void nc_warp_fwht(float* buf, int d, int lane) {
    if (d == 64) nc_warp_fwht_regs<2>(buf, lane);
    else if (d == 128) nc_warp_fwht_regs<4>(buf, lane);
    else nc_warp_fwht_regs<8>(buf, lane);
}

template <typename T>
__global__ void __launch_bounds__(kNcWarps * 32) write_nc_kernel(const __grid_constant__ NcWriteParams p) {
    __shared__ float buf_s[kNcWarps][kNcMaxDim];
    __shared__ uint8_t idx_s[kNcWarps][kNcMaxDim];
    __shared__ float bnd_s[16];
    if (threadIdx.x < 15) bnd_s[threadIdx.x] = p.boundaries[threadIdx.x];
    __syncthreads();
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
            // boundaries strictly below y (they ascend): a binary search over the shared copy
            int c = (bnd_s[7] < y) ? 8 : 0;
            c += (bnd_s[c + 3] < y) ? 4 : 0;
            c += (bnd_s[c + 1] < y) ? 2 : 0;
            c += (bnd_s[c] < y) ? 1 : 0;
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

// ---------------------------------------------------------------------------------------------
// decode: one block per (split, sequence, KV head); a warp takes whole pages.  Its 32 lanes load the
// page's code bytes (lane = token, half of the row; 16-bit loads, the slots being only 2-byte
// aligned), dequantize them into two small shared-memory tiles K^ and V^ ([16 tokens][PD dims] fp16,
// rows padded by 16 bytes) -- K through a byte-keyed table of centroid pairs, V as code * scale + zero
// in packed fp16 arithmetic -- and the products run as mma.sync.m16n8k16 on ldmatrix fragments:
// S = K^ Q^T (16 tokens x 8 query columns), O^T += V^^T P (PD dims x 8 columns, V^ read with
// ldmatrix.trans), P moved into place with movmatrix.  Online softmax in base 2 per page; the K norm
// is folded into the scores.  V was never rotated, so the partials are in the original domain.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t nct_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void nct_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void nct_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void nct_mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t nct_movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t nct_hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t nct_pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int PD>
struct NcTileShape {
    static constexpr int kRowBytes = (PD + 8) * 2;             // 16 mod 128: ldmatrix rows hit different banks
    static constexpr int kTileBytes = 16 * kRowBytes;
    static constexpr int kWords = PD / 16;                      // code words (4 bytes) per lane and operand
    static constexpr size_t kSmem = (size_t)kNcMaxGroup * PD * 4 + (size_t)kNcWarps * 2 * kTileBytes;
};

template <int PD>
__global__ void __launch_bounds__(kNcWarps * 32, PD == 256 ? 2 : 4) decode_nc_tiles_kernel(const __grid_constant__ NcDecodeParams p) {
    using T = NcTileShape<PD>;
    extern __shared__ __align__(16) uint8_t tsm[];
    __shared__ float m_s[kNcWarps][kNcMaxGroup], l_s[kNcWarps][kNcMaxGroup];
    __shared__ uint32_t lut_s[256];          // K code byte -> (centroid of the even dim = low nibble, of the odd dim) as half2
    __shared__ uint32_t lutv_s[256];         // V code byte -> (low nibble, high nibble) as half2 numbers 0..15
    __shared__ float nk_s[kNcWarps][16];
    constexpr int pd = PD;
    const int G = p.group;
    float* q_s = reinterpret_cast<float*>(tsm);                          // [G][pd] rotated queries
    uint8_t* tiles = tsm + (size_t)kNcMaxGroup * PD * 4;
    float* o_s = reinterpret_cast<float*>(tiles);                        // [warps][G][pd], after the loop
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int split = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    for (int v = tid; v < 256; v += blockDim.x) {
        lut_s[v] = nct_pack_half2(p.centroids[v & 15], p.centroids[v >> 4]);
        lutv_s[v] = nct_pack_half2((float)(v & 15), (float)(v >> 4));
    }

    // window of this split, in pages
    const int64_t len = p.seq_lens[b];
    const int64_t begin = 0;
    const int first_page = 0;
    int npages = (int)((len + kNcPage - 1) / kNcPage);
    const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
    const int have = p.page_indptr ? p.page_indptr[b + 1] - p.page_indptr[b] : p.max_pages;
    if (npages > have) {  // the table cannot back this length: read nothing
        if (tid == 0) atomicExch(&p.header[0], 4);
        npages = 0;
    }
    const int per = (npages + p.splits - 1) / p.splits;
    const int pg0 = first_page + split * per;
    const int pg1 = min(first_page + npages, pg0 + per);

    // rotate the group's queries: signs, butterflies, 1/sqrt(pd)
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int gg = i / pd, d = i - gg * pd;
        q_s[i] = nc_load(p.q, p.q_dtype, ((int64_t)b * p.num_q_heads + h * G + gg) * pd + d);
    }
    __syncthreads();
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
    // B fragments of Q^T: column g of the query tile (zero beyond the group), k-steps of 16 dims
    uint32_t qf[PD / 8];
#pragma unroll
    for (int s = 0; s < PD / 16; s++) {
        const float* row = q_s + g * pd + 16 * s + 2 * tg;
        const bool on = g < G;
        qf[2 * s] = on ? nct_pack_half2(row[0] * p.scale, row[1] * p.scale) : 0u;
        qf[2 * s + 1] = on ? nct_pack_half2(row[8] * p.scale, row[9] * p.scale) : 0u;
    }

    float o_acc[PD / 16][4];
#pragma unroll
    for (int i = 0; i < PD / 16; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o_acc[i][j] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const int tk = lane >> 1, hf = lane & 1;                       // loads: lane = (token, half of its code bytes)
    const uint32_t tile_k = nct_smem_u32(tiles) + (uint32_t)warp * 2 * T::kTileBytes, tile_v = tile_k + T::kTileBytes;
    const uint32_t st_k = tile_k + tk * T::kRowBytes + hf * PD, st_v = tile_v + tk * T::kRowBytes + hf * PD;
    const uint32_t lm_k = tile_k + (lane & 15) * T::kRowBytes + (lane >> 4) * 16;
    const uint32_t lm_v = tile_v + ((lane & 7) + 8 * (lane >> 4)) * T::kRowBytes + ((lane >> 3) & 1) * 16;
    bool bad_page = false;
    for (int pg = pg0 + warp; pg < pg1; pg += kNcWarps) {
        const int64_t page = p.page_indices[tbl + pg];
        if ((uint64_t)page >= (uint64_t)p.num_blocks) {  // never form an address from it
            bad_page = true;
            continue;
        }
        // ---- load and dequantize the page's codes into the two tiles ---------------------------------
        const uint8_t* ks = p.kv_cache + ((size_t)(page * kNcPage + tk) * p.num_kv_heads + h) * p.g.slot_bytes;
        const uint8_t* vs = ks + p.g.kps;
        // the slots of this format are only 2-byte aligned: 16-bit loads, two per code word
        uint4 kc[PD / 64], vc[PD / 64];
        {
            const uint16_t* k16 = reinterpret_cast<const uint16_t*>(ks + hf * (PD / 4));
            const uint16_t* v16 = reinterpret_cast<const uint16_t*>(vs + hf * (PD / 4));
            uint32_t* kd = reinterpret_cast<uint32_t*>(kc);
            uint32_t* vd = reinterpret_cast<uint32_t*>(vc);
#pragma unroll
            for (int i = 0; i < PD / 16; i++) {
                kd[i] = (uint32_t)k16[2 * i] | ((uint32_t)k16[2 * i + 1] << 16);
                vd[i] = (uint32_t)v16[2 * i] | ((uint32_t)v16[2 * i + 1] << 16);
            }
        }
        // (scale, scale) and (zero, zero) of this lane's token, as half2
        const uint32_t sc16 = *reinterpret_cast<const uint16_t*>(vs + p.g.qbytes), ze16 = *reinterpret_cast<const uint16_t*>(vs + p.g.qbytes + 2);
        const uint32_t vsz = sc16 | (sc16 << 16), vzz = ze16 | (ze16 << 16);
        if (hf == 0) nk_s[warp][tk] = __half2float(*reinterpret_cast<const __half*>(ks + p.g.qbytes));
#pragma unroll
        for (int i = 0; i < PD / 64; i++) {
            const uint32_t kw[4] = {kc[i].x, kc[i].y, kc[i].z, kc[i].w}, vw[4] = {vc[i].x, vc[i].y, vc[i].z, vc[i].w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t a[4], c[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    a[j] = lut_s[(kw[w] >> (8 * j)) & 0xFF];
                    c[j] = nct_hfma2(lutv_s[(vw[w] >> (8 * j)) & 0xFF], vsz, vzz);   // code * scale + zero
                }
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(st_k + (4 * i + w) * 16), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(st_v + (4 * i + w) * 16), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]) : "memory");
            }
        }
        __syncwarp();
        // ---- S = K^ Q^T ----------------------------------------------------------------------------------
        float s_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int s = 0; s < PD / 16; s++) {
            uint32_t a[4];
            nct_ldmatrix_x4(lm_k + s * 32, a);
            nct_mma16816(s_acc, a, qf[2 * s], qf[2 * s + 1]);
        }
        // ---- online softmax (base 2); rows g and g + 8 are tokens, columns 2tg and 2tg + 1 query heads -----
        const int64_t t0 = (int64_t)pg * kNcPage;
        const bool va = t0 + g >= begin && t0 + g < len, vb = t0 + g + 8 >= begin && t0 + g + 8 < len;
        const float kfa = va ? nk_s[warp][g] * p.score_scale : 0.0f, kfb = vb ? nk_s[warp][g + 8] * p.score_scale : 0.0f;
        const float x0 = va ? s_acc[0] * kfa : -INFINITY, x1 = va ? s_acc[1] * kfa : -INFINITY;
        const float x2 = vb ? s_acc[2] * kfb : -INFINITY, x3 = vb ? s_acc[3] * kfb : -INFINITY;
        float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float c0 = n0 > m0 ? nc_exp2(m0 - n0) : 1.0f, c1 = n1 > m1 ? nc_exp2(m1 - n1) : 1.0f;
        m0 = n0;
        m1 = n1;
        const float e0 = va ? nc_exp2(x0 - m0) : 0.0f, e1 = va ? nc_exp2(x1 - m1) : 0.0f;
        const float e2 = vb ? nc_exp2(x2 - m0) : 0.0f, e3 = vb ? nc_exp2(x3 - m1) : 0.0f;
        l0 = __fmaf_rn(l0, c0, e0 + e2);
        l1 = __fmaf_rn(l1, c1, e1 + e3);
        const uint32_t pb0 = nct_movmatrix_trans(nct_pack_half2(e0, e1));
        const uint32_t pb1 = nct_movmatrix_trans(nct_pack_half2(e2, e3));
        // ---- O^T += V^^T P ------------------------------------------------------------------------------------
#pragma unroll
        for (int mt = 0; mt < PD / 16; mt++) {
            uint32_t a[4];
            nct_ldmatrix_x4_trans(lm_v + mt * 32, a);
            o_acc[mt][0] *= c0; o_acc[mt][1] *= c1; o_acc[mt][2] *= c0; o_acc[mt][3] *= c1;
            nct_mma16816(o_acc[mt], a, pb0, pb1);
        }
        __syncwarp();   // the tiles are rewritten by the next page
    }
    if (bad_page && lane == 0) atomicExch(&p.header[0], 5);
    // this warp's sums over its token lanes, then everything to shared memory for the block's combine
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    __syncthreads();   // every warp has left its tiles: the region becomes o_s
    if (g == 0) {
        if (2 * tg < G) { m_s[warp][2 * tg] = m0; l_s[warp][2 * tg] = l0; }
        if (2 * tg + 1 < G) { m_s[warp][2 * tg + 1] = m1; l_s[warp][2 * tg + 1] = l1; }
    }
#pragma unroll
    for (int mt = 0; mt < PD / 16; mt++) {
        const int d0 = 16 * mt + g;
        if (2 * tg < G) {
            o_s[(warp * G + 2 * tg) * pd + d0] = o_acc[mt][0];
            o_s[(warp * G + 2 * tg) * pd + d0 + 8] = o_acc[mt][2];
        }
        if (2 * tg + 1 < G) {
            o_s[(warp * G + 2 * tg + 1) * pd + d0] = o_acc[mt][1];
            o_s[(warp * G + 2 * tg + 1) * pd + d0 + 8] = o_acc[mt][3];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * pd; i += blockDim.x) {
        const int gg = i / pd, d = i - gg * pd;
        float mm = -INFINITY;
        for (int w = 0; w < kNcWarps; w++) mm = fmaxf(mm, m_s[w][gg]);
        float ll = 0.0f, acc = 0.0f;
        if (mm > -INFINITY) {
            for (int w = 0; w < kNcWarps; w++) {
                const float sc = nc_exp2(m_s[w][gg] - mm);
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
    static bool configured[64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_tiles_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NcTileShape<64>::kSmem));
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_tiles_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NcTileShape<128>::kSmem));
        TQ_CUDA(cudaFuncSetAttribute(decode_nc_tiles_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NcTileShape<256>::kSmem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const dim3 grid((unsigned)p.splits, (unsigned)batch, (unsigned)num_kv_heads);
    switch (head_dim) {
        case 64: decode_nc_tiles_kernel<64><<<grid, kNcWarps * 32, NcTileShape<64>::kSmem, s>>>(p); break;
        case 128: decode_nc_tiles_kernel<128><<<grid, kNcWarps * 32, NcTileShape<128>::kSmem, s>>>(p); break;
        default: decode_nc_tiles_kernel<256><<<grid, kNcWarps * 32, NcTileShape<256>::kSmem, s>>>(p); break;
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
