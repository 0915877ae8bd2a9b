// Flat (non-paged) quantizer API kernels: TurboQuantMSE.quantize / dequantize and the
// Walsh-Hadamard rotation for any head size up to 256 and 1..4 bits
// (turboquant/quantizer.py:77-106, turboquant/hadamard.py:21-78 in the reference).
//
// These back the Python algorithm API; the paged cache write has its own specialised kernel.
// One warp owns one row, staged in a per-warp shared buffer; the arithmetic order is the same
// as in the cache-write kernel (eight interleaved no-FMA accumulators for the norm, IEEE
// division, butterflies in stage order, one scale multiply), so 4-bit codes agree with it
// bit for bit.  Compiled with -fmad=false.
#include <cmath>
#include <cstring>

#include "tq_common.cuh"

namespace tq {

constexpr int kMaxDim = 256;
constexpr int kFlatWarps = 4;

struct FlatParams {
    const void* x;         // quantize: input rows; fwht: fp32 input
    const float* signs;    // [padded] (pre-rotation signs); may be null for fwht
    const float* post_signs;
    uint8_t* packed;
    float* norms;
    float* out;
    int64_t n;
    int dim, padded, out_dim, bits, cache_order;
    float scale;           // (float)(1/sqrt(padded))
    float table[16];       // boundaries (quantize) or centroids (dequantize)
};

__device__ __forceinline__ void warp_fwht(float* buf, int padded, int lane) {
    for (int h = 1; h < padded; h <<= 1) {
        for (int idx = lane; idx < padded / 2; idx += 32) {
            const int i = (idx / h) * 2 * h + (idx % h);
            const float a = buf[i], b = buf[i + h];
            buf[i] = __fadd_rn(a, b);
            buf[i + h] = __fsub_rn(a, b);
        }
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(kFlatWarps * 32) quantize_flat_kernel(const __grid_constant__ FlatParams p) {
    __shared__ float buf_s[kFlatWarps][kMaxDim];
    __shared__ uint8_t idx_s[kFlatWarps][kMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = buf_s[warp];
    uint8_t* idx = idx_s[warp];
    const int nb = (1 << p.bits) - 1;
    const int vpb = 8 / p.bits;
    const int nbytes = (p.padded + vpb - 1) / vpb;
    for (int64_t r = (int64_t)blockIdx.x * kFlatWarps + warp; r < p.n; r += (int64_t)gridDim.x * kFlatWarps) {
        const T* row = reinterpret_cast<const T*>(p.x) + r * p.dim;
        for (int i = lane; i < p.padded; i += 32) buf[i] = i < p.dim ? to_f32(row[i]) : 0.0f;
        __syncwarp();
        // norm: eight interleaved accumulators over the first dim & ~7 elements, then the tail
        float acc = 0.0f;
        const int full = p.dim & ~7;
        if (lane < 8)
            for (int j = lane; j < full; j += 8) acc = __fadd_rn(acc, __fmul_rn(buf[j], buf[j]));
        float s = 0.0f;
        for (int k = 0; k < 8; k++) {
            const float a = __shfl_sync(0xffffffffu, acc, k);
            s = k == 0 ? a : __fadd_rn(s, a);
        }
        for (int j = full; j < p.dim; j++) s = __fadd_rn(s, __fmul_rn(buf[j], buf[j]));
        float norm = __fsqrt_rn(s);
        if (!(norm >= 1e-8f)) norm = (norm != norm) ? __uint_as_float(0x7fc00000u) : 1e-8f;
        for (int i = lane; i < p.padded; i += 32)
            buf[i] = i < p.dim ? __fmul_rn(__fdiv_rn(buf[i], norm), p.signs[i]) : 0.0f;
        __syncwarp();
        warp_fwht(buf, p.padded, lane);
        for (int i = lane; i < p.padded; i += 32) {
            const float y = __fmul_rn(buf[i], p.scale);
            int c = 0;
            for (int k = 0; k < nb; k++) c += (p.table[k] < y) ? 1 : 0;
            if (y != y) c = nb;  // torch's lower bound puts NaN in the last bucket
            idx[i] = (uint8_t)c;
        }
        __syncwarp();
        uint8_t* dst = p.packed + r * nbytes;
        for (int b = lane; b < nbytes; b += 32) {
            uint32_t v = 0;
            for (int i = 0; i < vpb; i++) {
                const int e = b * vpb + i;
                const uint32_t code = e < p.padded ? idx[e] : 0u;
                if (p.cache_order) v |= code << ((vpb - 1 - i) * p.bits);
                else v |= code << (i * p.bits);
            }
            dst[b] = (uint8_t)v;
        }
        if (lane == 0) p.norms[r] = norm;
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kFlatWarps * 32) dequantize_flat_kernel(const __grid_constant__ FlatParams p) {
    __shared__ float buf_s[kFlatWarps][kMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = buf_s[warp];
    const int vpb = 8 / p.bits, mask = (1 << p.bits) - 1;
    const int nbytes = (p.padded + vpb - 1) / vpb;
    for (int64_t r = (int64_t)blockIdx.x * kFlatWarps + warp; r < p.n; r += (int64_t)gridDim.x * kFlatWarps) {
        const uint8_t* src = p.packed + r * nbytes;
        for (int e = lane; e < p.padded; e += 32) {
            const int i = e % vpb;
            const int sh = p.cache_order ? (vpb - 1 - i) * p.bits : i * p.bits;
            buf[e] = p.table[(src[e / vpb] >> sh) & mask];
        }
        __syncwarp();
        warp_fwht(buf, p.padded, lane);
        const float norm = p.norms[r];
        for (int e = lane; e < p.dim; e += 32)
            p.out[r * p.dim + e] = __fmul_rn(__fmul_rn(__fmul_rn(buf[e], p.scale), p.signs[e]), norm);
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kFlatWarps * 32) fwht_kernel(const __grid_constant__ FlatParams p) {
    __shared__ float buf_s[kFlatWarps][kMaxDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = buf_s[warp];
    const float* x = reinterpret_cast<const float*>(p.x);
    for (int64_t r = (int64_t)blockIdx.x * kFlatWarps + warp; r < p.n; r += (int64_t)gridDim.x * kFlatWarps) {
        for (int i = lane; i < p.padded; i += 32) {
            float v = i < p.dim ? x[r * p.dim + i] : 0.0f;
            if (p.signs) v = __fmul_rn(v, p.signs[i]);
            buf[i] = v;
        }
        __syncwarp();
        warp_fwht(buf, p.padded, lane);
        for (int i = lane; i < p.out_dim; i += 32) {
            float v = __fmul_rn(buf[i], p.scale);
            if (p.post_signs) v = __fmul_rn(v, p.post_signs[i]);
            p.out[r * p.out_dim + i] = v;
        }
        __syncwarp();
    }
}

static int next_pow2(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

static unsigned flat_grid(int64_t n) {
    const int64_t blocks = (n + kFlatWarps - 1) / kFlatWarps;
    return (unsigned)(blocks < 148 * 16 ? (blocks > 0 ? blocks : 1) : 148 * 16);
}

}  // namespace tq

extern "C" int tq_quantize_flat(const void* x, int x_dtype, int64_t n, int dim, const float* signs,
                                int bits, int pack_order, uint8_t* packed, float* norms,
                                void* stream) {
    using namespace tq;
    if (n == 0) return TQ_OK;
    TQ_REQUIRE(x && signs && packed && norms, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(n > 0 && dim >= 1 && dim <= kMaxDim, TQ_ERR_INVALID, "dim must be 1..%d", kMaxDim);
    TQ_REQUIRE(bits >= 1 && bits <= 4, TQ_ERR_INVALID, "bits must be 1..4");
    FlatParams p{};
    p.x = x; p.signs = signs; p.packed = packed; p.norms = norms; p.n = n; p.dim = dim;
    p.padded = next_pow2(dim); p.bits = bits; p.cache_order = pack_order == TQ_PACK_CACHE;
    p.scale = (float)(1.0 / std::sqrt((double)p.padded));
    float cen[16];
    host_codebook(p.padded, bits, cen, p.table);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case TQ_F32: quantize_flat_kernel<float><<<flat_grid(n), kFlatWarps * 32, 0, s>>>(p); break;
        case TQ_F16: quantize_flat_kernel<__half><<<flat_grid(n), kFlatWarps * 32, 0, s>>>(p); break;
        case TQ_BF16: quantize_flat_kernel<__nv_bfloat16><<<flat_grid(n), kFlatWarps * 32, 0, s>>>(p); break;
        default: return fail(TQ_ERR_INVALID, "bad x_dtype %d", x_dtype);
    }
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

extern "C" int tq_dequantize_flat(const uint8_t* packed, const float* norms, int64_t n, int dim,
                                  const float* signs, int bits, int pack_order, float* out,
                                  void* stream) {
    using namespace tq;
    if (n == 0) return TQ_OK;
    TQ_REQUIRE(packed && norms && signs && out, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(n > 0 && dim >= 1 && dim <= kMaxDim, TQ_ERR_INVALID, "dim must be 1..%d", kMaxDim);
    TQ_REQUIRE(bits >= 1 && bits <= 4, TQ_ERR_INVALID, "bits must be 1..4");
    FlatParams p{};
    p.packed = const_cast<uint8_t*>(packed); p.norms = const_cast<float*>(norms); p.signs = signs;
    p.out = out; p.n = n; p.dim = dim; p.padded = next_pow2(dim); p.bits = bits;
    p.cache_order = pack_order == TQ_PACK_CACHE;
    p.scale = (float)(1.0 / std::sqrt((double)p.padded));
    float bnd[15];
    host_codebook(p.padded, bits, p.table, bnd);
    dequantize_flat_kernel<<<flat_grid(n), kFlatWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

extern "C" int tq_fwht(const float* x, int64_t n, int in_dim, int padded_dim, int out_dim,
                       const float* pre_signs, const float* post_signs, float* out, void* stream) {
    using namespace tq;
    if (n == 0) return TQ_OK;
    TQ_REQUIRE(x && out, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(padded_dim >= 1 && padded_dim <= kMaxDim && (padded_dim & (padded_dim - 1)) == 0,
               TQ_ERR_INVALID, "padded_dim must be a power of two <= %d, got %d", kMaxDim, padded_dim);
    TQ_REQUIRE(in_dim >= 1 && in_dim <= padded_dim && out_dim >= 1 && out_dim <= padded_dim,
               TQ_ERR_INVALID, "in_dim/out_dim must be within padded_dim");
    FlatParams p{};
    p.x = x; p.signs = pre_signs; p.post_signs = post_signs; p.out = out; p.n = n; p.dim = in_dim;
    p.padded = padded_dim; p.out_dim = out_dim;
    p.scale = (float)(1.0 / std::sqrt((double)padded_dim));
    fwht_kernel<<<flat_grid(n), kFlatWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}
