// Cache-write kernel: seeded signs -> FWHT -> L2 norm -> 4-bit Lloyd-Max code -> nibble pack ->
// scatter into the paged cache.  One launch covers K and V.
//
// Replaces the reference's quantize_write_hadamard_scatter_kernel
// (csrc/include/turboquant/quantize_write_kernel.cuh:332-431) but follows the arithmetic of the
// torch quantizer (turboquant/quantizer.py:77-91) so that codes and fp16 norms are bit-identical
// to it: eight interleaved sum-of-squares accumulators without FMA, IEEE sqrt and division,
// butterflies in stage order h = 1..64, one multiply by (float)(1/sqrt(128)), boundaries rounded
// from double, strict "boundary < value" tie rule.  This translation unit is compiled with
// -fmad=false and without fast-math.
//
// Mapping: one thread owns one 128-element row, so every butterfly is register-local.  Rows of a
// 128-row tile are staged into shared memory by per-row bulk async copies (each thread issues
// the copy of its own row, all complete on one mbarrier); a 16-byte row pad keeps the 16-byte
// shared loads conflict-free.  Two buffers overlap the copy of the next tile with the math.
#include <cmath>
#include <cstring>

#include "tq_common.cuh"

namespace tq {

constexpr int kWriteThreads = 128;
constexpr int kD = 128;

struct WriteParams {
    uint8_t* kv_cache;
    const void* src[2];       // key, value
    int64_t token_stride[2];  // elements
    const void* slot_mapping;
    int64_t num_tokens;
    int64_t slab_bytes;       // bytes between the K slab and the V slab
    int num_kv_heads;
    int block_size;
    int slot_bytes;
    int slot_is_i64;
    int zero_pad;
    const float* signs;           // [128] +-1, device
    uint32_t pos_bnd_bits[7];     // fp32 bit patterns of boundaries 8..14 (the positive ones)
    float fwht_scale;             // (float)(1/sqrt(128))
};

// Number of boundaries strictly below y, for the symmetric 15-boundary table
// (boundary 7 is exactly 0, boundary 14-i = -boundary i).  With a = |y| as an integer,
// y > 0: 8 + #{pb < a};  y <= 0: 7 - #{pb <= a} = 7 - #{pb < a + 1}.  A NaN goes to 15 like
// torch.bucketize's lower bound.
__device__ __forceinline__ uint32_t code4(float y, const uint32_t (&pb)[7]) {
    const uint32_t yb = __float_as_uint(y);
    const bool pos = !(y <= 0.0f);
    const uint32_t a = (yb & 0x7fffffffu) + (pos ? 0u : 1u);
    const bool c2 = a > pb[3];
    const uint32_t t1 = c2 ? pb[5] : pb[1];
    const bool c1 = a > t1;
    const uint32_t t0 = c2 ? (c1 ? pb[6] : pb[4]) : (c1 ? pb[2] : pb[0]);
    const bool c0 = a > t0;
    const uint32_t m = (c2 ? 4u : 0u) + (c1 ? 2u : 0u) + (c0 ? 1u : 0u);
    return pos ? 8u + m : 7u - m;
}

template <typename T>
struct RowLoad;

template <>
struct RowLoad<float> {
    static constexpr int kRowBytes = kD * 4;
    // chunk c (0..15) = elements 8c..8c+7
    static __device__ __forceinline__ void load8(const uint8_t* row, int c, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(row + c * 32);
        const float4 b = *reinterpret_cast<const float4*>(row + c * 32 + 16);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};

template <>
struct RowLoad<__nv_bfloat16> {
    static constexpr int kRowBytes = kD * 2;
    static __device__ __forceinline__ void load8(const uint8_t* row, int c, float (&v)[8]) {
        const uint4 a = *reinterpret_cast<const uint4*>(row + c * 16);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <>
struct RowLoad<__half> {
    static constexpr int kRowBytes = kD * 2;
    static __device__ __forceinline__ void load8(const uint8_t* row, int c, float (&v)[8]) {
        const uint4 a = *reinterpret_cast<const uint4*>(row + c * 16);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
};

// Quantize one 128-element row held in registers.  codes[16] are the 64 code bytes as
// little-endian words (byte b = (idx[2b] << 4) | idx[2b+1]); returns the fp32 norm.
__device__ __forceinline__ float quantize_row(float (&x)[kD], const WriteParams& p,
                                              const uint32_t (&sign_mask)[kD / 32],
                                              uint32_t (&codes)[16]) {
    // L2 norm: acc[k] += x[8j+k]^2 in order of j, product rounded before the add.
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++)
#pragma unroll
        for (int k = 0; k < 8; k++) acc[k] = __fadd_rn(acc[k], __fmul_rn(x[8 * j + k], x[8 * j + k]));
    float s = acc[0];
#pragma unroll
    for (int k = 1; k < 8; k++) s = __fadd_rn(s, acc[k]);
    float norm = __fsqrt_rn(s);
    // clamp(min=1e-8); a NaN stays a NaN, in the canonical quiet pattern torch produces
    if (!(norm >= 1e-8f)) norm = (norm != norm) ? __uint_as_float(0x7fc00000u) : 1e-8f;

    // normalise (IEEE division) and apply the +-1 signs (a sign-bit flip is an exact multiply)
#pragma unroll
    for (int d = 0; d < kD; d++) {
        const float u = __fdiv_rn(x[d], norm);
        const uint32_t flip = (sign_mask[d >> 5] << (31 - (d & 31))) & 0x80000000u;
        x[d] = __uint_as_float(__float_as_uint(u) ^ flip);
    }
    // butterflies, stage order h = 1, 2, ..., 64
#pragma unroll
    for (int h = 1; h < kD; h <<= 1)
#pragma unroll
        for (int i = 0; i < kD; i += 2 * h)
#pragma unroll
            for (int k = 0; k < h; k++) {
                const float a = x[i + k], b = x[i + k + h];
                x[i + k] = __fadd_rn(a, b);
                x[i + k + h] = __fsub_rn(a, b);
            }
    // scale, bucketize, pack
#pragma unroll
    for (int w = 0; w < 16; w++) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int d = 8 * w + 2 * b;
            const uint32_t hi = code4(__fmul_rn(x[d], p.fwht_scale), p.pos_bnd_bits);
            const uint32_t lo = code4(__fmul_rn(x[d + 1], p.fwht_scale), p.pos_bnd_bits);
            word |= ((hi << 4) | lo) << (8 * b);
        }
        codes[w] = word;
    }
    return norm;
}

template <typename T>
__global__ void __launch_bounds__(kWriteThreads)
write_kv_cache_kernel(const __grid_constant__ WriteParams p) {
    using L = RowLoad<T>;
    constexpr int kPitch = L::kRowBytes + 16;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[2];
    __shared__ int abort_flag;
    __shared__ uint32_t sign_mask_s[kD / 32];  // bit d set: signs[d] < 0

    const int tid = threadIdx.x;
    const int H = p.num_kv_heads;
    const int64_t rows = p.num_tokens * H;                               // per tensor
    const int64_t tiles_per_tensor = (rows + kWriteThreads - 1) / kWriteThreads;
    const int64_t num_tiles = 2 * tiles_per_tensor;

    if (tid == 0) {
        mbar_init(&full_bar[0], 1);
        mbar_init(&full_bar[1], 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    {
        const uint32_t neg = __ballot_sync(0xffffffffu, p.signs[tid] < 0.0f);
        if ((tid & 31) == 0) sign_mask_s[tid >> 5] = neg;
    }
    __syncthreads();
    uint32_t sign_mask[kD / 32];
#pragma unroll
    for (int i = 0; i < kD / 32; i++) sign_mask[i] = sign_mask_s[i];

    auto issue = [&](int64_t tile, int buf) {
        const int which = tile >= tiles_per_tensor ? 1 : 0;
        const int64_t row0 = (tile - which * tiles_per_tensor) * kWriteThreads;
        const int64_t left = rows - row0;
        const int64_t nrows = left < kWriteThreads ? left : (int64_t)kWriteThreads;
        if (tid == 0) mbar_arrive_expect_tx(&full_bar[buf], (uint32_t)(nrows * L::kRowBytes));
        if (tid < nrows) {
            const int64_t r = row0 + tid;
            const int64_t t = r / H;
            const int h = (int)(r - t * H);
            const T* src = reinterpret_cast<const T*>(p.src[which]) + t * p.token_stride[which] +
                           (int64_t)h * kD;
            bulk_g2s(smem + (size_t)buf * kWriteThreads * kPitch + (size_t)tid * kPitch, src,
                     L::kRowBytes, &full_bar[buf]);
        }
    };

    int64_t tile = blockIdx.x;
    if (tile < num_tiles) issue(tile, 0);
    for (int it = 0; tile < num_tiles; tile += gridDim.x, it++) {
        const int buf = it & 1;
        const int64_t next = tile + gridDim.x;
        if (next < num_tiles) issue(next, buf ^ 1);

        if (!mbar_wait(&full_bar[buf], (it >> 1) & 1)) abort_flag = 1;
        __syncthreads();
        if (abort_flag) return;  // copy never landed: leave without touching the cache

        const int which = tile >= tiles_per_tensor ? 1 : 0;
        const int64_t r = (tile - which * tiles_per_tensor) * kWriteThreads + tid;
        if (r < rows) {
            const int64_t t = r / H;
            const int h = (int)(r - t * H);
            const int64_t slot = p.slot_is_i64
                                     ? reinterpret_cast<const int64_t*>(p.slot_mapping)[t]
                                     : (int64_t) reinterpret_cast<const int32_t*>(p.slot_mapping)[t];
            if (slot >= 0) {
                const uint8_t* row = smem + (size_t)buf * kWriteThreads * kPitch + (size_t)tid * kPitch;
                float x[kD];
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    float v[8];
                    L::load8(row, c, v);
#pragma unroll
                    for (int k = 0; k < 8; k++) x[8 * c + k] = v[k];
                }
                uint32_t codes[16];
                const float norm = quantize_row(x, p, sign_mask, codes);
                const uint32_t nh = (norm != norm) ? 0x7e00u : (uint32_t)__half_as_ushort(__float2half_rn(norm));
                // slot = block * block_size + entry and the cache is [block][entry][head][slot_bytes]
                uint8_t* dst = p.kv_cache + (size_t)which * p.slab_bytes +
                               ((size_t)slot * H + h) * p.slot_bytes;
#pragma unroll
                for (int q = 0; q < 4; q++)
                    *reinterpret_cast<uint4*>(dst + 16 * q) =
                        make_uint4(codes[4 * q], codes[4 * q + 1], codes[4 * q + 2], codes[4 * q + 3]);
                if (p.zero_pad)
                    *reinterpret_cast<uint4*>(dst + 64) = make_uint4(nh | (nh << 16), 0u, 0u, 0u);
                else
                    *reinterpret_cast<uint32_t*>(dst + 64) = nh | (nh << 16);
            }
        }
        __syncthreads();  // everyone is done reading this buffer before it is refilled
    }
}

template <typename T>
static int launch_write(const WriteParams& p, int sm_count, cudaStream_t stream) {
    constexpr int kPitch = RowLoad<T>::kRowBytes + 16;
    const size_t smem = (size_t)2 * kWriteThreads * kPitch;
    static bool configured[64] = {};  // per template instance and device
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(write_kv_cache_kernel<T>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int64_t rows = p.num_tokens * p.num_kv_heads;
    const int64_t tiles = 2 * ((rows + kWriteThreads - 1) / kWriteThreads);
    const int per_sm = (int)(227 * 1024 / (smem + 1024));
    const int64_t grid = tiles < (int64_t)sm_count * per_sm ? tiles : (int64_t)sm_count * per_sm;
    write_kv_cache_kernel<T><<<(unsigned)grid, kWriteThreads, smem, stream>>>(p);
    TQ_CUDA(cudaGetLastError());
    return TQ_OK;
}

int device_sm_count(int* out);

}  // namespace tq

extern "C" int tq_write_kv_cache(void* kv_cache, int64_t num_blocks, int block_size,
                                 int num_kv_heads, int slot_bytes, const void* key,
                                 const void* value, int in_dtype, int64_t num_tokens,
                                 int64_t k_token_stride, int64_t v_token_stride, const float* signs,
                                 const void* slot_mapping, int slot_dtype, int head_dim, int flags,
                                 void* stream) {
    using namespace tq;
    TQ_REQUIRE(num_tokens >= 0 && num_blocks >= 0, TQ_ERR_INVALID, "negative size");
    if (num_tokens == 0) return TQ_OK;
    TQ_REQUIRE(kv_cache && key && value && signs && slot_mapping, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(head_dim == kD, TQ_ERR_UNSUPPORTED, "cache write supports head_dim 128, got %d", head_dim);
    TQ_REQUIRE(num_kv_heads >= 1 && block_size >= 1, TQ_ERR_INVALID, "bad geometry");
    TQ_REQUIRE(slot_bytes >= 80 && slot_bytes % 16 == 0, TQ_ERR_INVALID,
               "slot_bytes must be a multiple of 16 and >= 80, got %d", slot_bytes);
    TQ_REQUIRE(in_dtype == TQ_F32 || in_dtype == TQ_F16 || in_dtype == TQ_BF16, TQ_ERR_INVALID, "bad in_dtype");
    TQ_REQUIRE(slot_dtype == TQ_I32 || slot_dtype == TQ_I64, TQ_ERR_INVALID, "bad slot_dtype");
    const int esz = in_dtype == TQ_F32 ? 4 : 2;
    TQ_REQUIRE(((uintptr_t)key % 16) == 0 && ((uintptr_t)value % 16) == 0 &&
                   (k_token_stride * esz) % 16 == 0 && (v_token_stride * esz) % 16 == 0,
               TQ_ERR_INVALID, "key/value rows must be 16-byte aligned");
    TQ_REQUIRE(k_token_stride >= (int64_t)num_kv_heads * head_dim &&
                   v_token_stride >= (int64_t)num_kv_heads * head_dim,
               TQ_ERR_INVALID, "token stride smaller than one token");
    TQ_REQUIRE(((uintptr_t)kv_cache % 16) == 0, TQ_ERR_INVALID, "kv_cache must be 16-byte aligned");

    WriteParams p{};
    p.kv_cache = static_cast<uint8_t*>(kv_cache);
    p.src[0] = key;
    p.src[1] = value;
    p.token_stride[0] = k_token_stride;
    p.token_stride[1] = v_token_stride;
    p.slot_mapping = slot_mapping;
    p.num_tokens = num_tokens;
    p.slab_bytes = num_blocks * block_size * (int64_t)num_kv_heads * slot_bytes;
    p.num_kv_heads = num_kv_heads;
    p.block_size = block_size;
    p.slot_bytes = slot_bytes;
    p.slot_is_i64 = slot_dtype == TQ_I64;
    p.zero_pad = (flags & TQ_WRITE_ZERO_PAD) != 0;
    p.signs = signs;
    float cen[16], bnd[15];
    host_codebook(kD, 4, cen, bnd);
    for (int i = 0; i < 7; i++) {
        float b = bnd[8 + i];
        memcpy(&p.pos_bnd_bits[i], &b, 4);
    }
    p.fwht_scale = (float)(1.0 / sqrt((double)kD));
    int sms = 0;
    int rc = device_sm_count(&sms);
    if (rc != TQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case TQ_F32: return launch_write<float>(p, sms, s);
        case TQ_F16: return launch_write<__half>(p, sms, s);
        default: return launch_write<__nv_bfloat16>(p, sms, s);
    }
}
