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
// Mapping: two lanes own one 128-element row; lane m holds elements 8j + 4m .. 8j + 4m + 3
// (j = 0..15), i.e. four of the eight norm accumulators and code bytes 4j + 2m, 4j + 2m + 1.
// Butterfly stages 1, 2 and 8..64 are register-local, stage 4 is one shuffle per element.  A warp
// works on 16 rows per pass, which halves the per-row share of everything that is done once per
// pass (pipeline, slot lookup, norm reduction, store).  Rows are staged into shared memory by
// per-row bulk async copies, each warp running its own two-buffer pipeline.  Everything per
// element runs on the FP32 pipe where it can
// (the integer/logic pipe has half its rate):
//   * x / norm is q = x*r, e = fma(-q, norm, x), q' = fma(e, r, q) with r the correctly rounded
//     reciprocal, which equals the IEEE quotient whenever the intermediates stay normal and the
//     norm's significand is not all ones (checked per row; otherwise the row takes the division
//     instruction);
//   * the code index comes from a table over 1/64-wide bins of y (each bin holds at most one of
//     the 15 boundaries): boundaries below the bin + one exact comparison with the boundary inside.
#include <cuda.h>  // CUtensorMap and its enums only: the encoder is looked up at run time, nothing links against the driver

#include <cmath>
#include <cstring>
#include <type_traits>

#include "tq_common.cuh"

namespace tq {

constexpr int kD = 128;
// Bins of the code search: bin(y) = round(64 y) + kBinZero.  |y| <= 1 up to rounding for a
// normalized row, so kBins = 2 * 96 + 1 bins (|y| <= 1.5) cover every value the search can see.
constexpr int kBinZero = 96;
constexpr int kBins = 2 * kBinZero + 1;
constexpr float kBinMagic = 8388608.0f + (float)kBinZero;  // 2^23 + kBinZero: the sum's low mantissa bits are the bin

struct WriteParams {
    uint8_t* kv_cache;
    const void* src[2];       // key, value
    int64_t token_stride[2];  // elements
    const void* slot_mapping;
    int64_t num_tokens;
    int64_t slab_bytes;       // bytes between the K slab and the V slab
    int64_t total_slots;      // num_blocks * block_size: a slot at or beyond it is dropped and counted
    int num_kv_heads;
    int head_shift;           // log2(num_kv_heads) when that is a power of two, else -1
    int block_size;
    int slot_bytes;
    int slot_is_i64;
    int zero_pad;
    const float* signs;       // [128] +-1, device
    float2 bin_table[kBins];  // per bin of y: {boundary inside the bin or +inf, number of boundaries in lower bins}
    float fwht_scale;         // (float)(1/sqrt(128))
    // tensor-core kernel, dense inputs: key / value as [rows][128] tensors, boxes of 16 rows x 64 elements
    alignas(64) CUtensorMap tmap[2];
};

// Two fp32 values in one 64-bit register and the packed arithmetic of sm_100 (add/sub/mul/fma
// .f32x2): each lane of a pair is rounded to nearest exactly like the scalar instruction, at half
// the instruction count.  A lane's elements (8j + 2m, 8j + 2m + 1) form the natural pairs.
struct P2 { unsigned long long v; };
__device__ __forceinline__ P2 pk(float lo, float hi) {
    P2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void up(P2 a, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v)); }
__device__ __forceinline__ P2 add2(P2 a, P2 b) { P2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ P2 sub2(P2 a, P2 b) { P2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ P2 mul2(P2 a, P2 b) { P2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ P2 fma2(P2 a, P2 b, P2 c) {
    P2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
    return r;
}

// Code of y among the 15 boundaries: the number of boundaries strictly below y (torch.bucketize,
// right = False), as a float.  The boundaries are at least 1/64 apart, so the bin
// k = round(64 y) + kBinZero holds at most one of them; the binning is monotone in y, hence every
// boundary in a lower bin is below y and every boundary in a higher bin is not.  Table entry k =
// {the boundary inside bin k, or +inf; the number of boundaries in lower bins}: one lookup and one
// exact comparison finish the search.  The table has 16 columns (entry k of column c at
// k * 128 + 8 c; an 8-byte load is served half a warp at a time), so a warp's lookups never
// conflict, and the address is one integer multiply-add of the float's bit pattern:
// (0x4B000000 + k) * 128 wraps to 128 k + 2^31, and the column base has 2^31 subtracted.
// The host fills the table with the same float operations, which makes it consistent with this
// binning by construction.  NaN rows never get here.
__device__ __forceinline__ float code_lookup(float y, float kf, uint32_t table_lane) {
    const uint32_t addr = __float_as_uint(kf) * 128u + table_lane;
    float bnd, below;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(bnd), "=f"(below) : "r"(addr));
    return y > bnd ? __fadd_rn(below, 1.0f) : below;
}
// code byte of a pair (even dim in the high nibble), as a float in 0..255
__device__ __forceinline__ float code_byte(P2 y2, uint32_t table_lane) {
    float y0, y1, k0, k1;
    up(y2, y0, y1);
    up(fma2(y2, pk(64.0f, 64.0f), pk(kBinMagic, kBinMagic)), k0, k1);  // bins of both, one instruction
    return __fmaf_rn(code_lookup(y0, k0, table_lane), 16.0f, code_lookup(y1, k1, table_lane));
}

// row index -> (token, head).  A 64-bit division by a run-time value is a long subroutine; the
// usual head counts are powers of two (shift and mask), and below 2^31 rows a 32-bit division does.
__device__ __forceinline__ void split_row(int64_t r, int H, int head_shift, int64_t& t, int& h) {
    if (head_shift >= 0) {
        t = r >> head_shift;
        h = (int)r & (H - 1);
    } else if (r < 0x7fffffffLL) {
        const uint32_t q = (uint32_t)r / (uint32_t)H;
        t = q;
        h = (int)((uint32_t)r - q * (uint32_t)H);
    } else {
        t = r / H;
        h = (int)(r - t * H);
    }
}

// Rows dropped because their slot lay outside the cache (a stale or garbage slot id must never
// become a store address); read back by tq_fault_counts.
static __device__ int32_t g_write_dropped = 0;
// Rows the tensor-core kernel handled, and how many of them it re-derived with the exact path
// (read back by tq_write_guard_stats).
static __device__ unsigned long long g_guard_rows[2] = {0ull, 0ull};

template <typename T>
struct RowLoad;

// quad(row, j, m): elements 8j + 4m .. 8j + 4m + 3 of a staged row, as two pairs.  kPad keeps the
// loads of a warp (16 rows x 2 lanes) conflict free: 16-bit rows are read 8 bytes per lane in
// half-warps (8 rows: row * 68 words -> 4 banks apart), 32-bit rows 16 bytes per lane in
// quarter-warps (4 rows: row * 136 words -> 8 banks apart).
template <>
struct RowLoad<float> {
    static constexpr int kElemBytes = 4, kPad = 32;
    static __device__ __forceinline__ void quad(const uint8_t* row, int j, int m, float2& a, float2& b) {
        const float4 v = *reinterpret_cast<const float4*>(row + 32 * j + 16 * m);
        a = make_float2(v.x, v.y);
        b = make_float2(v.z, v.w);
    }
};
template <>
struct RowLoad<__nv_bfloat16> {
    static constexpr int kElemBytes = 2, kPad = 16;
    static __device__ __forceinline__ void quad(const uint8_t* row, int j, int m, float2& a, float2& b) {
        const uint2 w = *reinterpret_cast<const uint2*>(row + 16 * j + 8 * m);
        a = make_float2(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u));
        b = make_float2(__uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
    }
};
template <>
struct RowLoad<__half> {
    static constexpr int kElemBytes = 2, kPad = 16;
    static __device__ __forceinline__ void quad(const uint8_t* row, int j, int m, float2& a, float2& b) {
        const uint2 w = *reinterpret_cast<const uint2*>(row + 16 * j + 8 * m);
        a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
        b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    }
};

// Threads per block: one block per SM.  16-bit inputs run 16 warps; fp32 rows need twice the
// staging space, so they run 8.
// D = elements per input row: 128, or fewer (a multiple of 8) for heads that the rotation pads
// with zeros to 128 (turboquant/hadamard.py:66-68); the cache slot is the same either way.
template <typename T, int D>
struct WriteShape {
    static constexpr int kRowBytes = D * RowLoad<T>::kElemBytes;
    static constexpr int kThreads = sizeof(T) == 4 ? 256 : 512;
    static constexpr int kWarps = kThreads / 32;
    static constexpr int kPieceRows = 16;                 // rows per warp and pass: two lanes per row
    static constexpr int kTileRows = kWarps * kPieceRows;
    static constexpr int kPitch = kRowBytes + RowLoad<T>::kPad;
    static constexpr int kOutPitch = 72;                  // 18 words: 16 rows -> 16 different banks
    static constexpr size_t kStageBytes = (size_t)2 * kTileRows * kPitch;
    static constexpr size_t kTableBytes = (size_t)kBins * 16 * sizeof(float2);
    static constexpr size_t kOutBytes = (size_t)kTileRows * kOutPitch;
    static constexpr size_t kSmem = kStageBytes + kTableBytes + kOutBytes;
};

template <typename T, int D>
__global__ void __launch_bounds__(WriteShape<T, D>::kThreads, 1)
write_kv_cache_kernel(const __grid_constant__ WriteParams p) {
    using L = RowLoad<T>;
    using W = WriteShape<T, D>;
    constexpr int kPitch = W::kPitch, kPieceRows = W::kPieceRows;
    extern __shared__ __align__(128) uint8_t smem[];
    // every warp runs its own two-buffer pipeline over 16-row pieces: no block-wide barrier in the loop
    __shared__ __align__(8) uint64_t full_bar[W::kWarps][2];
    __shared__ __align__(16) float signs_s[kD];

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int m = lane & 1;              // lane within the row: elements 8j + 4m .. 8j + 4m + 3
    const int row_in_warp = lane >> 1;   // row of the warp's 16-row piece this lane works on
    const int row_in_tile = warp * kPieceRows + row_in_warp;
    const int H = p.num_kv_heads;
    const int64_t rows = p.num_tokens * H;  // per tensor
    const int64_t num_tiles = 2 * ((rows + kPieceRows - 1) / kPieceRows);  // K and V pieces alternate

    grid_launch_dependents();
    if (lane == 0) {
        mbar_init(&full_bar[warp][0], 1);
        mbar_init(&full_bar[warp][1], 1);
    }
    if (tid == 0) fence_barrier_init();
    // Code-search table behind the staging buffers: entry k of column c at (16 k + c) * 8 bytes.
    // An 8-byte load is served half a warp at a time, so 16 columns (lane & 15) are enough for
    // conflict-free lookups.
    float2* bins_s = reinterpret_cast<float2*>(smem + W::kStageBytes);
    for (int i = tid; i < kBins * 16; i += W::kThreads) bins_s[i] = p.bin_table[i >> 4];
    // (the bit pattern of 2^23 + k) * 128 = 2^31 + 128 k modulo 2^32: take the 2^31 out here
    const uint32_t table_lane = smem_u32(bins_s) + 8u * (lane & 15) - 0x80000000u;
    uint8_t* out_s = smem + W::kStageBytes + W::kTableBytes;
    // the signs, like the table, are constants of the context: both are read ahead of the wait
    if (tid < kD) signs_s[tid] = p.signs[tid];
    grid_dependency_wait();  // K, V, the slots and the cache belong to earlier kernels
    __syncthreads();

    // piece index -> tensor and rows: tile = 2 * piece + tensor
    auto issue = [&](int64_t tile, int buf) {
        const int which = (int)(tile & 1);
        const int64_t row0 = (tile >> 1) * kPieceRows;
        const int64_t left = rows - row0;
        const int64_t nrows = left < kPieceRows ? left : (int64_t)kPieceRows;
        fence_proxy_async();  // earlier shared-memory reads of this buffer precede the copy engine's writes
        if (lane == 0) mbar_arrive_expect_tx(&full_bar[warp][buf], (uint32_t)(nrows * W::kRowBytes));
        __syncwarp();
        if (lane < nrows) {
            const int64_t r = row0 + lane;
            int64_t t;
            int h;
            split_row(r, H, p.head_shift, t, h);
            const T* src = reinterpret_cast<const T*>(p.src[which]) + t * p.token_stride[which] + (int64_t)h * D;
            bulk_g2s(smem + (size_t)buf * W::kTileRows * kPitch + (size_t)(warp * kPieceRows + lane) * kPitch, src,
                     W::kRowBytes, &full_bar[warp][buf]);
        }
    };

    // consecutive pieces go to different blocks: a small write spreads over as many SMs as it has
    // pieces instead of filling the warps of one
    const int64_t warp_stride = (int64_t)gridDim.x * W::kWarps;
    int64_t tile = (int64_t)warp * gridDim.x + blockIdx.x;
    if (tile < num_tiles) issue(tile, 0);
    for (int it = 0; tile < num_tiles; tile += warp_stride, it++) {
        const int buf = it & 1;
        const int64_t next = tile + warp_stride;
        if (next < num_tiles) issue(next, buf ^ 1);  // that buffer was read out one iteration ago

        const int which = (int)(tile & 1);
        const int64_t r = (tile >> 1) * kPieceRows + row_in_warp;
        const bool row_ok = r < rows;  // uniform over the two lanes of a row
        int64_t slot = -1;
        int h = 0;
        if (row_ok) {  // the slot is fetched while the rows are still on their way
            int64_t t;
            split_row(r, H, p.head_shift, t, h);
            slot = p.slot_is_i64 ? reinterpret_cast<const int64_t*>(p.slot_mapping)[t]
                                 : (int64_t) reinterpret_cast<const int32_t*>(p.slot_mapping)[t];
        }

        if (!mbar_wait(&full_bar[warp][buf], (it >> 1) & 1)) return;  // copy never landed: touch nothing
        // All lanes run the arithmetic (the shuffles need whole pairs).  Rows past the end compute
        // on whatever the buffer holds (any bit pattern is handled: finite rows normalize to
        // |y| <= 1, anything else becomes an all-NaN row) and store nothing.
        const uint8_t* row = smem + (size_t)buf * W::kTileRows * kPitch + (size_t)row_in_tile * kPitch;
        P2 x[32];  // x[2j] = elements (8j+4m, 8j+4m+1), x[2j+1] = (8j+4m+2, 8j+4m+3)
        P2 acc_a = pk(0.0f, 0.0f), acc_b = pk(0.0f, 0.0f);  // accumulators 4m, 4m+1 and 4m+2, 4m+3 of the eight
        float minsq = 1.0f;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (8 * j >= D) {  // padding of a short head: zeros, which add nothing to the norm
                x[2 * j] = pk(0.0f, 0.0f);
                x[2 * j + 1] = pk(0.0f, 0.0f);
                continue;
            }
            float2 va, vb;
            L::quad(row, j, m, va, vb);
            x[2 * j] = pk(va.x, va.y);
            x[2 * j + 1] = pk(vb.x, vb.y);
            // in order of j, product rounded before the add
            const P2 sa = mul2(x[2 * j], x[2 * j]), sb = mul2(x[2 * j + 1], x[2 * j + 1]);
            acc_a = add2(acc_a, sa);
            acc_b = add2(acc_b, sb);
            float s0, s1, s2, s3;
            up(sa, s0, s1);
            up(sb, s2, s3);
            asm("min.f32 %0, %0, %1, %2;" : "+f"(minsq) : "f"(s0), "f"(s1));  // three-input minimum
            asm("min.f32 %0, %0, %1, %2;" : "+f"(minsq) : "f"(s2), "f"(s3));
        }
        // combine the eight accumulators left to right: lane m = 0 holds 0..3, lane m = 1 holds 4..7
        float mine[4], other[4];
        up(acc_a, mine[0], mine[1]);
        up(acc_b, mine[2], mine[3]);
#pragma unroll
        for (int k = 0; k < 4; k++) other[k] = __shfl_xor_sync(0xffffffffu, mine[k], 1);
        float s = m ? other[0] : mine[0];
#pragma unroll
        for (int k = 1; k < 4; k++) s = __fadd_rn(s, m ? other[k] : mine[k]);
#pragma unroll
        for (int k = 0; k < 4; k++) s = __fadd_rn(s, m ? mine[k] : other[k]);
        minsq = fminf(minsq, __shfl_xor_sync(0xffffffffu, minsq, 1));
        float norm = __fsqrt_rn(s);
        // clamp(min=1e-8); a NaN stays a NaN, in the canonical quiet pattern torch produces
        if (!(norm >= 1e-8f)) norm = (norm != norm) ? __uint_as_float(0x7fc00000u) : 1e-8f;

        // normalise.  Fast path: every square is a normal number (so |x| >= 2^-75 and nonzero)
        // and the norm is moderate with a significand that is not all ones.
        const uint32_t nbits = __float_as_uint(norm);
        const bool fast = minsq >= 1.1754944e-38f && norm >= 9.0949470e-13f && norm <= 1.0995116e12f &&
                          (nbits & 0x7fffffu) != 0x7fffffu;
        if (fast) {
            const float rcp = __frcp_rn(norm);
            const P2 rcp2 = pk(rcp, rcp), nneg2 = pk(-norm, -norm);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const P2 q = mul2(x[i], rcp2);
                const P2 err = fma2(q, nneg2, x[i]);   // x - q * norm, exact
                x[i] = fma2(err, rcp2, q);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) {
                float a, b;
                up(x[i], a, b);
                x[i] = pk(__fdiv_rn(a, norm), __fdiv_rn(b, norm));
            }
        }
        // signs, then butterflies in stage order: h = 1 inside a pair, h = 2 between the two pairs
        // of a j, h = 4 between the two lanes, h = 8..64 across j
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const float4 sg = *reinterpret_cast<const float4*>(&signs_s[8 * j + 4 * m]);
            float a, b, c, d;
            up(mul2(x[2 * j], pk(sg.x, sg.y)), a, b);
            up(mul2(x[2 * j + 1], pk(sg.z, sg.w)), c, d);
            const P2 lo = pk(__fadd_rn(a, b), __fsub_rn(a, b)), hi = pk(__fadd_rn(c, d), __fsub_rn(c, d));
            x[2 * j] = add2(lo, hi);
            x[2 * j + 1] = sub2(lo, hi);
        }
        {
            // upper partner: other - mine, lower partner: mine + other; one FMA with +-1 does both
            // (the product with +-1 is exact, so the rounding is that of the plain add/sub)
            const float sgn = m ? -1.0f : 1.0f;
            const P2 sgn2 = pk(sgn, sgn);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                float a, b;
                up(x[i], a, b);
                const float oa = __shfl_xor_sync(0xffffffffu, a, 1), ob = __shfl_xor_sync(0xffffffffu, b, 1);
                x[i] = fma2(x[i], sgn2, pk(oa, ob));
            }
        }
#pragma unroll
        for (int hj = 1; hj < 16; hj <<= 1)
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (!(j & hj)) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const P2 a = x[2 * j + e], b = x[2 * (j + hj) + e];
                        x[2 * j + e] = add2(a, b);
                        x[2 * (j + hj) + e] = sub2(a, b);
                    }
                }
        const P2 scale2 = pk(p.fwht_scale, p.fwht_scale);
        // scale, code, pack: code bytes 4j + 2m and 4j + 2m + 1 (even dim in the high nibble) as one
        // 16-bit store, taken from the low bits of a float with 2^23 added
        float y0, y1;
        up(mul2(x[0], scale2), y0, y1);
        // A non-finite input turns the whole row into NaN (every output of the transform depends
        // on every input); torch's bucketize sends NaN to the last bucket: every code is 15.
        const bool all_nan = y0 != y0;
        uint8_t* orow = out_s + (size_t)row_in_tile * W::kOutPitch;
        if (!all_nan) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const float b0 = code_byte(mul2(x[2 * j], scale2), table_lane);
                const float b1 = code_byte(mul2(x[2 * j + 1], scale2), table_lane);
                const float both = __fadd_rn(__fmaf_rn(b1, 256.0f, b0), 8388608.0f);
                *reinterpret_cast<uint16_t*>(orow + 4 * j + 2 * m) = (uint16_t)__float_as_uint(both);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) *reinterpret_cast<uint16_t*>(orow + 4 * j + 2 * m) = 0xffffu;
        }
        __syncwarp();
        if (row_ok && slot >= p.total_slots) {
            if (m == 0 && h == 0 && which == 0) atomicAdd(&g_write_dropped, 1);  // once per token
            slot = -1;
        }
        if (row_ok && slot >= 0) {
            // slot = block * block_size + entry and the cache is [block][entry][head][slot_bytes]
            uint8_t* dst = p.kv_cache + (size_t)which * p.slab_bytes + ((size_t)slot * H + h) * p.slot_bytes;
            const uint2* src8 = reinterpret_cast<const uint2*>(orow + 32 * m);
            const uint2 c0 = src8[0], c1 = src8[1], c2 = src8[2], c3 = src8[3];
            uint4* dst16 = reinterpret_cast<uint4*>(dst + 32 * m);
            dst16[0] = make_uint4(c0.x, c0.y, c1.x, c1.y);
            dst16[1] = make_uint4(c2.x, c2.y, c3.x, c3.y);
            if (m == 0) {
                const uint32_t nh = (norm != norm) ? 0x7e00u : (uint32_t)__half_as_ushort(__float2half_rn(norm));
                if (p.zero_pad) *reinterpret_cast<uint4*>(dst + 64) = make_uint4(nh | (nh << 16), 0u, 0u, 0u);
                else *reinterpret_cast<uint32_t*>(dst + 64) = nh | (nh << 16);
            }
        }
        __syncwarp();  // the warp is done with this buffer and with its rows of the output staging
    }
}

template <typename T, int D>
static int launch_write(const WriteParams& p, int sm_count, cudaStream_t stream) {
    using W = WriteShape<T, D>;
    const size_t smem = W::kSmem;
    static bool configured[64] = {};  // per template instance and device
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(write_kv_cache_kernel<T, D>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int64_t rows = p.num_tokens * p.num_kv_heads;
    const int64_t pieces = 2 * ((rows + W::kPieceRows - 1) / W::kPieceRows);  // one warp pass each
    const int64_t grid = pieces < (int64_t)sm_count ? pieces : (int64_t)sm_count;  // one block per SM
    TQ_CUDA(launch_serialized(write_kv_cache_kernel<T, D>, dim3((unsigned)grid), dim3(W::kThreads), smem, stream, p));
    return TQ_OK;
}


// =============================================================================================
// 16-bit inputs, head size 128: tensor-core transform with guarded codes.
//
// The kernel above spends about 23 instructions per element, most of them on arithmetic whose
// exact rounding only matters for the few elements that land next to a code boundary.  This
// kernel gets the same bytes with fewer instructions:
//
//   * The norm is computed exactly as above (bf16 / fp16 squares are exact in fp32; the adds run
//     in the reference order: eight interleaved accumulators over j, combined left to right).  A
//     thread of an MMA fragment holds, for its two rows, exactly the elements of accumulators
//     2tg and 2tg+1, in order of j; their fp32 values come from a tensor-core product with the
//     identity (one non-zero addend per output, hence exact), so no unpacking is needed.
//   * The transform is H128 = H8 (x) H16: the H16 factor (butterfly stages h = 1..8) is one
//     m16n8k16 tensor-core product per 16-element chunk of a 16-row tile against a +-1 matrix
//     with the sign vector folded in (products with +-1 are exact; the accumulator starts at zero),
//     the H8 factor (h = 16..64) is three register-local butterfly stages in fp32.  The result Y is
//     the transform of the raw row; y = Y * SCALE / norm is never formed: its bin and its distance
//     from the bin's boundary come from one FMA each with per-row constants.
//   * Guard.  Let y_ref be what the reference computes (division, seven rounded stages, one
//     multiply) and y_fast = Y * SCALE / norm as evaluated here, both with the same fp32 norm.
//     Against exact arithmetic on that norm, |y_ref - y| <= 26 u (u = 2^-24: 11.3 u from the
//     divisions, 282 u from the stage roundings, both in units of the unscaled transform, times
//     SCALE, plus the final multiply), and |y_fast - y| <= 29 u: 34 u * max|x| per chunk product --
//     the tensor core adds 16 exact addends after aligning them to the largest one and keeps at
//     least 24 bits, so each addend loses less than 2^-23 of that largest one -- times 8 chunks,
//     50 u * norm from the three fp32 stages, 1.5 u relative from the rounded scale factor.
//     Together |y_fast - y_ref| < 55 u = 3.3e-6.  A code is taken from y_fast only when y_fast is
//     farther than 2^-18 = 3.8e-6 from the boundary of its bin: z = (y_fast - b) * 2^17 + 1/2,
//     s = saturate(z) is exactly 0 or 1 then, and code = (boundaries in lower bins) + s.  Any
//     s strictly between 0 and 1 makes sum s (1 - s) positive for the row (non-negative terms, so
//     nothing cancels), and such a row is done again by the exact path below, 32 lanes on one row,
//     from the staged input.  About 3.6 % of N(0,1) rows take it.  Rows whose norm is not a
//     moderate finite number (zero rows, overflowing or non-finite rows) always take it.
//   * The bins of y_fast are formed from Y * (64 * f) rather than from the rounded y, so next to a
//     bin edge the two paths may pick neighbouring bins; the host checks that no boundary lies
//     within 2^-13 of a bin edge, which makes both bins give the same code there.
//   * Staging.  Dense inputs (token stride = heads x 128) are fetched by tiled tensor copies
//     (cp.async.bulk.tensor, two boxes of 16 rows x 128 bytes per tile, 128-byte swizzle, issued
//     by one lane); the swizzle makes the ldmatrix reads conflict free.  Strided inputs (K / V as
//     column slices of a fused projection) use one bulk copy per row into rows of 272 bytes.
// =============================================================================================
constexpr float kGuardBig = 131072.0f;  // 2^17

template <typename T>
struct MmaOps;
template <>
struct MmaOps<__nv_bfloat16> {
    static constexpr uint32_t kOne = 0x3F80u, kMinusOne = 0xBF80u;
    // the accumulator input is the constant zero: nothing has to be cleared first
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    }
    static __device__ __forceinline__ P2 unpack(uint32_t w) {
        return pk(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
};
template <>
struct MmaOps<__half> {
    static constexpr uint32_t kOne = 0x3C00u, kMinusOne = 0xBC00u;
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    }
    static __device__ __forceinline__ P2 unpack(uint32_t w) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        return pk(f.x, f.y);
    }
};

// Shared-memory map of the tensor-core kernel.  A warp's stage buffer holds its 16-row tile either
// as two swizzled halves of 16 rows x 128 bytes (tensor copies) or as rows of 272 bytes (per-row
// copies; 272 = 16 mod 128, so the eight rows of an ldmatrix hit different banks).
struct MmaShape {
    static constexpr int kThreads = 512, kWarps = 16, kRows = 16;
    static constexpr int kRowBytes = 256, kPitch = 272;
    static constexpr int kWarpStage = 5120;                        // >= 16 x 272, a multiple of 1024 (swizzle atom)
    static constexpr size_t kStageBytes = (size_t)2 * kWarps * kWarpStage;
    static constexpr size_t kTableBytes = (size_t)kBins * 16 * 8 + 1024;  // 16 columns of 8-byte entries + the boundaries
    static constexpr size_t kBfragBytes = (size_t)8 * 32 * 16;     // B fragments of the 8 chunks, per lane
    static constexpr int kOutPitch = 72;
    static constexpr size_t kOutBytes = (size_t)kWarps * kRows * kOutPitch;
    static constexpr size_t kSmem = kStageBytes + kTableBytes + kBfragBytes + kOutBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
}
// Tiled tensor copy global -> shared of one box at element coordinates (x, y), completing on an
// mbarrier.  x times the element size is a multiple of 16 bytes at both call sites (0 and 128).
__device__ __forceinline__ void tensor_g2s_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// One code byte (even dim in the high nibble) of the pair (Y0, Y1) of one row, as a float, and the
// row's ambiguity sum.  Table entry of a bin (8 bytes, 16 columns: an 8-byte load is served half a
// warp at a time, so lookups never conflict): {1/2 - b * 2^17 (or -inf), boundaries in lower bins}.
__device__ __forceinline__ float guarded_byte(P2 Y2, P2 kf2, float zf, uint32_t table_lane, P2& amb) {
    float Y0, Y1, k0, k1;
    up(Y2, Y0, Y1);
    up(fma2(Y2, kf2, pk(kBinMagic, kBinMagic)), k0, k1);
    float c0, below0, c1, below1;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(c0), "=f"(below0) : "r"(__float_as_uint(k0) * 128u + table_lane));
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(c1), "=f"(below1) : "r"(__float_as_uint(k1) * 128u + table_lane));
    const float s0 = fma_sat(Y0, zf, c0), s1 = fma_sat(Y1, zf, c1);
    const P2 s2 = pk(s0, s1);
    amb = fma2(s2, sub2(pk(1.0f, 1.0f), s2), amb);  // s (1 - s): zero exactly when s is 0 or 1
    return __fmaf_rn(__fadd_rn(s0, below0), 16.0f, __fadd_rn(s1, below1));
}

template <typename T, bool TMA>
__global__ void __launch_bounds__(MmaShape::kThreads, 1)
write_kv_cache_mma_kernel(const __grid_constant__ WriteParams p) {
    using O = MmaOps<T>;
    using W = MmaShape;
    constexpr int kPitch = W::kPitch, kRows = W::kRows;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[W::kWarps][2];
    __shared__ __align__(16) float signs_s[kD];
    // the swizzle pattern of a tensor copy is a function of the shared-memory address: 1024-byte aligned stages
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tg = lane & 3;   // fragment coordinates: rows g and g + 8, column pair tg
    const int m = lane & 1;                   // store phase: two lanes per row
    const int row_in_warp = lane >> 1;
    const int H = p.num_kv_heads;
    const int64_t rows = p.num_tokens * H;
    const int64_t num_tiles = 2 * ((rows + kRows - 1) / kRows);  // K and V tiles alternate

    grid_launch_dependents();
    if (lane == 0) {
        mbar_init(&full_bar[warp][0], 1);
        mbar_init(&full_bar[warp][1], 1);
    }
    if (tid == 0) fence_barrier_init();
    float2* tab_s = reinterpret_cast<float2*>(smem + W::kStageBytes);
    float* bnd_s = reinterpret_cast<float*>(smem + W::kStageBytes + (size_t)kBins * 16 * 8);  // exact path only
    for (int i = tid; i < kBins * 16; i += W::kThreads) {
        const float2 e = p.bin_table[i >> 4];  // {boundary inside the bin or +inf, boundaries in lower bins}
        tab_s[i] = make_float2(e.x < INFINITY ? __fmaf_rn(-e.x, kGuardBig, 0.5f) : -INFINITY, e.y);
        if ((i & 15) == 0) bnd_s[i >> 4] = e.x;
    }
    const uint32_t table_lane = smem_u32(tab_s) + 8u * (lane & 15) - 0x80000000u;
    uint4* bfrag_s = reinterpret_cast<uint4*>(smem + W::kStageBytes + W::kTableBytes);
    uint8_t* out_s = smem + W::kStageBytes + W::kTableBytes + W::kBfragBytes;
    if (tid < kD) signs_s[tid] = p.signs[tid];
    __syncthreads();
    // B fragments: column n of n-tile j computes output dim 4 (n / 2) + 2 j + (n % 2) of the chunk,
    // so that a thread ends up with four consecutive dims (two code bytes) of its rows.
    for (int i = tid; i < 8 * 32 * 4; i += W::kThreads) {
        const int c = i >> 7, l = (i >> 2) & 31, r = i & 3;
        const int j = r >> 1, n = l >> 2, k0 = 2 * (l & 3) + 8 * (r & 1);
        const int dout = 4 * (n >> 1) + 2 * j + (n & 1);
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int k = k0 + e;
            const bool neg = ((__popc(k & dout) & 1) != 0) != (signs_s[16 * c + k] < 0.0f);
            w |= (neg ? O::kMinusOne : O::kOne) << (16 * e);
        }
        reinterpret_cast<uint32_t*>(bfrag_s)[i] = w;
    }
    grid_dependency_wait();  // K, V, the slots and the cache belong to earlier kernels
    __syncthreads();

    auto issue = [&](int64_t tile, int buf) {
        const int which = (int)(tile & 1);
        const int64_t row0 = (tile >> 1) * kRows;
        uint8_t* dst0 = smem + ((size_t)buf * W::kWarps + warp) * W::kWarpStage;
        fence_proxy_async();  // earlier shared-memory reads of this buffer precede the copy engine's writes
        if (TMA) {
            // two boxes of 16 rows x 64 elements; rows past the end of the tensor arrive as zeros
            if (lane == 0) {
                mbar_arrive_expect_tx(&full_bar[warp][buf], (uint32_t)(kRows * W::kRowBytes));
                tensor_g2s_2d(dst0, &p.tmap[which], 0, (int)row0, &full_bar[warp][buf]);
                tensor_g2s_2d(dst0 + 2048, &p.tmap[which], 64, (int)row0, &full_bar[warp][buf]);
            }
        } else {
            const int64_t left = rows - row0;
            const int64_t nrows = left < kRows ? left : (int64_t)kRows;
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[warp][buf], (uint32_t)(nrows * W::kRowBytes));
            __syncwarp();
            if (lane < nrows) {
                const int64_t r = row0 + lane;
                int64_t t;
                int h;
                split_row(r, H, p.head_shift, t, h);
                const T* src = reinterpret_cast<const T*>(p.src[which]) + t * p.token_stride[which] + (int64_t)h * kD;
                bulk_g2s(dst0 + (size_t)lane * kPitch, src, W::kRowBytes, &full_bar[warp][buf]);
            }
        }
    };

    // B fragment of the 8 x 8 identity: rows 2tg, 2tg + 1 of column g
    const uint32_t ident = (g == 2 * tg ? O::kOne : 0u) | (g == 2 * tg + 1 ? O::kOne << 16 : 0u);
    // ldmatrix: lane l supplies the address of row (l & 7) + 8 ((l >> 3) & 1), 16-byte piece (l >> 4) of the chunk
    const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1), lm_hi = lane >> 4;
    const int64_t warp_stride = (int64_t)gridDim.x * W::kWarps;
    int64_t tile = (int64_t)warp * gridDim.x + blockIdx.x;
    if (tile < num_tiles) issue(tile, 0);
    unsigned int stat_rows = 0, stat_exact = 0;  // this warp's share of g_guard_rows, added once at the end
    for (int it = 0; tile < num_tiles; tile += warp_stride, it++) {
        const int buf = it & 1;
        const int64_t next = tile + warp_stride;
        if (next < num_tiles) issue(next, buf ^ 1);

        const int which = (int)(tile & 1);
        const int64_t r = (tile >> 1) * kRows + row_in_warp;  // the row this lane stores
        const bool row_ok = r < rows;
        int64_t slot = -1;
        int h = 0;
        if (row_ok) {
            int64_t t;
            split_row(r, H, p.head_shift, t, h);
            slot = p.slot_is_i64 ? reinterpret_cast<const int64_t*>(p.slot_mapping)[t]
                                 : (int64_t) reinterpret_cast<const int32_t*>(p.slot_mapping)[t];
        }
        if (!mbar_wait(&full_bar[warp][buf], (it >> 1) & 1)) return;
        const uint8_t* stage = smem + ((size_t)buf * W::kWarps + warp) * W::kWarpStage;
        // Rows past the end of the tensor hold zeros or stale bytes: they are computed like any
        // others (whatever they contain ends in a finite code or in the exact path) and never stored.
        // byte address of 16-byte piece `piece` (0..15) of row `row` of the staged tile
        auto piece_addr = [&](int row, int piece) -> uint32_t {
            if (TMA) return smem_u32(stage) + (piece >> 3) * 2048 + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
            return smem_u32(stage) + row * kPitch + piece * 16;
        };

        // ---- chunk products (stages h = 1..8) and the exact sums of squares -----------------------
        P2 v[8][2][2];  // [chunk][n-tile][row half]: {dims 4tg + 2j, 4tg + 2j + 1} of rows g / g + 8
        P2 n_lo = pk(0.0f, 0.0f), n_hi = pk(0.0f, 0.0f);  // accumulators 2tg, 2tg+1 of rows g and g + 8
#pragma unroll
        for (int c = 0; c < 8; c++) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(piece_addr(lm_row, 2 * c + lm_hi), a0, a1, a2, a3);
            const uint4 b = bfrag_s[c * 32 + lane];
            float d0[4], d1[4], e0[4], e1[4];
            O::mma(d0, a0, a1, a2, a3, b.x, b.y);
            O::mma(d1, a0, a1, a2, a3, b.z, b.w);
            v[c][0][0] = pk(d0[0], d0[1]); v[c][0][1] = pk(d0[2], d0[3]);
            v[c][1][0] = pk(d1[0], d1[1]); v[c][1][1] = pk(d1[2], d1[3]);
            // The fp32 values of the fragment's own elements, for the squares: e0 = rows g / g + 8,
            // elements 8 (2c) + 2tg, +1; e1 = elements 8 (2c + 1) + 2tg, +1.
            O::mma(e0, a0, a1, a2, a3, ident, 0u);
            O::mma(e1, a0, a1, a2, a3, 0u, ident);
            P2 x2 = pk(e0[0], e0[1]); n_lo = add2(n_lo, mul2(x2, x2));
            x2 = pk(e0[2], e0[3]); n_hi = add2(n_hi, mul2(x2, x2));
            x2 = pk(e1[0], e1[1]); n_lo = add2(n_lo, mul2(x2, x2));
            x2 = pk(e1[2], e1[3]); n_hi = add2(n_hi, mul2(x2, x2));
        }
        // the eight accumulators of a row sit in its quad, two per lane: combine them left to right
        float norm_lo, norm_hi;
        {
            float l0, l1, h0, h1;
            up(n_lo, l0, l1);
            up(n_hi, h0, h1);
            const int qb = lane & ~3;
            float s_lo = __shfl_sync(0xffffffffu, l0, qb), s_hi = __shfl_sync(0xffffffffu, h0, qb);
            s_lo = __fadd_rn(s_lo, __shfl_sync(0xffffffffu, l1, qb));
            s_hi = __fadd_rn(s_hi, __shfl_sync(0xffffffffu, h1, qb));
#pragma unroll
            for (int t = 1; t < 4; t++) {
                s_lo = __fadd_rn(s_lo, __shfl_sync(0xffffffffu, l0, qb + t));
                s_hi = __fadd_rn(s_hi, __shfl_sync(0xffffffffu, h0, qb + t));
                s_lo = __fadd_rn(s_lo, __shfl_sync(0xffffffffu, l1, qb + t));
                s_hi = __fadd_rn(s_hi, __shfl_sync(0xffffffffu, h1, qb + t));
            }
            norm_lo = __fsqrt_rn(s_lo);
            norm_hi = __fsqrt_rn(s_hi);
            if (!(norm_lo >= 1e-8f)) norm_lo = (norm_lo != norm_lo) ? __uint_as_float(0x7fc00000u) : 1e-8f;
            if (!(norm_hi >= 1e-8f)) norm_hi = (norm_hi != norm_hi) ? __uint_as_float(0x7fc00000u) : 1e-8f;
        }
        const bool fast_lo = norm_lo > 1e-8f && norm_lo < 1e30f, fast_hi = norm_hi > 1e-8f && norm_hi < 1e30f;
        const float f_lo = __fmul_rn(p.fwht_scale, __frcp_rn(norm_lo)), f_hi = __fmul_rn(p.fwht_scale, __frcp_rn(norm_hi));

        // ---- stages h = 16, 32, 64 across the chunks ------------------------------------------------
#pragma unroll
        for (int hc = 1; hc < 8; hc <<= 1)
#pragma unroll
            for (int c = 0; c < 8; c++)
                if (!(c & hc)) {
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const P2 a = v[c][j][e], b = v[c | hc][j][e];
                            v[c][j][e] = add2(a, b);
                            v[c | hc][j][e] = sub2(a, b);
                        }
                }

        // ---- guarded codes: bytes 8c + 2tg and 8c + 2tg + 1 of rows g and g + 8 ---------------------
        uint8_t* orow_lo = out_s + (size_t)(warp * kRows + g) * W::kOutPitch + 2 * tg;
        uint8_t* orow_hi = orow_lo + 8 * W::kOutPitch;
        P2 amb_lo = pk(0.0f, 0.0f), amb_hi = pk(0.0f, 0.0f);
        const float zf_lo = f_lo * kGuardBig, zf_hi = f_hi * kGuardBig;
        const P2 kf_lo = pk(f_lo * 64.0f, f_lo * 64.0f), kf_hi = pk(f_hi * 64.0f, f_hi * 64.0f);
        // A row off the fast path (norm zero, huge or not finite) may hold values whose bin is not a
        // table index: it forms no lookup address at all.  The branch is uniform unless such a row
        // exists (the four lanes of a quad agree on their rows' flags).
        if (__all_sync(0xffffffffu, fast_lo && fast_hi)) {
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float b0 = guarded_byte(v[c][0][0], kf_lo, zf_lo, table_lane, amb_lo);
                const float b1 = guarded_byte(v[c][1][0], kf_lo, zf_lo, table_lane, amb_lo);
                *reinterpret_cast<uint16_t*>(orow_lo + 8 * c) =
                    (uint16_t)__float_as_uint(__fadd_rn(__fmaf_rn(b1, 256.0f, b0), 8388608.0f));
                const float b2 = guarded_byte(v[c][0][1], kf_hi, zf_hi, table_lane, amb_hi);
                const float b3 = guarded_byte(v[c][1][1], kf_hi, zf_hi, table_lane, amb_hi);
                *reinterpret_cast<uint16_t*>(orow_hi + 8 * c) =
                    (uint16_t)__float_as_uint(__fadd_rn(__fmaf_rn(b3, 256.0f, b2), 8388608.0f));
            }
        } else {
            if (fast_lo) {
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float b0 = guarded_byte(v[c][0][0], kf_lo, zf_lo, table_lane, amb_lo);
                    const float b1 = guarded_byte(v[c][1][0], kf_lo, zf_lo, table_lane, amb_lo);
                    *reinterpret_cast<uint16_t*>(orow_lo + 8 * c) =
                        (uint16_t)__float_as_uint(__fadd_rn(__fmaf_rn(b1, 256.0f, b0), 8388608.0f));
                }
            }
            if (fast_hi) {
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float b2 = guarded_byte(v[c][0][1], kf_hi, zf_hi, table_lane, amb_hi);
                    const float b3 = guarded_byte(v[c][1][1], kf_hi, zf_hi, table_lane, amb_hi);
                    *reinterpret_cast<uint16_t*>(orow_hi + 8 * c) =
                        (uint16_t)__float_as_uint(__fadd_rn(__fmaf_rn(b3, 256.0f, b2), 8388608.0f));
                }
            }
        }
        float al0, al1, ah0, ah1;
        up(amb_lo, al0, al1);
        up(amb_hi, ah0, ah1);
        // NaN compares false on "== 0": a row that produced NaNs is flagged as well
        const bool flag_lo = !fast_lo || !(__fadd_rn(al0, al1) == 0.0f);
        const bool flag_hi = !fast_hi || !(__fadd_rn(ah0, ah1) == 0.0f);
        uint32_t m_lo = __ballot_sync(0xffffffffu, flag_lo), m_hi = __ballot_sync(0xffffffffu, flag_hi);
        m_lo = (m_lo | (m_lo >> 1) | (m_lo >> 2) | (m_lo >> 3)) & 0x11111111u;  // bit 4g: row g flagged
        m_hi = (m_hi | (m_hi >> 1) | (m_hi >> 2) | (m_hi >> 3)) & 0x11111111u;
        stat_rows += kRows;
        stat_exact += __popc(m_lo) + __popc(m_hi);
        __syncwarp();

        // ---- exact path for the flagged rows: the whole warp on one row, lane L on elements 4L..4L+3 ---
        for (int half = 0; half < 2; half++) {
            uint32_t todo = half ? m_hi : m_lo;
            while (todo) {
                const int rr = (__ffs(todo) - 1) >> 2;
                todo &= todo - 1;
                float norm = __shfl_sync(0xffffffffu, half ? norm_hi : norm_lo, 4 * rr);
                const int row = rr + 8 * half;
                uint2 w;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w.x), "=r"(w.y)
                             : "r"(piece_addr(row, lane >> 1) + 8 * (lane & 1)));
                float x0, x1, x2, x3;
                up(O::unpack(w.x), x0, x1);
                up(O::unpack(w.y), x2, x3);
                if (norm != norm) {
                    // The identity products turn a row with an infinite element into NaNs (inf x 0).
                    // The sum of squares is NaN only if an element is; with infinities alone it is +inf.
                    const bool has_nan = __any_sync(0xffffffffu, x0 != x0 || x1 != x1 || x2 != x2 || x3 != x3);
                    if (!has_nan) {
                        norm = INFINITY;
                        if ((lane >> 2) == rr) {
                            if (half) norm_hi = norm;
                            else norm_lo = norm;
                        }
                    }
                }
                const float4 sg = *reinterpret_cast<const float4*>(&signs_s[4 * lane]);
                x0 = __fmul_rn(__fdiv_rn(x0, norm), sg.x);
                x1 = __fmul_rn(__fdiv_rn(x1, norm), sg.y);
                x2 = __fmul_rn(__fdiv_rn(x2, norm), sg.z);
                x3 = __fmul_rn(__fdiv_rn(x3, norm), sg.w);
                const float a0 = __fadd_rn(x0, x1), a1 = __fsub_rn(x0, x1), a2 = __fadd_rn(x2, x3), a3 = __fsub_rn(x2, x3);
                float y[4] = {__fadd_rn(a0, a2), __fadd_rn(a1, a3), __fsub_rn(a0, a2), __fsub_rn(a1, a3)};
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float o = __shfl_xor_sync(0xffffffffu, y[i], d);
                        y[i] = (lane & d) ? __fsub_rn(o, y[i]) : __fadd_rn(y[i], o);
                    }
                }
                float code[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float yy = __fmul_rn(y[i], p.fwht_scale);
                    if (yy != yy) {  // torch's bucketize sends NaN to the last bucket
                        code[i] = 15.0f;
                    } else {
                        const float kf = __fmaf_rn(yy, 64.0f, kBinMagic);
                        const uint32_t bin = __float_as_uint(kf) - 0x4B000000u;
                        const float below = tab_s[bin * 16 + (lane & 15)].y;
                        code[i] = yy > bnd_s[bin] ? __fadd_rn(below, 1.0f) : below;
                    }
                }
                const float both = __fadd_rn(__fmaf_rn(__fmaf_rn(code[2], 16.0f, code[3]), 256.0f,
                                                        __fmaf_rn(code[0], 16.0f, code[1])), 8388608.0f);
                *reinterpret_cast<uint16_t*>(out_s + (size_t)(warp * kRows + row) * W::kOutPitch + 2 * lane) =
                    (uint16_t)__float_as_uint(both);
            }
        }
        __syncwarp();

        // ---- store: two lanes per row, 32 code bytes each, the norm from lane m = 0 ------------------
        const float na = __shfl_sync(0xffffffffu, norm_lo, 4 * (row_in_warp & 7));
        const float nb = __shfl_sync(0xffffffffu, norm_hi, 4 * (row_in_warp & 7));
        const float norm = (row_in_warp & 8) ? nb : na;
        if (row_ok && slot >= p.total_slots) {
            if (m == 0 && h == 0 && which == 0) atomicAdd(&g_write_dropped, 1);
            slot = -1;
        }
        if (row_ok && slot >= 0) {
            const uint8_t* orow = out_s + (size_t)(warp * kRows + row_in_warp) * W::kOutPitch;
            uint8_t* dst = p.kv_cache + (size_t)which * p.slab_bytes + ((size_t)slot * H + h) * p.slot_bytes;
            const uint2* src8 = reinterpret_cast<const uint2*>(orow + 32 * m);
            const uint2 c0 = src8[0], c1 = src8[1], c2 = src8[2], c3 = src8[3];
            uint4* dst16 = reinterpret_cast<uint4*>(dst + 32 * m);
            dst16[0] = make_uint4(c0.x, c0.y, c1.x, c1.y);
            dst16[1] = make_uint4(c2.x, c2.y, c3.x, c3.y);
            if (m == 0) {
                const uint32_t nh = (norm != norm) ? 0x7e00u : (uint32_t)__half_as_ushort(__float2half_rn(norm));
                if (p.zero_pad) *reinterpret_cast<uint4*>(dst + 64) = make_uint4(nh | (nh << 16), 0u, 0u, 0u);
                else *reinterpret_cast<uint32_t*>(dst + 64) = nh | (nh << 16);
            }
        }
        __syncwarp();
    }
    if (lane == 0 && stat_rows) {
        atomicAdd(&g_guard_rows[0], (unsigned long long)stat_rows);
        if (stat_exact) atomicAdd(&g_guard_rows[1], (unsigned long long)stat_exact);
    }
}

// cuTensorMapEncodeTiled, looked up through the runtime (no link-time dependency on the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        tried = true;
    }
    return fn;
}

// [rows][128] 16-bit elements, row pitch 256 bytes, boxes of 16 rows x 64 elements with the 128-byte swizzle
static bool encode_rows_map(CUtensorMap* map, const void* base, int64_t rows, bool is_bf16) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)kD * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)MmaShape::kRows};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T>
static int launch_write_mma(WriteParams& p, int sm_count, cudaStream_t stream) {
    using W = MmaShape;
    const int64_t rows = p.num_tokens * p.num_kv_heads;
    // tensor copies need dense [rows][128] tensors whose row index fits the copy's 32-bit coordinate
    const bool dense = p.token_stride[0] == (int64_t)p.num_kv_heads * kD && p.token_stride[1] == (int64_t)p.num_kv_heads * kD &&
                       rows < (int64_t)0x7fffffff;
    const bool tma = dense && encode_rows_map(&p.tmap[0], p.src[0], rows, sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) &&
                     encode_rows_map(&p.tmap[1], p.src[1], rows, std::is_same<T, __nv_bfloat16>::value);
    auto kernel = tma ? write_kv_cache_mma_kernel<T, true> : write_kv_cache_mma_kernel<T, false>;
    static bool configured[2][64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[tma][dev]) {
        TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)W::kSmem));
        if (dev >= 0 && dev < 64) configured[tma][dev] = true;
    }
    const int64_t tiles = 2 * ((rows + W::kRows - 1) / W::kRows);
    const int64_t grid = tiles < (int64_t)sm_count ? tiles : (int64_t)sm_count;
    TQ_CUDA(launch_serialized(kernel, dim3((unsigned)grid), dim3(W::kThreads), W::kSmem, stream, p));
    return TQ_OK;
}

int write_guard_stats(unsigned long long* out2) {
    TQ_CUDA(cudaMemcpyFromSymbol(out2, g_guard_rows, 2 * sizeof(unsigned long long)));
    return TQ_OK;
}

int device_sm_count(int* out);
int generic_write(void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads, int slot_bytes, const void* key,
                  const void* value, int in_dtype, int64_t num_tokens, int64_t k_token_stride, int64_t v_token_stride,
                  const float* signs, const void* slot_mapping, int slot_dtype, int head_dim, int flags, void* stream);
int generic_fault_counts(int32_t* write_dropped, int32_t* dequant_skipped);

int write_fault_count(int32_t* out) {
    int32_t a = 0, b = 0, c = 0;
    TQ_CUDA(cudaMemcpyFromSymbol(&a, g_write_dropped, sizeof(int32_t)));
    int rc = generic_fault_counts(&b, &c);
    if (rc != TQ_OK) return rc;
    *out = a + b;
    return TQ_OK;
}

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
    TQ_REQUIRE(num_kv_heads >= 1 && block_size >= 1, TQ_ERR_INVALID, "bad geometry");
    TQ_REQUIRE(in_dtype == TQ_F32 || in_dtype == TQ_F16 || in_dtype == TQ_BF16, TQ_ERR_INVALID, "bad in_dtype");
    TQ_REQUIRE(slot_dtype == TQ_I32 || slot_dtype == TQ_I64, TQ_ERR_INVALID, "bad slot_dtype");
    if (head_dim != 128 && head_dim != 96) {  // other head sizes (64, 256, ...): the plain kernels
        TQ_REQUIRE(k_token_stride >= (int64_t)num_kv_heads * head_dim && v_token_stride >= (int64_t)num_kv_heads * head_dim,
                   TQ_ERR_INVALID, "token stride smaller than one token");
        TQ_REQUIRE((flags & TQ_WRITE_TENSOR_PATH) == 0, TQ_ERR_UNSUPPORTED,
                   "the tensor-core write kernel takes fp16 / bf16 rows of 128 elements");
        return generic_write(kv_cache, num_blocks, block_size, num_kv_heads, slot_bytes, key, value, in_dtype, num_tokens,
                             k_token_stride, v_token_stride, signs, slot_mapping, slot_dtype, head_dim, flags, stream);
    }
    TQ_REQUIRE(slot_bytes >= 80 && slot_bytes % 16 == 0, TQ_ERR_INVALID,
               "slot_bytes must be a multiple of 16 and >= 80, got %d", slot_bytes);
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
    p.total_slots = num_blocks * (int64_t)block_size;
    p.num_kv_heads = num_kv_heads;
    p.head_shift = -1;
    for (int sft = 0; sft < 16; sft++)
        if ((1 << sft) == num_kv_heads) p.head_shift = sft;
    p.block_size = block_size;
    p.slot_bytes = slot_bytes;
    p.slot_is_i64 = slot_dtype == TQ_I64;
    p.zero_pad = (flags & TQ_WRITE_ZERO_PAD) != 0;
    p.signs = signs;
    float cen[16], bnd[15];
    host_codebook(kD, 4, cen, bnd);
    {   // bins of y (same float operations as the kernel's code_f)
        int bin_of[15];
        for (int i = 0; i < 15; i++) {
            volatile float kf = fmaf(bnd[i], 64.0f, kBinMagic);
            float kff = kf;
            uint32_t bits;
            memcpy(&bits, &kff, 4);
            bin_of[i] = (int)(bits - 0x4B000000u);
            TQ_REQUIRE(bin_of[i] >= 0 && bin_of[i] < kBins && (i == 0 || bin_of[i] > bin_of[i - 1]), TQ_ERR_UNSUPPORTED,
                       "boundaries too close for the bin table");
            // the guarded kernel may look a value next to a bin edge up in either neighbour: no
            // boundary may sit that close to an edge (edges are at (k +- 1/2) / 64)
            const double pos = (double)bnd[i] * 64.0 - std::floor((double)bnd[i] * 64.0 + 0.5);
            TQ_REQUIRE(std::fabs(std::fabs(pos) - 0.5) * (1.0 / 64.0) > 1.0 / 8192.0, TQ_ERR_UNSUPPORTED,
                       "a boundary lies next to a bin edge");
        }
        for (int k = 0; k < kBins; k++) {
            int below = 0;
            float inside = INFINITY;  // no boundary in this bin: the comparison is never true
            for (int i = 0; i < 15; i++) {
                if (bin_of[i] < k) below++;
                if (bin_of[i] == k) inside = bnd[i];
            }
            p.bin_table[k] = make_float2(inside, (float)below);
        }
    }
    p.fwht_scale = (float)(1.0 / sqrt((double)kD));
    int sms = 0;
    int rc = device_sm_count(&sms);
    if (rc != TQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Large writes of 16-bit rows go to the tensor-core kernel; small ones (a decode step's new
    // tokens), fp32 rows and padded heads keep the kernel that needs no tables beyond one.
    const bool exact_only = (flags & TQ_WRITE_EXACT_PATH) != 0, tensor_only = (flags & TQ_WRITE_TENSOR_PATH) != 0;
    TQ_REQUIRE(!(exact_only && tensor_only), TQ_ERR_INVALID, "TQ_WRITE_EXACT_PATH and TQ_WRITE_TENSOR_PATH exclude each other");
    TQ_REQUIRE(!tensor_only || (head_dim == 128 && in_dtype != TQ_F32), TQ_ERR_UNSUPPORTED,
               "the tensor-core write kernel takes fp16 / bf16 rows of 128 elements");
    if (!exact_only && head_dim == 128 && in_dtype != TQ_F32 && (tensor_only || num_tokens * num_kv_heads >= 4096))
        return in_dtype == TQ_F16 ? launch_write_mma<__half>(p, sms, s) : launch_write_mma<__nv_bfloat16>(p, sms, s);
    if (head_dim == 96) {
        switch (in_dtype) {
            case TQ_F32: return launch_write<float, 96>(p, sms, s);
            case TQ_F16: return launch_write<__half, 96>(p, sms, s);
            default: return launch_write<__nv_bfloat16, 96>(p, sms, s);
        }
    }
    switch (in_dtype) {
        case TQ_F32: return launch_write<float, 128>(p, sms, s);
        case TQ_F16: return launch_write<__half, 128>(p, sms, s);
        default: return launch_write<__nv_bfloat16, 128>(p, sms, s);
    }
}

extern "C" int tq_write_guard_stats(int64_t* rows_total, int64_t* rows_exact) {
    TQ_REQUIRE(rows_total && rows_exact, TQ_ERR_INVALID, "null pointer");
    unsigned long long v[2] = {0, 0};
    int rc = tq::write_guard_stats(v);
    if (rc != TQ_OK) return rc;
    *rows_total = (int64_t)v[0];
    *rows_exact = (int64_t)v[1];
    return TQ_OK;
}
