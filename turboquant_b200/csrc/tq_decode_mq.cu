// Paged decode attention for WIDE query tiles (more than 8 and up to 32 query columns per KV head:
// several decode queries that share one sequence's KV, times the GQA ratio; causal query chunks),
// on the 5th-generation tensor cores: tcgen05.mma with the accumulators and one operand in tensor
// memory.
//
// The mma.sync kernel (tq_decode.cu) holds eight query columns in registers; 32 columns would need
// 128 accumulator registers per thread, so a query tile of 8 queries x GQA 4 made four passes over
// the KV there.  Here one pass serves all 32 columns: S = K^ Q^T (128 tokens x 32 columns),
// O^T = V^^T P (128 dims x 32 columns) and the column sums of P all live in tensor memory.
//
// The reference has no counterpart: its decode op takes one query per batch row
// (csrc/src/decode_v5_tc_binding.cu:783-785) and re-reads the KV for each.  The per-tile arithmetic
// is that of csrc/include/flashinfer_decode_turboquant_v5_tc.cuh:307-627 (dequantize through the
// codebook, rotated-domain QK^T, online softmax, PV), the partial / LSE contract that of
// csrc/include/flashinfer_decode_turboquant_combine.cuh:18-79, merged by merge_kernel (tq_decode.cu).
//
// One thread block = one KV-head PAIR of a contiguous page range (the device-side plan of the
// other kernel, over gridDim.x / (heads / 2) ranges).  896 threads in seven warpgroups:
//   warps 0-3    control: warp 0 streams the raw K pages and warp 2 the raw V pages (tiled tensor
//                copies: boxes of 16 tokens x 160 bytes = both heads' slots, each into its own ring of
//                four 64-token stages); warp 1 issues S = K^ Q^T, warp 3 issues O^T += V^^T P and the
//                column sums (one elected lane, compile-time descriptors, tcgen05.commit on mbarriers);
//   warps 4-7    softmax of the pair's first head, warps 8-11 of its second head: thread t owns
//                token t of the 128-token tile: reads its row of S from tensor memory once, hands
//                the buffer back, applies the K norm and the scale, keeps a lazily raised running
//                maximum per column, writes P = exp2(x - m) as fp16 to shared memory;
//   warps 12-19  dequantize K, warps 20-27 dequantize V: 32 code bytes per thread and tile-head
//                through the lookup table (one lookup per code byte, as in the other kernel).
// K^ goes to TENSOR MEMORY with tcgen05.st: the A operand of S = K^ Q^T may live there (lane =
// token, two fp16 per column; 64 columns per head), which keeps it out of the shared-memory pipe.
// V^ (times the token's V norm, zero for tokens past the sequence) goes to shared memory in the
// un-swizzled MN-major core-matrix layout, 32 KB per head.  The column sums l = sum_t P[t][c] come
// from the tensor core as well: P against a block of ones in tensor memory, so every row of that
// accumulator holds the sums and the softmax threads keep no running sums in registers.
// S is double-buffered per head; K^, S and V^ of a head run ahead of its softmax.
// Q^T (per head: 32 columns x 128 dims, fp16), P of the first head (128 tokens x 32 columns) and
// the K norms live in the unused upper halves of the lookup table's 256-byte rows: a core matrix is
// exactly 128 bytes.  P of the second head has a buffer of its own.
// Tensor memory (512 columns allocated, 448 used): O^T 2 x 32, K^ 2 x 64, S 4 x 32, ones 64, sums 2 x 32.
//
// Every wait is bounded; a wait that runs out raises the sticky status word, the block stops
// taking work, frees its tensor memory and returns.
#include <cuda.h>  // CUtensorMap and its enums only: the encoder is looked up at run time

#include <cmath>
#include <cstring>

#include "tq_decode_common.cuh"

namespace tq {

constexpr int kMqThreads = 896;
constexpr int kMqCols = 32;            // query columns per KV head (shorter tiles are padded with zeros)
constexpr int kMqTile = 128;           // tokens per tile
constexpr int kMqStages = 4;           // per ring (K, V)
constexpr int kMqBoxBytes = 16 * 160;  // one page half of a head pair
constexpr int kMqStageBytes = 4 * kMqBoxBytes;  // 4 pages of K or of V
constexpr int kMqOperandHalf = 16384;  // half of one head's V^: 64 tokens x 128 dims x 2 bytes
constexpr uint32_t kMqWaitLimit = 1u << 18;   // tries per wait: at most about a quarter of a second
constexpr uint32_t kMqSuspendNs = 1000;       // suspend-time hint of one try
constexpr int kMqTmemCols = 512;       // O^T (32 columns per head), K^ (64 per head), S (2 x 32 per head), a block of
                                       // ones (64) and the column sums (32 per head): 448 used

// shared-window offsets: the K ring and half of the V ring below the table, the table (with Q^T, one P
// and the norms in its holes), then the operand buffers, the rest of the V ring and the other P
constexpr uint32_t kMqRawK = 4096;                              // 4 x 10240
constexpr uint32_t kMqRawV01 = kMqRawK + 4 * kMqStageBytes;     // 2 x 10240, ends at 65536
constexpr uint32_t kMqVhat = kLutAddr + kLutSpan;               // 32 KB per head: 64 KB
constexpr uint32_t kMqRawV23 = kMqVhat + 4 * kMqOperandHalf;    // 2 x 10240
constexpr uint32_t kMqP1 = kMqRawV23 + 2 * kMqStageBytes;       // 8 KB: [16 token groups][4 column groups][8][16 B]
constexpr uint32_t kMqSmemEnd = kMqP1 + 8192;                   // 225280
static_assert(kMqRawV01 + 2 * kMqStageBytes == kLutAddr, "the rings below the table end where it starts");

__device__ __forceinline__ uint32_t mq_hole(int i) { return kLutAddr + 256u * (uint32_t)i + 128u; }
// holes: [0, 128) Q^T of the two heads, [128, 192) P of the first head, [192, 224) K norms (8 tile-heads x 128
// floats: K^ of a head runs up to three tiles ahead of its softmax), [240, 248)
// per-column scratch of the two softmax groups, [248, 250) the running maxima
constexpr int kHoleQ = 0, kHoleP = 128, kHoleNormK = 192, kHoleCol = 240, kHoleMax = 248;

struct MqParams {
    DecodeParams d;
    alignas(64) CUtensorMap cache_map;  // uint8 [2][num_blocks * 16][H * 80], boxes of [1][16][160]
    int head_pairs;                     // KV heads / 2
    int ncols;                          // valid query columns per KV head (queries x GQA ratio)
    int causal;                         // query i of n sees the first len - (n - 1 - i) tokens of its sequence
};

// Bounded wait of a whole warp; the answer is the same in every lane.  The try carries a suspend-time
// hint: a waiting warp sleeps in the barrier unit until the phase completes (or the hint runs out)
// instead of spinning through the issue slots of the warps that have work.
__device__ __forceinline__ bool mq_try_wait_hint(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kMqSuspendNs)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mq_wait(uint64_t* bar, uint32_t parity) {
    bool done = false;
    for (uint32_t i = 0; i < kMqWaitLimit && !done; i++) done = mq_try_wait_hint(bar, parity);
    return __all_sync(0xffffffffu, done);
}

__host__ __device__ constexpr uint64_t mq_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46);  // version 1, no swizzle
}

__device__ __forceinline__ void mq_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// the same with the A operand in tensor memory (lane = row, two 16-bit elements per column)
__device__ __forceinline__ void mq_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mq_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
          "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&a)[4], const uint32_t (&b)[4]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                 ::"r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tiled tensor copy of one box [1][16 tokens][160 bytes] at (x = byte in the token row, y = token, z = K / V)
__device__ __forceinline__ void mq_box_g2s(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void bar_sync_named(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

__global__ void __launch_bounds__(kMqThreads, 1) decode_mq_kernel(const __grid_constant__ MqParams mp) {
    const DecodeParams& p = mp.d;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t rawk_full[kMqStages], rawk_empty[kMqStages], rawv_full[kMqStages], rawv_empty[kMqStages];
    __shared__ __align__(8) uint64_t kq_full[2], kq_empty[2], vq_full[2], vq_empty[2], s_full[4], s_empty[4], p_full[2], p_empty[2], o_done[2];
    __shared__ int seg_seq[kMaxSegments], seg_p0[kMaxSegments], seg_p1[kMaxSegments];
    __shared__ int num_segments, abort_flag;
    __shared__ uint32_t tmem_slot;
    __shared__ int raise_flag[16];   // [tile parity][head][warp]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = smem_u32(smem);
    grid_launch_dependents();
    // the map above assumes that the dynamic shared memory starts below kMqRawK of the shared window
    if (smem_base > kMqRawK) {
        grid_dependency_wait();
        if (tid == 0) atomicExch(&p.header[0], 3);
        return;
    }
    auto rawk_addr = [&](int s) -> uint32_t { return kMqRawK + (uint32_t)s * kMqStageBytes; };
    auto rawv_addr = [&](int s) -> uint32_t {
        return s < 2 ? kMqRawV01 + (uint32_t)s * kMqStageBytes : kMqRawV23 + (uint32_t)(s - 2) * kMqStageBytes;
    };
    uint32_t* lut_s = reinterpret_cast<uint32_t*>(smem + (kLutAddr - smem_base));

    if (tid == 0) {
        for (int s = 0; s < kMqStages; s++) {
            mbar_init(&rawk_full[s], 1);
            mbar_init(&rawk_empty[s], 4);   // the four K warps that read the stage's tokens
            mbar_init(&rawv_full[s], 1);
            mbar_init(&rawv_empty[s], 4);   // the four V warps that read the stage's tokens
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&kq_full[i], 8);    // per head: K^ of a tile-head is in tensor memory
            mbar_init(&kq_empty[i], 1);   // per head: its S has been computed
            mbar_init(&vq_full[i], 8);    // per head: V^ of a tile-head is in shared memory
            mbar_init(&vq_empty[i], 1);   // per head: its PV has been computed
            for (int j = 0; j < 2; j++) {
                mbar_init(&s_full[2 * i + j], 1);     // [head][parity of the tile]: S is double-buffered per head
                mbar_init(&s_empty[2 * i + j], 4);
            }
            mbar_init(&p_full[i], 4);
            mbar_init(&p_empty[i], 1);
            mbar_init(&o_done[i], 1);   // one phase per segment: the head's last PV has completed
        }
        num_segments = 0;
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // ---- plan (warp 0) and lookup table (the other warps), as in decode_paged_kernel ---------------
    const int hp = blockIdx.x % mp.head_pairs;       // KV-head pair of this block
    const int c = blockIdx.x / mp.head_pairs;        // page range of this block
    const int n_ranges = gridDim.x / mp.head_pairs;
    constexpr int PPS = kMqTile / kPageTokens;       // pages per tile
    if (warp != 0) {
        for (int i = tid - 32; i < 256 * 32; i += kMqThreads - 32) {
            const int v = i >> 5;
            lut_s[v * 64 + (i & 31)] = (uint32_t)p.centroid_h[v & 15] | ((uint32_t)p.centroid_h[v >> 4] << 16);
        }
        grid_dependency_wait();
    } else {
        grid_dependency_wait();
        int total_real = 0, nonempty = 0;
        bool too_long = false;
        for (int base = 0; base < p.batch; base += 32) {
            int np = 0, fp = 0, le;
            if (base + lane < p.batch) {
                seq_pages(p, base + lane, fp, np, le);
                const int have = p.page_indptr ? p.page_indptr[base + lane + 1] - p.page_indptr[base + lane] : p.max_pages;
                too_long |= np > 0 && fp + np > have;
            }
            nonempty += __popc(__ballot_sync(0xffffffffu, np > 0));
            for (int o = 16; o > 0; o >>= 1) np += __shfl_xor_sync(0xffffffffu, np, o);
            total_real += np;
        }
        if (__any_sync(0xffffffffu, too_long)) {
            if (blockIdx.x == 0) {
                for (int b = lane; b <= p.batch; b += 32) p.page_prefix[b] = 0;
                if (lane == 0) {
                    p.header[1] = 1;
                    p.header[2] = 0;
                    p.header[3] = 0;
                    atomicExch(&p.header[0], kStatusSeqTooLong);
                }
            }
            total_real = -1;
        }
        int n_eff = (total_real + PPS - 1) / PPS;   // at least one tile per block
        n_eff = n_eff < 1 ? 1 : (n_eff > n_ranges ? n_ranges : n_eff);
        const int seg_cost = total_real / n_eff >= 8 * PPS ? PPS : 0;   // a sequence start costs about one tile
        const int total = total_real + nonempty * seg_cost;
        const int64_t lo = c < n_eff ? ((int64_t)c * total) / n_eff : 0;
        const int64_t hi = c < n_eff ? ((int64_t)(c + 1) * total) / n_eff : 0;
        int run = 0, nseg = 0;
        for (int base = 0; base < p.batch && total_real >= 0; base += 32) {
            int np = 0, fp = 0, le;
            const int b = base + lane;
            if (b < p.batch) seq_pages(p, b, fp, np, le);
            const int vnp = np > 0 ? np + seg_cost : 0;
            int incl = vnp;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const int vstart = run + incl - vnp, end = run + incl, start = vstart + seg_cost;
            if (blockIdx.x == 0 && b < p.batch) p.page_prefix[b] = vstart;
            const bool hit = b < p.batch && np > 0 && start < hi && end > lo;
            const uint32_t mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int slot = nseg + __popc(mask & ((1u << lane) - 1u));
                if (slot < kMaxSegments) {
                    seg_seq[slot] = b;
                    seg_p0[slot] = (int)((lo > start ? lo : start) - start);
                    seg_p1[slot] = (int)((hi < end ? hi : end) - start);
                }
            }
            nseg += __popc(mask);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0 && total_real >= 0) {
            if (blockIdx.x == 0) {
                p.page_prefix[p.batch] = run;
                p.header[1] = n_eff;
                p.header[2] = total;
                p.header[3] = seg_cost;
            }
            if (nseg > kMaxSegments) {
                atomicExch(&p.header[0], 2);
                nseg = 0;
            }
            num_segments = nseg;
        }
    }
    __syncthreads();
    const int nseg = num_segments;
    if (nseg == 0) return;   // uniform: nothing allocated yet

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kMqTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // O^T at +32 h2, K^ at +64 h2, S at +64 h2 + 32 (tile parity)
    const uint32_t tm_o0 = tmem, tm_k0 = tmem + 64, tm_s0 = tmem + 192, tm_ones = tmem + 320, tm_l0 = tmem + 384;

    if (warp >= 4 && warp < 8) {   // 128 lanes x 64 columns of half2(1, 1)
        uint32_t ones[16];
#pragma unroll
        for (int i = 0; i < 16; i++) ones[i] = 0x3C003C00u;
#pragma unroll
        for (int i = 0; i < 4; i++) tmem_st16(tm_ones + 16 * i + ((uint32_t)((warp & 3) * 32) << 16), ones);
        tc_fence_before();
    }
    // The roles part here for good: each lowers or raises its register count first, runs its own loop
    // over the block's segments, and meets the others only at barrier 1 (twice per segment: the rotated
    // queries are in place / the segment has drained).  u counts tile-heads and tile_n tiles across the
    // segments; they fix the barrier phases and advance identically in every role.
    // Register budget per scheduler (one control, two softmax, four dequantize warps of the 512 warp-registers):
    // 40 + 2 x 104 + 4 x 64 = 504.  An exact fit (control at 48) never got its registers: setmaxnreg.inc waits.
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        int u = 0, tile_n = 0;
        for (int sg = 0; sg < nseg; sg++) {
            const int b = seg_seq[sg];
            int first_page, npages_b, len_eff;
            seq_pages(p, b, first_page, npages_b, len_eff);
            const int p0 = seg_p0[sg], p1 = seg_p1[sg];
            const int ntiles = (p1 - p0 + PPS - 1) / PPS;
            bar_sync_named(1, kMqThreads);
            if (warp == 0 || warp == 2) {
                // =============================== producers: raw K pages (warp 0), raw V pages (warp 2) =====
                const int z = warp >> 1;
                uint64_t* full = z ? rawv_full : rawk_full;
                uint64_t* empty = z ? rawv_empty : rawk_empty;
                const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
                bool bad_page = false;
                for (int t = 0; t < ntiles && !abort_flag; t++) {
                    const int n = tile_n + t;
                    for (int rs = 0; rs < 2; rs++) {
                        const int st = (2 * n + rs) & 3;
                        const int pg0 = p0 + t * PPS + rs * 4;
                        const int np = min(4, p1 - pg0);        // pages of this stage (may be <= 0 in the last tile)
                        if (n >= 2 && !mq_wait(&empty[st], ((n >> 1) - 1) & 1)) {
                            abort_flag = 1;
                            atomicExch(&p.header[0], 1);
                            break;
                        }
                        int page = 0;
                        if (lane < 4 && lane < np) {
                            page = p.page_indices[tbl + first_page + pg0 + lane];
                            if ((uint64_t)(int64_t)page >= (uint64_t)p.num_blocks) {
                                page = 0;
                                bad_page = true;
                            }
                        }
                        if (lane == 0) mbar_arrive_expect_tx(&full[st], (uint32_t)((np > 0 ? np : 0) * kMqBoxBytes));
                        __syncwarp();
                        if (lane < 4 && lane < np)
                            mq_box_g2s((z ? rawv_addr(st) : rawk_addr(st)) + lane * kMqBoxBytes, &mp.cache_map,
                                       hp * 160 + p.kv_head_off, page * kPageTokens, z, &full[st]);
                    }
                }
                if (bad_page && lane == 0) atomicExch(&p.header[0], kStatusBadPage);
            } else {
                // =============================== tensor-core issue ======================================
                // Warp 1 issues S = K^ Q^T and warp 3 O^T += V^^T P, each in tile-head order: S of a later
                // tile-head never waits behind a PV that is still waiting for its softmax.  One elected lane
                // issues; every descriptor is a compile-time constant (the head is unrolled).
                constexpr uint32_t idesc_qk = (1u << 4) | ((uint32_t)(kMqCols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                constexpr uint32_t idesc_pv = idesc_qk | (1u << 15) | (1u << 16);
                constexpr uint32_t idesc_l = idesc_qk | (1u << 16);   // A (ones) from tensor memory, B = P with the columns contiguous
                bool ok = true;
                for (int t = 0; t < ntiles && ok && !abort_flag; t++) {
#pragma unroll
                    for (int h2 = 0; h2 < 2; h2++) {
                        const int uu = u + 2 * t + h2;   // u is even: buffers that alternate with uu are the head's
                        if (warp == 1) {
                            if (ok) ok = mq_wait(&kq_full[h2], (uu >> 1) & 1);
                            const int tg = uu >> 1, sp = tg & 1;   // tile counter of the block, S buffer of the head
                            if (ok && tg >= 2) ok = mq_wait(&s_empty[2 * h2 + sp], ((tg >> 1) - 1) & 1);
                            if (!ok) break;
                            tc_fence_after();
                            if (elect_one()) {
#pragma unroll
                                for (int j = 0; j < 8; j++) {   // K^ from tensor memory, 8 columns (16 positions) per instruction
                                    constexpr uint64_t dq0 = mq_desc(kLutAddr + 128u, 1024, 256);
                                    const uint64_t db = dq0 + (uint64_t)(((h2 * 64 + 2 * j * 4) * 256) >> 4);
                                    mq_mma_ts(tm_s0 + 64 * h2 + 32 * sp, tm_k0 + 64 * h2 + 8 * j, db, idesc_qk, j ? 1u : 0u);
                                }
                                mq_commit(&kq_empty[h2]);
                                mq_commit(&s_full[2 * h2 + sp]);
                            }
                            __syncwarp();
                        } else {
                            if (ok) ok = mq_wait(&p_full[h2], (uu >> 1) & 1);
                            if (ok) ok = mq_wait(&vq_full[h2], (uu >> 1) & 1);
                            if (!ok) break;
                            tc_fence_after();
                            if (elect_one()) {
                                constexpr uint64_t dp0 = mq_desc(kLutAddr + 128u + 256u * kHoleP, 1024, 256);
                                constexpr uint64_t dp1 = mq_desc(kMqP1, 512, 128);
#pragma unroll
                                for (int j = 0; j < 8; j++) {   // 16 tokens per instruction
                                    const uint64_t da = mq_desc(kMqVhat + h2 * 2 * kMqOperandHalf, 2048, 128) + (uint64_t)((j * 4096) >> 4);
                                    const uint64_t db = h2 ? dp1 + (uint64_t)((j * 2 * 512) >> 4) : dp0 + (uint64_t)((j * 2 * 4 * 256) >> 4);
                                    mq_mma(tm_o0 + 32 * h2, da, db, idesc_pv, j ? 1u : (uint32_t)(t > 0));
                                }
                                // column sums of P: the same B operand against a block of ones in tensor memory; every
                                // row of the result holds l[column] = sum over the tile's tokens of P[token][column]
#pragma unroll
                                for (int j = 0; j < 8; j++) {
                                    const uint64_t db = h2 ? dp1 + (uint64_t)((j * 2 * 512) >> 4) : dp0 + (uint64_t)((j * 2 * 4 * 256) >> 4);
                                    mq_mma_ts(tm_l0 + 32 * h2, tm_ones + 8 * (j & 3), db, idesc_l, j ? 1u : (uint32_t)(t > 0));
                                }
                                mq_commit(&vq_empty[h2]);
                                mq_commit(&p_empty[h2]);
                                if (t == ntiles - 1) mq_commit(&o_done[h2]);
                            }
                            __syncwarp();
                        }
                    }
                }
                if (!ok && !abort_flag) {
                    abort_flag = 1;
                    if (lane == 0) atomicExch(&p.header[0], 1);
                }
            }
            u += 2 * ntiles;
            tile_n += ntiles;
            bar_sync_named(1, kMqThreads);   // every instruction of this segment has completed before Q^T and tensor memory are reused
            if (abort_flag) break;
        }
        tc_fence_before();
        bar_sync_named(1, kMqThreads);
        if (warp == 0) {
            tc_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kMqTmemCols));
        }
        return;
    }
    if (warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        const bool vteam = warp >= 20;
        const int dt = (tid - 384) & 255;   // thread of its team
        const uint32_t lut_lane = kLutAddr + 4u * lane;
        int u = 0, tile_n = 0;
        for (int sg = 0; sg < nseg; sg++) {
            const int b = seg_seq[sg];
            int first_page, npages_b, len_eff;
            seq_pages(p, b, first_page, npages_b, len_eff);
            const int p0 = seg_p0[sg], p1 = seg_p1[sg];
            const int ntiles = (p1 - p0 + PPS - 1) / PPS;
            // ---- rotated queries of both heads into the Q^T holes (4 columns per warp) ----------------
            {
            const float4 sg4 = reinterpret_cast<const float4*>(p.signs)[lane];
            for (int rr = warp - 12; rr < 2 * kMqCols; rr += 16) {
                const int h2 = rr >> 5, col = rr & 31;
                float w[4] = {0.f, 0.f, 0.f, 0.f};
                if (col < mp.ncols && 4 * lane < p.head_dim) {
                    const int qi = col / p.real_group, hh = col - qi * p.real_group;
                    const int64_t base = ((((int64_t)b * p.nq + qi) * p.real_heads) + (2 * hp + h2) * p.real_group + hh) *
                                             p.head_dim + 4 * lane;
#pragma unroll
                    for (int i = 0; i < 4; i++) w[i] = load_q(p.q, p.q_dtype, base + i);
                }
                w[0] *= sg4.x; w[1] *= sg4.y; w[2] *= sg4.z; w[3] *= sg4.w;
                const float a0 = w[0] + w[1], a1 = w[0] - w[1], a2 = w[2] + w[3], a3 = w[2] - w[3];
                w[0] = a0 + a2; w[1] = a1 + a3; w[2] = a0 - a2; w[3] = a1 - a3;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float o = __shfl_xor_sync(0xffffffffu, w[i], d);
                        w[i] = (lane & d) ? o - w[i] : w[i] + o;
                    }
                }
                // contraction position 2i holds dim 2i + 1 and vice versa (a code byte dequantizes to
                // {low half: odd dim, high half: even dim}); lane l has positions 4l .. 4l + 3 of unit l / 2
                const uint32_t lo = pack_half2(w[1] * 0.08838834764831845f, w[0] * 0.08838834764831845f);
                const uint32_t hi = pack_half2(w[3] * 0.08838834764831845f, w[2] * 0.08838834764831845f);
                const int kk = lane >> 1;
                const uint32_t addr = mq_hole(kHoleQ + h2 * 64 + kk * 4 + (col >> 3)) + (col & 7) * 16 + (lane & 1) * 8;
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
            }
            fence_proxy_async();
            }
            bar_sync_named(1, kMqThreads);
            bool ok = true;
            if (!vteam) {
                // =============================== dequantize K ========================================
                // thread = (token, 32 of its 64 code bytes): K^ goes to TENSOR MEMORY, where it is the A operand of
                // S = K^ Q^T: lane = token, column c = contraction positions 2c, 2c + 1 (one half2), 64 columns per
                // tile-head, one buffer per head of the pair.  The warp's 32 tokens are its lane quarter and lie in
                // one raw stage.  (Lanes four tokens apart would meet in the same banks, 4 x 160 bytes = 5 x 128:
                // they read their two 16-byte pieces in opposite order.)
                const int tok = dt & 127, piece = dt >> 7, swap = (tok >> 2) & 1;
                const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
                for (int t = 0; t < ntiles && ok && !abort_flag; t++) {
                    const int n = tile_n + t;
                    const int st = (2 * n + (tok >> 6)) & 3;
                    ok = mq_wait(&rawk_full[st], (n >> 1) & 1);
                    const uint32_t krow0 = rawk_addr(st) + ((tok & 63) >> 4) * kMqBoxBytes + (tok & 15) * 160;
                    for (int h2 = 0; h2 < 2 && ok; h2++) {
                        const int uu = u + 2 * t + h2;   // u is even: the head's own buffer and barriers
                        const uint32_t krow = krow0 + h2 * 80 + 16 * piece;
                        const uint4 ca = lds128(krow + 32 * swap), cb = lds128(krow + 32 * (swap ^ 1));
                        if (piece == 0)   // the K norms of the tile, times the scales, for the softmax warps
                            sts32f(mq_hole(kHoleNormK + (uu & 7) * 4 + (tok >> 5)) + (tok & 31) * 4, lds_half(krow0 + h2 * 80 + 64) * p.k_scale);
                        if ((uu >> 1) >= 1) ok = mq_wait(&kq_empty[h2], ((uu >> 1) - 1) & 1);   // S of the head's previous tile is done
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            const uint4 cw = (hh == 0) == (swap == 0) ? ca : cb;
                            const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                            for (int w2 = 0; w2 < 2; w2++) {   // eight columns (two code words) per store
                                uint32_t ra[4], rb[4];
                                dequant8(w4[2 * w2], lut_lane, ra);
                                dequant8(w4[2 * w2 + 1], lut_lane, rb);
                                tmem_st8(tm_k0 + 64 * h2 + 32 * hh + 16 * piece + 8 * w2 + lane_base, ra, rb);
                            }
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(&kq_full[h2]);
                            if (h2 == 1) mbar_arrive(&rawk_empty[st]);   // both heads have read this stage
                        }
                    }
                }
            } else {
                // =============================== dequantize V ========================================
                // thread = (token, 32 of its 64 code bytes): one step per tile-head.  The warp's 32 tokens lie in one
                // raw stage; lanes four tokens apart read their two 16-byte pieces in opposite order (banks).
                const int tok = dt & 127, pc2 = dt >> 7, swap = (tok >> 2) & 1;
                for (int t = 0; t < ntiles && ok && !abort_flag; t++) {
                    const int n = tile_n + t;
                    const int st = (2 * n + (tok >> 6)) & 3;
                    ok = mq_wait(&rawv_full[st], (n >> 1) & 1);
                    const uint32_t vrow0 = rawv_addr(st) + ((tok & 63) >> 4) * kMqBoxBytes + (tok & 15) * 160;
                    // The row's norm times the scale is folded into V^ (P then holds the bare weights, whose column
                    // sums the tensor core forms).  A token past the sequence or past this block's pages gets the
                    // factor zero: whatever its slot holds, its V^ row is exactly zero.
                    const int tok_rel = (p0 + t * PPS) * kPageTokens + tok;
                    const bool valid = first_page * kPageTokens + tok_rel < len_eff && tok_rel < p1 * kPageTokens;
                    for (int h2 = 0; h2 < 2 && ok; h2++) {
                        const int uu = u + 2 * t + h2;
                        const uint32_t vrow = vrow0 + h2 * 80 + 32 * pc2;
                        const uint4 ca = lds128(vrow + 16 * swap), cb = lds128(vrow + 16 * (swap ^ 1));
                        const float vf = valid ? lds_half(vrow0 + h2 * 80 + 64) * p.v_scale : 0.f;
                        const uint32_t vf2 = pack_half2(vf, vf);
                        if ((uu >> 1) >= 1) ok = mq_wait(&vq_empty[h2], ((uu >> 1) - 1) & 1);   // the head's PV of the tile before
                        if (!ok) break;
                        const uint32_t dst = kMqVhat + h2 * 2 * kMqOperandHalf + (tok >> 3) * 2048 + (8 * pc2) * 128 + (tok & 7) * 16;
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const uint4 cw = (q == 0) == (swap == 0) ? ca : cb;
                            const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                            for (int w = 0; w < 4; w++) {
                                uint32_t r[4];
                                dequant8(w4[w], lut_lane, r);
                                sts128(dst + (4 * q + w) * 128, hmul2(r[0], vf2), hmul2(r[1], vf2), hmul2(r[2], vf2), hmul2(r[3], vf2));
                            }
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(&vq_full[h2]);
                            if (h2 == 1) mbar_arrive(&rawv_empty[st]);   // both heads have read this stage
                        }
                    }
                }
            }
            if (!ok && !abort_flag) {
                abort_flag = 1;
                if (lane == 0) atomicExch(&p.header[0], 1);
            }
            u += 2 * ntiles;
            tile_n += ntiles;
            bar_sync_named(1, kMqThreads);   // every instruction of this segment has completed before Q^T and tensor memory are reused
            if (abort_flag) break;
        }
        tc_fence_before();
        bar_sync_named(1, kMqThreads);
        return;
    }
    // =============================== softmax ======================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    {
        int u = 0, tile_n = 0;
        for (int sg = 0; sg < nseg; sg++) {
            const int b = seg_seq[sg];
            int first_page, npages_b, len_eff;
            seq_pages(p, b, first_page, npages_b, len_eff);
            const int p0 = seg_p0[sg], p1 = seg_p1[sg];
            const int ntiles = (p1 - p0 + PPS - 1) / PPS;
            bar_sync_named(1, kMqThreads);
            {
            const int h2 = (warp - 4) >> 2;
            const int stid = (tid - 128) & 127;              // token of the tile = lane of tensor memory
            const int wq = warp & 3;
            const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
            const uint32_t tm_o = tm_o0 + 32 * h2, tm_l = tm_l0 + 32 * h2;
            const int bar_id = 2 + h2;
            const int hole_col = kHoleCol + 4 * h2;
            if (stid < kMqCols) sts32f(mq_hole(kHoleMax + h2) + stid * 4, -INFINITY);
            bar_sync_named(bar_id, 128);
            // The four warps of a group meet at named barriers inside this loop, so none of them may leave it
            // early: a warp whose wait ran out (or that saw another role give up) only stops waiting, working
            // and signalling, and still walks through every barrier of every tile.
            bool ok = true;
            for (int t = 0; t < ntiles; t++) {
                const int tok_global = (first_page + p0 + t * PPS) * kPageTokens + stid;
                const bool valid = tok_global < len_eff && (p0 + t * PPS) * kPageTokens + stid < (p1 * kPageTokens);
                const int uu = u + 2 * t + h2;
                // causal queries: column cc belongs to query cc / group, which sees this token iff cc >= cmin
                const int cmin = mp.causal ? (p.nq - len_eff + tok_global) * p.real_group : 0;
                if (abort_flag) ok = false;
                const int tg = uu >> 1, sp = tg & 1;
                if (ok) ok = mq_wait(&s_full[2 * h2 + sp], (tg >> 1) & 1);
                tc_fence_after();
                const float kf = lds32f(mq_hole(kHoleNormK + (uu & 7) * 4 + (stid >> 5)) + (stid & 31) * 4);
                // The token's row of S: read once, kept in registers (the column sums are not kept here: the tensor
                // core forms them, see the issue warp), and the S buffer is handed back at once.
                uint32_t sr[32];
                if (ok) tmem_ld32(tm_s0 + 64 * h2 + 32 * sp + lane_base, sr);
                tc_fence_before();
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&s_empty[2 * h2 + sp]);
                bool raise = false;
                if (ok) {
#pragma unroll
                    for (int cc = 0; cc < kMqCols; cc += 4) {
                        const uint4 mv = lds128(mq_hole(kHoleMax + h2) + cc * 4);
                        const float m4[4] = {__uint_as_float(mv.x), __uint_as_float(mv.y), __uint_as_float(mv.z), __uint_as_float(mv.w)};
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            raise |= valid && cc + i >= cmin && __uint_as_float(sr[cc + i]) * kf > m4[i] + kRaiseThreshold;
                    }
                }
                // does any token of the tile exceed the running maximum of its column by 2^6?  (flags by tile parity:
                // the common path has only this one barrier per tile)
                const bool wraise = __any_sync(0xffffffffu, raise);
                if (lane == 0) raise_flag[8 * sp + 4 * h2 + wq] = wraise;
                bar_sync_named(bar_id, 128);
                const int* rf = &raise_flag[8 * sp + 4 * h2];
                const bool any_raise = rf[0] | rf[1] | rf[2] | rf[3];
                if (ok && tg >= 1) ok = mq_wait(&p_empty[h2], (tg - 1) & 1);   // the head's P buffer is free, its PVs are done
                tc_fence_after();
                if (any_raise) {   // the same answer in the group's four warps
                    // column maxima over the 128 tokens: warp reduction, then across the four warps
#pragma unroll
                    for (int cc = 0; cc < kMqCols; cc++) {
                        float v = ok && valid && cc >= cmin ? __uint_as_float(sr[cc]) * kf : -INFINITY;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
                        if (lane == cc) sts32f(mq_hole(hole_col + wq) + lane * 4, v);
                    }
                    bar_sync_named(bar_id, 128);
                    float mine = 0.f;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t orow[16], lrow[16];
                        if (t > 0) {   // earlier tiles are rescaled: O^T (this thread's dim row) and the sums' row
                            tmem_ld16(tm_o + lane_base + 16 * half, orow);
                            tmem_ld16(tm_l + lane_base + 16 * half, lrow);
                        }
#pragma unroll
                        for (int c16 = 0; c16 < 16; c16++) {
                            const int cc = 16 * half + c16;
                            float v = lds32f(mq_hole(hole_col) + cc * 4);
                            v = fmaxf(v, lds32f(mq_hole(hole_col + 1) + cc * 4));
                            v = fmaxf(v, lds32f(mq_hole(hole_col + 2) + cc * 4));
                            v = fmaxf(v, lds32f(mq_hole(hole_col + 3) + cc * 4));
                            const float m_old = lds32f(mq_hole(kHoleMax + h2) + cc * 4);
                            const float m_new = fmaxf(m_old, v);
                            const float factor = m_new > m_old ? fast_exp2(m_old - m_new) : 1.f;   // exp2(-inf) = 0 the first time
                            if (cc == stid) mine = m_new;
                            if (t > 0) {
                                orow[c16] = __float_as_uint(__uint_as_float(orow[c16]) * factor);
                                lrow[c16] = __float_as_uint(__uint_as_float(lrow[c16]) * factor);
                            }
                        }
                        if (t > 0) {
                            tmem_st16(tm_o + lane_base + 16 * half, orow);
                            tmem_st16(tm_l + lane_base + 16 * half, lrow);
                        }
                    }
                    tc_fence_before();
                    bar_sync_named(bar_id, 128);   // every thread has read the old maxima
                    if (stid < kMqCols) sts32f(mq_hole(kHoleMax + h2) + stid * 4, mine);
                    bar_sync_named(bar_id, 128);   // maxima written
                }
                // P = exp2(x - m) as fp16 (the V norm is folded into V^): [token group][column group][token][8 columns];
                // the first head's in the table's holes
                if (ok) {
                    const uint32_t pdst = h2 ? kMqP1 + (stid >> 3) * 512 + (stid & 7) * 16 : mq_hole(kHoleP + (stid >> 3) * 4) + (stid & 7) * 16;
                    const uint32_t pcg = h2 ? 128u : 256u;
#pragma unroll
                    for (int cg = 0; cg < 4; cg++) {
                        uint32_t ph[4];
                        const uint4 ma = lds128(mq_hole(kHoleMax + h2) + cg * 32), mb = lds128(mq_hole(kHoleMax + h2) + cg * 32 + 16);
                        const float m8[8] = {__uint_as_float(ma.x), __uint_as_float(ma.y), __uint_as_float(ma.z), __uint_as_float(ma.w),
                                             __uint_as_float(mb.x), __uint_as_float(mb.y), __uint_as_float(mb.z), __uint_as_float(mb.w)};
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            const int cc = 8 * cg + i;
                            const float e0 = valid && cc >= cmin ? fast_exp2(__uint_as_float(sr[cc]) * kf - m8[i]) : 0.f;
                            const float e1 = valid && cc + 1 >= cmin ? fast_exp2(__uint_as_float(sr[cc + 1]) * kf - m8[i + 1]) : 0.f;
                            ph[i >> 1] = pack_half2(e0, e1);
                        }
                        sts128(pdst + cg * pcg, ph[0], ph[1], ph[2], ph[3]);
                    }
                }
                fence_proxy_async();
                tc_fence_before();
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&p_full[h2]);
            }
            // ---- segment epilogue: wait for this head's last PV, normalize, write the partials ---------
            // (a barrier of the head's own, one phase per segment: P's barrier may be a phase further on)
            if (abort_flag) ok = false;
            if (ok) ok = mq_wait(&o_done[h2], sg & 1);
            if (!ok) {
                abort_flag = 1;
                if (lane == 0) atomicExch(&p.header[0], 1);
            } else {
                tc_fence_after();
                const int64_t slot = (int64_t)c + b;   // one partial per (page range, sequence)
                const int kvh = 2 * hp + h2;
                const int dim = stid ^ 1;   // row 2i of O^T is dim 2i + 1 and vice versa
                float* po = p.partial_o + (slot * p.num_q_heads + (int64_t)kvh * mp.ncols) * kHeadDim + dim;
                float mine = 0.f;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t orow[16], lrow[16];   // every row of the sums' accumulator holds the column sums
                    tmem_ld16(tm_o + lane_base + 16 * half, orow);
                    tmem_ld16(tm_l + lane_base + 16 * half, lrow);
#pragma unroll
                    for (int c16 = 0; c16 < 16; c16++) {
                        const int cc = 16 * half + c16;
                        const float ls = __uint_as_float(lrow[c16]);
                        if (cc == stid) mine = ls;
                        if (cc < mp.ncols) po[(int64_t)cc * kHeadDim] = ls > 0.f ? __uint_as_float(orow[c16]) / ls : 0.f;
                    }
                }
                if (stid < mp.ncols) {
                    const float mm = lds32f(mq_hole(kHoleMax + h2) + stid * 4);
                    p.partial_lse[slot * p.num_q_heads + (int64_t)kvh * mp.ncols + stid] = mine > 0.f ? mm + log2f(mine) : -INFINITY;
                }
                tc_fence_before();
            }
            }
            u += 2 * ntiles;
            tile_n += ntiles;
            bar_sync_named(1, kMqThreads);   // every instruction of this segment has completed before Q^T and tensor memory are reused
            if (abort_flag) break;
        }
        tc_fence_before();
        bar_sync_named(1, kMqThreads);
    }
}

// cuTensorMapEncodeTiled through the runtime (no link-time dependency on the driver library)
typedef CUresult (*MqEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MqEncodeFn mq_encode_fn() {
    static MqEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<MqEncodeFn>(sym);
        tried = true;
    }
    return fn;
}

// Is the wide-tile kernel applicable?  Dense cache rows of 2, 4, 8 or 16 KV heads, padded head size 128.
bool mq_applicable(int num_kv_heads, int cols) {
    return cols > 8 && cols <= kMqCols && (num_kv_heads == 2 || num_kv_heads == 4 || num_kv_heads == 8 || num_kv_heads == 16);
}

int launch_decode_mq(const DecodeParams& d, int num_kv_heads, int64_t num_blocks, int grid, int causal, cudaStream_t stream) {
    MqParams mp{};
    mp.d = d;
    mp.head_pairs = num_kv_heads / 2;
    mp.ncols = d.group;
    mp.causal = causal;
    MqEncodeFn enc = mq_encode_fn();
    TQ_REQUIRE(enc != nullptr, TQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t row_bytes = (cuuint64_t)num_kv_heads * kSlotBytes;
    const cuuint64_t dims[3] = {row_bytes, (cuuint64_t)num_blocks * kPageTokens, 2};
    const cuuint64_t strides[2] = {row_bytes, (cuuint64_t)d.slab_bytes};
    const cuuint32_t box[3] = {160u, (cuuint32_t)kPageTokens, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult rc = enc(&mp.cache_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(d.kv_cache), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TQ_REQUIRE(rc == CUDA_SUCCESS, TQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the cache (%d)", (int)rc);
    const int smem = (int)kMqSmemEnd;
    static bool configured[64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(decode_mq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // whole page ranges for every head pair (a grid smaller than the head pairs is rounded up to one range)
    const int ranges = grid / mp.head_pairs > 0 ? grid / mp.head_pairs : 1;
    const int g = ranges * mp.head_pairs;
    TQ_CUDA(launch_serialized(decode_mq_kernel, dim3((unsigned)g), dim3(kMqThreads), (size_t)smem, stream, mp));
    return TQ_OK;
}

}  // namespace tq
