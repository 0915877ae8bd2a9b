// Paged decode attention over the 4-bit quantized KV cache, split-KV, for sm_100a.
//
// Replaces the reference's TurboQuantContiguousDecodeKernelV5TC<..., paged=true>
// (csrc/include/flashinfer_decode_turboquant_v5_tc.cuh:112-795), its launcher
// decode_v5_from_cache_paged_splitkv_ws (csrc/src/decode_v5_tc_binding.cu:754-874) and
// SplitKVCombineKernel (csrc/include/flashinfer_decode_turboquant_combine.cuh:18-79).
//
// Design (one thread block = all KV heads of a contiguous page range):
//   * The concatenated page list of the whole batch is cut into equal page ranges, one per
//     thread block, on the device (a warp scan over seq_lens): no host planning, no host sync,
//     balanced for mixed lengths.  "Equal" is measured with a charge for every sequence a block
//     has to start (kSegCostStages).  A block whose range spans several sequences processes them
//     as consecutive segments and writes one partial per (block, sequence).
//   * A producer warp streams pages with non-multicast 1-D bulk async copies (cp.async.bulk,
//     2560 bytes = a run of token rows per copy) into a ring of three shared-memory stages
//     guarded by full/empty mbarriers.  The runs are placed, and MMA rows mapped to tokens, such
//     that the fragment loads below are bank-conflict free (DecodeSmem).
//   * Sixteen consumer warps, one per (KV head, page lane).  Packed codes go from shared memory
//     straight into mma.sync.m16n8k16 A-fragments: a thread's 16-byte K chunk is exactly its
//     k-slices of the eight QK MMAs (the head-dim order inside the contraction is free because Q
//     is loaded in the same permuted order), and V nibbles of two tokens are zipped into bytes
//     so that one dequantized half2 is a (token, token+1) pair of the PV contraction.  Tokens
//     sit on the M axis (16) and the query columns of the KV head on N (8).
//   * Dequantization is a shared-memory table lookup per code BYTE: entry v holds the half2
//     {centroid(v & 15), centroid(v >> 4)}, one column per lane, so that every lookup of a warp
//     is bank-conflict free; entries are 256 bytes apart at a 64 KB boundary of the shared window,
//     which lets one byte permute build the address (dequant8).  The logic pipe of the SM runs at
//     half the FP32 rate, and a pure byte-permute (prmt) dequantizer needs ~17 logic instructions
//     per 8 codes, which capped the first version of this kernel at 31% of HBM peak with the ALU
//     pipe 65% busy.  Norms are folded into the scores (K) and into P (V), so there is no
//     per-element multiply.
//   * Online softmax in the base-2 domain with one consistent base everywhere; the running
//     max is only raised when the tile max exceeds it by more than 2^6, which makes rescaling of
//     the output accumulators rare.
//   * Partials (normalized, rotated domain, fp32) + base-2 LSE go to the workspace; the merge
//     kernel combines them, applies the inverse rotation once per (sequence, head) and casts.
//
// Tensor-core generation: the dequantized operands are produced in registers, so the
// register-operand mma.sync path is used; tcgen05 needs its A/B tiles in shared memory, which
// would add a 2-byte-per-element shared-memory round trip to a kernel whose limiters are the
// shared-memory lookups and instruction issue, not MMA throughput (the tensor pipe is 22% busy).
#include <cmath>
#include <cstring>

#include "tq_decode_common.cuh"

namespace tq {

// Shared-memory stage layout.  A stage holds kPPS pages; page lane `pp` has a K region and a V
// region.  Each page half is copied as runs of kRunTokens consecutive token rows, one bulk copy
// per run: 2560 bytes for 16, 8, 4 and 2 KV heads, 1280 for one (copies of a few hundred bytes were
// found to be limited by the copy engine's request rate, 2.5 KB and larger are not).  A run is
// dense, so the bank of a row is fixed by the row size (640, 320, 160, 80 bytes = 0, 64, 32, 80
// mod 128); the runs' base offsets and the map from MMA row r to token row_token(r) are chosen per
// head count such that every group of lanes served together reads different banks: rows
// (2p, 2p+1) of a K fragment load lie 64 bytes apart mod 128, the four tokens of a V fragment
// load 32 bytes apart (checked for every head by a bank simulation; the only exception is the K
// load with one KV head, two wavefronts instead of one).  Rows r and r + 8 map to tokens a fixed
// distance apart inside one run, so five address registers serve the twelve loads of a tile.
//
// STRIDED: the HKV heads are a slice of a wider token row (more KV heads in the cache than one
// launch handles), so consecutive tokens are not contiguous and every token row is its own copy
// (1280, 640 or 320 bytes: slower, bound by the copy engine's request rate).  Rows then sit at a
// padded pitch, 64 mod 128 for K and 16 mod 128 for V, with the identity row -> token map.
template <int HKV, bool STRIDED = false>
struct DecodeSmem {
    static constexpr int kPPS = kConsumerWarps / HKV;  // pages per stage
    static constexpr int kRowBytes = HKV * kSlotBytes;
    static constexpr int kRunTokens = STRIDED ? 1 : HKV == 16 ? 2 : HKV == 8 ? 4 : HKV == 4 ? 8 : 16;
    static constexpr int kRunsPerHalf = kPageTokens / kRunTokens;
    static constexpr int kCopyBytes = kRunTokens * kRowBytes;
    static constexpr int kCopiesPerPage = 2 * kRunsPerHalf;
    static constexpr int kCopiesPerStage = kPPS * kCopiesPerPage;  // 16 or 32 (dense), 32 .. 128 (strided)
    static constexpr int kKPitch = kRowBytes + (64 - kRowBytes % 128 + 128) % 128;  // strided rows
    static constexpr int kVPitch = kRowBytes + (16 - kRowBytes % 128 + 128) % 128;
    static constexpr int kKRegion = STRIDED ? kPageTokens * kKPitch
                                    : HKV == 16 ? 20736 : HKV == 8 ? 10496 : HKV == 4 ? 5248 : kPageTokens * kRowBytes;  // per page lane
    static constexpr int kVRegion = STRIDED ? kPageTokens * kVPitch
                                    : HKV == 16 ? 20736 : HKV == 8 ? 10368 : HKV == 4 ? 5248 : kPageTokens * kRowBytes;
    static constexpr int kKBytes = kPPS * kKRegion;
    static constexpr int kVBytes = kPPS * kVRegion;
    static constexpr int kStageBytes = kKBytes + kVBytes;

    // run q of a page half -> byte offset of its first row inside the page lane's region
    static __host__ __device__ __forceinline__ constexpr int k_run(int q) {
        return STRIDED    ? q * kKPitch
               : HKV == 16 ? q * 2560 + 32 * (q & 3) + 128 * (q >> 2)                              // eight runs, 32 bytes apart mod 128
               : HKV == 8 ? q * 2560 + ((q & 1) ? 64 : 0) + ((q & 2) ? 144 : 0)  // 0, 2624, 5264, 7888
               : HKV == 4 ? q * 2576                                             // 0, 2576
                          : 0;
    }
    static __host__ __device__ __forceinline__ constexpr int v_run(int q) {
        return STRIDED ? q * kVPitch
               : HKV == 16 ? q * 2560 + 32 * (q & 3) + 128 * (q >> 2) : HKV == 8 ? q * 2592 : HKV == 4 ? q * 2592 : 0;
    }
    // token (0..15 within its page) -> byte offset of its row inside the page lane's region
    static __host__ __device__ __forceinline__ constexpr int k_off(int t) {
        return k_run(t / kRunTokens) + (t % kRunTokens) * kRowBytes;
    }
    static __host__ __device__ __forceinline__ constexpr int v_off(int t) {
        return v_run(t / kRunTokens) + (t % kRunTokens) * kRowBytes;
    }
    // MMA row / contraction slot r (0..15) -> token within the page
    static __host__ __device__ __forceinline__ constexpr int row_token(int r) {
        const int r7 = r & 7, up = r >> 3;
        return STRIDED    ? r
               : HKV == 16 ? 2 * ((0x13467520u >> (4 * r7)) & 7) + up                  // runs 0,2,5,7,6,4,3,1
               : HKV == 8 ? 4 * ((0x23013210 >> (4 * r7)) & 3) + (r7 >> 2) + 2 * up   // runs 0,1,2,3,1,0,3,2
               : HKV == 4 ? ((0xAB239810u >> (4 * r7)) & 15) + 4 * up                 // 0,1,8,9,3,2,11,10
               : HKV == 2 ? ((0x53427160u >> (4 * r7)) & 7) + 8 * up                  // 0,6,1,7,2,4,3,5
                          : r;
    }
    // the runs of a region neither overlap nor leave it
    static constexpr bool runs_fit() {
        for (int q = 0; q + 1 < kRunsPerHalf; q++)
            if (k_run(q) + kCopyBytes > k_run(q + 1) || v_run(q) + kCopyBytes > v_run(q + 1)) return false;
        return k_run(kRunsPerHalf - 1) + kCopyBytes <= kKRegion && v_run(kRunsPerHalf - 1) + kCopyBytes <= kVRegion;
    }
    // MMA rows r and r+8 sit a fixed distance apart in both regions (runs: two tokens further in
    // the same run; pitched rows: eight rows further)
    static constexpr int kKRow8 = k_off(row_token(8)) - k_off(row_token(0));
    static constexpr int kVRow8 = v_off(row_token(8)) - v_off(row_token(0));
    // per-warp scratch: rotated Q (fp16, `group` rows), reused to transpose the partial output
    // (2 x 128 floats), hence at least four rows
    static constexpr int q_rows(int group) { return group < 4 ? 4 : group; }
    static constexpr int q_bytes(int group) { return kConsumerWarps * q_rows(group) * kHeadDim * 2; }
};

// Shared-memory map of this kernel.  The lookup table starts at offset 64 KB of the block's
// shared window, so stage 0 sits below it and stages 1, 2 follow it; the per-warp scratch
// (rotated Q, later the transposed partial output) uses the upper 128 bytes of the table's
// 256-byte rows:
//   [stage 0] ... | 64 KB: table + scratch (64 KB) | 128 KB: [stage 1][stage 2]

template <int HKV, bool STRIDED>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_paged_kernel(const __grid_constant__ DecodeParams p) {
    using S = DecodeSmem<HKV, STRIDED>;
    static_assert(S::runs_fit(), "stage layout: runs overlap or leave their region");
    constexpr int PPS = S::kPPS;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ int seg_seq[kMaxSegments], seg_p0[kMaxSegments], seg_p1[kMaxSegments];
    __shared__ int num_segments, abort_flag;
    __shared__ int n_eff_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int nstages = kStages;
    const uint32_t smem_base = smem_u32(smem);
    // stage st lives at stage0 + (st ? stage_gap + (st - 1) * kStageBytes : 0) (byte offsets from smem)
    const uint32_t stage0_off = 0u;
    const uint32_t stage_gap = kLutAddr + kLutSpan - smem_base - stage0_off;
    const uint32_t lut_off = kLutAddr - smem_base;
    uint8_t* stages = smem + stage0_off;
    uint32_t* lut_s = reinterpret_cast<uint32_t*>(smem + lut_off);
    // Per-warp scratch (rotated Q rows of 256 bytes, later the transposed partial output) in the
    // unused upper half of the table's 256-byte rows: byte `off` of warp w's scratch is in hole
    // w * holes_per_warp + off / 128 at offset off % 128 (every access below stays inside one
    // 128-byte hole).
    const uint32_t q_warp_bytes = (uint32_t)S::q_rows(p.group) * kHeadDim * 2;
    auto q_ptr = [&](int w, uint32_t off) -> uint8_t* {
        const uint32_t hole = (uint32_t)w * (q_warp_bytes >> 7) + (off >> 7);
        return smem + lut_off + (hole << 8) + 128u + (off & 127u);
    };
    grid_launch_dependents();  // the merge's blocks may be scheduled as soon as there is room
    if (smem_base + stage0_off + S::kStageBytes > kLutAddr) {  // the map above does not fit
        grid_dependency_wait();
        if (tid == 0) atomicExch(&p.header[0], 3);
        return;
    }

    // Warm L2 with the small inputs while the kernel before this one drains: a whole KV stream has
    // passed through the cache since they were last touched.  A prefetch hands no value to this
    // kernel, so it may precede the wait.
    {
        const size_t first = ((size_t)blockIdx.x * kDecodeThreads + tid) * 128;
        const size_t step = (size_t)gridDim.x * kDecodeThreads * 128;
        auto warm = [&](const void* base, size_t bytes) {
            for (size_t off = first; off < bytes; off += step) prefetch_l2(static_cast<const uint8_t*>(base) + off);
        };
        warm(p.seq_lens, (size_t)p.batch * 4);
        if (p.page_indptr) {
            warm(p.page_indptr, (size_t)(p.batch + 1) * 4);
        } else {
            const size_t table = (size_t)p.batch * p.max_pages * 4;
            warm(p.page_indices, table < ((size_t)8 << 20) ? table : ((size_t)8 << 20));
        }
        warm(p.q, (size_t)p.batch * p.nq * p.real_heads * p.head_dim * (p.q_dtype == TQ_F32 ? 4 : 2));
    }

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kConsumerWarps);
        }
        num_segments = 0;
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // ---- plan: warp 0 scans seq_lens, finds this block's page range and its segments; the other
    // warps meanwhile fill the lookup table: entry v, column c = {centroid(v & 15), centroid(v >> 4)}
    if (warp != 0) {
        for (int i = tid - 32; i < 256 * 32; i += kDecodeThreads - 32) {
            const int v = i >> 5;
            lut_s[v * 64 + (i & 31)] = (uint32_t)p.centroid_h[v & 15] | ((uint32_t)p.centroid_h[v >> 4] << 16);
        }
        grid_dependency_wait();
    } else {
        grid_dependency_wait();  // seq_lens, the page table, Q and the workspace belong to earlier kernels
        // pass 1: total pages and the number of non-empty sequences
        int total_real = 0, nonempty = 0;
        int np_first = 0;  // this lane's sequence of the first 32: kept for pass 2 (one global round trip less)
        bool too_long = false;
        for (int base = 0; base < p.batch; base += 32) {
            int np = 0, fp = 0, le;
            if (base + lane < p.batch) {
                seq_pages(p, base + lane, fp, np, le);
                // pages the sequence has in its table (dense: the row; CSR: its indptr span)
                const int have = p.page_indptr ? p.page_indptr[base + lane + 1] - p.page_indptr[base + lane] : p.max_pages;
                too_long |= np > 0 && fp + np > have;
            }
            if (base == 0) np_first = np;
            nonempty += __popc(__ballot_sync(0xffffffffu, np > 0));
            for (int o = 16; o > 0; o >>= 1) np += __shfl_xor_sync(0xffffffffu, np, o);
            total_real += np;
        }
        if (__any_sync(0xffffffffu, too_long)) {
            // A length that its page table cannot back would walk off the table: read nothing, let the
            // merge write zeros (no parts for any sequence) and say so in the status word.
            if (blockIdx.x == 0) {
                for (int b = lane; b <= p.batch; b += 32) p.page_prefix[b] = 0;
                if (lane == 0) {
                    p.header[1] = 1;
                    p.header[2] = 0;
                    p.header[3] = 0;
                    atomicExch(&p.header[0], kStatusSeqTooLong);
                }
            }
            if (lane == 0) num_segments = 0;
            total_real = -1;
        }
        int n_eff = (total_real + kMinPagesPerCta * PPS - 1) / (kMinPagesPerCta * PPS);
        n_eff = n_eff < 1 ? 1 : (n_eff > (int)gridDim.x ? (int)gridDim.x : n_eff);
        // the charge for a sequence start only makes sense against blocks that stream for a while
        const int kSegCost = total_real / n_eff >= kSegCostMinStages * PPS ? kSegCostStages * PPS : 0;
        const int total = total_real + nonempty * kSegCost;  // virtual pages
        const int c = blockIdx.x;
        const int64_t lo = c < n_eff ? ((int64_t)c * total) / n_eff : 0;
        const int64_t hi = c < n_eff ? ((int64_t)(c + 1) * total) / n_eff : 0;
        // pass 2: prefix sums, segments, and (block 0) the prefix array for the merge kernel
        int run = 0, nseg = 0;
        for (int base = 0; base < p.batch && total_real >= 0; base += 32) {
            int np = 0, fp = 0, le;
            const int b = base + lane;
            if (base == 0) np = np_first;
            else if (b < p.batch) seq_pages(p, b, fp, np, le);
            const int vnp = np > 0 ? np + kSegCost : 0;
            int incl = vnp;
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            // virtual span of the sequence [vstart, end); its real pages are [start, end)
            const int vstart = run + incl - vnp, end = run + incl, start = vstart + kSegCost;
            if (c == 0 && b < p.batch) p.page_prefix[b] = vstart;
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
            if (c == 0) {
                p.page_prefix[p.batch] = run;
                p.header[1] = n_eff;
                p.header[2] = total;
                p.header[3] = kSegCost;
            }
            if (nseg > kMaxSegments) {  // more sequences per block than the list holds
                atomicExch(&p.header[0], 2);
                nseg = 0;
            }
            num_segments = nseg;
            n_eff_s = n_eff;
        }
    }
    __syncthreads();
    const int nseg = num_segments;
    if (nseg == 0) return;

    if (warp >= kConsumerWarps) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");  // the whole producer warpgroup
        if (warp > kConsumerWarps) return;
        // =============================== producer warp ======================================
        int st = 0, round = 0;
        bool bad_page = false;
        const uint64_t stream_policy = l2_policy_evict_first();  // the cache is read once per launch
        for (int sg = 0; sg < nseg && !abort_flag; sg++) {
            const int b = seg_seq[sg];
            int first_page, npages_b, len_eff;
            seq_pages(p, b, first_page, npages_b, len_eff);
            const int64_t tbl = p.page_indptr ? (int64_t)p.page_indptr[b] : (int64_t)b * p.max_pages;
            const int p0 = seg_p0[sg], p1 = seg_p1[sg];
            constexpr int kIdBlock = (32 / PPS) * PPS;  // page ids fetched per round: a whole number of stages
            for (int base = p0; base < p1; base += kIdBlock) {
                const int mine = base + lane;
                int my_page = mine < p1 ? p.page_indices[tbl + first_page + mine] : 0;
                if ((uint64_t)(int64_t)my_page >= (uint64_t)p.num_blocks) {  // never form an address from it
                    my_page = 0;
                    bad_page = true;
                }
                const int cnt = (p1 - base) < kIdBlock ? (p1 - base) : kIdBlock;
                for (int j = 0; j < cnt; j += PPS) {
                    const int np = (cnt - j) < PPS ? (cnt - j) : PPS;
                    if (round > 0) {
                        if (!mbar_wait(&empty_bar[st], (round - 1) & 1)) {
                            abort_flag = 1;
                            atomicExch(&p.header[0], 1);
                        }
                    }
                    if (abort_flag) break;
                    uint8_t* sk = stages + (st ? stage_gap + (size_t)(st - 1) * S::kStageBytes : 0);
                    uint8_t* sv = sk + S::kKBytes;
                    if (lane == 0)
                        mbar_arrive_expect_tx(&full_bar[st], (uint32_t)(np * 2 * kPageTokens * S::kRowBytes));
                    __syncwarp();
#pragma unroll
                    for (int c0 = 0; c0 < S::kCopiesPerStage; c0 += 32) {
                        // copy index = page lane * copies per page + (K runs, then V runs), one per lane and pass
                        const int ci = c0 + lane;
                        const int pp = ci / S::kCopiesPerPage, c = ci % S::kCopiesPerPage;
                        const int page = __shfl_sync(0xffffffffu, my_page, (j + pp) & 31);
                        if (ci < S::kCopiesPerStage && pp < np) {
                            const bool is_v = c >= S::kRunsPerHalf;
                            const int tok = (c % S::kRunsPerHalf) * S::kRunTokens;  // first token of the run
                            const uint8_t* src = p.kv_cache + (is_v ? p.slab_bytes : 0) +
                                                 ((int64_t)page * kPageTokens + tok) * p.kv_row_bytes + p.kv_head_off;
                            uint8_t* dst = is_v ? sv + pp * S::kVRegion + S::v_off(tok)
                                                : sk + pp * S::kKRegion + S::k_off(tok);
                            bulk_g2s_hint(dst, src, S::kCopyBytes, &full_bar[st], stream_policy);
                        }
                    }
                    if (++st == nstages) { st = 0; round++; }
                }
                if (abort_flag) break;
            }
        }
        if (bad_page) atomicExch(&p.header[0], kStatusBadPage);
        return;
    }

    // ================================= consumer warps =======================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");  // 4 x 112 + 24 <= 5 x 96 per scheduler
    const int g = lane >> 2, tg = lane & 3;
    const int head = warp % HKV;   // KV head of this warp
    const int sub = warp / HKV;    // page lane inside a stage
    const uint32_t lut_lane = smem_u32(lut_s) + 4u * lane;

    // per-thread constants of the fragment loads (byte offsets inside a stage): MMA rows g and
    // g+8 of this lane and its four contraction slots, mapped to tokens of the page
    const int ta = S::row_token(g), tb = S::row_token(g + 8);
    const uint32_t k_base = smem_u32(stages) + sub * S::kKRegion + head * kSlotBytes;
    const uint32_t v_base = smem_u32(stages) + S::kKBytes + sub * S::kVRegion + head * kSlotBytes;
    // Rows g+8, 2tg+8 and 2tg+9 are a compile-time distance from rows g, 2tg and 2tg+1: five
    // address registers serve the twelve loads of a tile.
    const uint32_t ka_addr = k_base + S::k_off(ta) + 16 * tg;
    const uint32_t nka_addr = k_base + S::k_off(ta) + 64;
    const uint32_t nva_addr = v_base + S::v_off(ta) + 64;
    const uint32_t v0_addr = v_base + S::v_off(S::row_token(2 * tg)) + 8 * g;
    const uint32_t v1_addr = v_base + S::v_off(S::row_token(2 * tg + 1)) + 8 * g;

    int st = 0, round = 0;
    uint32_t st_off = 0;  // st * kStageBytes
    for (int sg = 0; sg < nseg; sg++) {
        const int b = seg_seq[sg];
        int first_page, npages_b, len_eff;
        seq_pages(p, b, first_page, npages_b, len_eff);
        const int p0 = seg_p0[sg], p1 = seg_p1[sg];

        // ---- rotate this KV head's query heads: signs -> FWHT -> 1/sqrt(128) -> fp16 -----------
        // lane holds elements 4*lane .. 4*lane+3; stages h=1,2 are local, h=4..64 by shuffle.
        // The loads of up to four heads are issued together (one memory round trip per batch).
        const float4 sg4 = reinterpret_cast<const float4*>(p.signs)[lane];
        for (int r0 = 0; r0 < p.group; r0 += 4) {
            float v[4][4];
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
                const int r = r0 + rr < p.group ? r0 + rr : p.group - 1;
                const int qi = r / p.real_group, hh = r - qi * p.real_group;
                const int64_t base = ((((int64_t)b * p.nq + qi) * p.real_heads) + p.q_head_base + head * p.real_group + hh) *
                                         p.head_dim + 4 * lane;
                if (4 * lane >= p.head_dim) {  // padding of a short head
                    v[rr][0] = v[rr][1] = v[rr][2] = v[rr][3] = 0.f;
                } else if (p.q_dtype == TQ_BF16) {
                    const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + base);
                    v[rr][0] = __uint_as_float(t.x << 16); v[rr][1] = __uint_as_float(t.x & 0xffff0000u);
                    v[rr][2] = __uint_as_float(t.y << 16); v[rr][3] = __uint_as_float(t.y & 0xffff0000u);
                } else if (p.q_dtype == TQ_F16) {
                    const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p.q) + base);
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
                    v[rr][0] = lo.x; v[rr][1] = lo.y; v[rr][2] = hi.x; v[rr][3] = hi.y;
                } else {
                    const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + base);
                    v[rr][0] = t.x; v[rr][1] = t.y; v[rr][2] = t.z; v[rr][3] = t.w;
                }
            }
#pragma unroll
            for (int rr = 0; rr < 4; rr++) {
                float* w = v[rr];
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
                if (r0 + rr < p.group) {
                    // stored with each (even, odd) pair swapped: a code byte dequantizes to
                    // {low half: odd dim (low nibble), high half: even dim (high nibble)}
                    __half2* dst = reinterpret_cast<__half2*>(q_ptr(warp, (uint32_t)(r0 + rr) * 256u + 8u * lane));
                    dst[0] = __floats2half2_rn(w[1] * 0.08838834764831845f, w[0] * 0.08838834764831845f);
                    dst[1] = __floats2half2_rn(w[3] * 0.08838834764831845f, w[2] * 0.08838834764831845f);
                }
            }
        }
        __syncwarp();
        // B fragments of the eight QK MMAs: pairs 16*tg .. 16*tg+15 of query head g
        uint32_t qf[16];
        {
            const uint4* src = reinterpret_cast<const uint4*>(q_ptr(warp, (uint32_t)g * 256u + 64u * tg));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 t = g < p.group ? src[i] : make_uint4(0u, 0u, 0u, 0u);  // padded heads
                qf[4 * i] = t.x; qf[4 * i + 1] = t.y; qf[4 * i + 2] = t.z; qf[4 * i + 3] = t.w;
            }
        }
        __syncwarp();

        float o_acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) o_acc[i][j] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        for (int pg = p0; pg < p1; pg += PPS) {
            if (!mbar_wait(&full_bar[st], round & 1)) {  // bounded; every other warp's waits run out too
                abort_flag = 1;
                atomicExch(&p.header[0], 1);
                return;
            }
            const bool have = pg + sub < p1;  // this warp's page lane holds a page
            if (have) {
                const int tok0 = (first_page + pg + sub) * kPageTokens;  // first token of the page
                // ---- K codes and norms for tokens ta, tb; V codes: bytes 8g..8g+7 of four tokens ----
                const uint32_t ka_at = ka_addr + st_off, nka_at = nka_addr + st_off, nva_at = nva_addr + st_off;
                const uint4 ka = lds128_at<0>(ka_at), kb = lds128_at<S::kKRow8>(ka_at);
                float nka = lds_half_at<0>(nka_at), nkb = lds_half_at<S::kKRow8>(nka_at);
                float nva = lds_half_at<0>(nva_at), nvb = lds_half_at<S::kVRow8>(nva_at);
                // Only the last page of a sequence can hold tokens past its length: their norms are
                // zeroed (whatever the unwritten slots contain) and their scores biased to -inf.
                float bias_a = 0.f, bias_b = 0.f;
                if (tok0 + kPageTokens > len_eff) {
                    if (tok0 + ta >= len_eff) { nka = 0.f; nva = 0.f; bias_a = -INFINITY; }
                    if (tok0 + tb >= len_eff) { nkb = 0.f; nvb = 0.f; bias_b = -INFINITY; }
                }
                const uint32_t v0_at = v0_addr + st_off, v1_at = v1_addr + st_off;
                const uint2 v0 = lds64_at<0>(v0_at), v1 = lds64_at<0>(v1_at);
                const uint2 v2 = lds64_at<S::kVRow8>(v0_at), v3 = lds64_at<S::kVRow8>(v1_at);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[st]);  // stage data is in registers now

                // ---- S = K^ Q^T : 16 tokens x 8 heads ---------------------------------------------
                float s_acc[4] = {0.f, 0.f, 0.f, 0.f}, s_acc2[4] = {0.f, 0.f, 0.f, 0.f};  // two MMA chains
                const uint32_t kwa[4] = {ka.x, ka.y, ka.z, ka.w};
                const uint32_t kwb[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    uint32_t ra[4], rb[4];
                    dequant8(kwa[w], lut_lane, ra);
                    dequant8(kwb[w], lut_lane, rb);
                    mma16816(s_acc, ra[0], rb[0], ra[1], rb[1], qf[4 * w], qf[4 * w + 1]);
                    mma16816(s_acc2, ra[2], rb[2], ra[3], rb[3], qf[4 * w + 2], qf[4 * w + 3]);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) s_acc[i] += s_acc2[i];
                // ---- online softmax (base 2) ------------------------------------------------------
                const float kfa = nka * p.k_scale, kfb = nkb * p.k_scale;
                const float x0 = fmaf(s_acc[0], kfa, bias_a), x1 = fmaf(s_acc[1], kfa, bias_a);
                const float x2 = fmaf(s_acc[2], kfb, bias_b), x3 = fmaf(s_acc[3], kfb, bias_b);
                // The running max of a head is raised only when some score of the tile exceeds it by
                // more than 2^6; one vote decides that, and only then is the tile max reduced across
                // the lanes (three shuffle rounds) and the accumulators rescaled.
                float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
                if (__any_sync(0xffffffffu, mx0 > m0 + kRaiseThreshold || mx1 > m1 + kRaiseThreshold)) {
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
                    }
                    const bool raise0 = mx0 > m0 + kRaiseThreshold, raise1 = mx1 > m1 + kRaiseThreshold;
                    const float c0 = raise0 ? fast_exp2(m0 - mx0) : 1.f, c1 = raise1 ? fast_exp2(m1 - mx1) : 1.f;
                    if (raise0) m0 = mx0;
                    if (raise1) m1 = mx1;
                    l0 *= c0;
                    l1 *= c1;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        o_acc[i][0] *= c0; o_acc[i][1] *= c1; o_acc[i][2] *= c0; o_acc[i][3] *= c1;
                    }
                }
                const float e0 = fast_exp2(x0 - m0), e1 = fast_exp2(x1 - m1);
                const float e2 = fast_exp2(x2 - m0), e3 = fast_exp2(x3 - m1);
                l0 += e0 + e2;
                l1 += e1 + e3;
                const float vfa = nva * p.v_scale, vfb = nvb * p.v_scale;
                // P (token rows g / g+8, head columns 2tg, 2tg+1) -> transposed B fragments
                const uint32_t pb0 = movmatrix_trans(pack_half2(e0 * vfa, e1 * vfa));
                const uint32_t pb1 = movmatrix_trans(pack_half2(e2 * vfb, e3 * vfb));

                // ---- O^T += V^^T P : zip the nibbles of a token pair into bytes, dequantize --------
                const uint32_t vw0[2] = {v0.x, v0.y}, vw1[2] = {v1.x, v1.y};
                const uint32_t vw2[2] = {v2.x, v2.y}, vw3[2] = {v3.x, v3.y};
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    // low nibbles = odd dims, high nibbles = even dims
                    const uint32_t lo01 = (vw0[i] & 0x0F0F0F0Fu) | ((vw1[i] << 4) & 0xF0F0F0F0u);
                    const uint32_t hi01 = ((vw0[i] >> 4) & 0x0F0F0F0Fu) | (vw1[i] & 0xF0F0F0F0u);
                    const uint32_t lo23 = (vw2[i] & 0x0F0F0F0Fu) | ((vw3[i] << 4) & 0xF0F0F0F0u);
                    const uint32_t hi23 = ((vw2[i] >> 4) & 0x0F0F0F0Fu) | (vw3[i] & 0xF0F0F0F0u);
                    uint32_t a_lo01[4], a_hi01[4], a_lo23[4], a_hi23[4];
                    dequant8(lo01, lut_lane, a_lo01);
                    dequant8(hi01, lut_lane, a_hi01);
                    dequant8(lo23, lut_lane, a_lo23);
                    dequant8(hi23, lut_lane, a_hi23);
#pragma unroll
                    for (int j = 0; j < 4; j++)  // rows: g <- odd dim, g+8 <- even dim of byte 4i+j
                        mma16816(o_acc[4 * i + j], a_lo01[j], a_hi01[j], a_lo23[j], a_hi23[j], pb0, pb1);
                }
            } else {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[st]);
            }
            st_off = st ? st_off + S::kStageBytes : stage_gap;
            if (++st == nstages) { st = 0; st_off = 0; round++; }
        }

        // ---- finish the segment: normalize, write the partial and its base-2 LSE ----------------
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, o);
            l1 += __shfl_xor_sync(0xffffffffu, l1, o);
        }
        const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
        const int64_t slot = ((int64_t)blockIdx.x + b) * PPS + sub;
        const int h0 = 2 * tg, h1 = 2 * tg + 1;
        float* po = p.partial_o + (slot * p.num_q_heads + head * p.group) * kHeadDim;
        // Two query heads at a time go through the warp's scratch (2 x 128 floats) so that the
        // global stores are full 512-byte rows instead of scattered words (which cost 7 us per
        // segment): the lanes with tg == pass own heads 2*pass and 2*pass+1.
        for (int pass = 0; 2 * pass < p.group; pass++) {
            __syncwarp();
            if (tg == pass) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int d_even = 16 * g + 2 * i;
                    *reinterpret_cast<float2*>(q_ptr(warp, 4u * d_even)) = make_float2(o_acc[i][2] * inv0, o_acc[i][0] * inv0);
                    *reinterpret_cast<float2*>(q_ptr(warp, 512u + 4u * d_even)) =
                        make_float2(o_acc[i][3] * inv1, o_acc[i][1] * inv1);
                }
            }
            __syncwarp();
            const float4 r0 = *reinterpret_cast<const float4*>(q_ptr(warp, 16u * lane));
            const float4 r1 = *reinterpret_cast<const float4*>(q_ptr(warp, 512u + 16u * lane));
            reinterpret_cast<float4*>(po + (2 * pass) * kHeadDim)[lane] = r0;
            if (2 * pass + 1 < p.group) reinterpret_cast<float4*>(po + (2 * pass + 1) * kHeadDim)[lane] = r1;
        }
        __syncwarp();
        if (g == 0) {
            float* pl = p.partial_lse + slot * p.num_q_heads + head * p.group;
            if (h0 < p.group) pl[h0] = l0 > 0.f ? m0 + log2f(l0) : -INFINITY;
            if (h1 < p.group) pl[h1] = l1 > 0.f ? m1 + log2f(l1) : -INFINITY;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Merge: one block per (row, query head), one thread per rotated dim.
// ---------------------------------------------------------------------------------------------
struct MergeParams {
    const float* partial_o;
    const float* partial_lse;
    const int32_t* header;       // decode workspace header (null for the generic merge)
    const int32_t* page_prefix;  // decode workspace prefix (null for the generic merge)
    const float* signs;
    void* out;
    float* out_lse;   // natural-log LSE (final) or base-2 LSE (rotated output), optional
    int64_t rows;     // batch (decode merge) or rows (generic merge)
    int num_q_heads, num_parts, pps, grid_ctas, out_dtype, emit_rotated;
    int nq, real_heads, real_group;  // virtual head -> (query, real head) of the output row; nq = 1: identity
    int head_dim;                    // elements per output row (128, or 96: the padded dims are dropped)
    int q_head_base;                 // first real query head of this launch (KV heads handled in several launches)
    // Exchange of rotated partials between the GPUs that split one KV axis (xmode != 0):
    // every rank owns an exchange buffer (ExchangeLayout) that all ranks have mapped.
    int xmode;                       // 0 none, 1 push this rank's partial to all ranks, 2 wait for all ranks and merge
    int xrank, xworld;
    int xspin;                       // polls (256 ns apart) the wait for a peer may take before it gives up
    int64_t xrows;                   // output rows (batch x queries x heads) of one rank's partial
    unsigned char* xbuf[kMaxExchangeRanks];  // xbuf[r] = rank r's exchange buffer as mapped here
};

// Exchange buffer of one rank: control words, one flag per source rank, then two generations
// (epoch parity) of [world][rows] base-2 LSEs and [world][rows][128] rotated partials.
//   ctrl[0] epoch of the last finished step   ctrl[1] sticky status (1 = a wait ran out)
//   ctrl[2] blocks done pushing               ctrl[3] blocks done merging
struct ExchangeLayout {
    size_t flags, lse, o, total;
    __host__ __device__ ExchangeLayout(int world, int64_t rows) {
        flags = 64;
        lse = 256;
        o = lse + (((size_t)2 * world * rows * sizeof(float) + 255) & ~(size_t)255);
        total = o + (size_t)2 * world * rows * kHeadDim * sizeof(float);
    }
};

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One block per (row, query head), kMergeWarps warps (4, or 16 when one sequence is spread over
// many blocks of the decode grid).  Warp w takes parts w, w + kMergeWarps, ...; lane l owns
// rotated dims 4l..4l+3.  A warp first fetches the LSEs of its parts (lane i: its i-th part),
// forms the weights, then fetches all its payloads with the loads in flight together: the
// kernel is a handful of L2 round trips long up to 32 parts per warp (one sequence spread over
// every block of the decode grid: 296 parts).  The warps' results are combined in shared memory, then
// the first four warps run the inverse rotation (FWHT, 1/sqrt(128), signs), one thread per dim.
__device__ __forceinline__ void sync_first_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int kMergeWarps>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const __grid_constant__ MergeParams p) {
    __shared__ float buf[kHeadDim];
    __shared__ float part_acc[kMergeWarps][kHeadDim];
    __shared__ float part_m[kMergeWarps], part_w[kMergeWarps];
    const int d = threadIdx.x, warp = d >> 5, lane = d & 31;
    const int64_t row = blockIdx.x;
    const int hq = blockIdx.y;
    grid_launch_dependents();
    grid_dependency_wait();  // the partials (and the exchange words) come from the kernel before
    const float* partial_o = p.partial_o;
    const float* partial_lse = p.partial_lse;
    int32_t* xctrl = nullptr;
    int32_t xepoch = 0;
    if (p.xmode) {
        xctrl = reinterpret_cast<int32_t*>(p.xbuf[p.xrank]);
        xepoch = *reinterpret_cast<volatile int32_t*>(xctrl) + 1;  // the step in progress
    }
    if (p.xmode == 2) {
        // Wait (bounded: about a second) until every rank's partial of this step has landed in
        // this rank's buffer, then merge the [world][rows] parts of the step's generation.
        __shared__ int x_ok;
        if (d == 0) {
            const int32_t* flags = reinterpret_cast<const int32_t*>(p.xbuf[p.xrank] + 64);
            int ok = 1;
            for (int w = 0; w < p.xworld && ok; w++) {
                int spins = 0;
                while ((int32_t)(ld_acquire_sys(flags + w) - xepoch) < 0) {
                    if (++spins > p.xspin) { ok = 0; break; }
                    __nanosleep(256);
                }
            }
            if (!ok) atomicExch(xctrl + 1, 1);
            x_ok = ok;
        }
        __syncthreads();
        if (!x_ok) return;
        const ExchangeLayout xl(p.xworld, p.xrows);
        const int64_t gen = (int64_t)(xepoch & 1) * p.xworld * p.xrows;
        partial_lse = reinterpret_cast<const float*>(p.xbuf[p.xrank] + xl.lse) + gen;
        partial_o = reinterpret_cast<const float*>(p.xbuf[p.xrank] + xl.o) + gen * kHeadDim;
    }
    // The parts of this row form an arithmetic slot sequence: slot(i) = first + i * stride.
    int64_t first = 0, stride = 1;
    int count = 0;
    if (p.header) {
        // partials of sequence `row` come from the blocks whose page range meets its pages
        const int64_t n = p.header[1], total = p.header[2];
        // virtual span [page_prefix[row], page_prefix[row + 1]); real pages start seg_cost further
        const int64_t e = p.page_prefix[row + 1];
        const int64_t s = p.page_prefix[row] + p.header[3];
        if (e > s && total > 0) {
            const int64_t c_first = ((s + 1) * n + total - 1) / total - 1;
            const int64_t c_last = (e * n + total - 1) / total - 1;
            first = (c_first + row) * p.pps;
            count = (int)(c_last - c_first + 1) * p.pps;
        }
    } else {
        // generic layout: partial_o [parts][rows][128]
        first = row;
        stride = p.rows;
        count = p.num_parts;
    }
    const float* lse_base = partial_lse + first * p.num_q_heads + hq;
    const int64_t lse_stride = stride * p.num_q_heads;
    const float4* o_base = reinterpret_cast<const float4*>(partial_o + (first * p.num_q_heads + hq) * kHeadDim) + lane;
    const int64_t o_stride = lse_stride * (kHeadDim / 4);
    float m = -INFINITY, wsum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = warp; i0 < count; i0 += kMergeWarps * 32) {  // this warp's parts i0, i0+16, ..., 32 per pass
        const int left = (count - i0 + kMergeWarps - 1) / kMergeWarps;
        const int n = left < 32 ? left : 32;
        const float my_lse = lane < n ? lse_base[(int64_t)(i0 + kMergeWarps * lane) * lse_stride] : -INFINITY;
        float mx = my_lse;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m, mx);
        if (m_new == -INFINITY) continue;                 // every part so far is empty
        const float rescale = exp2f(m - m_new);           // 0 on the first non-empty pass
        const float my_w = exp2f(my_lse - m_new);         // exp2(-inf) = 0 for empty parts
        float ws = my_w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
        wsum = wsum * rescale + ws;
        acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
        m = m_new;
        for (int j0 = 0; j0 < n; j0 += 8) {
            float4 o[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                o[j] = j0 + j < n ? o_base[(int64_t)(i0 + kMergeWarps * (j0 + j)) * o_stride] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float w = __shfl_sync(0xffffffffu, my_w, (j0 + j) & 31);
                if (j0 + j < n && w > 0.f) {              // an empty part's payload is never trusted
                    acc.x += w * o[j].x; acc.y += w * o[j].y; acc.z += w * o[j].z; acc.w += w * o[j].w;
                }
            }
        }
    }
    reinterpret_cast<float4*>(part_acc[warp])[lane] = acc;
    if (lane == 0) { part_m[warp] = m; part_w[warp] = wsum; }
    __syncthreads();
    if (d >= kHeadDim) return;  // the rest runs on one thread per dim; its barriers count 128 threads
    float mm = part_m[0];
#pragma unroll
    for (int w = 1; w < kMergeWarps; w++) mm = fmaxf(mm, part_m[w]);
    float o = 0.f, wtot = 0.f;
    if (mm > -INFINITY) {
#pragma unroll
        for (int w = 0; w < kMergeWarps; w++) {
            const float sc = exp2f(part_m[w] - mm);
            if (sc > 0.f) { o += sc * part_acc[w][d]; wtot += sc * part_w[w]; }
        }
    }
    o = wtot > 0.f ? o / wtot : 0.f;
    const float lse2 = wtot > 0.f ? mm + log2f(wtot) : -INFINITY;
    int64_t orow = row * p.num_q_heads + hq;
    if (p.header) {  // virtual head hq = kv_head * cols + (query * real_group + head_in_group) of this launch
        const int cols = p.nq * p.real_group;
        const int kvh = hq / cols, col = hq - kvh * cols;
        const int qi = col / p.real_group, hh = col - qi * p.real_group;
        orow = (row * p.nq + qi) * p.real_heads + p.q_head_base + kvh * p.real_group + hh;
    }
    if (p.xmode == 1) {
        // Push this rank's rotated partial into every rank's buffer (plain stores over NVLink, or
        // local), then publish: the last block to finish releases this rank's flag everywhere.
        const ExchangeLayout xl(p.xworld, p.xrows);
        const int64_t at = ((int64_t)(xepoch & 1) * p.xworld + p.xrank) * p.xrows + orow;
        for (int w = 0; w < p.xworld; w++) {
            reinterpret_cast<float*>(p.xbuf[w] + xl.o)[at * kHeadDim + d] = o;
            if (d == 0) reinterpret_cast<float*>(p.xbuf[w] + xl.lse)[at] = lse2;
        }
        __threadfence_system();
        sync_first_128();
        if (d == 0) {
            const int blocks = gridDim.x * gridDim.y;
            if (atomicAdd(xctrl + 2, 1) == blocks - 1) {
                xctrl[2] = 0;
                __threadfence_system();
                for (int w = 0; w < p.xworld; w++)
                    st_release_sys(reinterpret_cast<int32_t*>(p.xbuf[w] + 64) + p.xrank, xepoch);
            }
        }
        return;
    }
    if (p.emit_rotated) {
        reinterpret_cast<float*>(p.out)[orow * kHeadDim + d] = o;
        if (p.out_lse && d == 0) p.out_lse[orow] = lse2;
        return;
    }
    // inverse rotation: FWHT, 1/sqrt(128), signs
    buf[d] = o;
    sync_first_128();
    for (int h = 1; h < kHeadDim; h <<= 1) {
        const float a = buf[d & ~h], b2 = buf[d | h];
        sync_first_128();
        buf[d] = (d & h) ? a - b2 : a + b2;
        sync_first_128();
    }
    o = buf[d] * 0.08838834764831845f * p.signs[d];
    if (d < p.head_dim) {
        if (p.out_dtype == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[orow * p.head_dim + d] = __float2bfloat16_rn(o);
        else if (p.out_dtype == TQ_F16) reinterpret_cast<__half*>(p.out)[orow * p.head_dim + d] = __float2half_rn(o);
        else reinterpret_cast<float*>(p.out)[orow * p.head_dim + d] = o;
    }
    if (p.out_lse && d == 0) p.out_lse[orow] = lse2 * 0.6931471805599453f;
    if (p.xmode == 2) {  // the last block to finish closes the step
        sync_first_128();
        if (d == 0) {
            const int blocks = gridDim.x * gridDim.y;
            __threadfence();
            if (atomicAdd(xctrl + 3, 1) == blocks - 1) {
                xctrl[3] = 0;
                *reinterpret_cast<volatile int32_t*>(xctrl) = xepoch;
            }
        }
    }
}

int device_sm_count(int* out);
size_t generic_workspace_bytes(int batch, int num_q_heads, int num_kv_heads, int head_dim, int num_ctas);
int generic_merge_rotated(const float* partial_o, const float* partial_lse2, int num_parts, int64_t rows, int head_dim,
                          const float* signs, void* out, int out_dtype, float* out_lse, void* stream);
int generic_decode(const void* q, int q_dtype, int batch, int nq, int real_q_heads, int num_kv_heads, int head_dim,
                   const void* kv_cache, int64_t num_blocks, int block_size, int slot_bytes, const int32_t* page_indices,
                   const int32_t* page_indptr, int max_pages, const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                   const float* signs, float sm_scale, void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                   float* out_lse, int emit_rotated, int num_ctas, void* stream);

bool mq_applicable(int num_kv_heads, int cols);
int launch_decode_mq(const DecodeParams& d, int num_kv_heads, int64_t num_blocks, int grid, int causal, cudaStream_t stream);

static thread_local cudaEvent_t g_events[3] = {nullptr, nullptr, nullptr};
static int g_exchange_spin_limit = kExchangeSpinLimit;

struct WorkspaceLayout {
    size_t header, prefix, lse, o, total;
    int64_t slots;
};

static WorkspaceLayout workspace_layout(int batch, int num_q_heads, int num_kv_heads, int num_ctas) {
    WorkspaceLayout w;
    const int pps = kConsumerWarps / num_kv_heads;
    w.slots = ((int64_t)num_ctas + batch) * pps;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    w.header = 0;
    w.prefix = up(64);
    w.lse = w.prefix + up(sizeof(int32_t) * ((size_t)batch + 1));
    w.o = w.lse + up(sizeof(float) * (size_t)w.slots * num_q_heads);
    w.total = w.o + up(sizeof(float) * (size_t)w.slots * num_q_heads * kHeadDim);
    return w;
}

static int resolve_ctas(int num_ctas, int* out) {
    if (num_ctas > 0) {
        *out = num_ctas;
        return TQ_OK;
    }
    int sms = 0;
    int rc = device_sm_count(&sms);
    if (rc != TQ_OK) return rc;
    *out = sms;  // one thread block per SM
    return TQ_OK;
}

template <int HKV, bool STRIDED>
static int launch_decode(DecodeParams& p, int grid, cudaStream_t stream) {
    using S = DecodeSmem<HKV, STRIDED>;
    const int smem = (int)(kLutAddr + kLutSpan) + (kStages - 1) * S::kStageBytes;  // from offset 0: ample
    static bool configured[64] = {};  // the attribute is per device
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        TQ_CUDA(cudaFuncSetAttribute(decode_paged_kernel<HKV, STRIDED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    TQ_CUDA(launch_serialized(decode_paged_kernel<HKV, STRIDED>, dim3(grid), dim3(kDecodeThreads), smem, stream, p));
    return TQ_OK;
}

// KV heads one launch handles.  Up to 16 heads that fill the token rows of the cache: one launch
// on dense rows.  More heads (a multiple of 4): launches of 16, 8 or 4 heads on strided rows.
static bool single_launch(int num_kv_heads) {
    return num_kv_heads == 1 || num_kv_heads == 2 || num_kv_heads == 4 || num_kv_heads == 8 || num_kv_heads == 16;
}
static int chunk_heads(int remaining) { return remaining >= 16 ? 16 : remaining >= 8 ? 8 : 4; }
static int largest_chunk(int num_kv_heads) { return single_launch(num_kv_heads) ? num_kv_heads : chunk_heads(num_kv_heads); }

struct ExchangeArgs {
    int rank, world;
    void* const* bufs;  // host array [world]: every rank's exchange buffer as mapped in this process
    size_t bytes;       // size of each buffer
};

static int decode_common(const void* q, int q_dtype, int batch, int nq, int real_q_heads, int num_kv_heads,
                         int head_dim, const void* kv_cache, int64_t num_blocks, int block_size,
                         int slot_bytes, const int32_t* page_indices, const int32_t* page_indptr,
                         int max_pages, const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                         const float* signs, float sm_scale, void* workspace, size_t workspace_bytes,
                         void* out, int out_dtype, float* out_lse, int emit_rotated, int num_ctas,
                         void* stream, const ExchangeArgs* x = nullptr, int causal = 0) {
    TQ_REQUIRE(batch >= 0, TQ_ERR_INVALID, "negative batch");
    if (batch == 0) return TQ_OK;
    if (x) {
        TQ_REQUIRE(x->world >= 1 && x->world <= kMaxExchangeRanks && x->rank >= 0 && x->rank < x->world && x->bufs,
                   TQ_ERR_INVALID, "exchange: rank %d of %d (at most %d ranks)", x->rank, x->world, kMaxExchangeRanks);
        const ExchangeLayout xl(x->world, (int64_t)batch * nq * real_q_heads);
        TQ_REQUIRE(x->bytes >= xl.total, TQ_ERR_WORKSPACE, "exchange buffer too small: %zu < %zu", x->bytes, xl.total);
        for (int w = 0; w < x->world; w++)
            TQ_REQUIRE(x->bufs[w] && ((uintptr_t)x->bufs[w] % 256) == 0, TQ_ERR_INVALID,
                       "exchange buffer %d is null or not 256-byte aligned", w);
    }
    TQ_REQUIRE(q && kv_cache && page_indices && seq_lens && signs && workspace && out, TQ_ERR_INVALID, "null pointer");
    if (head_dim != kHeadDim && head_dim != 96) {  // other head sizes (64, 256, ...): the plain kernels
        TQ_REQUIRE(!x && !causal, TQ_ERR_UNSUPPORTED,
                   "head size %d: no causal queries and no KV-split exchange (those are built for padded size 128)", head_dim);
        TQ_REQUIRE(q_dtype >= TQ_F32 && q_dtype <= TQ_BF16 && out_dtype >= TQ_F32 && out_dtype <= TQ_BF16, TQ_ERR_INVALID, "bad dtype");
        TQ_REQUIRE(((uintptr_t)workspace % 256) == 0, TQ_ERR_INVALID, "workspace must be 256-byte aligned");
        return generic_decode(q, q_dtype, batch, nq, real_q_heads, num_kv_heads, head_dim, kv_cache, num_blocks, block_size,
                              slot_bytes, page_indices, page_indptr, max_pages, seq_lens, kv_begin, kv_end, signs, sm_scale,
                              workspace, workspace_bytes, out, out_dtype, out_lse, emit_rotated, num_ctas, stream);
    }
    TQ_REQUIRE(block_size == kPageTokens, TQ_ERR_UNSUPPORTED, "decode supports 16-token pages, got %d", block_size);
    TQ_REQUIRE(slot_bytes == kSlotBytes, TQ_ERR_UNSUPPORTED, "decode supports 80-byte slots, got %d", slot_bytes);
    TQ_REQUIRE(single_launch(num_kv_heads) || (num_kv_heads > 8 && num_kv_heads % 4 == 0), TQ_ERR_UNSUPPORTED,
               "num_kv_heads must be 1, 2, 4, 8, 16 or a larger multiple of 4, got %d", num_kv_heads);
    TQ_REQUIRE(!x || single_launch(num_kv_heads), TQ_ERR_UNSUPPORTED,
               "the kernel-side exchange takes at most 16 KV heads per GPU, got %d", num_kv_heads);
    TQ_REQUIRE(nq >= 1 && real_q_heads >= 1 && real_q_heads % num_kv_heads == 0, TQ_ERR_INVALID,
               "query heads must be a positive multiple of the KV heads, queries_per_seq >= 1");
    // up to 8 query columns per KV head: the mma.sync kernel; up to 32: the tcgen05 kernel
    const int cols = nq * (real_q_heads / num_kv_heads);
    // (causal queries always take the wide-tile kernel: it masks per column)
    const bool wide = cols > 8 || causal;
    TQ_REQUIRE(!causal || (mq_applicable(num_kv_heads, cols < 9 ? 9 : cols) && !x && kv_begin == 0 && kv_end < 0 && !emit_rotated),
               TQ_ERR_UNSUPPORTED, "causal queries: queries_per_seq x query heads per KV head up to 32, 2, 4, 8 or 16 KV heads, "
               "whole sequences (got %d x %d, %d KV heads)", nq, real_q_heads / num_kv_heads, num_kv_heads);
    TQ_REQUIRE(cols <= 8 || mq_applicable(num_kv_heads, cols), TQ_ERR_UNSUPPORTED,
               "queries_per_seq x query heads per KV head must be 1..8, or up to 32 with 2, 4, 8 or 16 KV heads (got %d x %d, "
               "%d KV heads)", nq, real_q_heads / num_kv_heads, num_kv_heads);
    const int real_group = real_q_heads / num_kv_heads;
    const int first_chunk = largest_chunk(num_kv_heads);
    TQ_REQUIRE(q_dtype >= TQ_F32 && q_dtype <= TQ_BF16 && out_dtype >= TQ_F32 && out_dtype <= TQ_BF16,
               TQ_ERR_INVALID, "bad dtype");
    TQ_REQUIRE(((uintptr_t)kv_cache % 16) == 0 && ((uintptr_t)workspace % 256) == 0, TQ_ERR_INVALID,
               "kv_cache must be 16-byte and workspace 256-byte aligned");
    TQ_REQUIRE(kv_begin >= 0 && kv_begin % kPageTokens == 0, TQ_ERR_INVALID, "kv_begin must be a multiple of 16");
    TQ_REQUIRE(page_indptr || max_pages > 0, TQ_ERR_INVALID, "max_pages must be positive for a dense block table");
    TQ_REQUIRE(num_blocks >= 1, TQ_ERR_INVALID, "the cache has no pages (num_blocks = %lld)", (long long)num_blocks);
    int ctas = 0;
    int rc = resolve_ctas(num_ctas, &ctas);
    if (rc != TQ_OK) return rc;
    // the workspace is sized for the largest launch and reused by the others (stream order)
    const WorkspaceLayout w = workspace_layout(batch, nq * real_group * first_chunk, first_chunk, ctas);
    TQ_REQUIRE(workspace_bytes >= w.total, TQ_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.total);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);

    DecodeParams p{};
    p.q = q;
    p.kv_cache = static_cast<const uint8_t*>(kv_cache);
    p.page_indices = page_indices;
    p.page_indptr = page_indptr;
    p.seq_lens = seq_lens;
    p.signs = signs;
    p.header = reinterpret_cast<int32_t*>(ws + w.header);
    p.page_prefix = reinterpret_cast<int32_t*>(ws + w.prefix);
    p.partial_lse = reinterpret_cast<float*>(ws + w.lse);
    p.partial_o = reinterpret_cast<float*>(ws + w.o);
    p.slab_bytes = num_blocks * (int64_t)block_size * num_kv_heads * slot_bytes;
    p.num_blocks = num_blocks;
    p.kv_begin = kv_begin;
    p.kv_end = kv_end;
    p.batch = batch;
    p.nq = nq;
    p.real_heads = real_q_heads;
    p.real_group = real_group;
    p.group = nq * real_group;
    p.max_pages = max_pages;
    p.q_dtype = q_dtype;
    p.head_dim = head_dim;
    p.kv_row_bytes = (int64_t)num_kv_heads * slot_bytes;
    const double inv_sqrt_d = 1.0 / std::sqrt((double)kHeadDim);
    p.k_scale = (float)(inv_sqrt_d * (double)sm_scale * 1.4426950408889634);
    p.v_scale = (float)inv_sqrt_d;
    for (int k = 0; k < 16; k++) {
        const __half h = __float2half_rn((float)kCentroidsN01_4bit[k]);
        p.centroid_h[k] = *reinterpret_cast<const uint16_t*>(&h);
    }
    // The status word (header[0]) is sticky: the kernels only ever raise it, nobody clears it here
    // (a memset node per call costs more than it is worth); it means something to a caller who
    // zeroed the first bytes of the workspace once.
    if (g_events[0]) TQ_CUDA(cudaEventRecord(g_events[0], s));
    const bool strided = !single_launch(num_kv_heads);
    for (int kv0 = 0; kv0 < num_kv_heads;) {
        const int hk = strided ? chunk_heads(num_kv_heads - kv0) : num_kv_heads;  // KV heads of this launch
        const int vheads = nq * real_group * hk;                                    // its virtual query heads
        p.num_q_heads = vheads;
        p.kv_head_off = kv0 * slot_bytes;
        p.q_head_base = kv0 * real_group;
        if (wide) {
            rc = launch_decode_mq(p, num_kv_heads, num_blocks, ctas, causal, s);
        } else if (strided) {
            switch (hk) {
                case 16: rc = launch_decode<16, true>(p, ctas, s); break;
                case 8: rc = launch_decode<8, true>(p, ctas, s); break;
                default: rc = launch_decode<4, true>(p, ctas, s); break;
            }
        } else {
            switch (hk) {
                case 16: rc = launch_decode<16, false>(p, ctas, s); break;
                case 8: rc = launch_decode<8, false>(p, ctas, s); break;
                case 4: rc = launch_decode<4, false>(p, ctas, s); break;
                case 2: rc = launch_decode<2, false>(p, ctas, s); break;
                default: rc = launch_decode<1, false>(p, ctas, s); break;
            }
        }
        if (rc != TQ_OK) return rc;
        if (g_events[1] && kv0 == 0) TQ_CUDA(cudaEventRecord(g_events[1], s));

        MergeParams m{};
        m.partial_o = p.partial_o;
        m.partial_lse = p.partial_lse;
        m.header = p.header;
        m.page_prefix = p.page_prefix;
        m.signs = signs;
        m.out = out;
        m.out_lse = out_lse;
        m.rows = batch;
        m.num_q_heads = vheads;
        m.nq = nq;
        m.real_heads = real_q_heads;
        m.real_group = real_group;
        m.q_head_base = p.q_head_base;
        m.head_dim = emit_rotated ? kHeadDim : head_dim;
        m.pps = wide ? 1 : kConsumerWarps / hk;   // partial slots per (block, sequence)
        m.grid_ctas = ctas;
        m.out_dtype = out_dtype;
        m.emit_rotated = emit_rotated;
        if (x) {
            m.xmode = 1;
            m.xrank = x->rank;
            m.xworld = x->world;
            m.xrows = (int64_t)batch * nq * real_q_heads;
            m.xspin = g_exchange_spin_limit;
            for (int w = 0; w < x->world; w++) m.xbuf[w] = static_cast<unsigned char*>(x->bufs[w]);
        }
        // parts per sequence: about (blocks x page lanes) / batch; many of them -> the wide merge
        if ((int64_t)ctas * m.pps > (int64_t)64 * batch)
            TQ_CUDA(launch_serialized(merge_kernel<16>, dim3((unsigned)batch, (unsigned)vheads), dim3(512), 0, s, m));
        else
            TQ_CUDA(launch_serialized(merge_kernel<4>, dim3((unsigned)batch, (unsigned)vheads), dim3(128), 0, s, m));
        if (x) {
            // second pass: wait for every rank's partial in this rank's buffer, merge, rotate back
            MergeParams f = m;
            f.xmode = 2;
            f.header = nullptr;
            f.page_prefix = nullptr;
            f.rows = m.xrows;
            f.num_q_heads = 1;
            f.nq = 1;
            f.num_parts = x->world;
            f.emit_rotated = 0;
            TQ_CUDA(launch_serialized(merge_kernel<4>, dim3((unsigned)m.xrows, 1), dim3(128), 0, s, f));
        }
        kv0 += hk;
    }
    if (g_events[2]) TQ_CUDA(cudaEventRecord(g_events[2], s));
    return TQ_OK;
}

}  // namespace tq

extern "C" int tq_debug_set_decode_events(void* ev_start, void* ev_mid, void* ev_end) {
    tq::g_events[0] = static_cast<cudaEvent_t>(ev_start);
    tq::g_events[1] = static_cast<cudaEvent_t>(ev_mid);
    tq::g_events[2] = static_cast<cudaEvent_t>(ev_end);
    return TQ_OK;
}

extern "C" int tq_decode_max_query_columns(void) { return 32; }

extern "C" size_t tq_decode_workspace_bytes(int batch, int num_q_heads, int num_kv_heads,
                                            int head_dim, int num_ctas) {
    if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return 0;
    if (head_dim != tq::kHeadDim && head_dim != 96 && head_dim > 0)
        return head_dim > 32 && head_dim <= 256 ? tq::generic_workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, num_ctas) : 0;
    if (!tq::single_launch(num_kv_heads) && !(num_kv_heads > 8 && num_kv_heads % 4 == 0)) return 0;
    int ctas = 0;
    if (tq::resolve_ctas(num_ctas, &ctas) != TQ_OK) return 0;
    const int chunk = tq::largest_chunk(num_kv_heads);  // the launches of a call share the workspace
    return tq::workspace_layout(batch, num_q_heads / num_kv_heads * chunk, chunk, ctas).total;
}

extern "C" int tq_decode_paged(const void* q, int q_dtype, int batch, int num_q_heads,
                               int num_kv_heads, int head_dim, const void* kv_cache,
                               int64_t num_blocks, int block_size, int slot_bytes,
                               const int32_t* page_indices, const int32_t* page_indptr,
                               int max_pages, const int32_t* seq_lens, const float* signs,
                               float sm_scale, void* workspace, size_t workspace_bytes, void* out,
                               int out_dtype, float* out_lse, int num_ctas, void* stream) {
    return tq::decode_common(q, q_dtype, batch, 1, num_q_heads, num_kv_heads, head_dim, kv_cache,
                             num_blocks, block_size, slot_bytes, page_indices, page_indptr,
                             max_pages, seq_lens, 0, -1, signs, sm_scale, workspace, workspace_bytes,
                             out, out_dtype, out_lse, 0, num_ctas, stream);
}

extern "C" int tq_decode_paged_multi(const void* q, int q_dtype, int batch, int queries_per_seq,
                                     int num_q_heads, int num_kv_heads, int head_dim, const void* kv_cache,
                                     int64_t num_blocks, int block_size, int slot_bytes,
                                     const int32_t* page_indices, const int32_t* page_indptr, int max_pages,
                                     const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                                     const float* signs, float sm_scale, void* workspace,
                                     size_t workspace_bytes, void* out, int out_dtype, float* out_lse,
                                     int rotated_partial, int num_ctas, void* stream) {
    if (rotated_partial) {
        TQ_REQUIRE(out_lse != nullptr && out_dtype == TQ_F32, TQ_ERR_INVALID,
                   "a rotated partial needs fp32 out and out_lse");
    }
    return tq::decode_common(q, q_dtype, batch, queries_per_seq, num_q_heads, num_kv_heads, head_dim, kv_cache,
                             num_blocks, block_size, slot_bytes, page_indices, page_indptr, max_pages,
                             seq_lens, kv_begin, kv_end, signs, sm_scale, workspace, workspace_bytes, out,
                             out_dtype, out_lse, rotated_partial ? 1 : 0, num_ctas, stream);
}

extern "C" int tq_set_exchange_wait_limit(int polls) {
    tq::g_exchange_spin_limit = polls > 0 ? polls : tq::kExchangeSpinLimit;
    return TQ_OK;
}

extern "C" size_t tq_exchange_bytes(int64_t rows, int world) {
    if (rows <= 0 || world < 1 || world > tq::kMaxExchangeRanks) return 0;
    return tq::ExchangeLayout(world, rows).total;
}

extern "C" int tq_decode_paged_causal(const void* q, int q_dtype, int batch, int queries_per_seq, int num_q_heads,
                                      int num_kv_heads, int head_dim, const void* kv_cache, int64_t num_blocks,
                                      int block_size, int slot_bytes, const int32_t* page_indices,
                                      const int32_t* page_indptr, int max_pages, const int32_t* seq_lens,
                                      const float* signs, float sm_scale, void* workspace, size_t workspace_bytes,
                                      void* out, int out_dtype, float* out_lse, int num_ctas, void* stream) {
    TQ_REQUIRE(queries_per_seq >= 1, TQ_ERR_INVALID, "queries_per_seq must be positive");
    return tq::decode_common(q, q_dtype, batch, queries_per_seq, num_q_heads, num_kv_heads, head_dim, kv_cache,
                             num_blocks, block_size, slot_bytes, page_indices, page_indptr, max_pages, seq_lens, 0,
                             -1, signs, sm_scale, workspace, workspace_bytes, out, out_dtype, out_lse, 0, num_ctas,
                             stream, nullptr, 1);
}

extern "C" int tq_decode_paged_exchange(const void* q, int q_dtype, int batch, int queries_per_seq,
                                        int num_q_heads, int num_kv_heads, int head_dim, const void* kv_cache,
                                        int64_t num_blocks, int block_size, int slot_bytes,
                                        const int32_t* page_indices, const int32_t* page_indptr, int max_pages,
                                        const int32_t* seq_lens, int64_t kv_begin, int64_t kv_end,
                                        const float* signs, float sm_scale, void* workspace,
                                        size_t workspace_bytes, int rank, int world, void* const* exchange_bufs,
                                        size_t exchange_bytes, void* out, int out_dtype, float* out_lse,
                                        int num_ctas, void* stream) {
    const tq::ExchangeArgs x{rank, world, exchange_bufs, exchange_bytes};
    return tq::decode_common(q, q_dtype, batch, queries_per_seq, num_q_heads, num_kv_heads, head_dim, kv_cache,
                             num_blocks, block_size, slot_bytes, page_indices, page_indptr, max_pages,
                             seq_lens, kv_begin, kv_end, signs, sm_scale, workspace, workspace_bytes, out,
                             out_dtype, out_lse, 0, num_ctas, stream, &x);
}

extern "C" int tq_decode_paged_partial(const void* q, int q_dtype, int batch, int num_q_heads,
                                       int num_kv_heads, int head_dim, const void* kv_cache,
                                       int64_t num_blocks, int block_size, int slot_bytes,
                                       const int32_t* page_indices, const int32_t* page_indptr,
                                       int max_pages, const int32_t* seq_lens, int64_t kv_begin,
                                       int64_t kv_end, const float* signs, float sm_scale,
                                       void* workspace, size_t workspace_bytes, float* out_rot,
                                       float* out_lse2, int num_ctas, void* stream) {
    return tq::decode_common(q, q_dtype, batch, 1, num_q_heads, num_kv_heads, head_dim, kv_cache,
                             num_blocks, block_size, slot_bytes, page_indices, page_indptr,
                             max_pages, seq_lens, kv_begin, kv_end, signs, sm_scale, workspace,
                             workspace_bytes, out_rot, TQ_F32, out_lse2, 1, num_ctas, stream);
}

extern "C" int tq_merge_rotated(const float* partial_o, const float* partial_lse2, int num_parts,
                                int64_t rows, int head_dim, const float* signs, void* out,
                                int out_dtype, float* out_lse, void* stream) {
    using namespace tq;
    if (rows == 0) return TQ_OK;
    TQ_REQUIRE(partial_o && partial_lse2 && signs && out, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(num_parts >= 1 && rows > 0, TQ_ERR_INVALID, "num_parts and rows must be positive");
    TQ_REQUIRE(out_dtype >= TQ_F32 && out_dtype <= TQ_BF16, TQ_ERR_INVALID, "bad out_dtype");
    if (head_dim != kHeadDim && head_dim != 96)   // partials of the other head sizes are [..][padded] wide
        return generic_merge_rotated(partial_o, partial_lse2, num_parts, rows, head_dim, signs, out, out_dtype, out_lse, stream);
    MergeParams m{};
    m.partial_o = partial_o;
    m.partial_lse = partial_lse2;
    m.signs = signs;
    m.out = out;
    m.out_lse = out_lse;
    m.rows = rows;
    m.num_q_heads = 1;
    m.nq = 1;
    m.head_dim = head_dim;
    m.num_parts = num_parts;
    m.out_dtype = out_dtype;
    if (num_parts > 64)
        TQ_CUDA(launch_serialized(merge_kernel<16>, dim3((unsigned)rows, 1), dim3(512), 0, static_cast<cudaStream_t>(stream), m));
    else
        TQ_CUDA(launch_serialized(merge_kernel<4>, dim3((unsigned)rows, 1), dim3(128), 0, static_cast<cudaStream_t>(stream), m));
    return TQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode without any caller-side or library-side allocation.
//
// Some hosts of this library may not create device memory at the time they call it: code that
// runs inside an engine whose memory pool has already been handed out in full, a plugin that is
// only given the tensors of the model and may not grow the footprint, or a caller on a path
// where cudaMalloc (an implicitly synchronising call) is forbidden.  For them the split-KV
// scratch (partials, LSEs, the small header) lives in a fixed array inside the library image.
// Every GPU that loads the library carries these kStaticScratchBytes until the process exits.
// ---------------------------------------------------------------------------------------------
namespace tq {
constexpr size_t kStaticScratchBytes = TQ_STATIC_SCRATCH_BYTES;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the
// address is looked up once per device (with that device current) and cached.
static int static_scratch_pointer(void** out) {
    static void* cached[64] = {};
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    TQ_REQUIRE(dev >= 0 && dev < 64, TQ_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!cached[dev]) {
        void* ptr = nullptr;
        TQ_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        TQ_REQUIRE(ptr != nullptr, TQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return TQ_OK;
}
}  // namespace tq

extern "C" int tq_decode_paged_static(const void* q, int q_dtype, int batch, int num_q_heads,
                                      int num_kv_heads, int head_dim, const void* kv_cache,
                                      int64_t num_blocks, int block_size, int slot_bytes,
                                      const int32_t* page_indices, const int32_t* page_indptr,
                                      int max_pages, const int32_t* seq_lens, const float* signs,
                                      float sm_scale, void* out, int out_dtype, float* out_lse,
                                      int num_ctas, void* stream) {
    using namespace tq;
    TQ_REQUIRE(batch >= 0, TQ_ERR_INVALID, "negative batch");
    if (batch == 0) return TQ_OK;
    TQ_REQUIRE(num_kv_heads == 1 || num_kv_heads == 2 || num_kv_heads == 4 || num_kv_heads == 8 || num_kv_heads == 16,
               TQ_ERR_UNSUPPORTED, "num_kv_heads must be 1, 2, 4, 8 or 16, got %d", num_kv_heads);
    TQ_REQUIRE(num_q_heads > 0, TQ_ERR_INVALID, "num_q_heads must be positive");
    int ctas = 0;
    int rc = resolve_ctas(num_ctas, &ctas);
    if (rc != TQ_OK) return rc;
    const size_t need = workspace_layout(batch, num_q_heads, num_kv_heads, ctas).total;
    TQ_REQUIRE(need <= kStaticScratchBytes, TQ_ERR_WORKSPACE,
               "this call needs %zu bytes of split-KV scratch but the built-in scratch holds %zu: lower batch "
               "(%d), num_q_heads (%d) or num_ctas (%d), or use tq_decode_paged with your own workspace",
               need, kStaticScratchBytes, batch, num_q_heads, ctas);
    void* scratch = nullptr;
    rc = static_scratch_pointer(&scratch);
    if (rc != TQ_OK) return rc;
    return decode_common(q, q_dtype, batch, 1, num_q_heads, num_kv_heads, head_dim, kv_cache, num_blocks,
                         block_size, slot_bytes, page_indices, page_indptr, max_pages, seq_lens, 0, -1,
                         signs, sm_scale, scratch, kStaticScratchBytes, out, out_dtype, out_lse, 0, ctas,
                         stream);
}

extern "C" int tq_decode_static_status(int32_t* status_out, void* stream) {
    using namespace tq;
    TQ_REQUIRE(status_out != nullptr, TQ_ERR_INVALID, "null pointer");
    void* scratch = nullptr;
    int rc = static_scratch_pointer(&scratch);
    if (rc != TQ_OK) return rc;
    TQ_CUDA(cudaMemcpyAsync(status_out, scratch, sizeof(int32_t), cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return TQ_OK;
}
