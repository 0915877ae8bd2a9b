// Offload / restore of packed cache pages.
//
// A page of the quantized cache is the natural unit to spill to host memory (or to a peer) and to
// bring back instead of re-running the prefill: the reference measures exactly that trade with a
// raw copy of a whole cache slab (tests/bench_kv_offload.py:23-62).  Here the pages of one or more
// sequences are gathered by page id into one contiguous buffer and scattered back:
//
//   packed[n][2 (K, V)][block_size][num_kv_heads][68]     68 = 64 code bytes + fp16 norm twice
//
// The 12 pad bytes of every 80-byte slot never carry information and are not moved (15 % less
// traffic over the host link); on restore they are left as they are in the destination slots.
// `packed` may be device memory (copied on by the caller) or pinned host memory mapped into the
// device's address space, in which case the kernels move the bytes over the host link themselves.
#include "tq_common.cuh"

namespace tq {

constexpr int kPagePayload = 68;  // bytes of an 80-byte slot that carry information
// Payload of the other slot sizes: 48 bytes (head size 64) carry 32 code bytes + one fp16 norm,
// moved as 36; 144 bytes (head size 256) carry 128 + 8; anything else is moved whole.
static __host__ __device__ inline int slot_payload(int slot_bytes) {
    return slot_bytes == 80 ? kPagePayload : slot_bytes == 48 ? 36 : slot_bytes == 144 ? 136 : slot_bytes;
}

struct PageMoveParams {
    uint8_t* kv_cache;
    uint8_t* packed;
    const int32_t* page_ids;
    int64_t slab_bytes;   // K slab -> V slab
    int64_t half_bytes;   // one page half in the cache: block_size * H * slot_bytes
    int64_t num_blocks;   // page ids outside [0, num_blocks) are skipped and counted
    int n_pages, slots_per_half, slot_bytes, payload_words;
};

// Pages skipped because their id lay outside the cache; read back by tq_fault_counts.
static __device__ int32_t g_pages_skipped = 0;

// One block per (page, K / V); thread i moves word i % 17 of slot i / 17.
template <bool GATHER>
__global__ void __launch_bounds__(256) page_move_kernel(const __grid_constant__ PageMoveParams p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int n = blockIdx.x, which = blockIdx.y;
    const int64_t page = p.page_ids[n];
    if ((uint64_t)page >= (uint64_t)p.num_blocks) {
        if (threadIdx.x == 0 && which == 0) atomicAdd(&g_pages_skipped, 1);
        return;
    }
    uint8_t* cache_half = p.kv_cache + (size_t)which * p.slab_bytes + (size_t)page * p.half_bytes;
    const int pw = p.payload_words;
    uint8_t* packed_half = p.packed + ((size_t)n * 2 + which) * (size_t)p.slots_per_half * pw * 4;
    const int words = p.slots_per_half * pw;
    for (int i = threadIdx.x; i < words; i += blockDim.x) {
        const int slot = i / pw, w = i - slot * pw;
        uint32_t* c = reinterpret_cast<uint32_t*>(cache_half + (size_t)slot * p.slot_bytes) + w;
        uint32_t* q = reinterpret_cast<uint32_t*>(packed_half) + i;
        if (GATHER) *q = *c;
        else *c = *q;
    }
}

static int page_move(bool gather, void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                     int slot_bytes, const int32_t* page_ids, int n_pages, void* packed, size_t packed_bytes,
                     void* stream) {
    TQ_REQUIRE(n_pages >= 0 && num_blocks >= 0, TQ_ERR_INVALID, "negative size");
    if (n_pages == 0) return TQ_OK;
    TQ_REQUIRE(kv_cache && page_ids && packed, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(block_size >= 1 && num_kv_heads >= 1 && slot_bytes >= 4 && slot_bytes % 4 == 0,
               TQ_ERR_INVALID, "bad geometry");
    TQ_REQUIRE(((uintptr_t)kv_cache % 4) == 0 && ((uintptr_t)packed % 4) == 0, TQ_ERR_INVALID,
               "kv_cache and packed must be 4-byte aligned");
    const size_t need = (size_t)n_pages * 2 * block_size * num_kv_heads * slot_payload(slot_bytes);
    TQ_REQUIRE(packed_bytes >= need, TQ_ERR_WORKSPACE, "packed buffer too small: %zu < %zu", packed_bytes, need);
    PageMoveParams p{};
    p.kv_cache = static_cast<uint8_t*>(kv_cache);
    p.packed = static_cast<uint8_t*>(packed);
    p.page_ids = page_ids;
    p.half_bytes = (int64_t)block_size * num_kv_heads * slot_bytes;
    p.slab_bytes = num_blocks * p.half_bytes;
    p.num_blocks = num_blocks;
    p.n_pages = n_pages;
    p.slots_per_half = block_size * num_kv_heads;
    p.slot_bytes = slot_bytes;
    p.payload_words = slot_payload(slot_bytes) / 4;
    const dim3 grid((unsigned)n_pages, 2);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gather) TQ_CUDA(launch_serialized(page_move_kernel<true>, grid, dim3(256), 0, s, p));
    else TQ_CUDA(launch_serialized(page_move_kernel<false>, grid, dim3(256), 0, s, p));
    return TQ_OK;
}

int pages_fault_count(int32_t* out) {
    TQ_CUDA(cudaMemcpyFromSymbol(out, g_pages_skipped, sizeof(int32_t)));
    return TQ_OK;
}

}  // namespace tq

extern "C" size_t tq_pages_packed_bytes(int n_pages, int block_size, int num_kv_heads) {
    if (n_pages <= 0 || block_size <= 0 || num_kv_heads <= 0) return 0;
    return (size_t)n_pages * 2 * block_size * num_kv_heads * tq::kPagePayload;
}

extern "C" size_t tq_pages_packed_bytes_for_slot(int n_pages, int block_size, int num_kv_heads, int slot_bytes) {
    if (n_pages <= 0 || block_size <= 0 || num_kv_heads <= 0 || slot_bytes < 4 || slot_bytes % 4) return 0;
    return (size_t)n_pages * 2 * block_size * num_kv_heads * tq::slot_payload(slot_bytes);
}

extern "C" int tq_pages_gather(const void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                               int slot_bytes, const int32_t* page_ids, int n_pages, void* packed,
                               size_t packed_bytes, void* stream) {
    return tq::page_move(true, const_cast<void*>(kv_cache), num_blocks, block_size, num_kv_heads, slot_bytes, page_ids,
                         n_pages, packed, packed_bytes, stream);
}

extern "C" int tq_pages_scatter(void* kv_cache, int64_t num_blocks, int block_size, int num_kv_heads,
                                int slot_bytes, const int32_t* page_ids, int n_pages, const void* packed,
                                size_t packed_bytes, void* stream) {
    return tq::page_move(false, kv_cache, num_blocks, block_size, num_kv_heads, slot_bytes, page_ids, n_pages,
                         const_cast<void*>(packed), packed_bytes, stream);
}
