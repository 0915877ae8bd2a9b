// Shared device/host helpers for the sm_100a kernels: error plumbing, mbarrier and bulk-copy
// PTX wrappers (non-multicast), small conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/turboquant_b200.h"

namespace tq {

// ---------------------------------------------------------------------------------------
// host-side error reporting (thread-local message returned by tq_last_error)
// ---------------------------------------------------------------------------------------
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define TQ_REQUIRE(cond, code, ...)                    \
    do {                                               \
        if (!(cond)) return ::tq::fail(code, __VA_ARGS__); \
    } while (0)

#define TQ_CUDA(call)                                                                         \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return ::tq::fail(TQ_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

// Codebook constants shared by every translation unit (defined in tq_api.cu).
void host_codebook(int dim, int bits, float* centroids, float* boundaries);
extern const double kCentroidsN01_4bit[16];

// ---------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One try.  The suspend-time hint (nanoseconds) lets the waiting warp sleep in the barrier unit until
// the phase completes or the hint runs out, instead of spinning through the issue slots of the
// warps that have work.
#ifndef TQ_WAIT_HINT_NS
#define TQ_WAIT_HINT_NS 0
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
#if TQ_WAIT_HINT_NS > 0
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)TQ_WAIT_HINT_NS)
        : "memory");
#else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
#endif
    return ok != 0;
}

// Bounded wait: gives up after kSpinLimit polls (each poll itself blocks for a
// hardware-defined time slice), so a lost copy can never hang the GPU.  Returns false on
// timeout; the caller raises the CTA's abort flag and unwinds.
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Brings one line into L2 without handing a value to the kernel (L2 is the point of coherence, so a
// line fetched early still shows later writes of other kernels).
__device__ __forceinline__ void prefetch_l2(const void* ptr) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

// Programmatic dependent launch: the write, decode and merge kernels are launched with programmatic
// stream serialization, so a kernel's blocks may be scheduled (and run their on-chip prologue)
// while the kernel before it in the stream drains.  grid_dependency_wait() returns once that
// kernel has completed and its writes are visible; nothing before it may touch global memory.
// Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename P>
static cudaError_t launch_serialized(void (*kernel)(P), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     const P& params) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

// 1-D bulk async copy global -> this CTA's shared memory, completing on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// The same with an L2 eviction priority for the lines it brings in (data that is read once should
// not push out what the neighbouring kernels reuse).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                              uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t hi16) { return __uint_as_float(hi16 << 16); }

template <int DT>
struct InType;
template <>
struct InType<TQ_F32> { using type = float; };
template <>
struct InType<TQ_F16> { using type = __half; };
template <>
struct InType<TQ_BF16> { using type = __nv_bfloat16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

}  // namespace tq
