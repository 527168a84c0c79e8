// Shared device helpers for the sm_100a kernels: mbarrier and bulk-copy (TMA) PTX wrappers,
// programmatic dependent launch, bounded waits, status codes.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/llm_b200.h"

namespace llmb {

// ---------------------------------------------------------------------------------------
// Host side: per-device status word that kernels set when a bounded wait gives up.
// ---------------------------------------------------------------------------------------
int *device_status_ptr();  // address of the status word (a module variable: one per device, zero at load)

#define LLMB_CUDA_OK(expr)                                                   \
    do {                                                                     \
        cudaError_t _e = (expr);                                             \
        if (_e != cudaSuccess) return ::llmb::cuda_fail(_e, __FILE__, __LINE__); \
    } while (0)

int cuda_fail(cudaError_t e, const char *file, int line);
void set_last_error(const char *msg);
int sm_count_cached();

// A kernel's opt-in to more than 48 KB of dynamic shared memory is a per-device attribute.  `have` is a
// per-kernel table indexed by device ordinal; returns true when the current device's entry is below
// `bytes` (the caller then sets the attribute and records it with smem_attr_set).
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, size_t (&have)[kMaxDevices], size_t bytes) {
    const int dev = current_device_slot();
    if (dev >= 0 && have[dev] >= bytes) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && dev >= 0) have[dev] = bytes;
    return e;
}

// ---------------------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------------------
#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in these kernels is bounded.  try_wait suspends for a hardware-defined time slice
// per call, so the cap below is on the order of seconds; a wait that runs out records `code`
// in the status word and returns false, and the caller winds the kernel down.
constexpr uint32_t kWaitSpins = 1u << 20;

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *status, int code) {
    for (uint32_t i = 0; i < kWaitSpins; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicExch(status, code);
    return false;
}

// Warp-collective wait: every lane tries once (the common case: the data is already there); if not,
// lane 0 alone polls, so a waiting CTA does not flood the shared-memory pipe that the bulk copies
// need to land their data, and the other lanes take one more try_wait afterwards to acquire the
// phase themselves.  All 32 lanes must call it.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, int *status, int code, int lane) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, status, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok && lane != 0) ok = mbar_wait(bar, parity, status, code) ? 1 : 0;  // already complete: returns at once
    return ok != 0;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Source,
// destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue now /
// wait until every kernel this one depends on has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

#endif  // __CUDACC__

// Launch helper: kernel launch with the programmatic-stream-serialization attribute, so that
// consecutive kernels in a stream (or captured graph) overlap prologue and epilogue.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the CTAs grouped into thread-block clusters of `cluster` CTAs (a grid dimension must be a
// multiple of the cluster's); (1, 1, 1) is a plain launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      bool pdl, dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster.x;
    attr[1].val.clusterDim.y = cluster.y;
    attr[1].val.clusterDim.z = cluster.z;
    cfg.attrs = attr;
    cfg.numAttrs = cluster.x * cluster.y * cluster.z > 1 ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace llmb
