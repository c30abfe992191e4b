// Shared launch helpers, status codes and the last-error slot for the C-ABI library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/splatad_b200.h"

namespace splatad {

constexpr int kThreads = 256;
// B200 has 148 SMs; persistent kernels use a fixed grid that is a multiple of it.
constexpr int kNumSMs = 148;

void set_last_error(const char *fmt, ...);

inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("%s: %s", what, cudaGetErrorString(e));
        return SPLATAD_ERR_CUDA;
    }
    return SPLATAD_OK;
}

#define SPL_REQUIRE(cond, code, ...)                                                             \
    do {                                                                                         \
        if (!(cond)) {                                                                           \
            ::splatad::set_last_error(__VA_ARGS__);                                              \
            return (code);                                                                       \
        }                                                                                        \
    } while (0)

inline uint32_t div_up(uint64_t a, uint64_t b) { return (uint32_t)((a + b - 1) / b); }

// Optional per-kernel timing (off by default, see splatad_profile_enable): while enabled every
// launch site wrapped in SPL_PROF records a CUDA event pair on the launching stream.
bool prof_enabled();
void prof_begin(const char *name, cudaStream_t st);
void prof_end(cudaStream_t st);
struct ProfScope {
    cudaStream_t st;
    bool on;
    ProfScope(const char *name, cudaStream_t s) : st(s), on(prof_enabled()) {
        if (on) prof_begin(name, st);
    }
    ~ProfScope() {
        if (on) prof_end(st);
    }
};
#define SPL_PROF_CAT2(a, b) a##b
#define SPL_PROF_CAT(a, b) SPL_PROF_CAT2(a, b)
#define SPL_PROF(name, st) ::splatad::ProfScope SPL_PROF_CAT(_prof_, __LINE__)(name, st)

// Programmatic dependent launch for chains of short kernels on one stream. A kernel started with
// launch_chained() may have its blocks placed on the SMs while the kernel before it is still
// draining; it must call chain_enter() before it touches anything, which waits (in hardware) until
// the whole preceding kernel has finished and its writes are visible, and then lets the kernel
// behind it start the same way. Started with <<<>>> instead, chain_enter() does nothing.
__device__ __forceinline__ void chain_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KP, typename... A>
inline void launch_chained(void (*kernel)(KP...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                           A &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KP>(args)...);   // errors surface in check_launch()
}

// ---------------------------------------------------------------------------------------------
// Bulk asynchronous copies global -> shared (the TMA engine's one-dimensional form) completing on
// an mbarrier, for kernels that prefetch their next slab of inputs while they compute on the
// current one. Source, destination and size must be multiples of 16 bytes. Every wait is bounded:
// after kAsyncWaitLimit polls the caller gives up, counts a timeout (splatad_async_copy_timeouts)
// and leaves without touching the data.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kAsyncWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// makes the initialised barriers visible to the asynchronous proxy (follow with __syncthreads())
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_global, uint32_t bytes,
                                              unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(__cvta_generic_to_global(src_global)), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// true when the barrier's phase `parity` has completed; false after kAsyncWaitLimit polls
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t i = 0; i < kAsyncWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Cooperative copy of `nfl` contiguous floats global -> shared with 128-bit loads when the
// source is 16-byte aligned (it is whenever the tensor base is, because block slabs start at
// multiples of 256 rows).
__device__ __forceinline__ void stage_in(const float *__restrict__ src, float *smem, uint32_t nfl) {
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const uint32_t nvec = nfl >> 2;
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(smem);
        for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x) d4[i] = __ldg(s4 + i);
        for (uint32_t i = (nvec << 2) + threadIdx.x; i < nfl; i += blockDim.x) smem[i] = __ldg(src + i);
    } else {
        for (uint32_t i = threadIdx.x; i < nfl; i += blockDim.x) smem[i] = __ldg(src + i);
    }
}

// Cooperative copy shared -> global, 128-bit stores when aligned.
__device__ __forceinline__ void stage_out(float *__restrict__ dst, const float *smem, uint32_t nfl) {
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        const uint32_t nvec = nfl >> 2;
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        const float4 *s4 = reinterpret_cast<const float4 *>(smem);
        for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x) d4[i] = s4[i];
        for (uint32_t i = (nvec << 2) + threadIdx.x; i < nfl; i += blockDim.x) dst[i] = smem[i];
    } else {
        for (uint32_t i = threadIdx.x; i < nfl; i += blockDim.x) dst[i] = smem[i];
    }
}

} // namespace splatad
