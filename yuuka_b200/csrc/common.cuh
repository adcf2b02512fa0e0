// Shared host-side plumbing of libyuuka_cuda: handle types, error reporting
// and the guard that keeps C++ exceptions behind the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <exception>
#include <new>
#include <string>
#include <utility>

#include "yuuka_cuda.h"

namespace yk {

// Thread-local message of the most recent failed call (the reference keeps the
// same contract: backend/hip/bridge/bridge.cpp:47-57).
std::string & last_error_ref();
yuuka_status fail(yuuka_status code, const char * fmt, ...);

struct StatusError {
    yuuka_status code;
};

#define YK_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t err__ = (expr);                                                           \
        if (err__ != cudaSuccess) {                                                           \
            yk::fail(YUUKA_ERR_DEVICE, "%s failed: %s", #expr, cudaGetErrorString(err__));    \
            throw yk::StatusError{YUUKA_ERR_DEVICE};                                          \
        }                                                                                     \
    } while (0)

#define YK_REQUIRE(cond, code, ...)                                                           \
    do {                                                                                      \
        if (!(cond)) {                                                                        \
            yk::fail(code, __VA_ARGS__);                                                      \
            throw yk::StatusError{code};                                                      \
        }                                                                                     \
    } while (0)

// Runs fn and converts every failure into a status (bridge.cpp:1893-1904).
template <typename F>
yuuka_status guard(F && fn) {
    try {
        fn();
        return YUUKA_OK;
    } catch (const StatusError & e) {
        return e.code;
    } catch (const std::bad_alloc &) {
        return fail(YUUKA_ERR_ALLOCATION, "host allocation failed");
    } catch (const std::exception & e) {
        return fail(YUUKA_ERR_INTERNAL, "%s", e.what());
    } catch (...) {
        return fail(YUUKA_ERR_INTERNAL, "unknown failure");
    }
}

inline uint64_t row_bytes(uint32_t dtype, uint64_t cols) {
    switch (dtype) {
    case YUUKA_DTYPE_F32: return cols * 4;
    case YUUKA_DTYPE_F16: return cols * 2;
    case YUUKA_DTYPE_BF16: return cols * 2;
    case YUUKA_DTYPE_Q8_0: return cols % 32 ? 0 : cols / 32 * 34;
    case YUUKA_DTYPE_Q4_K: return cols % 256 ? 0 : cols / 256 * 144;
    case YUUKA_DTYPE_Q5_K: return cols % 256 ? 0 : cols / 256 * 176;
    case YUUKA_DTYPE_Q6_K: return cols % 256 ? 0 : cols / 256 * 210;
    default: return 0;
    }
}

}  // namespace yk

struct yuuka_device {
    int index = 0;
    cudaDeviceProp prop{};
    int sm_count = 0;
};

struct yuuka_buffer {
    yuuka_device * dev = nullptr;
    void * ptr = nullptr;
    uint64_t bytes = 0;
};

struct yuuka_stream {
    yuuka_device * dev = nullptr;
    cudaStream_t s = nullptr;
};

struct yuuka_event {
    yuuka_device * dev = nullptr;
    cudaEvent_t e = nullptr;
};

namespace yk {
inline void record_completion(yuuka_stream * stream, yuuka_event * completion) {
    if (completion) YK_CUDA(cudaEventRecord(completion->e, stream->s));
}
inline void set_device(const yuuka_device * dev) { YK_CUDA(cudaSetDevice(dev->index)); }

// Programmatic dependent launch. Every kernel of the step calls pdl_entry() (or
// pdl_trigger() ... pdl_wait()) before it reads anything a previous kernel wrote.
// The launch attribute lets the next kernel's CTAs take the SM slots that this
// kernel's finished CTAs free, and the wait holds them until this kernel has
// completed and its writes are visible; the GEMM issues its first weight loads
// before the wait. A kernel launched without the attribute sees the instructions
// as no-ops and keeps plain stream order.
// An explicit early trigger (griddepcontrol.launch_dependents at kernel entry)
// measured slower on the 4B verify step (3.9 ms with it in every kernel, 3.3 ms
// with it in the small kernels only, 3.1 ms with none), so both switches are 0:
// a dependent grid that is resident early and has to block in griddepcontrol.wait
// for microseconds resumes late (about 7 us per occurrence on the delta-net pair).
#ifdef __CUDACC__
#ifndef YK_PDL_EARLY_TRIGGER
#define YK_PDL_EARLY_TRIGGER 0
#endif
__device__ __forceinline__ void pdl_trigger() {
#if YK_PDL_EARLY_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A late trigger: a kernel calls this once its long part is over (a GEMM after its last row group, the
// delta-net scan after the recurrence). The dependent grid is released when every CTA has passed this
// point or exited, so its launch latency overlaps the epilogues of the slowest CTAs instead of following them.
#ifndef YK_PDL_LATE_TRIGGER
#define YK_PDL_LATE_TRIGGER 1
#endif
__device__ __forceinline__ void pdl_trigger_late() {
#if YK_PDL_LATE_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
#ifndef YK_PDL_EARLY_SMALL
#define YK_PDL_EARLY_SMALL 0
#endif
__device__ __forceinline__ void pdl_entry() {
#if YK_PDL_EARLY_SMALL
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
    pdl_wait();
}
#endif

bool pdl_enabled();  // false when YUUKA_CUDA_NO_PDL=1

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    YK_CUDA(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...));
}

// The same with thread-block clusters of cluster_x CTAs along x (gridDim.x a multiple of cluster_x).
template <typename... KArgs, typename... Args>
inline void launch_k_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, unsigned cluster_x,
                             Args &&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cluster_x;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    YK_CUDA(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...));
}

#if defined(__CUDACC__)
// All threads of all CTAs of the cluster (hardware barrier; every CTA must reach it).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A double in the shared memory of CTA `rank` of this cluster, at the address `p` has in this CTA.
__device__ __forceinline__ double ld_cluster_f64(const double * p, unsigned rank) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    double v;
    asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(const unsigned long long * p, unsigned rank) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return v;
}
// Stores a float at the address `p` has in this CTA, in the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ void st_cluster_f32(float * p, unsigned rank, float v) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float * p, unsigned rank) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(const float * p, unsigned rank) {  // p 16-byte aligned
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ unsigned cluster_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
#endif
}  // namespace yk
