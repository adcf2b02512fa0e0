// What one dependency point between two phases of a verify step costs on this device, in the two forms a step can
// take: (a) a chain of kernels launched with programmatic stream serialization inside a CUDA graph (what the
// library does: every kernel starts with griddepcontrol.wait), and (b) one persistent kernel, launched
// cooperatively so that all its CTAs are resident, whose phases are separated by a grid-wide barrier (an
// arrival counter and a bounded acquire spin). Both run one CTA of 512 threads with 160 KB of shared memory per
// SM, the shape of the quantized GEMM kernel, and a body that reads a neighbour's slot and writes its own, so
// that each phase really depends on the one before. Prints microseconds per dependency point.
#include <cstdio>
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e)); return 1; } } while (0)

__global__ void __launch_bounds__(512, 1) step_kernel(float * buf, int n) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // every CTA reads what the previous kernel wrote and writes its own slot
    float v = buf[(blockIdx.x + 1) % gridDim.x * 32 + (threadIdx.x & 31)];
    if (threadIdx.x < 32) buf[blockIdx.x * 32 + threadIdx.x] = v + 1.0f;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ unsigned g_bar;
__device__ int g_err;
__global__ void __launch_bounds__(512, 1) persistent_kernel(float * buf, int steps) {
    const unsigned nb = gridDim.x;
    for (int s = 0; s < steps; s++) {
        float v = buf[(blockIdx.x + 1) % nb * 32 + (threadIdx.x & 31)];
        if (threadIdx.x < 32) buf[blockIdx.x * 32 + threadIdx.x] = v + 1.0f;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(&g_bar, 1u);
            const unsigned target = (unsigned)(s + 1) * nb;
            unsigned seen = 0, spins = 0;
            do {
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(seen) : "l"(&g_bar) : "memory");
            } while (seen < target && ++spins < (1u << 22));
            if (seen < target) atomicExch(&g_err, 1);
        }
        __syncthreads();
    }
}

int main() {
    int sm = 0;
    CK(cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, 0));
    float * buf;
    CK(cudaMalloc(&buf, sm * 32 * sizeof(float)));
    CK(cudaMemset(buf, 0, sm * 32 * sizeof(float)));
    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    const int steps = 200;
    // (a) graph of dependent launches
    CK(cudaFuncSetAttribute(step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal));
    for (int i = 0; i < steps; i++) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(sm); cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = 160 * 1024; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        CK(cudaLaunchKernelEx(&cfg, step_kernel, buf, steps));
    }
    CK(cudaStreamEndCapture(st, &graph));
    CK(cudaGraphInstantiate(&exec, graph, 0));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int rep = 0; rep < 3; rep++) {
        CK(cudaEventRecord(e0, st));
        CK(cudaGraphLaunch(exec, st));
        CK(cudaEventRecord(e1, st));
        CK(cudaStreamSynchronize(st));
        float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
        printf("graph of %d dependent launches (148 x 512 threads, 160 KB smem): %.3f us per launch\n", steps, ms * 1000 / steps);
    }
    // (b) cooperative kernel with grid barriers
    CK(cudaFuncSetAttribute(persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    for (int rep = 0; rep < 3; rep++) {
        unsigned zero = 0;
        CK(cudaMemcpyToSymbolAsync(g_bar, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
        int nsteps = steps;
        void * args[] = {&buf, &nsteps};
        CK(cudaEventRecord(e0, st));
        CK(cudaLaunchCooperativeKernel((void *)persistent_kernel, dim3(sm), dim3(512), args, 160 * 1024, st));
        CK(cudaEventRecord(e1, st));
        CK(cudaStreamSynchronize(st));
        float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
        int err = 0; CK(cudaMemcpyFromSymbol(&err, g_err, sizeof(err)));
        printf("cooperative kernel with %d grid barriers: %.3f us per barrier (expired %d)\n", steps, ms * 1000 / steps, err);
    }
    return 0;
}
