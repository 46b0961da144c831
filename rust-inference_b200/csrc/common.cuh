// Shared helpers of the sm_100a kernels: element types, reductions, error reporting.
//
// Every kernel file exports plain C functions that take device pointers, sizes
// and a CUDA stream, launch on that stream and return 0 or a non-zero code;
// `ri_last_error()` of the same library gives the message.  Nothing here
// allocates or synchronises.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define RI_DTYPE_F32 0
#define RI_DTYPE_BF16 1

#ifndef RI_ERRBUF_DEFINED
#define RI_ERRBUF_DEFINED
static thread_local char ri_errbuf[512];
extern "C" const char* ri_last_error() { return ri_errbuf; }
#endif

#define RI_FAIL(code, ...)                                  \
    do {                                                    \
        snprintf(ri_errbuf, sizeof(ri_errbuf), __VA_ARGS__); \
        return (code);                                      \
    } while (0)

#define RI_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) RI_FAIL(-1, __VA_ARGS__); \
    } while (0)

// after a launch: report a launch error without synchronising
#define RI_CHECK_LAUNCH(name)                                                              \
    do {                                                                                   \
        cudaError_t e_ = cudaGetLastError();                                               \
        if (e_ != cudaSuccess) RI_FAIL((int)e_, "%s: %s", name, cudaGetErrorString(e_));   \
    } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched with ri_launch_pdl may start while the kernel before it in the stream is
// still running.  It must call pdl_wait() before it reads anything that kernel (or any
// earlier one) wrote and before its first write to global memory; what it does before that
// (index arithmetic, loads of what no kernel of the step writes) overlaps the predecessor's
// tail.  pdl_trigger() lets the blocks of the kernel after this one start in the same way.
// Both are no-ops for a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
// Where a kernel lets its successor start: early (at its top) the successor's blocks take
// places on the SMs while this kernel still has blocks waiting for one; late (after its main
// loop) they only overlap its tail.
#ifndef RI_PDL_EARLY_TRIGGER
#define RI_PDL_EARLY_TRIGGER 0
#endif
__device__ __forceinline__ void pdl_trigger_early() { if (RI_PDL_EARLY_TRIGGER) pdl_trigger(); }
__device__ __forceinline__ void pdl_trigger_late() { if (!RI_PDL_EARLY_TRIGGER) pdl_trigger(); }

#include <stdlib.h>
static inline int ri_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RUST_INFERENCE_B200_NO_PDL");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t ri_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ri_pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- bounded wait on an mbarrier ---------------------------------------------------------------
// True when the phase with this parity has completed.  Gives up after about four milliseconds
// (a copy or a tensor-core batch takes microseconds), so that a mistake in the bookkeeping of a
// kernel ends in an error code and a wrong result, never in a kernel that does not return.
__device__ __forceinline__ unsigned long long ri_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool ri_mbar_wait(unsigned long long* bar, unsigned parity) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    unsigned long long start = 0;
    for (int i = 0;; i++) {
        unsigned ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 63) == 63) {
            unsigned long long now = ri_globaltimer();
            if (start == 0) start = now;
            else if (now - start > 4000000ull) return false;
        }
    }
}

__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024).  `red` holds 33 floats.
// The order of the additions depends only on the block size, not on the data.
__device__ __forceinline__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                 // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int nw = blockDim.x >> 5;
    if (warp == 0) {
        float t = (lane < nw) ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
