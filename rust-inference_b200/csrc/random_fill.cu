// Fills a device tensor with the random values of random_fill.cuh (one thread per element, grid-stride).
#include "common.cuh"
#include "random_fill.cuh"

#define RF_NORMAL 0
#define RF_UNIFORM 1

template <typename T>
__global__ void __launch_bounds__(256)
random_fill_kernel(T* __restrict__ out, unsigned long long key, unsigned long long first, unsigned long long count,
                   int kind, double a, double b) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = kind == RF_NORMAL ? rf_normal(key, first + i, a) : rf_uniform(key, first + i, a, b);
        st_f(out + i, v);
    }
}

// out[i] = value of element first + i, i < count.  kind 0: N(0, a); kind 1: a + U(-b/2, b/2).
// dtype 0: float32, 1: bfloat16 (rounded to nearest even from the float32 value).
extern "C" int ri_random_fill(void* out, unsigned long long key, unsigned long long first, unsigned long long count,
                              int kind, double a, double b, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    RI_REQUIRE(out != nullptr, "random_fill: null output");
    RI_REQUIRE(kind == RF_NORMAL || kind == RF_UNIFORM, "random_fill: kind %d", kind);
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "random_fill: dtype %d", dtype);
    unsigned long long blocks = (count + 255) / 256;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    if (dtype == RI_DTYPE_F32)
        random_fill_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, key, first, count, kind, a, b);
    else
        random_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, key, first, count, kind, a, b);
    RI_CHECK_LAUNCH("random_fill");
    return 0;
}
