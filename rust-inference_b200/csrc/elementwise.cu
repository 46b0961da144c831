// Embedding gather, RMSNorm (with the residual add fused in) and SiLU-gated product.
//
// The residual stream is float32 in every mode; the parts between two norms
// work in the compute type T (float or bfloat16).  All sums of squares,
// reciprocal roots and gains are float32.
//
// Formulas: thanhauco/rust-inference src/ops/embedding.rs:10-42,
// src/ops/norm.rs:7-62, src/ops/elementwise.rs:10-52 (kernels.cu:89-148 there).
#include "common.cuh"
#include "linear_skinny_geometry.cuh"

// ---------------------------------------------------------------------------
// out[t, :] = float(table[ids[t], :])
// ---------------------------------------------------------------------------
__device__ __forceinline__ void embed_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void embed_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __bfloat1622float2(h[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}

template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                  int dim, int vocab, int* __restrict__ bad) {
    pdl_trigger();
    pdl_wait();
    int id = ids[blockIdx.x];
    if (id < 0 || id >= vocab) {          // checked on the host as well; never read out of range
        if (threadIdx.x == 0) atomicExch(bad, 1);
        return;
    }
    const T* src = table + (size_t)id * dim;
    float* dst = out + (size_t)blockIdx.x * dim;
    if (dim % 8 == 0 && ((((uintptr_t)table | (uintptr_t)out)) & 15) == 0) {
        // 16 bytes per load: a row of 4,096 elements is one or two loads per thread instead of sixteen in a row
        for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
            float v[8];
            embed_load8(src + i, v);
            *reinterpret_cast<float4*>(dst + i) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
        return;
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ld_f(src + i);
}

extern "C" int ri_embed_rows(const int* ids, const void* table, float* out, int tokens, int dim, int vocab,
                             int dtype, int* bad_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && dim > 0 && vocab > 0, "embed_rows: bad sizes tokens=%d dim=%d vocab=%d", tokens, dim, vocab);
    int threads = dim >= 1024 ? 256 : 128;
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(embed_rows_kernel<float>, dim3(tokens), dim3(threads), 0, stream, ids, (const float*)table, out, dim, vocab, bad_flag);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(embed_rows_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out, dim, vocab, bad_flag);
    else
        RI_FAIL(-1, "embed_rows: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("embed_rows");
    return 0;
}

// ---------------------------------------------------------------------------
// RMSNorm of the residual stream.
//   x = resid[r] (+ delta[r]);  if delta and write_back: resid[r] = x
//   out[i] = T(x * (1 / sqrt(mean(x^2) + eps)) * gain)
// r = rows ? rows[i] : i.  With `rows` nothing is written back.
// One block per row, the row staged in shared memory (dim floats).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const int* __restrict__ rows,
                               const float* __restrict__ gain, T* __restrict__ out, int dim, float eps,
                               int write_back) {
    extern __shared__ float row[];
    __shared__ float red[33];
    size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* rp = resid + r * dim;
    const T* dp = delta ? delta + r * dim : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = rp[i];
        if (dp) {
            v += ld_f(dp + i);
            if (write_back) rp[i] = v;
        }
        row[i] = v;
        ss += v * v;
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)dim + eps);
    T* op = out + (size_t)blockIdx.x * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) st_f(op + i, row[i] * inv * gain[i]);
}

// The same for rows whose length is a multiple of 4 and at most 4 * NV * blockDim: the row
// stays in registers (NV float4 per thread), loads and stores are 16 / 8 bytes wide.  The
// order of the additions (a thread's elements in rising order, then the block's tree) is
// fixed by the row length alone.
__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    uint2 u = *(const uint2*)p;
    __nv_bfloat162 a = *(__nv_bfloat162*)&u.x, b = *(__nv_bfloat162*)&u.y;
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(unsigned*)&a;
    u.y = *(unsigned*)&b;
    *(uint2*)p = u;
}

#ifndef RMS_HINT_PER_THREAD
#define RMS_HINT_PER_THREAD 2
#endif

template <typename T, int NV>
__global__ void rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const int* __restrict__ rows,
                                   const float* __restrict__ gain, T* __restrict__ out, int dim, float eps,
                                   int write_back, int n_rows, WeightHint next) {
    __shared__ float red[33];
    pdl_trigger();
    const int nvec = dim >> 2;
    // the gains (and which row this block norms: a table of the step) are not the work of the kernel before this
    // one: they are read before the wait for it, which takes a load from memory out of the chain behind the wait
    float4 g[NV];
    size_t r = blockIdx.x;
    if ((int)blockIdx.x < n_rows) {
#pragma unroll
        for (int j = 0; j < NV; j++) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) g[j] = ld4(gain + 4 * i);
        }
        if (rows) r = (size_t)rows[blockIdx.x];
    }
    pdl_wait();
    if ((int)blockIdx.x >= n_rows) {
        // the blocks beyond the rows ask for the weights that the linear after this norm reads
        weight_hint_prefetch(next, ((int)blockIdx.x - n_rows) * (int)blockDim.x + (int)threadIdx.x,
                             ((int)gridDim.x - n_rows) * (int)blockDim.x);
        return;
    }
    float* rp = resid + r * dim;
    const T* dp = delta ? delta + r * dim : nullptr;
    float4 v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
            float4 a = ld4(rp + 4 * i);
            if (dp) {
                float4 d = ld4(dp + 4 * i);
                a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
                if (write_back) st4(rp + 4 * i, a);
            }
            v[j] = a;
            ss += a.x * a.x;
            ss += a.y * a.y;
            ss += a.z * a.z;
            ss += a.w * a.w;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)dim + eps);
    T* op = out + (size_t)blockIdx.x * dim;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        int i = threadIdx.x + j * blockDim.x;
        if (i < nvec)
            st4(op + 4 * i, make_float4(v[j].x * inv * g[j].x, v[j].y * inv * g[j].y, v[j].z * inv * g[j].z, v[j].w * inv * g[j].w));
    }
}

// Many rows (a prompt step): a block of 256 threads takes a row, each thread doing the work of the four threads
// t, t+256, t+512, t+768 of the 1,024-thread kernel above: the same partial sums, the same warp trees (a warp here
// computes those of warps w, w+8, w+16 and w+24 there) and the same last tree, so every bit is as above.  Several
// such blocks fit on an SM, so that one block's loads are on their way while another reduces or stores, and each
// thread has four times the bytes in flight.
constexpr int RMS_VT = 4;
template <typename T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_many_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                                           const float* __restrict__ gain, T* __restrict__ out, int dim,
                                                           float eps, int write_back) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int nvec = dim >> 2;
    const int r = blockIdx.x;
    float* rp = resid + (size_t)r * dim;
    const T* dp = delta ? delta + (size_t)r * dim : nullptr;
    float4 v[RMS_VT][NV];
    float ss[RMS_VT];
#pragma unroll
    for (int q = 0; q < RMS_VT; q++)
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = threadIdx.x + 256 * q + j * 1024;
            if (i < nvec) {
                v[q][j] = ld4(rp + 4 * i);
                if (dp) {
                    float4 d = ld4(dp + 4 * i);
                    v[q][j].x += d.x; v[q][j].y += d.y; v[q][j].z += d.z; v[q][j].w += d.w;
                }
            }
        }
#pragma unroll
    for (int q = 0; q < RMS_VT; q++) {
        ss[q] = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = threadIdx.x + 256 * q + j * 1024;
            if (i < nvec) {
                const float4 a = v[q][j];
                if (dp && write_back) st4(rp + 4 * i, a);
                ss[q] += a.x * a.x;
                ss[q] += a.y * a.y;
                ss[q] += a.z * a.z;
                ss[q] += a.w * a.w;
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int q = 0; q < RMS_VT; q++) {
        ss[q] = warp_sum(ss[q]);
        if (lane == 0) red[warp + 8 * q] = ss[q];
    }
    __syncthreads();
    if (warp == 0) {
        float t = warp_sum(red[lane]);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(red[32] / (float)dim + eps);
    T* op = out + (size_t)r * dim;
#pragma unroll
    for (int q = 0; q < RMS_VT; q++)
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = threadIdx.x + 256 * q + j * 1024;
            if (i < nvec) {
                const float4 g = ld4(gain + 4 * i);
                st4(op + 4 * i, make_float4(v[q][j].x * inv * g.x, v[q][j].y * inv * g.y, v[q][j].z * inv * g.z,
                                            v[q][j].w * inv * g.w));
            }
        }
}

template <typename T>
static bool launch_rmsnorm_vec(float* resid, const void* delta, const int* rows, const float* gain, void* out,
                               int n_rows, int dim, float eps, int write_back, const WeightHint& next, cudaStream_t stream) {
    if (dim % 4) return false;
    uintptr_t al = (uintptr_t)resid | (uintptr_t)gain | (uintptr_t)out | (uintptr_t)delta;
    if (al & 15) return false;
    int nvec = dim / 4;
    int threads = nvec >= 1024 ? 1024 : ((nvec + 31) / 32) * 32;
    int nv = (nvec + threads - 1) / threads;
    const T* d = (const T*)delta;
    T* o = (T*)out;
    if (nv > 4) return false;
    if (!rows && !next.base && n_rows >= 512 && threads == 1024 && nv <= 2) {
        if (nv == 1) ri_launch_pdl(rmsnorm_many_kernel<T, 1>, dim3(n_rows), dim3(256), 0, stream, resid, d, gain, o, dim, eps, write_back);
        else ri_launch_pdl(rmsnorm_many_kernel<T, 2>, dim3(n_rows), dim3(256), 0, stream, resid, d, gain, o, dim, eps, write_back);
        return true;
    }
    // with a hint: as many more blocks as give each thread a few requests
    int extra = 0;
    if (next.base) {
        const long long lines = (long long)next.rows * SK_WARPS * (SK_HINT_STAGES * SK_STAGE_K * 2 / SK_HINT_LINE);
        const int want = (int)((lines + (long long)threads * RMS_HINT_PER_THREAD - 1) / ((long long)threads * RMS_HINT_PER_THREAD));
        extra = want < 1 ? 1 : (want > 256 ? 256 : want);
    }
    const dim3 grid(n_rows + extra);
    if (nv == 1) ri_launch_pdl(rmsnorm_vec_kernel<T, 1>, grid, dim3(threads), 0, stream, resid, d, rows, gain, o, dim, eps, write_back, n_rows, next);
    else if (nv == 2) ri_launch_pdl(rmsnorm_vec_kernel<T, 2>, grid, dim3(threads), 0, stream, resid, d, rows, gain, o, dim, eps, write_back, n_rows, next);
    else ri_launch_pdl(rmsnorm_vec_kernel<T, 4>, grid, dim3(threads), 0, stream, resid, d, rows, gain, o, dim, eps, write_back, n_rows, next);
    return true;
}

// next_w [next_n, next_k] (bfloat16, or null): the weights of the skinny linear that reads this norm's output;
// the kernel asks for the part of them that the linear wants first after what it holds itself.
extern "C" int ri_rmsnorm(float* resid, const void* delta, const int* rows, const float* gain, void* out, int n_rows,
                          int dim, float eps, int write_back, int dtype, const void* next_w, int next_n, int next_k,
                          cudaStream_t stream) {
    if (n_rows == 0) return 0;
    RI_REQUIRE(n_rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", n_rows, dim);
    if (rows) write_back = 0;
    WeightHint next = make_weight_hint(nullptr, 0, 0, 0);
    if (next_w) {
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        }
        next = make_weight_hint(next_w, next_n, next_k, sms);
    }
    if (dtype == RI_DTYPE_F32 && launch_rmsnorm_vec<float>(resid, delta, rows, gain, out, n_rows, dim, eps, write_back, next, stream)) {
        RI_CHECK_LAUNCH("rmsnorm");
        return 0;
    }
    if (dtype == RI_DTYPE_BF16 && launch_rmsnorm_vec<__nv_bfloat16>(resid, delta, rows, gain, out, n_rows, dim, eps, write_back, next, stream)) {
        RI_CHECK_LAUNCH("rmsnorm");
        return 0;
    }
    size_t smem = (size_t)dim * sizeof(float);
    RI_REQUIRE(smem <= 200 * 1024, "rmsnorm: a row of %d elements does not fit in shared memory (limit 51200)", dim);
    int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    if (rows) write_back = 0;
    cudaError_t e = cudaSuccess;
    if (dtype == RI_DTYPE_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "rmsnorm: %s", cudaGetErrorString(e));
        rmsnorm_kernel<float><<<n_rows, threads, smem, stream>>>(resid, (const float*)delta, rows, gain, (float*)out, dim, eps, write_back);
    } else if (dtype == RI_DTYPE_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "rmsnorm: %s", cudaGetErrorString(e));
        rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(resid, (const __nv_bfloat16*)delta, rows, gain, (__nv_bfloat16*)out, dim, eps, write_back);
    } else {
        RI_FAIL(-1, "rmsnorm: unknown dtype %d", dtype);
    }
    RI_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------
// resid[r] += delta[r] for whole rows (used when no norm follows an addition)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_rows_kernel(float* __restrict__ resid, const T* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += ld_f(delta + i);
}

extern "C" int ri_add_rows(float* resid, const void* delta, long long n, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == RI_DTYPE_F32) add_rows_kernel<float><<<blocks, 256, 0, stream>>>(resid, (const float*)delta, (size_t)n);
    else if (dtype == RI_DTYPE_BF16) add_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(resid, (const __nv_bfloat16*)delta, (size_t)n);
    else RI_FAIL(-1, "add_rows: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("add_rows");
    return 0;
}

// ---------------------------------------------------------------------------
// out[m, c] = silu(gate[m, c]) * up[m, c],  silu(t) = t / (1 + exp(-t))
// `gu` [m, 2*inter] holds gate and up in alternating blocks of `block` channels:
// gate of channel c at column (c / block) * 2 * block + c % block, up `block` columns further.
// block = inter is "all gates, then all ups"; block = 8 is the layout the skinny linear's
// fused epilogue wants (a block of 16 output rows = 8 gates and their 8 ups).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int block, size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t m = i / inter;
    int c = (int)(i - m * inter);
    int gc = (c / block) * 2 * block + c % block;
    float g = ld_f(gu + m * 2 * inter + gc);
    float u = ld_f(gu + m * 2 * inter + gc + block);
    st_f(out + i, (g / (1.0f + expf(-g))) * u);
}

// eight outputs per thread with 16-byte loads and stores, when the sizes and addresses allow it
template <typename T>
struct Pack8;
template <>
struct Pack8<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *(const uint4*)p; }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *(uint4*)p = raw; }
    __device__ __forceinline__ float get(int i) const {
        unsigned w = (&raw.x)[i >> 1];
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    __device__ __forceinline__ void set2(int i, float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        (&raw.x)[i] = *(unsigned*)&v;
    }
};
template <>
struct Pack8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *(const float4*)p; b = *(const float4*)(p + 4); }
    __device__ __forceinline__ void store(float* p) const { *(float4*)p = a; *(float4*)(p + 4) = b; }
    __device__ __forceinline__ float get(int i) const { return (&a.x)[i]; }        // a and b are adjacent members
    __device__ __forceinline__ void set2(int i, float lo, float hi) { (&a.x)[2 * i] = lo; (&a.x)[2 * i + 1] = hi; }
};

// silu(t) = t / (1 + exp(-t)).  float32: as written (expf, a true division).  bfloat16: the hardware's exp2 and
// reciprocal approximations, whose errors (2^-22 relative) vanish in the rounding of the result to 8 bits.
template <typename T>
__device__ __forceinline__ float silu_of(float t) { return t / (1.0f + expf(-t)); }
template <>
__device__ __forceinline__ float silu_of<__nv_bfloat16>(float t) { return __fdividef(t, 1.0f + __expf(-t)); }

template <typename T>
__global__ void silu_mul_vec8_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int block, size_t total8) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = inter >> 3;
    size_t m = i / per_row;
    int c = (int)(i - m * per_row) << 3;
    Pack8<T> g, u, o;
    const int gc = (c / block) * 2 * block + c % block;        // block is a multiple of 8: the 8 channels stay together
    g.load(gu + m * 2 * inter + gc);
    u.load(gu + m * 2 * inter + gc + block);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float g0 = g.get(2 * j), g1 = g.get(2 * j + 1);
        o.set2(j, silu_of<T>(g0) * u.get(2 * j), silu_of<T>(g1) * u.get(2 * j + 1));
    }
    o.store(out + m * inter + c);
}

extern "C" int ri_silu_mul(const void* gu, void* out, int rows, int inter, int block, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    RI_REQUIRE(rows > 0 && inter > 0, "silu_mul: bad sizes rows=%d inter=%d", rows, inter);
    RI_REQUIRE(block > 0 && inter % block == 0, "silu_mul: %d channels are not whole blocks of %d", inter, block);
    size_t total = (size_t)rows * inter;
    if (block % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        size_t total8 = total / 8;
        unsigned blocks8 = (unsigned)((total8 + 255) / 256);
        if (dtype == RI_DTYPE_F32) ri_launch_pdl(silu_mul_vec8_kernel<float>, dim3(blocks8), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, block, total8);
        else if (dtype == RI_DTYPE_BF16) ri_launch_pdl(silu_mul_vec8_kernel<__nv_bfloat16>, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, block, total8);
        else RI_FAIL(-1, "silu_mul: unknown dtype %d", dtype);
        RI_CHECK_LAUNCH("silu_mul");
        return 0;
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == RI_DTYPE_F32) ri_launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, block, total);
    else if (dtype == RI_DTYPE_BF16) ri_launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, block, total);
    else RI_FAIL(-1, "silu_mul: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("silu_mul");
    return 0;
}
