// y[M, N] = x[M, K] . W[N, K]^T in true float32 (FMA on the CUDA cores, no tensor
// cores, no reduced-precision mode).  Every output element is the sum over
// k = 0..K-1 in that order with one accumulator, whatever M, N and the tile a
// row falls into: a token's result does not depend on what it is batched with.
// Formula: thanhauco/rust-inference src/ops/linear.rs:7-20.
#include "common.cuh"

#define LF_BM 64
#define LF_BN 64
#define LF_BK 16
#define LF_THREADS 256

__global__ void __launch_bounds__(LF_THREADS)
linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M, int N, int K,
                  int vec_ok) {
    __shared__ float xs[LF_BK][LF_BM + 4];
    __shared__ float ws[LF_BK][LF_BN + 4];
    int m0 = blockIdx.y * LF_BM, n0 = blockIdx.x * LF_BN;
    int tid = threadIdx.x;
    int tx = tid % 16, ty = tid / 16;          // thread owns rows ty*4.., cols tx*4..
    int lrow = tid / 4, lk = (tid % 4) * 4;    // loader: row of the tile, 4 consecutive k
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += LF_BK) {
        float xv[4], wv[4];
        int gm = m0 + lrow, gn = n0 + lrow, gk = k0 + lk;
        if (vec_ok && gk + 3 < K) {
            float4 a = gm < M ? *(const float4*)(x + (size_t)gm * K + gk) : make_float4(0, 0, 0, 0);
            float4 b = gn < N ? *(const float4*)(w + (size_t)gn * K + gk) : make_float4(0, 0, 0, 0);
            xv[0] = a.x; xv[1] = a.y; xv[2] = a.z; xv[3] = a.w;
            wv[0] = b.x; wv[1] = b.y; wv[2] = b.z; wv[3] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                xv[i] = (gm < M && gk + i < K) ? x[(size_t)gm * K + gk + i] : 0.0f;
                wv[i] = (gn < N && gk + i < K) ? w[(size_t)gn * K + gk + i] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            xs[lk + i][lrow] = xv[i];
            ws[lk + i][lrow] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < LF_BK; kk++) {
            float4 a = *(const float4*)&xs[kk][ty * 4];
            float4 b = *(const float4*)&ws[kk][tx * 4];
            float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) y[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

extern "C" int ri_linear_f32(const float* x, const float* w, float* y, int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    RI_REQUIRE(M > 0 && N > 0 && K > 0, "linear_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    dim3 grid((N + LF_BN - 1) / LF_BN, (M + LF_BM - 1) / LF_BM);
    RI_REQUIRE(grid.y <= 65535, "linear_f32: too many rows (%d)", M);
    int vec_ok = (K % 4 == 0) && (((uintptr_t)x | (uintptr_t)w) % 16 == 0);
    linear_f32_kernel<<<grid, LF_THREADS, 0, stream>>>(x, w, y, M, N, K, vec_ok);
    RI_CHECK_LAUNCH("linear_f32");
    return 0;
}
