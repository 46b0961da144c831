// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 for a handful of tokens (M <= 16): the
// decode-time linear, bound by reading W once from memory.
//
// A block owns 16 rows of W (16 outputs) and all of K; its eight warps each take an
// eighth of K and stream their part of the 16 rows straight from global memory into
// registers, 16 bytes per lane per load, several loads in flight.  The products run
// on the tensor cores (mma.sync m16n8k16, W rows as the 16 MMA rows, tokens as the 8
// columns).  No shared-memory staging of W is needed: within a group of 32 k the
// order of the k index is permuted the same way for W and for x, which a dot product
// does not notice, so that what a lane loads (8 consecutive k of one row) is exactly
// its MMA fragment.  The eight partial sums are added in warp order in shared memory.
//
// A token's result does not depend on M or on the other tokens.
// Output is bfloat16 or float32 (the float32 accumulator, for the logits).
#include "common.cuh"
#include "mma_helpers.cuh"

#define SK_WARPS 8
#define SK_ROWS 16

__device__ __forceinline__ uint4 ld_nc16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_ca16(const void* p) { return __ldg((const uint4*)p); }

// NT: token tiles of 8 (1 or 2); U: groups of 32 k in flight per warp
template <int NT, int U, typename OutT>
__global__ void __launch_bounds__(32 * SK_WARPS)
linear_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ y, int M, int N, int K) {
    __shared__ float part[SK_WARPS][SK_ROWS][NT * 8 + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    const int n0 = blockIdx.x * SK_ROWS;
    pdl_trigger_early();
    pdl_wait();
    const int steps = (K + 31) / 32;                        // groups of 32 k
    const int s_lo = (int)((long long)steps * warp / SK_WARPS), s_hi = (int)((long long)steps * (warp + 1) / SK_WARPS);
    // rows past N and tokens past M are computed on row 0 / token 0 and never written
    const int rowA = n0 + quad, rowB = n0 + quad + 8;
    const bf16* wA = w + (size_t)(rowA < N ? rowA : 0) * K + qc * 8;
    const bf16* wB = w + (size_t)(rowB < N ? rowB : 0) * K + qc * 8;
    const bf16* xr[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        int tok = t * 8 + quad;
        xr[t] = x + (size_t)(tok < M ? tok : 0) * K + qc * 8;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[t][e] = 0.0f;

    const int full = K / 32;                                 // groups in which every lane has its 8 k
    const int s_full = s_hi < full ? s_hi : full;
    int s = s_lo;
    for (; s + U <= s_full; s += U) {                        // U groups in flight, no conditions
        uint4 a[U], b[U], xv[U][NT];
#pragma unroll
        for (int u = 0; u < U; u++) {
            a[u] = ld_nc16(wA + (s + u) * 32);
            b[u] = ld_nc16(wB + (s + u) * 32);
#pragma unroll
            for (int t = 0; t < NT; t++) xv[u][t] = ld_ca16(xr[t] + (s + u) * 32);
        }
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int t = 0; t < NT; t++) {
                mma_bf16(acc[t], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][t].x, xv[u][t].y);
                mma_bf16(acc[t], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][t].z, xv[u][t].w);
            }
    }
    for (; s < s_hi; s++) {                                  // what is left, one group at a time
        const bool in = s * 32 + qc * 8 < K;                 // K is a multiple of 8: a lane's 8 k are whole or absent
        const uint4 zero = make_uint4(0, 0, 0, 0);
        uint4 a = in ? ld_nc16(wA + s * 32) : zero, b = in ? ld_nc16(wB + s * 32) : zero;
#pragma unroll
        for (int t = 0; t < NT; t++) {
            uint4 xv = in ? ld_ca16(xr[t] + s * 32) : zero;
            mma_bf16(acc[t], a.x, b.x, a.y, b.y, xv.x, xv.y);
            mma_bf16(acc[t], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
    }
    pdl_trigger_late();
    // acc[t][0,1]: (row quad, tokens t*8 + 2qc, +1); acc[t][2,3]: (row quad+8, same tokens)
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) part[warp][quad + (e >> 1) * 8][t * 8 + qc * 2 + (e & 1)] = acc[t][e];
    __syncthreads();
    for (int i = threadIdx.x; i < SK_ROWS * NT * 8; i += blockDim.x) {
        int tok = i / SK_ROWS, row = i % SK_ROWS;              // consecutive threads: consecutive outputs of one token
        if (tok >= M || n0 + row >= N) continue;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < SK_WARPS; wi++) v += part[wi][row][tok];
        st_f(y + (size_t)tok * N + n0 + row, v);
    }
}

template <int NT, int U, typename OutT>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + SK_ROWS - 1) / SK_ROWS);
    ri_launch_pdl(linear_skinny_kernel<NT, U, OutT>, grid, dim3(32 * SK_WARPS), 0, stream, (const bf16*)x, (const bf16*)w, (OutT*)y, M, N, K);
    return 0;
}

extern "C" int ri_linear_skinny_max_tokens() { return 16; }

// out_f32: 0 = bfloat16 output, 1 = float32 output
extern "C" int ri_linear_skinny(const void* x, const void* w, void* y, int M, int N, int K, int out_f32,
                                cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    RI_REQUIRE(M > 0 && N > 0 && K > 0, "linear_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    RI_REQUIRE(M <= 16, "linear_skinny: at most 16 tokens, got %d", M);
    RI_REQUIRE(K % 8 == 0, "linear_skinny: K=%d must be a multiple of 8", K);
    RI_REQUIRE((((uintptr_t)x | (uintptr_t)w) & 15) == 0, "linear_skinny: x and w must be 16-byte aligned");
    if (M <= 8) {
        if (out_f32) launch_skinny<1, 8, float>(x, w, y, M, N, K, stream);
        else launch_skinny<1, 8, bf16>(x, w, y, M, N, K, stream);
    } else {
        if (out_f32) launch_skinny<2, 4, float>(x, w, y, M, N, K, stream);
        else launch_skinny<2, 4, bf16>(x, w, y, M, N, K, stream);
    }
    RI_CHECK_LAUNCH("linear_skinny");
    return 0;
}
