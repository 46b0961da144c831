// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 for a handful of tokens (M <= 16): the
// decode-time linear, bound by reading W once from memory.
//
// A block owns 16 rows of W (16 outputs) and all of K; its four warps each take a
// quarter of K.  A warp streams its part of the 16 rows through a ring of two stages
// in shared memory: per stage each of 16 lanes starts one bulk copy (cp.async.bulk,
// 512 bytes of one row, completion counted on the stage's mbarrier), so 16 KB per
// warp are in flight without holding a register, and three blocks share an SM.  The copies of the first stages are
// started before the kernel waits for its predecessor (programmatic dependent
// launch): W is never written, so they overlap the predecessor's tail.
//
// The products run on the tensor cores (mma.sync m16n8k16, W rows as the 16 MMA rows,
// tokens as the 8 columns).  Within a group of 32 k the order of the k index is
// permuted the same way for W and for x, which a dot product does not notice, so
// that the 16 bytes a lane reads (8 consecutive k of one row) are exactly its MMA
// fragment; rows sit 576 bytes apart in shared memory, which makes those reads free
// of bank conflicts.  The warps' partial sums are added in warp order.
//
// A token's result does not depend on M or on the other tokens.  Output is bfloat16
// or float32 (the float32 accumulator, for the logits).  Waits are bounded: if one
// runs out the kernel sets the error word (5) and finishes.
#include "common.cuh"
#include "mma_helpers.cuh"

#ifndef SK_WARPS
#define SK_WARPS 4
#endif
#define SK_ROWS 16
#ifndef SK_STAGE_K
#define SK_STAGE_K 256                       // k per stage
#endif
#define SK_GROUPS (SK_STAGE_K / 32)          // groups of 32 k in a stage
#define SK_STAGE_BYTES (SK_STAGE_K * 2)      // bytes of a row in a stage
#define SK_PITCH (SK_STAGE_BYTES + 64)       // rows 64 bytes apart modulo 128: no bank conflicts
#ifndef SK_STAGES
#define SK_STAGES 2
#endif
#ifndef SK_MIN_BLOCKS
#define SK_MIN_BLOCKS 3
#endif

__device__ __forceinline__ uint4 ld_ca16(const void* p) { return __ldg((const uint4*)p); }
__device__ __forceinline__ uint4 lds16(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void sk_mbar_init(unsigned long long* bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void sk_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool sk_wait(unsigned long long* bar, unsigned parity) { return ri_mbar_wait(bar, parity); }

struct __align__(16) SkinnyWarpSmem {
    unsigned char w[SK_STAGES][SK_ROWS][SK_PITCH];
};
struct __align__(16) SkinnySmem {
    SkinnyWarpSmem warp[SK_WARPS];
    unsigned long long bar[SK_WARPS][SK_STAGES];
    float part[SK_WARPS][SK_ROWS][17];
};

// NT: token tiles of 8 (1 or 2).  SWIGLU: the 16 rows of a block are 8 gate rows followed by their 8 up rows;
// the block writes silu(gate) * up, 8 outputs per token, into y [M, N/2].
template <int NT, typename OutT, bool SWIGLU>
__global__ void __launch_bounds__(32 * SK_WARPS, SK_MIN_BLOCKS)
linear_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ y, int M, int N, int K,
                     int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char sk_raw[];
    SkinnySmem& sm = *reinterpret_cast<SkinnySmem*>(sk_raw);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    const int n0 = blockIdx.x * SK_ROWS;
    const int rows_here = min(SK_ROWS, N - n0);
    // this warp's share of K, in stages of 128 k
    const int stages_total = (K + SK_STAGE_K - 1) / SK_STAGE_K;
    const int st_lo = (int)((long long)stages_total * warp / SK_WARPS), st_hi = (int)((long long)stages_total * (warp + 1) / SK_WARPS);
    const int my_stages = st_hi - st_lo;
    SkinnyWarpSmem& ws = sm.warp[warp];
    unsigned long long* bar = sm.bar[warp];

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < SK_STAGES; s++) sk_mbar_init(&bar[s]);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();

    // start the copy of stage `i` (counted from this warp's first) into ring slot i % SK_STAGES
    auto issue = [&](int i) {
        const int slot = i % SK_STAGES;
        const int k0 = (st_lo + i) * SK_STAGE_K;
        const int kbytes = min(SK_STAGE_K, K - k0) * 2;                 // K is a multiple of 8: a multiple of 16 bytes
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // earlier reads and writes of the slot come first
        if (lane == 0) sk_expect_tx(&bar[slot], (unsigned)(rows_here * kbytes));
        __syncwarp();
        if (lane < rows_here) {
            sk_bulk_g2s(&ws.w[slot][lane][0], w + (size_t)(n0 + lane) * K + k0, (unsigned)kbytes, &bar[slot]);
            // the tail of a partial stage is read as zeros
            for (int bofs = kbytes; bofs < SK_STAGE_BYTES; bofs += 16) *(uint4*)&ws.w[slot][lane][bofs] = make_uint4(0, 0, 0, 0);
        } else if (lane < SK_ROWS) {
            for (int bofs = 0; bofs < SK_STAGE_BYTES; bofs += 16) *(uint4*)&ws.w[slot][lane][bofs] = make_uint4(0, 0, 0, 0);
        }
    };
    const int prefill = my_stages < SK_STAGES ? my_stages : SK_STAGES;
    for (int i = 0; i < prefill; i++) issue(i);       // W is read-only for every kernel: no need to wait first
    pdl_wait();                                        // x comes from the kernel before

    const bf16* xr[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        int tok = t * 8 + quad;
        xr[t] = x + (size_t)(tok < M ? tok : 0) * K + qc * 8;          // tokens past M: token 0, never written
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[t][e] = 0.0f;

    bool dead = false;
    for (int i = 0; i < my_stages; i++) {
        const int slot = i % SK_STAGES;
        const int k0 = (st_lo + i) * SK_STAGE_K;
        // x for this stage (L1/L2), asked for before the wait
        uint4 xv[SK_GROUPS][NT];
#pragma unroll
        for (int g = 0; g < SK_GROUPS; g++)
#pragma unroll
            for (int t = 0; t < NT; t++) {
                int k = k0 + g * 32 + qc * 8;
                xv[g][t] = k < K ? ld_ca16(xr[t] + k0 + g * 32) : make_uint4(0, 0, 0, 0);
            }
        if (!dead && !sk_wait(&bar[slot], (unsigned)((i / SK_STAGES) & 1))) {
            if (lane == 0) atomicExch(err, 5);
            dead = true;
        }
        __syncwarp();                                   // zero tails written by other lanes
#pragma unroll
        for (int g = 0; g < SK_GROUPS; g++) {
            uint4 a = lds16(&ws.w[slot][quad][g * 64 + qc * 16]);
            uint4 b = lds16(&ws.w[slot][quad + 8][g * 64 + qc * 16]);
#pragma unroll
            for (int t = 0; t < NT; t++) {
                mma_bf16(acc[t], a.x, b.x, a.y, b.y, xv[g][t].x, xv[g][t].y);
                mma_bf16(acc[t], a.z, b.z, a.w, b.w, xv[g][t].z, xv[g][t].w);
            }
        }
        __syncwarp();                                   // every lane has read the slot
        if (i + SK_STAGES < my_stages) issue(i + SK_STAGES);
    }
    pdl_trigger_late();
    // acc[t][0,1]: (row quad, tokens t*8 + 2qc, +1); acc[t][2,3]: (row quad+8, same tokens)
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) sm.part[warp][quad + (e >> 1) * 8][t * 8 + qc * 2 + (e & 1)] = acc[t][e];
    __syncthreads();
    if constexpr (SWIGLU) {
        for (int i = threadIdx.x; i < 8 * NT * 8; i += blockDim.x) {
            int tok = i / 8, r = i % 8;
            if (tok >= M || n0 + 8 + r >= N) continue;
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int wi = 0; wi < SK_WARPS; wi++) {
                g += sm.part[wi][r][tok];
                u += sm.part[wi][r + 8][tok];
            }
            st_f(y + (size_t)tok * (N / 2) + n0 / 2 + r, (g / (1.0f + expf(-g))) * u);
        }
    } else {
        for (int i = threadIdx.x; i < SK_ROWS * NT * 8; i += blockDim.x) {
            int tok = i / SK_ROWS, row = i % SK_ROWS;          // consecutive threads: consecutive outputs of one token
            if (tok >= M || n0 + row >= N) continue;
            float v = 0.0f;
#pragma unroll
            for (int wi = 0; wi < SK_WARPS; wi++) v += sm.part[wi][row][tok];
            st_f(y + (size_t)tok * N + n0 + row, v);
        }
    }
}

template <int NT, typename OutT, bool SWIGLU>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, int* err, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<NT, OutT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SkinnySmem));
        if (e != cudaSuccess) RI_FAIL((int)e, "linear_skinny: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((N + SK_ROWS - 1) / SK_ROWS);
    ri_launch_pdl(linear_skinny_kernel<NT, OutT, SWIGLU>, grid, dim3(32 * SK_WARPS), sizeof(SkinnySmem), stream, (const bf16*)x,
                  (const bf16*)w, (OutT*)y, M, N, K, err);
    return 0;
}

extern "C" int ri_linear_skinny_max_tokens() { return 16; }

// out_f32: 0 = bfloat16 output, 1 = float32 output.  swiglu: 1 = w holds gate and up rows in alternating
// blocks of 8 and y [M, N/2] gets silu(gate) * up (bfloat16 only).
extern "C" int ri_linear_skinny(const void* x, const void* w, void* y, int M, int N, int K, int out_f32, int swiglu,
                                int* err_flag, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    RI_REQUIRE(M > 0 && N > 0 && K > 0, "linear_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    RI_REQUIRE(M <= 16, "linear_skinny: at most 16 tokens, got %d", M);
    RI_REQUIRE(K % 8 == 0, "linear_skinny: K=%d must be a multiple of 8", K);
    RI_REQUIRE((((uintptr_t)x | (uintptr_t)w) & 15) == 0, "linear_skinny: x and w must be 16-byte aligned");
    int rc;
    if (swiglu) {
        RI_REQUIRE(!out_f32 && N % 16 == 0, "linear_skinny: the fused SiLU-gate epilogue needs bfloat16 output and N a multiple of 16 (N=%d)", N);
        rc = M <= 8 ? launch_skinny<1, bf16, true>(x, w, y, M, N, K, err_flag, stream) : launch_skinny<2, bf16, true>(x, w, y, M, N, K, err_flag, stream);
    } else if (M <= 8) {
        rc = out_f32 ? launch_skinny<1, float, false>(x, w, y, M, N, K, err_flag, stream) : launch_skinny<1, bf16, false>(x, w, y, M, N, K, err_flag, stream);
    } else {
        rc = out_f32 ? launch_skinny<2, float, false>(x, w, y, M, N, K, err_flag, stream) : launch_skinny<2, bf16, false>(x, w, y, M, N, K, err_flag, stream);
    }
    if (rc) return rc;
    RI_CHECK_LAUNCH("linear_skinny");
    return 0;
}
