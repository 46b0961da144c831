// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 for a handful of tokens (M <= 16): the
// decode-time linear, bound by reading W once from memory.
//
// A block owns 16 rows of W (16 outputs) and all of K; its four warps each take a
// quarter of K.  A warp streams its part of the 16 rows through a ring of two stages
// of 256 k in shared memory: per stage one lane starts four TMA tensor copies
// (cp.async.bulk.tensor.2d, boxes of 16 rows x 64 k with the 128-byte swizzle,
// completion counted on the stage's mbarrier), so 16 KB per warp are in flight without
// holding a register, and three blocks share an SM (a grid that leaves an SM two blocks at
// most takes a ring of three stages: 24 KB per warp).  What a box holds beyond N or K is
// filled with zeros by the copy.  The copies of the first stages are started before
// the kernel waits for its predecessor (programmatic dependent launch): W is never
// written, so they overlap the predecessor's tail.
//
// The products run on the tensor cores (mma.sync m16n8k16, W rows as the 16 MMA rows,
// tokens as the 8 columns).  Within a group of 32 k the order of the k index is
// permuted the same way for W and for x, which a dot product does not notice, so
// that the 16 bytes a lane reads (8 consecutive k of one row) are exactly its MMA
// fragment.  MMA row r is W row rho(r) = (r >> 1) | ((r & 1) << 2) of its half of the
// tile: with the swizzle that makes the eight lanes of a shared-memory transaction
// read eight different 16-byte columns.  The warps' partial sums are added in warp
// order.
//
// A token's result does not depend on M or on the other tokens.  Output is bfloat16
// or float32 (the float32 accumulator, for the logits).  Waits are bounded: if one
// runs out the warp sets the error word (5), starts no further copies, waits (bounded
// again) for the copies it has started, and the kernel finishes with a wrong result for
// that block.  -DSK_TEST_DROP_COPY_K=<k> (tests only; nothing in an ordinary build) makes
// block 0 leave out one copy of its first stage in launches with K == k, so that this path
// can be run: the barrier of that stage then never completes.
#include "common.cuh"
#include "mma_helpers.cuh"
#include "linear_skinny_geometry.cuh"
#include <cuda.h>

#define SK_GROUPS (SK_STAGE_K / 32)          // groups of 32 k in a stage
#define SK_BOXES (SK_STAGE_K / 64)           // copies per stage: 16 rows x 64 k (128 bytes) each
#define SK_BOX_BYTES (SK_ROWS * 128)
#define SK_STAGE_TOTAL (SK_BOXES * SK_BOX_BYTES)

// 16 bytes of x by an ordinary (coherent, L1-cached) load.  Not __ldg: x is written by the kernel before this one while
// this kernel is already on the SMs (programmatic dependent launch), and the non-coherent path is only right for what
// nobody writes during the kernel's life.
__device__ __forceinline__ uint4 ld_ca16(const void* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
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
// one box of the tensor map into shared memory: x in elements (a multiple of 64 here, so of 16 bytes), y the row
__device__ __forceinline__ void sk_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool sk_wait(unsigned long long* bar, unsigned parity) { return ri_mbar_wait(bar, parity); }

// STAGES: the depth of a warp's ring.  SK_STAGES (two stages, three blocks per SM) for grids of more than two
// blocks per SM; a grid that leaves an SM two blocks at most (the matrices of 4,096 rows: 256 blocks) takes
// SK_DEEP_STAGES, so that the blocks that are there have half as many bytes again on their way.
#define SK_DEEP_STAGES 3
template <int STAGES>
struct __align__(1024) SkinnySmem {
    unsigned char w[SK_WARPS][STAGES][SK_STAGE_TOTAL];         // boxes start on multiples of 1024 bytes (the swizzle's period)
    unsigned long long bar[SK_WARPS][STAGES];
    float part[SK_WARPS][SK_ROWS][17];
};
#define SK_SMEM_BYTES(STAGES) (sizeof(SkinnySmem<STAGES>) + 1024)

// NT: token tiles of 8 (1 or 2).  SWIGLU: the 16 rows of a block are 8 gate rows followed by their 8 up rows;
// the block writes silu(gate) * up, 8 outputs per token, into y [M, N/2].
template <int NT, typename OutT, bool SWIGLU, int STAGES>
__global__ void __launch_bounds__(32 * SK_WARPS, STAGES == SK_STAGES ? SK_MIN_BLOCKS : 2)
linear_skinny_kernel(const bf16* __restrict__ x, const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ y, int M, int N,
                     int K, int early_from, int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char sk_raw[];
    SkinnySmem<STAGES>& sm = *reinterpret_cast<SkinnySmem<STAGES>*>(sk_raw + ((1024u - (smem_u32(sk_raw) & 1023u)) & 1023u));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    const int rho = (quad >> 1) | ((quad & 1) << 2);          // the W row (of 8) behind MMA row `quad`
    const int n0 = blockIdx.x * SK_ROWS;
    // The kernel after this one may start when every block of this grid has said so (or has ended).  The blocks of
    // the grid's last wave (`early_from` on: by then no block of this grid waits for a place on an SM) say so at
    // once, the earlier ones when their loops are done: so the successor's blocks come in as the last wave drains,
    // read what they can before their own wait (their first weight stages, their tables) and then sit in it, and a
    // grid of several waves still keeps the SMs to itself while it has blocks waiting.
    const bool trigger_early = (int)blockIdx.x >= early_from;
    if (trigger_early) pdl_trigger();
    // this warp's share of K, in stages of 128 k
    const int stages_total = (K + SK_STAGE_K - 1) / SK_STAGE_K;
    const int st_lo = (int)((long long)stages_total * warp / SK_WARPS), st_hi = (int)((long long)stages_total * (warp + 1) / SK_WARPS);
    const int my_stages = st_hi - st_lo;
    unsigned char (*ws)[SK_STAGE_TOTAL] = sm.w[warp];
    unsigned long long* bar = sm.bar[warp];

    if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_w) : "memory");
#pragma unroll
        for (int s = 0; s < STAGES; s++) sk_mbar_init(&bar[s]);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();

    // start the copies of stage `i` (counted from this warp's first) into ring slot i % STAGES
    auto issue = [&](int i) {
        if (lane == 0) {
            const int slot = i % STAGES;
            const int k0 = (st_lo + i) * SK_STAGE_K;
            sk_expect_tx(&bar[slot], SK_STAGE_TOTAL);
#pragma unroll
            for (int j = 0; j < SK_BOXES; j++) {
#ifdef SK_TEST_DROP_COPY_K
                if (K == SK_TEST_DROP_COPY_K && blockIdx.x == 0 && warp == 0 && i == 0 && j == 0) continue;
#endif
                sk_tma_2d(&ws[slot][j * SK_BOX_BYTES], &map_w, k0 + j * 64, n0, &bar[slot]);
            }
        }
    };
    const int prefill = my_stages < STAGES ? my_stages : STAGES;
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
    int started = prefill;                              // stages whose copies have been started
    for (int i = 0; i < started; i++) {
        const int slot = i % STAGES;
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
        // after a wait has run out the stages already started are still waited for (their copies must not
        // outlive the block), each with its own limit, and no further stage is started
        if (!sk_wait(&bar[slot], (unsigned)((i / STAGES) & 1))) {
            if (lane == 0) atomicExch(err, 5);
            dead = true;
        }
#pragma unroll
        for (int g = 0; g < SK_GROUPS; g++) {
            // box g / 2, row rho (and rho + 8), 16-byte column (g % 2) * 4 + qc, swizzled by the row
            const unsigned char* pw = &ws[slot][(g >> 1) * SK_BOX_BYTES + rho * 128 + (((((g & 1) << 2) | qc) ^ rho) << 4)];
            uint4 a = lds16(pw);
            uint4 b = lds16(pw + 8 * 128);
#pragma unroll
            for (int t = 0; t < NT; t++) {
                mma_bf16(acc[t], a.x, b.x, a.y, b.y, xv[g][t].x, xv[g][t].y);
                mma_bf16(acc[t], a.z, b.z, a.w, b.w, xv[g][t].z, xv[g][t].w);
            }
        }
        __syncwarp();                                   // every lane has read the slot
        if (!dead && i + STAGES < my_stages) {
            issue(i + STAGES);
            started = i + STAGES + 1;
        }
    }
    if (!trigger_early) pdl_trigger_late();
    // acc[t][0,1]: (W row rho, tokens t*8 + 2qc, +1); acc[t][2,3]: (W row rho + 8, same tokens)
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) sm.part[warp][rho + (e >> 1) * 8][t * 8 + qc * 2 + (e & 1)] = acc[t][e];
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

// ---- the tensor map of W, made on the host and kept for the next call with the same matrix --------------
typedef CUresult (*sk_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct SkMapEntry {
    const void* w;
    int N, K;
    CUtensorMap map;
};
#define SK_MAP_CACHE 1024

// W [N, K] bfloat16, row-major, copied in boxes of 16 rows x 64 k; out-of-range parts of a box read as zeros
static int weight_tensor_map(const CUtensorMap** out, const void* w, int N, int K) {
    static sk_encode_tiled_fn encode = nullptr;
    static thread_local SkMapEntry cache[SK_MAP_CACHE];
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !fn)
            RI_FAIL(-1, "linear_skinny: the driver has no cuTensorMapEncodeTiled");
        encode = (sk_encode_tiled_fn)fn;
    }
    SkMapEntry& slot = cache[(((uintptr_t)w >> 8) ^ ((uintptr_t)w >> 20)) % SK_MAP_CACHE];
    if (slot.w != w || slot.N != N || slot.K != K) {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        cuuint32_t box[2] = {64, SK_ROWS};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&slot.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            slot.w = nullptr;
            RI_FAIL(-1, "linear_skinny: cuTensorMapEncodeTiled failed with %d (N=%d, K=%d)", (int)r, N, K);
        }
        slot.w = w;
        slot.N = N;
        slot.K = K;
    }
    *out = &slot.map;
    return 0;
}

template <int NT, typename OutT, bool SWIGLU, int STAGES>
static int launch_skinny_ring(const CUtensorMap* map, dim3 grid, int early_from, const void* x, void* y, int M, int N, int K, int* err,
                              cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<NT, OutT, SWIGLU, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SK_SMEM_BYTES(STAGES));
        if (e != cudaSuccess) RI_FAIL((int)e, "linear_skinny: %s", cudaGetErrorString(e));
        configured = true;
    }
    ri_launch_pdl(linear_skinny_kernel<NT, OutT, SWIGLU, STAGES>, grid, dim3(32 * SK_WARPS), SK_SMEM_BYTES(STAGES), stream, (const bf16*)x,
                  *map, (OutT*)y, M, N, K, early_from, err);
    return 0;
}

template <int NT, typename OutT, bool SWIGLU>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, int* err, cudaStream_t stream) {
    const CUtensorMap* map = nullptr;
    int rc = weight_tensor_map(&map, w, N, K);
    if (rc) return rc;
    dim3 grid((N + SK_ROWS - 1) / SK_ROWS);
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
#ifndef SK_NO_DEEP_RING      // (-DSK_NO_DEEP_RING: two stages everywhere, for comparisons)
    // a grid of at most two blocks per SM: the deeper ring (its blocks are all on the SMs at once: early_from 0)
    if ((long long)grid.x <= 2ll * sms) return launch_skinny_ring<NT, OutT, SWIGLU, SK_DEEP_STAGES>(map, grid, 0, x, y, M, N, K, err, stream);
#endif
    const long long resident = (long long)sms * SK_MIN_BLOCKS;                // blocks on the device at once
    const int early_from = (long long)grid.x > resident ? (int)((long long)grid.x - resident) : 0;
    return launch_skinny_ring<NT, OutT, SWIGLU, SK_STAGES>(map, grid, early_from, x, y, M, N, K, err, stream);
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
