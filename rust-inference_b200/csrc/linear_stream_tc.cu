// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 for 13 to 128 tokens: the decode-time linear of larger
// batches, still bound by reading W once from memory, on the 5th-generation tensor cores (tcgen05).
//
// A block owns 128 rows of W (128 outputs) and a share of K: the blocks that share a tile of outputs form a
// thread-block cluster (up to 8, chosen by the launcher so that about three blocks per SM are at work).  One lane
// starts the TMA tensor copies (cp.async.bulk.tensor.2d, 128-byte swizzle) of a stage: 128 rows x 64 k of W
// and the tokens' 64 k of x; another lane issues tcgen05.mma with the W tile as the A operand (M = 128), the
// tokens as B (N = tokens rounded up to 16) and the accumulator [128 outputs x tokens] in tensor memory; a
// tcgen05.commit hands the stage back to the copying lane.  The copies of W start before the kernel waits for
// its predecessor (programmatic dependent launch): W is never written.  When its share of K is done, every
// thread reads one output row of the accumulator (tcgen05.ld).  A block that is alone writes it straight to y;
// the blocks of a cluster put their partial tiles into their own shared memory, meet at the cluster's barrier,
// and each adds a share of the tokens over all partial tiles, read through distributed shared memory in the
// order of the shares of K: no scratch memory, no atomics, and a result that does not depend on the timing.
//
// With `gated` the rows of W are gate and up rows of a SwiGLU feed-forward alternating in blocks of 8 (so a tile of
// 128 rows holds 64 channels with both their rows), and the kernel writes silu(gate) * up into y [M, N / 2].
//
// Rows past N and columns past K or M read as zeros (the copies fill them).  Output is bfloat16 or float32.
// Waits on mbarriers are bounded: if one runs out the kernel sets the error word (5) and finishes (the
// cluster's barrier is a hardware barrier that every block reaches on every path).  -DLT_TEST_DROP_COPY_K=<k>
// (tests only; nothing in an ordinary build) makes the first block of launches with K == k leave out the copy
// of W of its first stage, so that this path can be run: that stage's barrier then never completes, the issuing
// lane gives up, the copying lane gives up waiting for the stage to come back, the accumulator is read as it is,
// the cluster's barriers are met and the tensor memory is given back.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <cuda.h>

#define LT_ROWS 128                        // rows of W per block (the MMA's M)
#define LT_STAGE_K 64                      // k per stage: 128 bytes, one swizzle row
#define LT_A_BYTES (LT_ROWS * 128)         // 16 KB
#define LT_MAX_TOKENS 128
#define LT_THREADS 128
#define LT_MAX_STAGES 6
#define LT_MAX_SPLITS 8                     // the portable limit of a cluster
#ifndef LT_BLOCKS_PER_SM
#define LT_BLOCKS_PER_SM 3
#endif
#ifndef LT_MIN_SHARE
#define LT_MIN_SHARE 512                   // k per share of K, at least
#endif
#ifndef LT_SMEM_KB
#define LT_SMEM_KB 72                      // shared memory for the stages of a block: three blocks per SM
#endif

__device__ __forceinline__ unsigned long long lt_desc(unsigned addr) {
    // shared-memory matrix descriptor: K-major, 128-byte swizzle (layout type 2), descriptor version 1,
    // 8 rows of 128 bytes (1024 bytes) between row groups
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)(16 >> 4) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// instruction descriptor of kind::f16: bf16 x bf16 -> f32, A and B K-major
__device__ __forceinline__ unsigned lt_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}
__device__ __forceinline__ void lt_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}
__device__ __forceinline__ void lt_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void lt_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lt_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void lt_tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float lt_silu(float t) { return t / (1.0f + expf(-t)); }

struct LtTail {
    unsigned long long full[LT_MAX_STAGES], empty[LT_MAX_STAGES], done;
    unsigned tmem_base;
    int dead;
};

template <typename OutT>
__global__ void __launch_bounds__(LT_THREADS)
linear_stream_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        OutT* __restrict__ y, int M, int Mp, int N, int K, int splits, int stages, int tmem_cols,
                        int gated, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char lt_smem[];
    if (smem_u32(lt_smem) & 1023u) {                               // the swizzle's period
        if (threadIdx.x == 0) atomicExch(err, 6);
        return;
    }
    const int b_bytes = Mp * 128, stage_bytes = LT_A_BYTES + b_bytes;
    LtTail& tail = *reinterpret_cast<LtTail*>(lt_smem + (size_t)stages * stage_bytes);
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * LT_ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // this block's share of K, in stages of 64 k
    const int stages_total = (K + LT_STAGE_K - 1) / LT_STAGE_K;
    const int st_lo = (int)((long long)stages_total * split / splits), st_hi = (int)((long long)stages_total * (split + 1) / splits);
    const int my_stages = st_hi - st_lo;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tail.tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 32) {
        for (int s = 0; s < stages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.empty[s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.done)));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tail.dead = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem = tail.tmem_base;
    // the launcher sizes the grid so that all its blocks are on the SMs at once: the kernel after this one (small
    // blocks that read their tables and wait) may come in right away
    pdl_trigger();

    int issued = 0;                                // stages whose copies the copying lane has started
    if (warp == 0 && lane == 0) {
        // ---- the copying lane ---------------------------------------------------------------------------------
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_x) : "memory");
        // W of the first stages before the wait for the kernel that makes x, x of those stages after it
        const int first = my_stages < stages ? my_stages : stages;
        for (int i = 0; i < first; i++) {
            lt_expect_tx(&tail.full[i], (unsigned)stage_bytes);
#ifdef LT_TEST_DROP_COPY_K
            if (K == LT_TEST_DROP_COPY_K && tile == 0 && split == 0 && i == 0) continue;      // tests only: see the top
#endif
            lt_tma_2d(lt_smem + (size_t)i * stage_bytes, &map_w, (st_lo + i) * LT_STAGE_K, n0, &tail.full[i]);
        }
        pdl_wait();
        for (int i = 0; i < first; i++)
            lt_tma_2d(lt_smem + (size_t)i * stage_bytes + LT_A_BYTES, &map_x, (st_lo + i) * LT_STAGE_K, 0, &tail.full[i]);
        issued = first;
        bool dead = false;
        for (int i = stages; i < my_stages && !dead; i++) {
            const int s = i % stages;
            if (!ri_mbar_wait(&tail.empty[s], (unsigned)((i / stages - 1) & 1))) { atomicExch(err, 5); tail.dead = 1; dead = true; }
            // After a wait has run out (here or in the issuing lane) no further stage is started: a stage's barrier
            // whose copies never all came is still in its old phase, and a second arrival in that phase is one more
            // than the barrier was set up for.
            if (dead || *(volatile int*)&tail.dead) break;
            lt_expect_tx(&tail.full[s], (unsigned)stage_bytes);
            lt_tma_2d(lt_smem + (size_t)s * stage_bytes, &map_w, (st_lo + i) * LT_STAGE_K, n0, &tail.full[s]);
            lt_tma_2d(lt_smem + (size_t)s * stage_bytes + LT_A_BYTES, &map_x, (st_lo + i) * LT_STAGE_K, 0, &tail.full[s]);
            issued = i + 1;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- the issuing lane -----------------------------------------------------------------------------------
        const unsigned idesc = lt_idesc(LT_ROWS, Mp);
        const unsigned long long a0 = lt_desc(smem_u32(lt_smem)), b0 = lt_desc(smem_u32(lt_smem + LT_A_BYTES));
        bool dead = false;
        for (int i = 0; i < my_stages && !dead; i++) {
            const int s = i % stages;
            if (!ri_mbar_wait(&tail.full[s], (unsigned)((i / stages) & 1))) { atomicExch(err, 5); tail.dead = 1; dead = true; }
            if (dead) break;                        // the stage is not there: no product on it, and it is not handed back
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned long long off = (unsigned long long)((s * stage_bytes) >> 4);
#pragma unroll
            for (int j = 0; j < LT_STAGE_K / 16; j++)
                lt_mma(tmem, a0 + off + (unsigned)((j * 32) >> 4), b0 + off + (unsigned)((j * 32) >> 4), idesc, (i > 0 || j > 0) ? 1u : 0u);
            lt_commit(&tail.empty[s]);
        }
        // (after a wait that ran out there may be no product at all behind this: then a plain arrival)
        if (dead) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.done)) : "memory");
        else lt_commit(&tail.done);
    }
    // (the other threads of warps 0 and 1 wait with everybody else)
    pdl_wait();                                    // before the first write to global memory
    if (!ri_mbar_wait(&tail.done, 0)) {
        if (lane == 0) atomicExch(err, 5);
        tail.dead = 1;
    }
    if (tid == 0 && *(volatile int*)&tail.dead) {
        // Somebody gave up: the copies that were started are waited for once more, each with the same limit, before
        // the shared memory they land in is used for the partial tile or given back (everybody meets at a barrier
        // further down).
        for (int i = issued > stages ? issued - stages : 0; i < issued; i++) ri_mbar_wait(&tail.full[i % stages], (unsigned)((i / stages) & 1));
    }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    // ---- the accumulator: thread = output row (tensor-memory lane), columns = tokens ----------------------------
    const int row = tid;                           // warp w reads lanes 32 w .. 32 w + 31
    const unsigned taddr = tmem + ((unsigned)(warp * 32) << 16);
    const bool row_ok = n0 + row < N;
    if (splits == 1) {
        // gated: rows 16 i .. 16 i + 7 of the tile are gate rows and the 8 after them the up rows of the same channels,
        // held by the lane 8 further on in the same warp
        const bool gate_row = ((row >> 3) & 1) == 0;
        const size_t ch = (size_t)((n0 + row) >> 4) * 8 + (row & 7);          // the channel of a gate row
        for (int c = 0; c < Mp; c += 16) {
            float v[16];
            lt_tmem_ld16(taddr + c, v);
            if (gated) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float g = my_stages > 0 ? v[i] : 0.0f;
                    const float u = __shfl_down_sync(0xffffffffu, g, 8);
                    if (gate_row && row_ok && c + i < M) st_f(y + (size_t)(c + i) * (N / 2) + ch, lt_silu(g) * u);
                }
            } else if (row_ok) {
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (c + i < M) st_f(y + (size_t)(c + i) * N + n0 + row, my_stages > 0 ? v[i] : 0.0f);
            }
        }
    } else if (gated) {
        float* part = reinterpret_cast<float*>(lt_smem);
        for (int c = 0; c < Mp; c += 16) {
            float v[16];
            lt_tmem_ld16(taddr + c, v);
#pragma unroll
            for (int i = 0; i < 16; i++) part[(size_t)(c + i) * LT_ROWS + row] = my_stages > 0 ? v[i] : 0.0f;
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        unsigned peer[LT_MAX_SPLITS];
#pragma unroll
        for (int sp = 0; sp < LT_MAX_SPLITS; sp++) {
            peer[sp] = 0;
            if (sp < splits)
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(peer[sp]) : "r"(smem_u32(lt_smem)), "r"(sp));
        }
        // four channels per thread and step: their gate rows and, 8 rows on, their up rows, over the shares of K in order
        const int o4 = (tid % (LT_ROWS / 8)) * 4;                             // channel of the tile, 0 .. 60
        const int rg = (o4 >> 3) * 16 + (o4 & 7);                             // its gate row in the tile
        for (int t = split + (tid / (LT_ROWS / 8)) * splits; t < M; t += (LT_THREADS / (LT_ROWS / 8)) * splits) {
            float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f), u = g;
#pragma unroll
            for (int sp = 0; sp < LT_MAX_SPLITS; sp++) {
                if (sp < splits) {
                    float4 a, b;
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                                 : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w)
                                 : "r"(peer[sp] + (unsigned)((t * LT_ROWS + rg) * 4)) : "memory");
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                                 : "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w)
                                 : "r"(peer[sp] + (unsigned)((t * LT_ROWS + rg + 8) * 4)) : "memory");
                    g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                    u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                }
            }
            OutT* dst = y + (size_t)t * (N / 2) + (n0 >> 1) + o4;
            if (n0 + rg + 8 < N) st_f(dst, lt_silu(g.x) * u.x);
            if (n0 + rg + 9 < N) st_f(dst + 1, lt_silu(g.y) * u.y);
            if (n0 + rg + 10 < N) st_f(dst + 2, lt_silu(g.z) * u.z);
            if (n0 + rg + 11 < N) st_f(dst + 3, lt_silu(g.w) * u.w);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    } else {
        // the partial tile [token][row] of this share of K goes into this block's shared memory (the stages are
        // done with: every copy has landed and every product has read it)
        float* part = reinterpret_cast<float*>(lt_smem);
        for (int c = 0; c < Mp; c += 16) {
            float v[16];
            lt_tmem_ld16(taddr + c, v);
#pragma unroll
            for (int i = 0; i < 16; i++) part[(size_t)(c + i) * LT_ROWS + row] = my_stages > 0 ? v[i] : 0.0f;
        }
        // all blocks of the cluster have written their tiles
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        // this block adds the tokens split, split + splits, ...: four outputs per thread and step, the shares of K
        // in their own order, read from the other blocks' shared memory
        unsigned peer[LT_MAX_SPLITS];
#pragma unroll
        for (int sp = 0; sp < LT_MAX_SPLITS; sp++) {
            peer[sp] = 0;
            if (sp < splits)
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(peer[sp]) : "r"(smem_u32(lt_smem)), "r"(sp));
        }
        const int r4 = (tid % (LT_ROWS / 4)) * 4;
        for (int t = split + (tid / (LT_ROWS / 4)) * splits; t < M; t += (LT_THREADS / (LT_ROWS / 4)) * splits) {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int sp = 0; sp < LT_MAX_SPLITS; sp++) {
                if (sp < splits) {
                    float4 v;
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                                 : "r"(peer[sp] + (unsigned)((t * LT_ROWS + r4) * 4)) : "memory");
                    acc.x += v.x;
                    acc.y += v.y;
                    acc.z += v.z;
                    acc.w += v.w;
                }
            }
            OutT* dst = y + (size_t)t * N + n0 + r4;
            if (n0 + r4 < N) st_f(dst, acc.x);
            if (n0 + r4 + 1 < N) st_f(dst + 1, acc.y);
            if (n0 + r4 + 2 < N) st_f(dst + 2, acc.z);
            if (n0 + r4 + 3 < N) st_f(dst + 3, acc.w);
        }
        // nobody leaves while its shared memory may still be read
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// ---- host ----------------------------------------------------------------------------------------------------------
typedef CUresult (*lt_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// a row-major bfloat16 matrix [rows, K], copied in boxes of box_rows rows x 64 k; what lies outside reads as zeros
static int lt_tensor_map(CUtensorMap* map, const void* p, int rows, int K, int box_rows) {
    static lt_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !fn)
            RI_FAIL(-1, "linear_stream_tc: the driver has no cuTensorMapEncodeTiled");
        encode = (lt_encode_tiled_fn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {LT_STAGE_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RI_FAIL(-1, "linear_stream_tc: cuTensorMapEncodeTiled failed with %d (rows=%d, K=%d)", (int)r, rows, K);
    return 0;
}

extern "C" int ri_linear_stream_tc_max_tokens() { return LT_MAX_TOKENS; }

// how K is split for a matrix of N rows: about two blocks per SM, at most 8 shares (a cluster), every share at
// least 512 k
static int lt_splits(int N, int K, int sms) {
    const int tiles = (N + LT_ROWS - 1) / LT_ROWS;
    int s = (LT_BLOCKS_PER_SM * sms) / tiles;
    const int most = K / LT_MIN_SHARE > 0 ? K / LT_MIN_SHARE : 1;
    if (s > most) s = most;
    if (s > LT_MAX_SPLITS) s = LT_MAX_SPLITS;
    if (s < 1) s = 1;
    return s;
}

// the number of shares of K that a launch for a matrix [N, K] takes on a device of `sms` SMs (for callers that choose
// between this kernel and another by how well its grid fills the device)
extern "C" int ri_linear_stream_tc_splits(int N, int K, int sms) { return lt_splits(N, K, sms > 0 ? sms : 148); }

template <typename OutT>
static cudaError_t lt_launch(dim3 grid, int splits, size_t smem, cudaStream_t stream, const CUtensorMap& map_w,
                             const CUtensorMap& map_x, OutT* y, int M, int Mp, int N, int K, int stages, int tmem_cols, int gated,
                             int* err) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(LT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ri_pdl_enabled();
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = (unsigned)splits;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, linear_stream_tc_kernel<OutT>, map_w, map_x, y, M, Mp, N, K, splits, stages, tmem_cols, gated, err);
}

// gated != 0: W [N, K] holds gate and up rows alternating in blocks of 8 and y [M, N / 2] gets silu(gate) * up
extern "C" int ri_linear_stream_tc(const void* x, const void* w, void* y, int M, int N, int K, int out_f32, int gated,
                                   int* err_flag, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    RI_REQUIRE(M > 0 && N > 0 && K > 0, "linear_stream_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    RI_REQUIRE(M <= LT_MAX_TOKENS, "linear_stream_tc: at most %d tokens, got %d", LT_MAX_TOKENS, M);
    RI_REQUIRE(K % 8 == 0, "linear_stream_tc: K=%d must be a multiple of 8", K);
    RI_REQUIRE(!gated || N % 16 == 0, "linear_stream_tc: %d gate and up rows are not whole blocks of 8 and 8", N);
    RI_REQUIRE((((uintptr_t)x | (uintptr_t)w) & 15) == 0, "linear_stream_tc: x and w must be 16-byte aligned");
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int Mp = (M + 15) / 16 * 16;
    const int tiles = (N + LT_ROWS - 1) / LT_ROWS, splits = lt_splits(N, K, sms);
    const int stage_bytes = LT_A_BYTES + Mp * 128;
    int stages = (LT_SMEM_KB * 1024) / stage_bytes;
    if (stages > LT_MAX_STAGES) stages = LT_MAX_STAGES;
    const size_t smem = (size_t)stages * stage_bytes + sizeof(LtTail);
    int tmem_cols = 32;
    while (tmem_cols < Mp) tmem_cols *= 2;
    CUtensorMap map_w, map_x;
    int rc = lt_tensor_map(&map_w, w, N, K, LT_ROWS);
    if (rc) return rc;
    rc = lt_tensor_map(&map_x, x, M, K, Mp);
    if (rc) return rc;
    static bool configured[2] = {false, false};
    if (!configured[out_f32 ? 1 : 0]) {
        cudaError_t e = out_f32 ? cudaFuncSetAttribute(linear_stream_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (LT_SMEM_KB + 2) * 1024)
                                : cudaFuncSetAttribute(linear_stream_tc_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (LT_SMEM_KB + 2) * 1024);
        if (e != cudaSuccess) RI_FAIL((int)e, "linear_stream_tc: %s", cudaGetErrorString(e));
        configured[out_f32 ? 1 : 0] = true;
    }
    dim3 grid(tiles, splits);
    cudaError_t le = out_f32 ? lt_launch<float>(grid, splits, smem, stream, map_w, map_x, (float*)y, M, Mp, N, K, stages, tmem_cols, gated, err_flag)
                             : lt_launch<bf16>(grid, splits, smem, stream, map_w, map_x, (bf16*)y, M, Mp, N, K, stages, tmem_cols, gated, err_flag);
    if (le != cudaSuccess) RI_FAIL((int)le, "linear_stream_tc: %s", cudaGetErrorString(le));
    RI_CHECK_LAUNCH("linear_stream_tc");
    return 0;
}
