// Decode attention over the paged cache for bfloat16: one new token per sequence,
// the keys split into chunks of 128 (four pages), partial results merged afterwards.
//
// Grid (chunk, kv head, sequence), four warps.  Warp w owns page w of the chunk.
//  * Values: each lane starts one bulk copy (cp.async.bulk, completion on an mbarrier)
//    of one 2*Dh-byte row of the page into padded shared memory; they are read back
//    transposed with ldmatrix for P.V.
//  * Keys and queries never touch shared memory: a lane loads 16 bytes (8 consecutive
//    head elements of one key) straight into registers, which is exactly its fragment
//    of the tensor-core product once the order of the head elements inside a group of
//    32 is permuted the same way for q and k (a dot product does not notice).
//  * S = Q K^T with all query heads that share this kv head as the rows of the MMA
//    (mma.sync m16n8k16; more than 16 heads per kv head take several passes), softmax
//    of the warp's 32 scores in float32, O = P V.
//  * The four warps' results are combined in shared memory in warp order and written
//    as one partial result (maximum, sum, unnormalised output) per (sequence, head,
//    chunk); `attention_decode_merge` adds the chunks in rising order.
// Each K/V byte is read from memory once for all heads of the group.
//
// Which keys a chunk holds depends on the sequence's own length only (chunk c is
// keys 128c .. 128c+127), so a sequence's result does not depend on the batch.
//
// Scratch memory: o_part [seqs, H, max_chunks, Dh] and ml_part [seqs, H,
// max_chunks, 2], float32, given by the caller.
//
// Every wait on an mbarrier is bounded; if it runs out the kernel reports error 5
// through the error word and goes on (its output is then wrong, the context is not).
//
// Compile with -DRI_HEAD_DIM=<multiple of 16, at most 256>.  Page size is 32.
// Formula: thanhauco/rust-inference src/attention.rs:111-150.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <float.h>

#ifndef RI_HEAD_DIM
#define RI_HEAD_DIM 128
#endif
static_assert(RI_HEAD_DIM % 16 == 0 && RI_HEAD_DIM >= 16 && RI_HEAD_DIM <= 256, "head_dim: multiple of 16 up to 256");

#define AD_DH RI_HEAD_DIM
#define AD_PAGE 32
#define AD_WARPS 4
#define AD_CHUNK (AD_PAGE * AD_WARPS)
#define AD_PITCH (AD_DH + 8)                 // bf16 elements per shared row: 16 bytes of padding, no bank conflicts
#define AD_ROWS 16                           // query heads per pass (rows of the MMA)
#define AD_GROUPS ((AD_DH + 31) / 32)        // groups of 32 head elements (the last may be half)
#define AD_CPITCH (AD_DH + 4)                // floats per row of the combine area
#define AD_MERGE_THREADS 128
#define AD_MERGE_TILE 128                    // chunks whose weights are staged at a time

struct __align__(16) DecodeSmem {
    bf16 v[AD_CHUNK][AD_PITCH];
    unsigned long long bar[AD_WARPS];
    float wm[AD_WARPS][AD_ROWS];
    float wl[AD_WARPS][AD_ROWS];
    // followed by the combine area: [warps][rows of a pass][AD_CPITCH] float
};

__host__ __device__ inline size_t decode_smem_bytes(int group_rows) {
    return sizeof(DecodeSmem) + sizeof(float) * AD_WARPS * (size_t)group_rows * AD_CPITCH;
}

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) { return ri_mbar_wait(bar, parity); }

__global__ void __launch_bounds__(32 * AD_WARPS)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        float* __restrict__ o_part, float* __restrict__ ml_part, const int* __restrict__ page_table,
                        const int* __restrict__ seq_slot, const int* __restrict__ seq_len, int H, int KV, int mpps,
                        int num_pages, int max_chunks, float scale_log2, int window, int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw);
    float* comb = reinterpret_cast<float*>(smem_raw + sizeof(DecodeSmem));
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int len = seq_len[b];                      // keys 0 .. len-1; the query is at position len-1
    const int first_key = (window > 0 && len - window > 0) ? len - window : 0;
    const int c0 = chunk * AD_CHUNK;
    if (c0 >= len || c0 + AD_CHUNK <= first_key) return;       // nothing of this chunk is visible
    const int G = H / KV;
    const int rows_pass = G < AD_ROWS ? G : AD_ROWS;           // rows of the combine area
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    const int slot = seq_slot[b];
    pdl_trigger_early();

    const int key0 = c0 + warp * AD_PAGE;
    const bool page_live = key0 < len && key0 + AD_PAGE > first_key;
    int page = -1;
    if (page_live) {
        page = page_table[(size_t)slot * mpps + key0 / AD_PAGE];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicExch(err, 4);
            page = -1;
        }
    }
    const size_t page_base = (((size_t)(page < 0 ? 0 : page) * KV + kvh) * AD_PAGE) * AD_DH;
    const int valid_rows = page < 0 ? 0 : min(AD_PAGE, len - key0);   // rows of the page that hold keys
    // The kernel before this one wrote the newest key and value (position len-1) and the
    // queries.  A warp whose page holds that position waits for it before it reads the
    // page; the other warps read keys and values of earlier steps and wait only before
    // they read the queries.
    const bool newest_page = key0 + AD_PAGE >= len;
    if (newest_page) pdl_wait();

    // ---- values: one bulk copy per row into padded shared memory; rows without a key are zeroed ----
    if (lane == 0) {
        mbar_init(&sm.bar[warp], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    if (lane == 0 && valid_rows > 0) mbar_expect_tx(&sm.bar[warp], (unsigned)valid_rows * AD_DH * 2);
    __syncwarp();
    if (lane < valid_rows) {
        bulk_copy_g2s(&sm.v[warp * AD_PAGE + lane][0], v_pool + page_base + (size_t)lane * AD_DH, AD_DH * 2, &sm.bar[warp]);
    } else {
        for (int c = 0; c < AD_DH; c += 8) *(uint4*)&sm.v[warp * AD_PAGE + lane][c] = make_uint4(0, 0, 0, 0);
    }

    bool waited = false;
    for (int g0 = 0; g0 < G; g0 += AD_ROWS) {
        // ---- query fragments of this pass: rows quad and quad+8 of the group (zero past its end) ----
        uint4 qa[AD_GROUPS], qb[AD_GROUPS];
        uint4 kf[4][AD_GROUPS];
#pragma unroll
        for (int t = 0; t < 4; t++) {                              // keys straight from global memory
            const int r = t * 8 + quad;                            // row of the page = key key0 + r
            const bool okr = r < valid_rows;
            const bf16* pk = k_pool + page_base + (size_t)(okr ? r : 0) * AD_DH;
#pragma unroll
            for (int g = 0; g < AD_GROUPS; g++) {
                int d = g * 32 + qc * 8;
                kf[t][g] = (okr && d < AD_DH) ? ldg_nc16(pk + d) : make_uint4(0, 0, 0, 0);
            }
        }
        if (g0 == 0 && !newest_page) pdl_wait();                   // the queries come from the kernel before
        {
            const bool okA = g0 + quad < G, okB = g0 + quad + 8 < G;
            const bf16* pa = q + ((size_t)b * H + kvh * G + g0 + (okA ? quad : 0)) * AD_DH;
            const bf16* pb = q + ((size_t)b * H + kvh * G + g0 + (okB ? quad + 8 : 0)) * AD_DH;
#pragma unroll
            for (int g = 0; g < AD_GROUPS; g++) {
                int d = g * 32 + qc * 8;
                bool in = d < AD_DH;
                qa[g] = (in && okA) ? *(const uint4*)(pa + d) : make_uint4(0, 0, 0, 0);
                qb[g] = (in && okB) ? *(const uint4*)(pb + d) : make_uint4(0, 0, 0, 0);
            }
        }
        // ---- S[16 rows, 32 keys] = Q K^T ------------------------------------------------------------
        float s[4][4];
        {
#pragma unroll
            for (int t = 0; t < 4; t++) {
#pragma unroll
                for (int e = 0; e < 4; e++) s[t][e] = 0.0f;
#pragma unroll
                for (int g = 0; g < AD_GROUPS; g++) {
                    mma_bf16(s[t], qa[g].x, qb[g].x, qa[g].y, qb[g].y, kf[t][g].x, kf[t][g].y);
                    mma_bf16(s[t], qa[g].z, qb[g].z, qa[g].w, qb[g].w, kf[t][g].z, kf[t][g].w);
                }
            }
        }
        // ---- mask, softmax over this warp's 32 keys (rows quad and quad+8) ---------------------------
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int key = key0 + t * 8 + qc * 2 + (e & 1);
                bool vis = page >= 0 && key < len && key >= first_key;
                s[t][e] = vis ? s[t][e] * scale_log2 : -FLT_MAX;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[t][e]);
            }
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float p = s[t][e] == -FLT_MAX ? 0.0f : exp2f(s[t][e] - mx[e >> 1]);
                s[t][e] = p;
                sum[e >> 1] += p;
            }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        }
        // ---- O[16, Dh] = P V: wait for the values (once), read them transposed ------------------------
        if (!waited) {
            if (valid_rows > 0 && !mbar_wait(&sm.bar[warp], 0) && lane == 0) atomicExch(err, 5);
            __syncwarp();                     // also orders the zero rows written by other lanes
            waited = true;
        }
        float o[AD_DH / 8][4];
#pragma unroll
        for (int t = 0; t < AD_DH / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) o[t][e] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {           // 16 keys at a time
            unsigned a0 = pack_bf16(s[kk * 2][0], s[kk * 2][1]), a1 = pack_bf16(s[kk * 2][2], s[kk * 2][3]);
            unsigned a2 = pack_bf16(s[kk * 2 + 1][0], s[kk * 2 + 1][1]), a3 = pack_bf16(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < AD_DH / 16; dp++) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3,
                                  &sm.v[warp * AD_PAGE + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][dp * 16 + (lane >> 4) * 8]);
                mma_bf16(o[dp * 2], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[dp * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- combine the four warps in warp order (only the rows that are heads) ---------------------
        if (g0 + AD_ROWS >= G) pdl_trigger_late();
        if (g0 > 0) __syncthreads();          // the pass before has finished reading the combine area
        if (qc == 0) {
            sm.wm[warp][quad] = mx[0];
            sm.wm[warp][quad + 8] = mx[1];
            sm.wl[warp][quad] = sum[0];
            sm.wl[warp][quad + 8] = sum[1];
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = quad + r * 8;
            if (g0 + row < G) {
                float M = -FLT_MAX;
#pragma unroll
                for (int w = 0; w < AD_WARPS; w++) M = fmaxf(M, sm.wm[w][row]);
                const float f = mx[r] == -FLT_MAX ? 0.0f : exp2f(mx[r] - M);
                float* dst = comb + ((size_t)warp * rows_pass + row) * AD_CPITCH + qc * 2;
#pragma unroll
                for (int t = 0; t < AD_DH / 8; t++)
                    *(float2*)(dst + t * 8) = make_float2(o[t][r * 2] * f, o[t][r * 2 + 1] * f);
            }
        }
        __syncthreads();
        const int live_rows = min(rows_pass, G - g0);
        for (int i = threadIdx.x; i < live_rows * AD_DH; i += blockDim.x) {
            int row = i / AD_DH, col = i % AD_DH;
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; w++) acc += comb[((size_t)w * rows_pass + row) * AD_CPITCH + col];
            int h = kvh * G + g0 + row;
            o_part[(((size_t)b * H + h) * max_chunks + chunk) * AD_DH + col] = acc;
        }
        if (threadIdx.x < live_rows) {
            int row = threadIdx.x;
            float M = -FLT_MAX;
#pragma unroll
            for (int w = 0; w < AD_WARPS; w++) M = fmaxf(M, sm.wm[w][row]);
            float L = 0.0f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; w++) L += sm.wm[w][row] == -FLT_MAX ? 0.0f : sm.wl[w][row] * exp2f(sm.wm[w][row] - M);
            int h = kvh * G + g0 + row;
            float* ml = ml_part + (((size_t)b * H + h) * max_chunks + chunk) * 2;
            ml[0] = M;
            ml[1] = L;
        }
    }
}

// out[b, h, :] = sum over the visible chunks, in rising order, of the partial results
__global__ void __launch_bounds__(AD_MERGE_THREADS)
attention_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                              bf16* __restrict__ out, const int* __restrict__ seq_len, int H, int max_chunks,
                              int window) {
    const int h = blockIdx.x, b = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    const int len = seq_len[b];
    const int first_key = (window > 0 && len - window > 0) ? len - window : 0;
    const int c_lo = first_key / AD_CHUNK, c_hi = (len + AD_CHUNK - 1) / AD_CHUNK;     // [c_lo, c_hi)
    const float* ml = ml_part + ((size_t)b * H + h) * max_chunks * 2;
    const float* op = o_part + ((size_t)b * H + h) * max_chunks * AD_DH;
    __shared__ float s_w[AD_MERGE_TILE], s_lw[AD_MERGE_TILE], s_red[32];
    // the maximum over the visible chunks
    float M = -FLT_MAX;
    for (int c = c_lo + (int)threadIdx.x; c < c_hi; c += blockDim.x) M = fmaxf(M, ml[c * 2]);
    M = warp_max(M);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = M;
    __syncthreads();
    M = s_red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) M = fmaxf(M, s_red[w]);
    // weights of a tile of chunks into shared memory, then sums in rising chunk order
    constexpr int PER = (AD_DH + AD_MERGE_THREADS - 1) / AD_MERGE_THREADS;
    float L = 0.0f;
    float acc[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) acc[j] = 0.0f;
    for (int t0 = c_lo; t0 < c_hi; t0 += AD_MERGE_TILE) {
        const int n = min(AD_MERGE_TILE, c_hi - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float m = ml[(t0 + i) * 2];
            float w = m == -FLT_MAX ? 0.0f : exp2f(m - M);
            s_w[i] = w;
            s_lw[i] = ml[(t0 + i) * 2 + 1] * w;
        }
        __syncthreads();
        for (int i = 0; i < n; i++) L += s_lw[i];
#pragma unroll
        for (int j = 0; j < PER; j++) {
            int d = threadIdx.x + j * AD_MERGE_THREADS;
            if (d < AD_DH) {
                float a = acc[j];
#pragma unroll 8
                for (int i = 0; i < n; i++) a += op[(size_t)(t0 + i) * AD_DH + d] * s_w[i];
                acc[j] = a;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        int d = threadIdx.x + j * AD_MERGE_THREADS;
        if (d < AD_DH) out[((size_t)b * H + h) * AD_DH + d] = __float2bfloat16_rn(acc[j] / L);
    }
}

extern "C" int ri_attention_decode_head_dim() { return AD_DH; }
extern "C" int ri_attention_decode_chunk() { return AD_CHUNK; }

// shared memory of a launch with G query heads per kv head; raises the kernel's limit when it grows
static int decode_configure(int G, size_t* smem_out) {
    static size_t configured = 0;
    size_t smem = decode_smem_bytes(G < AD_ROWS ? G : AD_ROWS);
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode: shared memory limit: %s", cudaGetErrorString(e));
        configured = smem;
    }
    *smem_out = smem;
    return 0;
}

// q, out [seqs, H, Dh] bf16; o_part [seqs, H, max_chunks, Dh] f32; ml_part [seqs, H, max_chunks, 2] f32.
// max_chunks * 128 must cover the longest sequence of the step.
extern "C" int ri_attention_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* o_part,
                                   float* ml_part, const int* page_table, const int* seq_slot, const int* seq_len,
                                   int seqs, int H, int KV, int Dh, int mpps, int page_size, int num_pages,
                                   int max_chunks, float scale, int window, int* err_flag, cudaStream_t stream) {
    if (seqs == 0) return 0;
    RI_REQUIRE(Dh == AD_DH, "attention_decode: built for head_dim %d, called with %d", AD_DH, Dh);
    RI_REQUIRE(page_size == AD_PAGE, "attention_decode: pages of %d tokens, this kernel needs %d", page_size, AD_PAGE);
    RI_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_decode: %d heads over %d kv heads", H, KV);
    RI_REQUIRE(max_chunks > 0 && seqs <= 65535 && KV <= 65535, "attention_decode: bad grid");
    RI_REQUIRE(window >= 0, "attention_decode: negative window");
    RI_REQUIRE((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0, "attention_decode: q and the pools must be 16-byte aligned");
    size_t smem = 0;
    int rc = decode_configure(H / KV, &smem);
    if (rc) return rc;
    dim3 grid(max_chunks, KV, seqs);
    ri_launch_pdl(attention_decode_kernel, grid, dim3(32 * AD_WARPS), smem, stream,
                  (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, o_part, ml_part, page_table, seq_slot, seq_len,
                  H, KV, mpps, num_pages, max_chunks, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_decode");
    ri_launch_pdl(attention_decode_merge_kernel, dim3(H, seqs), dim3(AD_MERGE_THREADS), 0, stream,
                  (const float*)o_part, (const float*)ml_part, (bf16*)out, seq_len, H, max_chunks, window);
    RI_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}
