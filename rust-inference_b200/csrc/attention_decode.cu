// Decode attention over the paged cache for bfloat16: one new token per sequence,
// the keys split into chunks of 128 (four pages), partial results merged afterwards.
//
// Grid (chunk, kv head, sequence), four warps.  Warp w owns page w of the chunk:
// it brings the page's keys and values into shared memory with cp.async (keys
// first, so the scores are computed while the values arrive), multiplies all
// query heads that share this kv head with the keys at once on the tensor cores
// (mma.sync m16n8k16, query heads as the 16 rows), takes the softmax of its 32
// scores in float32 and multiplies with the values.  The four warps' results are
// combined in shared memory in warp order and written as one partial result
// (running maximum, sum, unnormalised output) per (sequence, head, chunk).
// `attention_decode_merge` adds the chunks in rising order.  Each K/V byte is
// read from memory once for all heads of the group.
//
// Which keys a chunk holds depends on the sequence's own length only (chunk c is
// keys 128c .. 128c+127), so a sequence's result does not depend on the batch.
//
// Scratch memory: o_part [seqs, H, max_chunks, Dh] and ml_part [seqs, H,
// max_chunks, 2], float32, given by the caller.
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
#define AD_MERGE_THREADS 128
#define AD_MERGE_TILE 128                    // chunks whose weights are staged at a time

struct __align__(16) DecodeSmem {
    bf16 k[AD_CHUNK][AD_PITCH];
    bf16 v[AD_CHUNK][AD_PITCH];
    bf16 q[AD_ROWS][AD_PITCH];
    float wm[AD_WARPS][AD_ROWS];
    float wl[AD_WARPS][AD_ROWS];
};
// after the products, the k/v area is reused for the warps' outputs: [warps][rows][Dh] float
static_assert(sizeof(float) * AD_WARPS * AD_ROWS * AD_DH <= sizeof(bf16) * 2 * AD_CHUNK * AD_PITCH, "combine area");

__global__ void __launch_bounds__(32 * AD_WARPS)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        float* __restrict__ o_part, float* __restrict__ ml_part, const int* __restrict__ page_table,
                        const int* __restrict__ seq_slot, const int* __restrict__ seq_len, int H, int KV, int mpps,
                        int num_pages, int max_chunks, float scale_log2, int window, int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw);
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int len = seq_len[b];                      // keys 0 .. len-1; the query is at position len-1
    const int first_key = (window > 0 && len - window > 0) ? len - window : 0;
    const int c0 = chunk * AD_CHUNK;
    if (c0 >= len || c0 + AD_CHUNK <= first_key) return;       // nothing of this chunk is visible
    const int G = H / KV;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = seq_slot[b];

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
    const int quad = lane >> 2, qc = lane & 3;
    for (int g0 = 0; g0 < G; g0 += AD_ROWS) {
        __syncthreads();             // a pass before this one has finished with the shared memory
        // ---- this warp's page: keys, then values, 16 bytes per cp.async -------------------------------
        {
        constexpr int VEC_PER_ROW = AD_DH / 8;
        const size_t base = (((size_t)(page < 0 ? 0 : page) * KV + kvh) * AD_PAGE) * AD_DH;
        for (int i = lane; i < AD_PAGE * VEC_PER_ROW; i += 32) {
            int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
            bool ok = page >= 0 && key0 + r < len;
            cp_async16(&sm.k[warp * AD_PAGE + r][c], k_pool + base + (size_t)r * AD_DH + c, ok);
        }
        cp_async_commit();
        for (int i = lane; i < AD_PAGE * VEC_PER_ROW; i += 32) {
            int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
            bool ok = page >= 0 && key0 + r < len;
            cp_async16(&sm.v[warp * AD_PAGE + r][c], v_pool + base + (size_t)r * AD_DH + c, ok);
        }
        cp_async_commit();
        }

        // ---- the group's query heads as rows of a 16 x Dh tile (rows past the group are zero) ----
        for (int i = threadIdx.x; i < AD_ROWS * (AD_DH / 8); i += blockDim.x) {
            int r = i / (AD_DH / 8), c = (i % (AD_DH / 8)) * 8;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (g0 + r < G) val = *(const uint4*)(q + ((size_t)b * H + kvh * G + g0 + r) * AD_DH + c);
            *(uint4*)&sm.q[r][c] = val;
        }
        cp_async_wait<1>();          // this warp's keys have arrived (own copies only ...)
        __syncthreads();             // ... and the block barrier makes the query tile visible

        // ---- scores S[16 rows, 32 keys] = Q K^T ----------------------------------------------------
        float s[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[t][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < AD_DH / 16; ks++) {
            unsigned a0, a1, a2, a3;
            ldmatrix_x4(a0, a1, a2, a3, &sm.q[(lane & 7) + ((lane >> 3) & 1) * 8][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int tp = 0; tp < 2; tp++) {       // 16 keys at a time: two 8-key tiles
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3,
                            &sm.k[warp * AD_PAGE + tp * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
                mma_bf16(s[tp * 2], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[tp * 2 + 1], a0, a1, a2, a3, b2, b3);
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
        // ---- O[16, Dh] = P V ------------------------------------------------------------------------
        cp_async_wait<0>();
        __syncwarp();
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
        // ---- combine the four warps in warp order ---------------------------------------------------
        if (qc == 0) {
            sm.wm[warp][quad] = mx[0];
            sm.wm[warp][quad + 8] = mx[1];
            sm.wl[warp][quad] = sum[0];
            sm.wl[warp][quad + 8] = sum[1];
        }
        __syncthreads();             // all products are done: the k/v area may be overwritten
        float* comb = reinterpret_cast<float*>(smem_raw);       // [warps][rows][Dh]
        float f[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            int row = quad + r * 8;
            float M = -FLT_MAX;
            for (int w = 0; w < AD_WARPS; w++) M = fmaxf(M, sm.wm[w][row]);
            f[r] = mx[r] == -FLT_MAX ? 0.0f : exp2f(mx[r] - M);
        }
#pragma unroll
        for (int t = 0; t < AD_DH / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int row = quad + (e >> 1) * 8, col = t * 8 + qc * 2 + (e & 1);
                comb[((size_t)warp * AD_ROWS + row) * AD_DH + col] = o[t][e] * f[e >> 1];
            }
        __syncthreads();
        for (int i = threadIdx.x; i < AD_ROWS * AD_DH; i += blockDim.x) {
            int row = i / AD_DH, col = i % AD_DH;
            if (g0 + row >= G) continue;
            float acc = 0.0f;
            for (int w = 0; w < AD_WARPS; w++) acc += comb[((size_t)w * AD_ROWS + row) * AD_DH + col];
            int h = kvh * G + g0 + row;
            o_part[(((size_t)b * H + h) * max_chunks + chunk) * AD_DH + col] = acc;
        }
        if (threadIdx.x < AD_ROWS && g0 + threadIdx.x < G) {
            int row = threadIdx.x;
            float M = -FLT_MAX;
            for (int w = 0; w < AD_WARPS; w++) M = fmaxf(M, sm.wm[w][row]);
            float L = 0.0f;
            for (int w = 0; w < AD_WARPS; w++) L += sm.wm[w][row] == -FLT_MAX ? 0.0f : sm.wl[w][row] * exp2f(sm.wm[w][row] - M);
            int h = kvh * G + g0 + row;
            float* ml = ml_part + (((size_t)b * H + h) * max_chunks + chunk) * 2;
            ml[0] = M;
            ml[1] = L;
        }
    }
}

// out[b, h, :] = sum over the visible chunks, in rising order, of the partial results
__global__ void attention_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                              bf16* __restrict__ out, const int* __restrict__ seq_len, int H,
                                              int max_chunks, int window) {
    const int h = blockIdx.x, b = blockIdx.y;
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
    float L = 0.0f;
    float acc[(AD_DH + AD_MERGE_THREADS - 1) / AD_MERGE_THREADS];
#pragma unroll
    for (int j = 0; j < (AD_DH + AD_MERGE_THREADS - 1) / AD_MERGE_THREADS; j++) acc[j] = 0.0f;
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
        for (int j = 0; j < (AD_DH + AD_MERGE_THREADS - 1) / AD_MERGE_THREADS; j++) {
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
    for (int j = 0; j < (AD_DH + AD_MERGE_THREADS - 1) / AD_MERGE_THREADS; j++) {
        int d = threadIdx.x + j * AD_MERGE_THREADS;
        if (d < AD_DH) out[((size_t)b * H + h) * AD_DH + d] = __float2bfloat16_rn(acc[j] / L);
    }
}

extern "C" int ri_attention_decode_head_dim() { return AD_DH; }
extern "C" int ri_attention_decode_chunk() { return AD_CHUNK; }

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
    size_t smem = sizeof(DecodeSmem);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(max_chunks, KV, seqs);
    attention_decode_kernel<<<grid, 32 * AD_WARPS, smem, stream>>>(
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, o_part, ml_part, page_table, seq_slot, seq_len, H, KV,
        mpps, num_pages, max_chunks, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_decode");
    attention_decode_merge_kernel<<<dim3(H, seqs), AD_MERGE_THREADS, 0, stream>>>(
        o_part, ml_part, (bf16*)out, seq_len, H, max_chunks, window);
    RI_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}
