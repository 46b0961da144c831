// Prefill attention over the paged cache for bfloat16: many new tokens per sequence.
//
// Grid (query tile, head, sequence); a tile is 64 consecutive new tokens of one
// sequence, 16 per warp.  The block walks the keys it may see in blocks of 64
// (two pages) from the cache, where this step's keys already are: keys and values
// come in with cp.async, double buffered; S = Q K^T and O += P V run on the tensor
// cores (mma.sync m16n8k16), the softmax is the online one in float32 (running
// maximum and sum per query row).  Causal and window masks are applied only in the
// key blocks that touch an edge.  A query's result depends on its own position and
// on the tile it falls into (position within the step's tokens), not on the batch.
//
// Token t of sequence b: q row seq_start[b] + t, position seq_len[b] - n_b + t,
// where n_b = seq_start[b+1] - seq_start[b].  It sees keys max(0, pos-window+1)..pos.
//
// Compile with -DRI_HEAD_DIM=<multiple of 16, at most 256>.  Page size is 32.
// Formula: thanhauco/rust-inference src/attention.rs:4-8, 111-150.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <float.h>

#ifndef RI_HEAD_DIM
#define RI_HEAD_DIM 128
#endif
static_assert(RI_HEAD_DIM % 16 == 0 && RI_HEAD_DIM >= 16 && RI_HEAD_DIM <= 256, "head_dim: multiple of 16 up to 256");

#define PF_DH RI_HEAD_DIM
#define PF_PAGE 32
#define PF_WARPS 4
#define PF_BM (16 * PF_WARPS)          // queries per block
#define PF_BN 64                       // keys per step (two pages)
#define PF_PITCH (PF_DH + 8)

struct __align__(16) PrefillSmem {
    bf16 q[PF_BM][PF_PITCH];
    bf16 k[2][PF_BN][PF_PITCH];
    bf16 v[2][PF_BN][PF_PITCH];
};

// keys [kb*64, kb*64+63] of one kv head into buffer `buf`: two pages, 16 bytes per copy
__device__ __forceinline__ void load_kv_block(PrefillSmem& sm, int buf, int kb, const bf16* __restrict__ k_pool,
                                              const bf16* __restrict__ v_pool, const int* __restrict__ table, int kvh,
                                              int KV, int num_pages, int len, int key_lo, int* err) {
    constexpr int VEC = PF_DH / 8;
    for (int i = threadIdx.x; i < PF_BN * VEC; i += blockDim.x) {
        int r = i / VEC, c = (i % VEC) * 8;
        int key = kb * PF_BN + r;
        // a page that lies wholly before the first key any query of the tile sees may have been given back by a
        // window group already: it is not looked up, its rows are zeros (and masked)
        bool ok = key < len && (key / PF_PAGE + 1) * PF_PAGE > key_lo;
        size_t off = 0;
        if (ok) {
            int page = table[key / PF_PAGE];
            if (page < 0 || page >= num_pages) {
                atomicExch(err, 4);
                ok = false;
            } else {
                off = (((size_t)page * KV + kvh) * PF_PAGE + key % PF_PAGE) * PF_DH + c;
            }
        }
        cp_async16(&sm.k[buf][r][c], k_pool + off, ok);
        cp_async16(&sm.v[buf][r][c], v_pool + off, ok);
    }
}

__global__ void __launch_bounds__(32 * PF_WARPS)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                         bf16* __restrict__ out, const int* __restrict__ page_table, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_len, int H, int KV, int mpps,
                         int num_pages, float scale_log2, int window, int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw);
    const int b = blockIdx.z, h = blockIdx.y;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin;
    const int tiles = (n_new + PF_BM - 1) / PF_BM;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;       // late tiles see the most keys: start them first
    if (tile >= tiles) return;
    const int len = seq_len[b];
    const int r_base = tile * PF_BM;
    const int rows = min(PF_BM, n_new - r_base);
    const int pos_first = len - n_new + r_base, pos_last = pos_first + rows - 1;
    const int key_lo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int kb_lo = key_lo / PF_BN, kb_hi = pos_last / PF_BN;
    const int kvh = h / (H / KV);
    const int* table = page_table + (size_t)seq_slot[b] * mpps;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;

    // ---- queries of the tile (rows past the sequence's end are zero), first key block -----------
    for (int i = threadIdx.x; i < PF_BM * (PF_DH / 8); i += blockDim.x) {
        int r = i / (PF_DH / 8), c = (i % (PF_DH / 8)) * 8;
        bool ok = r < rows;
        const bf16* src = q + ((size_t)(t_begin + r_base + (ok ? r : 0)) * H + h) * PF_DH + c;
        cp_async16(&sm.q[r][c], src, ok);
    }
    load_kv_block(sm, 0, kb_lo, k_pool, v_pool, table, kvh, KV, num_pages, len, key_lo, err);
    cp_async_commit();

    float o[PF_DH / 8][4];
#pragma unroll
    for (int t = 0; t < PF_DH / 8; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[t][e] = 0.0f;
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.0f, 0.0f};
    const int my_pos[2] = {pos_first + warp * 16 + quad, pos_first + warp * 16 + quad + 8};

    for (int kb = kb_lo; kb <= kb_hi; kb++) {
        const int buf = (kb - kb_lo) & 1;
        if (kb < kb_hi) load_kv_block(sm, buf ^ 1, kb + 1, k_pool, v_pool, table, kvh, KV, num_pages, len, key_lo, err);
        cp_async_commit();
        cp_async_wait<1>();              // everything but the block just asked for has arrived
        __syncthreads();

        // ---- S[16 x 64] = Q K^T ---------------------------------------------------------------------
        float s[PF_BN / 8][4];
#pragma unroll
        for (int t = 0; t < PF_BN / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[t][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < PF_DH / 16; ks++) {
            unsigned a0, a1, a2, a3;
            ldmatrix_x4(a0, a1, a2, a3, &sm.q[warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int tp = 0; tp < PF_BN / 16; tp++) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3,
                            &sm.k[buf][tp * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
                mma_bf16(s[tp * 2], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[tp * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- scale, mask where the block touches an edge, online softmax -----------------------------
        const int k0 = kb * PF_BN;
        const bool edge = (k0 + PF_BN - 1 > pos_first) || (window > 0 && k0 < pos_last - window + 1);
        float mx[2] = {m[0], m[1]};
#pragma unroll
        for (int t = 0; t < PF_BN / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float val = s[t][e] * scale_log2;
                if (edge) {
                    int key = k0 + t * 8 + qc * 2 + (e & 1);
                    int p = my_pos[e >> 1];
                    bool vis = key <= p && (window <= 0 || key > p - window);
                    val = vis ? val : -FLT_MAX;
                }
                s[t][e] = val;
                mx[e >> 1] = fmaxf(mx[e >> 1], val);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            corr[r] = (m[r] == -FLT_MAX) ? 0.0f : exp2f(m[r] - mx[r]);
            m[r] = mx[r];
            l[r] *= corr[r];
        }
#pragma unroll
        for (int t = 0; t < PF_DH / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) o[t][e] *= corr[e >> 1];
#pragma unroll
        for (int t = 0; t < PF_BN / 8; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float p = s[t][e] == -FLT_MAX ? 0.0f : exp2f(s[t][e] - m[e >> 1]);
                s[t][e] = p;
                l[e >> 1] += p;
            }
        // ---- O += P V ---------------------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < PF_BN / 16; kk++) {
            unsigned a0 = pack_bf16(s[kk * 2][0], s[kk * 2][1]), a1 = pack_bf16(s[kk * 2][2], s[kk * 2][3]);
            unsigned a2 = pack_bf16(s[kk * 2 + 1][0], s[kk * 2 + 1][1]), a3 = pack_bf16(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < PF_DH / 16; dp++) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3,
                                  &sm.v[buf][kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][dp * 16 + (lane >> 4) * 8]);
                mma_bf16(o[dp * 2], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[dp * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();                 // the buffer is free for the block after next
    }
    cp_async_wait<0>();

    // ---- out = O / l --------------------------------------------------------------------------------
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        int row = warp * 16 + quad + r * 8;
        if (row >= rows) continue;
        float inv = 1.0f / l[r];
        bf16* dst = out + ((size_t)(t_begin + r_base + row) * H + h) * PF_DH;
#pragma unroll
        for (int t = 0; t < PF_DH / 8; t++) {
            __nv_bfloat162 v = __floats2bfloat162_rn(o[t][r * 2] * inv, o[t][r * 2 + 1] * inv);
            *(__nv_bfloat162*)(dst + t * 8 + qc * 2) = v;
        }
    }
}

extern "C" int ri_attention_prefill_head_dim() { return PF_DH; }

// q, out [tokens, H, Dh] bf16; max_new = the most tokens one sequence brings in this step
extern "C" int ri_attention_prefill(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* page_table, const int* seq_slot, const int* seq_start,
                                    const int* seq_len, int seqs, int max_new, int H, int KV, int Dh, int mpps,
                                    int page_size, int num_pages, float scale, int window, int* err_flag,
                                    cudaStream_t stream) {
    if (seqs == 0 || max_new == 0) return 0;
    RI_REQUIRE(Dh == PF_DH, "attention_prefill: built for head_dim %d, called with %d", PF_DH, Dh);
    RI_REQUIRE(page_size == PF_PAGE, "attention_prefill: pages of %d tokens, this kernel needs %d", page_size, PF_PAGE);
    RI_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_prefill: %d heads over %d kv heads", H, KV);
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "attention_prefill: bad grid");
    RI_REQUIRE(window >= 0, "attention_prefill: negative window");
    size_t smem = sizeof(PrefillSmem);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_prefill: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((max_new + PF_BM - 1) / PF_BM, H, seqs);
    attention_prefill_kernel<<<grid, 32 * PF_WARPS, smem, stream>>>(
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, page_table, seq_slot, seq_start, seq_len,
        H, KV, mpps, num_pages, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_prefill");
    return 0;
}
