// Causal grouped-query attention over the paged cache, one fixed order of arithmetic per row.
//
// This is the attention of the float32 path, and of bfloat16 models whose head size or page size the
// tensor-core kernels do not take.  A "row" is one (new token, query head).  What a row computes, and
// in which order, depends on the row's own position and on the cache's page size only: the keys it
// sees are walked in strips (32 consecutive keys of one page, at fixed places of the sequence), and
// for every strip
//     score_j = (sum over d ascending of q[d] k_j[d], one accumulator) * scale       lane j = key j of the strip
//     m' = max(m, max_j score_j);  c = exp(m - m');  p_j = exp(score_j - m')
//     l = l c + (sum of the p_j over the warp's shuffle tree);  acc[d] = acc[d] c, then += p_j v_j[d] for j ascending
// with exp the full-precision function, as thanhauco/rust-inference's CPU attention does a page at a
// time (src/attention.rs:111-150).  So the logits of a token are the same bits however the tokens were cut
// into steps and whatever else is in the batch.
//
// Work is shared between rows, not split inside one: a block takes up to `tile_q` consecutive new tokens
// of one sequence and up to `group_chunk` query heads of one kv head, stages each strip of keys and
// values once in shared memory (as float32) for all of them, and every warp then takes the rows
// w, w + 8, ... two at a time (two query heads of one token: what is read of a key or a value from shared memory
// serves both): a row belongs to one warp from start to end, its running maximum, sum and output live in shared
// memory between strips.  Keys and values are thus read from memory once per
// (tile, kv head) where one block per (token, head) would read them tile_q x group size times.
//
//   q, out  [tokens, H, Dh];  k_pool, v_pool [pages, KV, page_size, Dh]
//   sequence b: slot seq_slot[b], new tokens seq_start[b] .. seq_start[b+1]-1 of the packed arrays,
//   length seq_len[b] after the step; new token i sits at position seq_len[b] - n_b + i and sees keys
//   max(0, pos-window+1) .. pos  (window 0: all keys 0..pos).  kv head = h / (H / KV).
// A page index outside the pool (or -1) among the pages a tile needs: error word 4, the strip is left
// out.  Pages wholly before the first key that the tile sees are not looked up (a window group may have
// given them back).
#include "common.cuh"
#include <float.h>
#include <math.h>

#define AR_WARPS 8
#define AR_STRIP 32
#define AR_MAX_DH 512
#define AR_MAX_TILE 16
#define AR_SMEM_BUDGET (200 * 1024)

template <typename T> struct ArVec;                    // four consecutive elements from global memory as floats
template <> struct ArVec<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct ArVec<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
};

__host__ __device__ inline int ar_key_pitch(int Dh, bool vec4) { return vec4 ? Dh + 4 : Dh + 1; }    // floats per staged key

// One strip of keys for R (1 or 2) rows that follow each other in shared memory and see the same keys j_lo .. j_hi of
// the strip: scores (lane j = key j), the online-softmax update of each row's maximum and sum, and the rows' outputs
// (a lane owns head elements lane, lane + 32, ...; the keys are added in rising order).
template <bool VEC4, int R>
__device__ __forceinline__ void ar_strip(const float* __restrict__ qs, float* __restrict__ accs, float* __restrict__ ms,
                                         float* __restrict__ ls, const float* __restrict__ ks, const float* __restrict__ vs,
                                         int row, int Dh, int kpitch, int j_lo, int j_hi, float scale, int lane) {
    const bool mine = lane >= j_lo && lane <= j_hi;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; r++) s[r] = -INFINITY;
    if (mine) {
        const float* qr = qs + (size_t)row * Dh;
        const float* kr = ks + lane * kpitch;
        float dot[R];
#pragma unroll
        for (int r = 0; r < R; r++) dot[r] = 0.0f;
        if (VEC4) {
            for (int c = 0; c < Dh; c += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kr + c);
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const float4 a = *reinterpret_cast<const float4*>(qr + (size_t)r * Dh + c);
                    dot[r] = fmaf(a.x, k4.x, dot[r]);
                    dot[r] = fmaf(a.y, k4.y, dot[r]);
                    dot[r] = fmaf(a.z, k4.z, dot[r]);
                    dot[r] = fmaf(a.w, k4.w, dot[r]);
                }
            }
        } else {
            for (int d = 0; d < Dh; d++) {
                const float kd = kr[d];
#pragma unroll
                for (int r = 0; r < R; r++) dot[r] = fmaf(qr[(size_t)r * Dh + d], kd, dot[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) s[r] = dot[r] * scale;
    }
    float corr[R], p[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const float m_old = ms[row + r];
        const float m_new = fmaxf(m_old, warp_max(s[r]));
        corr[r] = expf(m_old - m_new);                            // 0 at the row's first strip (m_old is -inf)
        p[r] = mine ? expf(s[r] - m_new) : 0.0f;
        const float p_sum = warp_sum(p[r]);
        __syncwarp();
        if (lane == 0) {
            ms[row + r] = m_new;
            ls[row + r] = ls[row + r] * corr[r] + p_sum;
        }
    }
    // the outputs: four head elements per lane and row at a time, the strip's keys in rising order
    float* ar = accs + (size_t)row * Dh;
    for (int d0 = 0; d0 < Dh; d0 += 128) {
        float a[R][4];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int d = d0 + c * 32 + lane;
                a[r][c] = d < Dh ? ar[(size_t)r * Dh + d] * corr[r] : 0.0f;
            }
        for (int j = j_lo; j <= j_hi; j++) {
            float pj[R];
#pragma unroll
            for (int r = 0; r < R; r++) pj[r] = __shfl_sync(0xffffffffu, p[r], j);
            const float* vr = vs + j * Dh + d0 + lane;
#pragma unroll
            for (int c = 0; c < 4; c++)
                if (d0 + c * 32 + lane < Dh) {
                    const float v = vr[c * 32];
#pragma unroll
                    for (int r = 0; r < R; r++) a[r][c] = fmaf(pj[r], v, a[r][c]);
                }
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int d = d0 + c * 32 + lane;
                if (d < Dh) ar[(size_t)r * Dh + d] = a[r][c];
            }
    }
}

// VEC4: the head size is a multiple of 4 (vector loads, and a staged key's row starts on 16 bytes)
template <typename T, bool VEC4>
__global__ void __launch_bounds__(32 * AR_WARPS)
attention_rows_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                      T* __restrict__ out, const int* __restrict__ page_table, const int* __restrict__ seq_slot,
                      const int* __restrict__ seq_start, const int* __restrict__ seq_len, int H, int KV, int Dh,
                      int mpps, int page_size, int num_pages, int tile_q, int group_chunk, float scale, int window,
                      int* __restrict__ err) {
    extern __shared__ __align__(16) float ar_smem[];
    const int b = blockIdx.z;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin;
    const int r_base = blockIdx.x * tile_q;
    if (r_base >= n_new) return;
    const int nq = min(tile_q, n_new - r_base);
    const int G = H / KV, chunks = (G + group_chunk - 1) / group_chunk;
    const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y % chunks) * group_chunk;
    const int ng = min(group_chunk, G - g0);
    const int rows = nq * ng, rows_max = tile_q * group_chunk;
    const int kpitch = ar_key_pitch(Dh, VEC4);
    float* ks = ar_smem;                              // [32][kpitch]
    float* vs = ks + AR_STRIP * kpitch;               // [32][Dh]
    float* qs = vs + AR_STRIP * Dh;                   // [rows][Dh]
    float* accs = qs + (size_t)rows_max * Dh;         // [rows][Dh]
    float* ms = accs + (size_t)rows_max * Dh;         // [rows]
    float* ls = ms + rows_max;                        // [rows]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int len = seq_len[b];
    const int pos0 = len - n_new + r_base, pos_last = pos0 + nq - 1;       // positions of the tile's queries
    const int key_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int* table = page_table + (size_t)seq_slot[b] * mpps;

    // row = i * ng + g: new token r_base + i, query head kvh * G + g0 + g
    for (int idx = tid; idx < rows * Dh; idx += blockDim.x) {
        const int row = idx / Dh, d = idx - row * Dh;
        const int i = row / ng, g = row - i * ng;
        qs[idx] = ld_f(q + ((size_t)(t_begin + r_base + i) * H + kvh * G + g0 + g) * Dh + d);
        accs[idx] = 0.0f;
    }
    for (int row = tid; row < rows; row += blockDim.x) {
        ms[row] = -INFINITY;
        ls[row] = 0.0f;
    }

    // strips: 32 consecutive keys of one page (the last strip of a page may be shorter), at places that
    // depend on the page size only
    int key0 = key_lo - (key_lo % page_size) % AR_STRIP;              // start of the strip that holds key_lo
    while (key0 <= pos_last) {
        const int page_idx = key0 / page_size, in_page = key0 - page_idx * page_size;
        const int width = min(AR_STRIP, page_size - in_page);
        const int page = page_idx < mpps ? table[page_idx] : -1;
        if (page < 0 || page >= num_pages) {
            if (tid == 0) atomicExch(err, 4);
            key0 += width;
            continue;
        }
        __syncthreads();                                              // the strip before has been used (and q, acc are set)
        const size_t base = (((size_t)page * KV + kvh) * page_size + in_page) * Dh;
        if (VEC4) {
            const int per = Dh >> 2;
            for (int idx = tid; idx < width * per; idx += blockDim.x) {
                const int r = idx / per, c = idx - r * per;
                *reinterpret_cast<float4*>(ks + r * kpitch + 4 * c) = ArVec<T>::load(k_pool + base + (size_t)r * Dh + 4 * c);
                *reinterpret_cast<float4*>(vs + r * Dh + 4 * c) = ArVec<T>::load(v_pool + base + (size_t)r * Dh + 4 * c);
            }
        } else {
            for (int idx = tid; idx < width * Dh; idx += blockDim.x) {
                const int r = idx / Dh, d = idx - r * Dh;
                ks[r * kpitch + d] = ld_f(k_pool + base + idx);
                vs[idx] = ld_f(v_pool + base + idx);
            }
        }
        __syncthreads();
        // a warp takes two query heads of one token at a time (they see the same keys): a key or a value read from
        // shared memory then serves both rows; each row's own arithmetic and its order are what they would be alone
        const int pairs = (ng + 1) >> 1;
        for (int unit = warp; unit < nq * pairs; unit += AR_WARPS) {
            const int i = unit / pairs, g_first = 2 * (unit - i * pairs);
            const int pos = pos0 + i;
            const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            const int j_lo = max(first - key0, 0), j_hi = min(pos - key0, width - 1);       // the token's keys in this strip
            if (j_lo > j_hi) continue;                                // none: the rows' state stays as it is
            const int row_a = i * ng + g_first;
            if (g_first + 1 < ng)
                ar_strip<VEC4, 2>(qs, accs, ms, ls, ks, vs, row_a, Dh, kpitch, j_lo, j_hi, scale, lane);
            else
                ar_strip<VEC4, 1>(qs, accs, ms, ls, ks, vs, row_a, Dh, kpitch, j_lo, j_hi, scale, lane);
        }
        key0 += width;
    }
    __syncthreads();
    for (int row = warp; row < rows; row += AR_WARPS) {
        const int i = row / ng, g = row - i * ng;
        const float l = ls[row];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;                 // no key at all: only after error 4
        T* dst = out + ((size_t)(t_begin + r_base + i) * H + kvh * G + g0 + g) * Dh;
        for (int d = lane; d < Dh; d += 32) st_f(dst + d, accs[(size_t)row * Dh + d] * inv);
    }
}

// how a launch is cut: rows per block from the shared memory that the staged strip leaves
static void ar_geometry(int G, int Dh, int max_new, bool vec4, int* tile_q, int* group_chunk, size_t* smem) {
    const size_t strip = (size_t)AR_STRIP * (ar_key_pitch(Dh, vec4) + Dh) * sizeof(float);
    const size_t per_row = (size_t)(2 * Dh + 2) * sizeof(float);
    int rows_max = (int)((AR_SMEM_BUDGET - strip) / per_row);          // at least 17 (head size 512)
    int gc = G < rows_max ? G : rows_max;
    int tq = rows_max / gc;
    tq = tq > AR_MAX_TILE ? AR_MAX_TILE : tq;
    tq = tq > max_new ? max_new : tq;
    tq = tq < 1 ? 1 : tq;
    *tile_q = tq;
    *group_chunk = gc;
    *smem = strip + (size_t)tq * gc * per_row;
}

template <typename T, bool VEC4>
static int ar_launch(const void* q, const void* k_pool, const void* v_pool, void* out, const int* page_table,
                     const int* seq_slot, const int* seq_start, const int* seq_len, int seqs, int max_new, int H, int KV,
                     int Dh, int mpps, int page_size, int num_pages, float scale, int window, int* err_flag,
                     cudaStream_t stream) {
    int tile_q, group_chunk;
    size_t smem;
    const int G = H / KV;
    ar_geometry(G, Dh, max_new, VEC4, &tile_q, &group_chunk, &smem);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_rows_kernel<T, VEC4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AR_SMEM_BUDGET + 1024);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_rows: shared memory limit: %s", cudaGetErrorString(e));
        configured = true;
    }
    const long long gy = (long long)KV * ((G + group_chunk - 1) / group_chunk);
    RI_REQUIRE(gy <= 65535 && seqs <= 65535, "attention_rows: %d heads, %d sequences: too many for one launch", H, seqs);
    dim3 grid((max_new + tile_q - 1) / tile_q, (unsigned)gy, seqs);
    attention_rows_kernel<T, VEC4><<<grid, 32 * AR_WARPS, smem, stream>>>(
        (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, page_table, seq_slot, seq_start, seq_len, H, KV, Dh, mpps,
        page_size, num_pages, tile_q, group_chunk, scale, window, err_flag);
    RI_CHECK_LAUNCH("attention_rows");
    return 0;
}

// q, out [tokens, H, Dh]; max_new = the most tokens one sequence brings in this step
extern "C" int ri_attention_rows(const void* q, const void* k_pool, const void* v_pool, void* out, const int* page_table,
                                 const int* seq_slot, const int* seq_start, const int* seq_len, int seqs, int max_new,
                                 int H, int KV, int Dh, int mpps, int page_size, int num_pages, float scale, int window,
                                 int dtype, int* err_flag, cudaStream_t stream) {
    if (seqs == 0 || max_new == 0) return 0;
    RI_REQUIRE(seqs > 0 && max_new > 0 && H > 0 && KV > 0 && Dh > 0 && page_size > 0 && mpps > 0, "attention_rows: bad sizes");
    RI_REQUIRE(H % KV == 0, "attention_rows: %d heads are not a multiple of %d kv heads", H, KV);
    RI_REQUIRE(Dh <= AR_MAX_DH, "attention_rows: head_dim %d exceeds the limit %d", Dh, AR_MAX_DH);
    RI_REQUIRE(window >= 0, "attention_rows: negative window");
    const bool f32 = dtype == RI_DTYPE_F32;
    RI_REQUIRE(f32 || dtype == RI_DTYPE_BF16, "attention_rows: unknown dtype %d", dtype);
    // vector loads need rows of the pools and of q that start on 16 bytes (float32) or 8 bytes (bfloat16)
    const uintptr_t align = f32 ? 15 : 7;
    const bool vec4 = Dh % 4 == 0 && (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & align) == 0;
#define AR_GO(T, V) ar_launch<T, V>(q, k_pool, v_pool, out, page_table, seq_slot, seq_start, seq_len, seqs, max_new, H, KV, \
                                    Dh, mpps, page_size, num_pages, scale, window, err_flag, stream)
    if (f32) return vec4 ? AR_GO(float, true) : AR_GO(float, false);
    return vec4 ? AR_GO(__nv_bfloat16, true) : AR_GO(__nv_bfloat16, false);
#undef AR_GO
}
