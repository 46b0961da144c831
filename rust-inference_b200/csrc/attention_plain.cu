// Causal grouped-query attention over the paged cache: the plain kernel.
//
// One block per (head, token) with four warps; warp w takes the keys whose
// position j has j % 4 == w, each key a warp-wide dot product, softmax state
// (running maximum, sum, weighted values) in float32 per warp, merged at the
// end in warp order.  The order of every addition depends on the query's
// position only, so a token's output is the same whatever else is in the step.
// It serves the float32 path and is the fallback of the bfloat16 path.
//
//   q, out  [tokens, H, Dh];  k_pool, v_pool [pages, KV, page_size, Dh]
//   token t: sequence tok_seq[t] in slot seq_slot[.], position p = tok_pos[t];
//   it sees keys max(0, p-window+1) .. p  (window 0: all keys 0..p).
// score = (q . k) * scale;  kv head = h / (H / KV).
// Formulas: thanhauco/rust-inference src/attention.rs:4-8, 111-150
// (kernels.cu:338-405 there).
#include "common.cuh"
#include <float.h>

#define AP_WARPS 4
#define AP_MAX_DH 512
#define AP_PER_LANE (AP_MAX_DH / 32)

template <typename T>
__global__ void attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                       const T* __restrict__ v_pool, T* __restrict__ out,
                                       const int* __restrict__ page_table, const int* __restrict__ tok_seq,
                                       const int* __restrict__ tok_pos, const int* __restrict__ seq_slot, int H,
                                       int KV, int Dh, int mpps, int page_size, int num_pages, float scale, int window,
                                       int* __restrict__ err) {
    __shared__ float qs[AP_MAX_DH];
    __shared__ float wm[AP_WARPS], wl[AP_WARPS];
    __shared__ float wacc[AP_WARPS][AP_MAX_DH];

    int h = blockIdx.x, t = blockIdx.y;
    int kvh = h / (H / KV);
    int pos = tok_pos[t];
    int slot = seq_slot[tok_seq[t]];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* qrow = q + ((size_t)t * H + h) * Dh;
    for (int i = threadIdx.x; i < Dh; i += blockDim.x) qs[i] = ld_f(qrow + i);
    __syncthreads();

    const int per_lane = (Dh + 31) / 32;
    float acc[AP_PER_LANE];
#pragma unroll
    for (int i = 0; i < AP_PER_LANE; i++) acc[i] = 0.0f;
    float m = -FLT_MAX, l = 0.0f;
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = page_table + (size_t)slot * mpps;

    int j0 = first + ((warp - first) % AP_WARPS + AP_WARPS) % AP_WARPS;   // first j >= first with j % 4 == warp
    for (int j = j0; j <= pos; j += AP_WARPS) {
        int page = table[j / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicExch(err, 4);
            continue;
        }
        size_t off = (((size_t)page * KV + kvh) * page_size + j % page_size) * Dh;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < AP_PER_LANE; i++) {
            int d = lane + i * 32;
            if (i < per_lane && d < Dh) s += qs[d] * ld_f(k_pool + off + d);
        }
        s = warp_sum(s) * scale;
        float m_new = fmaxf(m, s);
        float corr = expf(m - m_new);
        float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < AP_PER_LANE; i++) {
            int d = lane + i * 32;
            if (i < per_lane && d < Dh) acc[i] = acc[i] * corr + p * ld_f(v_pool + off + d);
        }
        m = m_new;
    }

    if (lane == 0) { wm[warp] = m; wl[warp] = l; }
#pragma unroll
    for (int i = 0; i < AP_PER_LANE; i++) {
        int d = lane + i * 32;
        if (i < per_lane && d < Dh) wacc[warp][d] = acc[i];
    }
    __syncthreads();

    float mx = wm[0];
    for (int w = 1; w < AP_WARPS; w++) mx = fmaxf(mx, wm[w]);
    float denom = 0.0f;
    float f[AP_WARPS];
    for (int w = 0; w < AP_WARPS; w++) {
        f[w] = wl[w] > 0.0f ? expf(wm[w] - mx) : 0.0f;     // a warp that saw no key has weight 0
        denom += wl[w] * f[w];
    }
    T* orow = out + ((size_t)t * H + h) * Dh;
    for (int i = threadIdx.x; i < Dh; i += blockDim.x) {
        float v = 0.0f;
        for (int w = 0; w < AP_WARPS; w++) v += wacc[w][i] * f[w];
        st_f(orow + i, v / denom);
    }
}

extern "C" int ri_attention_plain(const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const int* page_table, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                                  int tokens, int H, int KV, int Dh, int mpps, int page_size, int num_pages,
                                  float scale, int window, int dtype, int* err_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && H > 0 && KV > 0 && Dh > 0, "attention_plain: bad sizes");
    RI_REQUIRE(H % KV == 0, "attention_plain: %d heads are not a multiple of %d kv heads", H, KV);
    RI_REQUIRE(Dh <= AP_MAX_DH, "attention_plain: head_dim %d exceeds the limit %d", Dh, AP_MAX_DH);
    RI_REQUIRE(tokens <= 65535 * 1024, "attention_plain: too many tokens in one step");
    RI_REQUIRE(window >= 0, "attention_plain: negative window");
    dim3 grid(H, tokens);
    RI_REQUIRE(tokens <= 65535, "attention_plain: at most 65535 tokens per step, got %d", tokens);
    if (dtype == RI_DTYPE_F32)
        attention_plain_kernel<float><<<grid, 32 * AP_WARPS, 0, stream>>>(
            (const float*)q, (const float*)k_pool, (const float*)v_pool, (float*)out, page_table, tok_seq, tok_pos,
            seq_slot, H, KV, Dh, mpps, page_size, num_pages, scale, window, err_flag);
    else if (dtype == RI_DTYPE_BF16)
        attention_plain_kernel<__nv_bfloat16><<<grid, 32 * AP_WARPS, 0, stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out,
            page_table, tok_seq, tok_pos, seq_slot, H, KV, Dh, mpps, page_size, num_pages, scale, window, err_flag);
    else
        RI_FAIL(-1, "attention_plain: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("attention_plain");
    return 0;
}
