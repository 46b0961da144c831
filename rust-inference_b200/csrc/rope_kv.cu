// Per-head RMSNorm of queries and keys, rotary position encoding and the append
// of keys and values to the paged cache, in one pass over the fused projection.
//
//   qkv  [tokens, (H + 2*KV) * Dh]   q heads, then k heads, then v heads
//   q_out[tokens, H, Dh]
//   k_pool, v_pool [pages, KV, page_size, Dh]  (one layer's pools)
//
// For a head vector x of q or k:  y = x * (1/sqrt(mean(x^2)+eps)) * gain  (if a
// gain is given), then for d < rot/2 with (c, s) = table[pos][d]:
//   z[d] = y[d]*c - y[d+rot/2]*s ;  z[d+rot/2] = y[d+rot/2]*c + y[d]*s
// and elements from `rot` on are left as they are.  All of it in float32.
// Formulas: thanhauco/rust-inference src/ops/norm.rs:14-32, src/ops/rope.rs:52-79,
// src/kvcache.rs:145-189 (kernels.cu:97-142, 321-336 there).
#include "common.cuh"

#define RK_WARPS 4
#define RK_MAX_DH 512

template <typename T>
__global__ void qk_norm_rope_append_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool,
                                           T* __restrict__ v_pool, const int* __restrict__ page_table,
                                           const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                           const int* __restrict__ seq_slot, const float* __restrict__ q_gain,
                                           const float* __restrict__ k_gain, float eps,
                                           const float2* __restrict__ rope, int rope_rows, int rot, int H, int KV,
                                           int Dh, int mpps, int page_size, int num_pages, int write_kv,
                                           int* __restrict__ err) {
    __shared__ float buf[RK_WARPS][RK_MAX_DH];
    pdl_trigger();
    pdl_wait();
    int t = blockIdx.x;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int pos = tok_pos[t];
    int slot = seq_slot[tok_seq[t]];
    int page = -1;
    if (write_kv) {
        page = page_table[(size_t)slot * mpps + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(err, 2);   // unmapped page: skip the write, report
            page = -1;
        }
    }
    if (rope && (pos < 0 || pos >= rope_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    int heads_total = H + 2 * KV;
    int half = rot / 2;
    const T* row = qkv + (size_t)t * heads_total * Dh;
    float* x = buf[warp];
    for (int h = blockIdx.y * RK_WARPS + warp; h < heads_total; h += RK_WARPS * gridDim.y) {
        const T* src = row + (size_t)h * Dh;
        int which = h < H ? 0 : (h < H + KV ? 1 : 2);      // q, k, v
        T* dst;
        if (which == 0) {
            dst = q_out + ((size_t)t * H + h) * Dh;
        } else {
            if (!write_kv || page < 0) continue;
            int kvh = which == 1 ? h - H : h - H - KV;
            T* pool = which == 1 ? k_pool : v_pool;
            dst = pool + (((size_t)page * KV + kvh) * page_size + pos % page_size) * Dh;
        }
        if (which == 2) {
            for (int d = lane; d < Dh; d += 32) dst[d] = src[d];
            continue;
        }
        const float* gain = which == 0 ? q_gain : k_gain;
        float ss = 0.0f;
        for (int d = lane; d < Dh; d += 32) {
            float v = ld_f(src + d);
            x[d] = v;
            ss += v * v;
        }
        if (gain) {
            ss = warp_sum(ss);
            float inv = 1.0f / sqrtf(ss / (float)Dh + eps);
            for (int d = lane; d < Dh; d += 32) x[d] = x[d] * inv * gain[d];
        }
        __syncwarp();
        if (rope) {
            const float2* cs = rope + (size_t)pos * half;
            for (int d = lane; d < half; d += 32) {
                float a = x[d], b = x[d + half];
                float2 c = cs[d];
                st_f(dst + d, a * c.x - b * c.y);
                st_f(dst + d + half, b * c.x + a * c.y);
            }
            for (int d = rot + lane; d < Dh; d += 32) st_f(dst + d, x[d]);
        } else {
            for (int d = lane; d < Dh; d += 32) st_f(dst + d, x[d]);
        }
        __syncwarp();
    }
}

// The same for head sizes of 64, 128 or 256 with the whole head rotated: a lane holds VEC
// consecutive elements (Dh = 32 * VEC), loads and stores are VEC elements wide, and the
// rotation partner of an element (half a head away) sits in lane ^ 16.
template <typename T, int V>
struct alignas(sizeof(T) * V) VecOf {
    T v[V];
};

#define RK_UNROLL 4
template <typename T, int VEC>
__global__ void qk_norm_rope_append_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool,
                                               T* __restrict__ v_pool, const int* __restrict__ page_table,
                                               const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                               const int* __restrict__ seq_slot, const float* __restrict__ q_gain,
                                               const float* __restrict__ k_gain, float eps,
                                               const float2* __restrict__ rope, int rope_rows, int H, int KV, int mpps,
                                               int page_size, int num_pages, int write_kv, int* __restrict__ err) {
    constexpr int Dh = 32 * VEC;
    pdl_trigger();
    // What the kernel before this one does not write is read before the wait for it: the step's tables (copied to
    // the device before the step's first kernel), the page table, the angles of this position and the gains.  With
    // a handful of tokens this kernel is a chain of dependent loads, and these are three links of it.
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    int page = -1, bad = 0;
    if (write_kv) {
        page = page_table[(size_t)slot * mpps + pos / page_size];
        if (page < 0 || page >= num_pages) {
            bad = 2;                                             // unmapped page: skip the write, report
            page = -1;
        }
    }
    const bool rope_ok = !rope || (pos >= 0 && pos < rope_rows);
    const int heads_total = H + 2 * KV;
    const T* row = qkv + (size_t)t * heads_total * Dh;
    const int d0 = lane * VEC;                                   // this lane's first element
    float cs_c[VEC], cs_s[VEC], gq[VEC], gk[VEC];
    if (rope && rope_ok) {
        const float2* cs = rope + (size_t)pos * (Dh / 2) + (lane & 15) * VEC;
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            float2 c = cs[j];
            cs_c[j] = c.x;
            cs_s[j] = (lane < 16) ? -c.y : c.y;                  // low half: a*c - b*s; high half: b*c + a*s
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        gq[j] = q_gain ? q_gain[d0 + j] : 1.0f;
        gk[j] = k_gain ? k_gain[d0 + j] : 1.0f;
    }
    pdl_wait();
    if (bad && threadIdx.x == 0) atomicExch(err, bad);
    if (!rope_ok) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    // heads in batches of RK_UNROLL: all their loads are started before the first is worked on
    const int stride = RK_WARPS * gridDim.y;
    for (int h0 = blockIdx.y * RK_WARPS + warp; h0 < heads_total; h0 += stride * RK_UNROLL) {
        VecOf<T, VEC> in[RK_UNROLL];
#pragma unroll
        for (int u = 0; u < RK_UNROLL; u++) {
            const int h = h0 + u * stride;
            if (h < heads_total) in[u] = *(const VecOf<T, VEC>*)(row + (size_t)h * Dh + d0);
        }
#pragma unroll
        for (int u = 0; u < RK_UNROLL; u++) {
            const int h = h0 + u * stride;
            if (h >= heads_total) break;
            const int which = h < H ? 0 : (h < H + KV ? 1 : 2);
            T* dst;
            if (which == 0) {
                dst = q_out + ((size_t)t * H + h) * Dh;
            } else {
                if (!write_kv || page < 0) continue;
                const int kvh = which == 1 ? h - H : h - H - KV;
                T* pool = which == 1 ? k_pool : v_pool;
                dst = pool + (((size_t)page * KV + kvh) * page_size + pos % page_size) * Dh;
            }
            if (which == 2) {
                *(VecOf<T, VEC>*)(dst + d0) = in[u];
                continue;
            }
            float x[VEC];
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                x[j] = ld_f(&in[u].v[j]);
                ss += x[j] * x[j];
            }
            if (which == 0 ? q_gain != nullptr : k_gain != nullptr) {
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)Dh + eps);
#pragma unroll
                for (int j = 0; j < VEC; j++) x[j] = x[j] * inv * (which == 0 ? gq[j] : gk[j]);
            }
            VecOf<T, VEC> o;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                float v = x[j];
                if (rope) {
                    float other = __shfl_xor_sync(0xffffffffu, x[j], 16);
                    v = x[j] * cs_c[j] + other * cs_s[j];
                }
                st_f(&o.v[j], v);
            }
            *(VecOf<T, VEC>*)(dst + d0) = o;
        }
    }
}

// bfloat16 with 16 bytes per lane: a head of DH elements takes DH / 8 lanes, a warp works on 32 / (DH / 8) heads
// at a time; the rotation partner of a lane's eight elements sits DH / 16 lanes away.  Used for many tokens
// (prefill), where the 8-byte loads of the kernel above leave half of the memory bandwidth unused.
template <int DH>
__global__ void qk_norm_rope_append_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                                  __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                                                  const int* __restrict__ page_table, const int* __restrict__ tok_seq,
                                                  const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                                  const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                                  float eps, const float2* __restrict__ rope, int rope_rows, int H, int KV,
                                                  int mpps, int page_size, int num_pages, int write_kv,
                                                  int* __restrict__ err) {
    constexpr int LPH = DH / 8;                  // lanes per head
    constexpr int HPW = 32 / LPH;                // heads per warp at a time
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LPH, ln = lane % LPH; // which of the warp's heads, which part of it
    const int heads_total = H + 2 * KV;
    const __nv_bfloat16* row = qkv + (size_t)t * heads_total * DH;
    const int d0 = ln * 8;
    // the loads of the first batch of heads start before anything else is known
    const int stride = RK_WARPS * HPW * gridDim.y;
    const int h_first = (blockIdx.y * RK_WARPS + warp) * HPW + sub;
    uint4 in[RK_UNROLL];
#pragma unroll
    for (int u = 0; u < RK_UNROLL; u++) {
        const int h = h_first + u * stride;
        if (h < heads_total) in[u] = *(const uint4*)(row + (size_t)h * DH + d0);
    }
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    int page = -1;
    if (write_kv) {
        page = page_table[(size_t)slot * mpps + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            page = -1;
        }
    }
    if (rope && (pos < 0 || pos >= rope_rows)) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    float cs_c[8], cs_s[8];
    if (rope) {
        const float2* cs = rope + (size_t)pos * (DH / 2) + (d0 % (DH / 2));
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            const float4 c = *(const float4*)(cs + j);           // two (cos, sin) pairs
            cs_c[j] = c.x;
            cs_s[j] = (d0 < DH / 2) ? -c.y : c.y;                // low half: a*c - b*s; high half: b*c + a*s
            cs_c[j + 1] = c.z;
            cs_s[j + 1] = (d0 < DH / 2) ? -c.w : c.w;
        }
    }
    for (int h0 = h_first, first = 1; h0 < heads_total; h0 += stride * RK_UNROLL, first = 0) {
        if (!first) {
#pragma unroll
            for (int u = 0; u < RK_UNROLL; u++) {
                const int h = h0 + u * stride;
                if (h < heads_total) in[u] = *(const uint4*)(row + (size_t)h * DH + d0);
            }
        }
#pragma unroll
        for (int u = 0; u < RK_UNROLL; u++) {
            const int h = h0 + u * stride;
            // the lanes of one head go together; a head past the end still takes part in the shuffles below
            const bool live = h < heads_total;
            const int which = !live ? 3 : (h < H ? 0 : (h < H + KV ? 1 : 2));
            __nv_bfloat16* dst = nullptr;
            if (which == 0) {
                dst = q_out + ((size_t)t * H + h) * DH;
            } else if (which < 3 && write_kv && page >= 0) {
                const int kvh = which == 1 ? h - H : h - H - KV;
                dst = (which == 1 ? k_pool : v_pool) + (((size_t)page * KV + kvh) * page_size + pos % page_size) * DH;
            }
            // (no lane leaves early: the shuffles below are the whole warp's, and its heads may be of different kinds)
            float x[8];
            {
                const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&in[u]);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __bfloat1622float2(live ? p2[j] : __nv_bfloat162());
                    x[2 * j] = f.x;
                    x[2 * j + 1] = f.y;
                }
            }
            const float* gain = which == 0 ? q_gain : (which == 1 ? k_gain : nullptr);
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss += x[j] * x[j];
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (gain) {
                const float inv = 1.0f / sqrtf(ss / (float)DH + eps);
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = x[j] * inv * gain[d0 + j];
            }
            uint4 o;
            unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                float v0 = x[j], v1 = x[j + 1];
                if (rope) {
                    const float o0 = __shfl_xor_sync(0xffffffffu, x[j], LPH / 2);
                    const float o1 = __shfl_xor_sync(0xffffffffu, x[j + 1], LPH / 2);
                    v0 = x[j] * cs_c[j] + o0 * cs_s[j];
                    v1 = x[j + 1] * cs_c[j + 1] + o1 * cs_s[j + 1];
                }
                const __nv_bfloat162 pk = __floats2bfloat162_rn(v0, v1);
                ow[j / 2] = *reinterpret_cast<const unsigned*>(&pk);
            }
            if (dst) *(uint4*)(dst + d0) = which == 2 ? in[u] : o;      // values are copied as they are
        }
    }
}

template <typename T, int VEC>
static void launch_rope_vec(dim3 grid, cudaStream_t stream, const void* qkv, void* q_out, void* k_pool, void* v_pool,
                            const int* page_table, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                            const float* q_gain, const float* k_gain, float eps, const float* rope_table, int rope_rows,
                            int H, int KV, int mpps, int page_size, int num_pages, int write_kv, int* err_flag) {
    ri_launch_pdl(qk_norm_rope_append_vec_kernel<T, VEC>, grid, dim3(32 * RK_WARPS), 0, stream, (const T*)qkv, (T*)q_out,
                  (T*)k_pool, (T*)v_pool, page_table, tok_seq, tok_pos, seq_slot, q_gain, k_gain, eps,
                  (const float2*)rope_table, rope_rows, H, KV, mpps, page_size, num_pages, write_kv, err_flag);
}

extern "C" int ri_qk_norm_rope_append(const void* qkv, void* q_out, void* k_pool, void* v_pool, const int* page_table,
                                      const int* tok_seq, const int* tok_pos, const int* seq_slot, const float* q_gain,
                                      const float* k_gain, float eps, const float* rope_table, int rope_rows, int rot,
                                      int tokens, int H, int KV, int Dh, int mpps, int page_size, int num_pages,
                                      int write_kv, int dtype, int* err_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    // H or KV may be 0 (only queries, or only keys and values); without kv heads nothing is appended
    RI_REQUIRE(tokens > 0 && H >= 0 && KV >= 0 && H + KV > 0 && Dh > 0, "qk_norm_rope_append: bad sizes");
    if (KV == 0) write_kv = 0;
    RI_REQUIRE(Dh <= RK_MAX_DH, "qk_norm_rope_append: head_dim %d exceeds the limit %d", Dh, RK_MAX_DH);
    RI_REQUIRE(rot >= 0 && rot <= Dh && rot % 2 == 0, "qk_norm_rope_append: rotary_dim %d must be even and <= head_dim %d", rot, Dh);
    RI_REQUIRE(!rope_table || rot > 0, "qk_norm_rope_append: a rope table needs rotary_dim > 0");
    RI_REQUIRE(page_size > 0 && mpps > 0, "qk_norm_rope_append: bad page sizes");
    // few tokens: spread the heads of a token over several blocks (one head per warp)
    int head_blocks = (H + 2 * KV + RK_WARPS - 1) / RK_WARPS;
    if ((long long)tokens * head_blocks > 4096) head_blocks = 1 > 4096 / tokens ? 1 : 4096 / tokens;
    RI_REQUIRE(tokens <= 2147483647 && head_blocks <= 65535, "qk_norm_rope_append: bad grid");
    dim3 grid(tokens, head_blocks);
    const bool whole = !rope_table || rot == Dh;
    const bool aligned = ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 31) == 0);
    if (whole && aligned && (Dh == 64 || Dh == 128 || Dh == 256) && (dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16)) {
#define RI_ROPE_VEC(T, V) launch_rope_vec<T, V>(grid, stream, qkv, q_out, k_pool, v_pool, page_table, tok_seq, tok_pos, \
                                                seq_slot, q_gain, k_gain, eps, rope_table, rope_rows, H, KV, mpps,      \
                                                page_size, num_pages, write_kv, err_flag)
        if (dtype == RI_DTYPE_F32) {
            if (Dh == 64) RI_ROPE_VEC(float, 2); else if (Dh == 128) RI_ROPE_VEC(float, 4); else RI_ROPE_VEC(float, 8);
        } else if (tokens >= 64) {
            // many tokens: 16 bytes per lane, several heads per warp at a time
            const int hpw = 32 / (Dh / 8);
            int hb = (H + 2 * KV + RK_WARPS * hpw - 1) / (RK_WARPS * hpw);
            if ((long long)tokens * hb > 2048) hb = 1 > 2048 / tokens ? 1 : 2048 / tokens;    // few blocks per token: the rotary table is read once per warp
            dim3 grid8(tokens, hb);
#define RI_ROPE_X8(D) ri_launch_pdl(qk_norm_rope_append_bf16x8_kernel<D>, grid8, dim3(32 * RK_WARPS), 0, stream,            \
                                    (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,              \
                                    (__nv_bfloat16*)v_pool, page_table, tok_seq, tok_pos, seq_slot, q_gain, k_gain, eps,   \
                                    (const float2*)rope_table, rope_rows, H, KV, mpps, page_size, num_pages, write_kv,     \
                                    err_flag)
            if (Dh == 64) RI_ROPE_X8(64); else if (Dh == 128) RI_ROPE_X8(128); else RI_ROPE_X8(256);
#undef RI_ROPE_X8
        } else {
            if (Dh == 64) RI_ROPE_VEC(__nv_bfloat16, 2); else if (Dh == 128) RI_ROPE_VEC(__nv_bfloat16, 4); else RI_ROPE_VEC(__nv_bfloat16, 8);
        }
#undef RI_ROPE_VEC
        RI_CHECK_LAUNCH("qk_norm_rope_append");
        return 0;
    }
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(qk_norm_rope_append_kernel<float>, grid, dim3(32 * RK_WARPS), 0, stream,
            (const float*)qkv, (float*)q_out, (float*)k_pool, (float*)v_pool, page_table, tok_seq, tok_pos, seq_slot,
            q_gain, k_gain, eps, (const float2*)rope_table, rope_rows, rot, H, KV, Dh, mpps, page_size, num_pages,
            write_kv, err_flag);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(qk_norm_rope_append_kernel<__nv_bfloat16>, grid, dim3(32 * RK_WARPS), 0, stream,
            (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
            page_table, tok_seq, tok_pos, seq_slot, q_gain, k_gain, eps, (const float2*)rope_table, rope_rows, rot, H,
            KV, Dh, mpps, page_size, num_pages, write_kv, err_flag);
    else
        RI_FAIL(-1, "qk_norm_rope_append: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("qk_norm_rope_append");
    return 0;
}
