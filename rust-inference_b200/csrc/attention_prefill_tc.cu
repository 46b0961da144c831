// Prefill attention on the 5th-generation tensor cores (tcgen05) for bfloat16, head size 64 or 128.
//
// Grid (head, query tile, sequence); a tile is 128 consecutive new tokens of one
// sequence, two threads per token (8 warps).  For every block of 64 keys the block
//   1. brings the keys and values from the paged cache into shared memory in the
//      128-byte-swizzled layout the tensor core reads (cp.async; the next block's keys
//      are asked for as soon as S is done, its values as soon as O_blk is done);
//   2. S = Q K^T: one thread issues tcgen05.mma (M 128 queries, N 64 keys), the
//      accumulator lives in tensor memory (TMEM columns 0..63);
//   3. every thread reads its own row of S from TMEM (tcgen05.ld), takes the online
//      softmax in float32 (maximum, then exp2 and sum), and writes its row of P as
//      bfloat16 into shared memory, again in the swizzled operand layout;
//   4. O_blk = P V: tcgen05.mma with V read as an MN-major operand straight from the
//      [key][element] tile (TMEM columns 64..), read back and added to the thread's
//      running output, rescaled by exp2(old maximum - new maximum).
// Completion of the MMAs is signalled through tcgen05.commit on an mbarrier; every
// wait is bounded and ends in an error code, not a hang.
//
// Token t of sequence b: q row seq_start[b] + t, position seq_len[b] - n_b + t;
// it sees keys max(0, pos-window+1)..pos.  A query's result depends on its position
// and its place in the step, not on the batch.
//
// Compile with -DRI_HEAD_DIM=64 or 128.  Page size is 32.
// Formula: thanhauco/rust-inference src/attention.rs:4-8, 111-150.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <float.h>

#ifndef RI_HEAD_DIM
#define RI_HEAD_DIM 128
#endif
static_assert(RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128, "tcgen05 prefill attention: head_dim 64 or 128");

#define TC_DH RI_HEAD_DIM
#define TC_PAGE 32
#define TC_BM 128                       // queries per block
#define TC_THREADS 256                  // two threads per query row
#define TC_BN 64                        // keys per step
#define TC_SLABS (TC_DH / 64)           // 64-element (128-byte) slabs along the head
#define TC_Q_SLAB (TC_BM * 128)         // a slab of the query tile: 128 rows of 128 bytes
#define TC_KV_SLAB (TC_BN * 128)        // a slab of a key or value tile: 64 rows of 128 bytes
#define TC_Q_BYTES (TC_SLABS * TC_Q_SLAB)
#define TC_KV_BYTES (TC_SLABS * TC_KV_SLAB)
#define TC_P_BYTES (TC_BM * 128)        // P [128 x 64 keys]: one slab
#define TC_TMEM_COLS 256                // S: columns 0..63, O_blk: columns 64..64+Dh-1

// dynamic shared memory, 1024-byte aligned (swizzle atoms):
//   q | k | v | p      then the small things
struct TcTail {
    unsigned long long mma_bar;
    unsigned tmem_base;
    int dead;
    float rowmax[2][128];             // exchange between the two threads of a row
};
#define TC_OFF_Q 0
#define TC_OFF_K (TC_OFF_Q + TC_Q_BYTES)
#define TC_OFF_V (TC_OFF_K + TC_KV_BYTES)
#define TC_OFF_P (TC_OFF_V + TC_KV_BYTES)
#define TC_OFF_TAIL (TC_OFF_P + TC_P_BYTES)
#define TC_SMEM_BYTES (TC_OFF_TAIL + 1088 + 1024)   // + slack to align the base to 1024

// The swizzled operand layout: a tile is cut into slabs of 64 elements (128 bytes) along its rows;
// inside a slab rows are 128 bytes apart and the 16-byte chunk c of a row sits at chunk position
// c ^ (row % 8).  Tiles start on 1024-byte boundaries.

// shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// instruction descriptor of kind::f16: bf16 x bf16 -> f32, A K-major, B K-major or MN-major
__host__ __device__ constexpr unsigned instr_desc(int M, int N, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_mn_major << 16) | ((unsigned)(N >> 3) << 17) |
           ((unsigned)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ bool tc_mbar_wait(unsigned long long* bar, unsigned parity) { return ri_mbar_wait(bar, parity); }

// A piece of a row of a [rows x Dh] tile from global memory into the swizzled layout: `chunks`
// 16-byte chunks starting at chunk `c0` of row `r`; `ok` false writes zeros.  `slab_bytes` is the
// size of one 64-element slab of the tile (rows * 128).
__device__ __forceinline__ void copy_row_piece(unsigned char* tile, int slab_bytes, int r, int c0, int chunks,
                                               const bf16* src_row, bool ok) {
    unsigned char* dst_row = tile + r * 128;
    for (int j = 0; j < chunks; j++) {
        int c = c0 + j;                                 // chunk of the row, 0 .. Dh/8 - 1
        cp_async16(dst_row + (c >> 3) * slab_bytes + (((c & 7) ^ (r & 7)) << 4), src_row + c * 8, ok);
    }
}
// keys [key0, key0+64) of one kv head: thread t copies a quarter of row t/4
__device__ __forceinline__ void load_kv_tile(unsigned char* tile, const bf16* __restrict__ pool,
                                             const int* __restrict__ table, int kvh, int KV, int num_pages, int key0,
                                             int len, int* err) {
    constexpr int Q4 = TC_DH / 32;                      // chunks in a quarter row
    const int r = threadIdx.x >> 2;
    const int key = key0 + r;
    bool ok = key < len;
    size_t off = 0;
    if (ok) {
        int page = table[key / TC_PAGE];
        if (page < 0 || page >= num_pages) {
            atomicExch(err, 4);
            ok = false;
        } else {
            off = (((size_t)page * KV + kvh) * TC_PAGE + key % TC_PAGE) * TC_DH;
        }
    }
    copy_row_piece(tile, TC_KV_SLAB, r, (threadIdx.x & 3) * Q4, Q4, pool + off, ok);
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// 256 threads: thread t works on query row t % 128; threads t and t + 128 share a row, the first
// takes keys 0..31 of a block and the first half of the output elements, the second the rest.
// Two blocks fit on an SM: while one waits for the tensor core the other does its softmax.
__global__ void __launch_bounds__(TC_THREADS, 2)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool,
                            const bf16* __restrict__ v_pool, bf16* __restrict__ out,
                            const int* __restrict__ page_table, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_len, int H, int KV, int mpps,
                            int num_pages, float scale_log2, int window, int* __restrict__ err) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    TcTail& tail = *reinterpret_cast<TcTail*>(smem + TC_OFF_TAIL);
    // blocks start in the order of blockIdx.x, then y: heads vary fastest, so the late tiles of all
    // heads, which see the most keys, start first
    const int b = blockIdx.z, h = blockIdx.x;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin;
    const int tiles = (n_new + TC_BM - 1) / TC_BM;
    const int tile = (int)gridDim.y - 1 - (int)blockIdx.y;
    if (tile >= tiles) return;
    const int len = seq_len[b];
    const int r_base = tile * TC_BM;
    const int rows = min(TC_BM, n_new - r_base);
    const int pos_first = len - n_new + r_base, pos_last = pos_first + rows - 1;
    const int key_lo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int kb_lo = key_lo / TC_BN, kb_hi = pos_last / TC_BN;
    const int kvh = h / (H / KV);
    const int* table = page_table + (size_t)seq_slot[b] * mpps;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (TC_BM - 1), half = tid >> 7;            // my query row, my half of keys / elements
    const int my_pos = pos_first + row;
    unsigned char* k_tile = smem + TC_OFF_K;
    unsigned char* v_tile = smem + TC_OFF_V;

    // ---- set-up: tensor memory, the MMA barrier --------------------------------------------------
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tail.tmem_base)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.mma_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tail.dead = 0;
    }
    // ---- copies in flight: group 1 = queries and the first keys, group 2 = the first values --------
    {
        const int r = tid >> 1;
        const bool ok = r < rows;
        copy_row_piece(smem + TC_OFF_Q, TC_Q_SLAB, r, (tid & 1) * (TC_DH / 16), TC_DH / 16,
                       q + ((size_t)(t_begin + r_base + (ok ? r : 0)) * H + h) * TC_DH, ok);
    }
    load_kv_tile(k_tile, k_pool, table, kvh, KV, num_pages, kb_lo * TC_BN, len, err);
    cp_async_commit();
    load_kv_tile(v_tile, v_pool, table, kvh, KV, num_pages, kb_lo * TC_BN, len, err);
    cp_async_commit();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tail.tmem_base;
    const unsigned tmem_row = tmem + ((unsigned)((warp & 3) * 32) << 16);      // this warp's 32 lanes
    const unsigned q_addr = smem_u32(smem + TC_OFF_Q), p_addr = smem_u32(smem + TC_OFF_P);
    const unsigned k_addr = smem_u32(k_tile), v_addr = smem_u32(v_tile);
    constexpr unsigned IDESC_QK = instr_desc(TC_BM, TC_BN, 0);
    constexpr unsigned IDESC_PV = instr_desc(TC_BM, TC_DH, 1);
    constexpr int OW = TC_DH / 2;                                  // output elements per thread
    constexpr int SW = TC_BN / 2;                                  // scores per thread (32)

    float o[OW];
#pragma unroll
    for (int i = 0; i < OW; i++) o[i] = 0.0f;
    float m = -FLT_MAX, l = 0.0f;                                  // m: in units of scaled log2 scores
    unsigned phase = 0;
    bool dead = false;

    for (int kb = kb_lo; kb <= kb_hi && !dead; kb++) {
        // the keys of this block have arrived (the values may still be on their way)
        cp_async_wait<1>();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        // ---- S = Q K^T ---------------------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < TC_DH / 16; j++) {
                unsigned qo = (unsigned)((j >> 2) * TC_Q_SLAB + (j & 3) * 32), ko = (unsigned)((j >> 2) * TC_KV_SLAB + (j & 3) * 32);
                umma_bf16(tmem, smem_desc(q_addr + qo, 16, 1024), smem_desc(k_addr + ko, 16, 1024), IDESC_QK, j > 0);
            }
            umma_commit(&tail.mma_bar);
        }
        if (!tc_mbar_wait(&tail.mma_bar, phase)) { atomicExch(err, 5); tail.dead = 1; }
        phase ^= 1;
        tc_fence_after();
        // the key tile is free: ask for the next block's keys (an empty group after the last block)
        if (kb < kb_hi) load_kv_tile(k_tile, k_pool, table, kvh, KV, num_pages, (kb + 1) * TC_BN, len, err);
        cp_async_commit();
        // ---- my 32 scores of the row: mask, maximum (shared with the row's other thread) --------------
        const int k0 = kb * TC_BN + half * SW;                     // my first key
        const bool edge = (kb * TC_BN + TC_BN - 1 > pos_first) || (window > 0 && kb * TC_BN < pos_last - window + 1);
        float s[SW];
        tmem_ld32(tmem_row + half * SW, s);
        float mx = -FLT_MAX;
        if (edge) {
#pragma unroll
            for (int i = 0; i < SW; i++) {
                int key = k0 + i;
                bool vis = key <= my_pos && (window <= 0 || key > my_pos - window);
                s[i] = vis ? s[i] : -FLT_MAX;
                mx = fmaxf(mx, s[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < SW; i++) mx = fmaxf(mx, s[i]);
        }
        tail.rowmax[half][row] = mx;
        __syncthreads();
        mx = fmaxf(mx, tail.rowmax[half ^ 1][row]);
        mx = mx == -FLT_MAX ? -FLT_MAX : mx * scale_log2;          // scale > 0: the maximum of the scaled scores
        mx = fmaxf(mx, m);
        const float corr = (m == -FLT_MAX) ? 0.0f : ex2_approx(m - mx);
        m = mx;
        l *= corr;
        // ---- P = exp2(S * scale - m) as bfloat16 into the operand layout; sum --------------------------
        {
            const float neg_m = (m == -FLT_MAX) ? 0.0f : -m;
            unsigned char* p_row = smem + TC_OFF_P + row * 128;
#pragma unroll
            for (int c = 0; c < SW / 8; c++) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    float x = s[c * 8 + e];
                    p[e] = (x == -FLT_MAX) ? 0.0f : ex2_approx(fmaf(x, scale_log2, neg_m));
                    l += p[e];
                }
                const int chunk = half * (SW / 8) + c;             // 16-byte chunk of the 64-key row
                *(uint4*)(p_row + ((chunk ^ (row & 7)) << 4)) =
                    make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
            }
        }
        cp_async_wait<1>();              // the values of this block have arrived (the next keys may be on their way)
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        // ---- O_blk = P V --------------------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < TC_BN / 16; j++) {
                umma_bf16(tmem + TC_BN, smem_desc(p_addr + j * 32, 16, 1024),
                          smem_desc(v_addr + j * 16 * 128, TC_KV_SLAB, 1024), IDESC_PV, j > 0);
            }
            umma_commit(&tail.mma_bar);
        }
        if (!tc_mbar_wait(&tail.mma_bar, phase)) { atomicExch(err, 5); tail.dead = 1; }
        phase ^= 1;
        tc_fence_after();
        // the value tile is free: ask for the next block's values
        if (kb < kb_hi) load_kv_tile(v_tile, v_pool, table, kvh, KV, num_pages, (kb + 1) * TC_BN, len, err);
        cp_async_commit();
#pragma unroll
        for (int c = 0; c < OW / 32; c++) {
            float ob[32];
            tmem_ld32(tmem_row + TC_BN + half * OW + c * 32, ob);
#pragma unroll
            for (int i = 0; i < 32; i++) o[c * 32 + i] = fmaf(o[c * 32 + i], corr, ob[i]);
        }
        dead = tail.dead != 0;
        // the next iteration's first barrier comes before anything of S, O_blk or P is overwritten
    }
    cp_async_wait<0>();
    // ---- out = O / l (l: both halves of the row) ---------------------------------------------------------
    __syncthreads();
    tail.rowmax[half][row] = l;
    __syncthreads();
    l += tail.rowmax[half ^ 1][row];
    if (row < rows && !dead) {
        const float inv = 1.0f / l;
        bf16* dst = out + ((size_t)(t_begin + r_base + row) * H + h) * TC_DH + half * OW;
#pragma unroll
        for (int i = 0; i < OW; i += 8) {
            uint4 w;
            w.x = pack_bf16(o[i] * inv, o[i + 1] * inv);
            w.y = pack_bf16(o[i + 2] * inv, o[i + 3] * inv);
            w.z = pack_bf16(o[i + 4] * inv, o[i + 5] * inv);
            w.w = pack_bf16(o[i + 6] * inv, o[i + 7] * inv);
            *(uint4*)(dst + i) = w;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

extern "C" int ri_attention_prefill_tc_head_dim() { return TC_DH; }

// q, out [tokens, H, Dh] bf16; max_new = the most tokens one sequence brings in this step
extern "C" int ri_attention_prefill_tc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       const int* page_table, const int* seq_slot, const int* seq_start,
                                       const int* seq_len, int seqs, int max_new, int H, int KV, int Dh, int mpps,
                                       int page_size, int num_pages, float scale, int window, int* err_flag,
                                       cudaStream_t stream) {
    if (seqs == 0 || max_new == 0) return 0;
    RI_REQUIRE(Dh == TC_DH, "attention_prefill_tc: built for head_dim %d, called with %d", TC_DH, Dh);
    RI_REQUIRE(page_size == TC_PAGE, "attention_prefill_tc: pages of %d tokens, this kernel needs %d", page_size, TC_PAGE);
    RI_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_prefill_tc: %d heads over %d kv heads", H, KV);
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "attention_prefill_tc: bad grid");
    RI_REQUIRE(window >= 0, "attention_prefill_tc: negative window");
    RI_REQUIRE(scale > 0.0f, "attention_prefill_tc: the score scale must be positive");
    RI_REQUIRE((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) == 0,
               "attention_prefill_tc: q, out and the pools must be 16-byte aligned");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_prefill_tc: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(H, (max_new + TC_BM - 1) / TC_BM, seqs);
    RI_REQUIRE(grid.y <= 65535, "attention_prefill_tc: too many tokens in one sequence of a step");
    attention_prefill_tc_kernel<<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, page_table, seq_slot, seq_start, seq_len,
        H, KV, mpps, num_pages, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_prefill_tc");
    return 0;
}
