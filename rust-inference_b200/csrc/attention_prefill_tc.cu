// Prefill attention on the 5th-generation tensor cores (tcgen05) for bfloat16, head size 64 or 128.
//
// Grid (head, query tile, sequence); a tile is 128 consecutive new tokens of one
// sequence, two threads per token (8 warps), two blocks per SM.  For every block of
// 64 keys
//   1. one thread starts TMA tensor copies (cp.async.bulk.tensor.2d, 128-byte swizzle:
//      the layout the tensor core reads) of the two pages of keys and of values from
//      the paged cache, two blocks ahead for the keys and one for the values (two
//      buffers each);
//   2. S = Q K^T: one thread issues tcgen05.mma (M 128 queries, N 64 keys), the
//      accumulator lives in tensor memory.  There are two S buffers (TMEM columns 0..63
//      and 64..127): S of the next block is issued as soon as every thread has read S
//      of this block, so the tensor core works on it and on the last P V while the
//      threads are busy with this block's softmax;
//   3. every thread reads its half row of S from TMEM (tcgen05.ld), and writes its
//      part of P = exp2(S * scale - m) as bfloat16 into shared memory in the operand
//      layout.  m is the row's running maximum, raised only when some row of the tile
//      meets a score more than 2^8 above its own (then every row takes its true
//      maximum and rescales its output in TMEM with tcgen05.ld / tcgen05.st); weights
//      up to 2^8 are exact in float32 and as good as any in bfloat16;
//   4. O += P V: tcgen05.mma with V read as an MN-major operand straight from the
//      [key][element] tile, accumulated in TMEM columns 128.. over all blocks.
// Completion of the products is signalled through tcgen05.commit on mbarriers (one for
// S, one for P V).  Every wait is bounded and ends in an error code, not a hang.
// The block's shared memory (112.6 KB, two blocks per SM) leaves no room for slack: the
// dynamic shared memory must start on a multiple of 1024 bytes, else the kernel reports
// error 6 and does nothing.
//
// Token t of sequence b: q row seq_start[b] + t, position seq_len[b] - n_b + t;
// it sees keys max(0, pos-window+1)..pos.  A query's result depends on its position
// and its place in the step, not on the batch.
//
// Compile with -DRI_HEAD_DIM=64 or 128.  Page size is 32.
// Formula: thanhauco/rust-inference src/attention.rs:4-8, 111-150.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <cuda.h>
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
#define TC_TMEM_COLS 256                // S: columns 0..63 and 64..127, O: columns 128..128+Dh-1
#define TC_O_COL (2 * TC_BN)
#define TC_LAZY 8.0f                    // log2 of how far a score may exceed the running maximum

// dynamic shared memory, 1024-byte aligned (swizzle atoms):
//   q | k0 | k1 | v0 | v1 | p      then the small things
struct TcTail {
    unsigned long long s_bar, pv_bar, p_bar, k_bar[2], v_bar[2];
    unsigned tmem_base;
    int dead;
    float rowmax[128];                // exchange between the two threads of a row
};
#define TC_OFF_Q 0
#define TC_OFF_K (TC_OFF_Q + TC_Q_BYTES)
#define TC_OFF_V (TC_OFF_K + 2 * TC_KV_BYTES)
#define TC_OFF_P (TC_OFF_V + 2 * TC_KV_BYTES)
#define TC_OFF_TAIL (TC_OFF_P + TC_P_BYTES)
#define TC_SMEM_BYTES (TC_OFF_TAIL + 576)

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
__device__ __forceinline__ void tmem_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one box (32 rows x 64 elements) of a pool's tensor map into shared memory: x in elements (0 or 64: a multiple
// of 16 bytes), y the row of the pool seen as a matrix [pages * KV * 32, Dh]
__device__ __forceinline__ void tc_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// block-wide barrier that also tells every thread whether any thread's predicate was set
__device__ __forceinline__ bool sync_or(bool pred) { return __syncthreads_or(pred ? 1 : 0) != 0; }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// The places in the pool of the two pages that hold keys 64 kb .. 64 kb + 63 (-1: the sequence has no such page)
struct TcPages {
    int id[2];
};
__device__ __forceinline__ TcPages tc_pages(const int* __restrict__ table, int kb, int len, int num_pages, int* err) {
    TcPages r;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int pg = kb * (TC_BN / TC_PAGE) + j;
        int id = -1;
        if (pg * TC_PAGE < len) {
            id = table[pg];
            if (id < 0 || id >= num_pages) {
                atomicExch(err, 4);
                id = -1;
            }
        }
        r.id[j] = id;
    }
    return r;
}
// starts the copies of a tile of 64 keys (or values): per page and per slab of 64 head elements one box
__device__ __forceinline__ void tc_load_tile(unsigned char* tile, const CUtensorMap* map, const TcPages& pg, int kvh, int KV,
                                             unsigned long long* bar) {
    const int boxes = ((pg.id[0] >= 0) + (pg.id[1] >= 0)) * TC_SLABS;
    tc_expect_tx(bar, (unsigned)boxes * (TC_PAGE * 128));       // also completes the phase when there is nothing to copy
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (pg.id[j] < 0) continue;
        const int row = (pg.id[j] * KV + kvh) * TC_PAGE;
#pragma unroll
        for (int sl = 0; sl < TC_SLABS; sl++)
            tc_tma_2d(tile + sl * TC_KV_SLAB + j * (TC_PAGE * 128), map, sl * 64, row, bar);
    }
}

// 256 threads: thread t works on query row t % 128; threads t and t + 128 share a row, the first
// takes keys 0..31 of a block and the first half of the output elements, the second the rest.
// Two blocks fit on an SM: while one waits for the tensor core the other does its softmax.
__global__ void __launch_bounds__(TC_THREADS, 2)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ page_table, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_len, int H, int KV, int mpps,
                            int num_pages, float scale_log2, int window, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem[];
    if (smem_u32(smem) & 1023u) {                                  // see the note on shared memory at the top
        if (threadIdx.x == 0) atomicExch(err, 6);
        return;
    }
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
    unsigned char* k_tiles = smem + TC_OFF_K;
    unsigned char* v_tiles = smem + TC_OFF_V;

    // ---- set-up: tensor memory, the barriers, the first copies ----------------------------------------
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tail.tmem_base)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_v) : "memory");
        unsigned long long* bars[6] = {&tail.s_bar, &tail.pv_bar, &tail.k_bar[0], &tail.k_bar[1], &tail.v_bar[0], &tail.v_bar[1]};
#pragma unroll
        for (int i = 0; i < 6; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(bars[i])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.p_bar)), "r"(TC_THREADS));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tail.dead = 0;
        const TcPages first = tc_pages(table, kb_lo, len, num_pages, err);
        tc_load_tile(k_tiles, &map_k, first, kvh, KV, &tail.k_bar[0]);
        tc_load_tile(v_tiles, &map_v, first, kvh, KV, &tail.v_bar[0]);
        if (kb_lo < kb_hi) {
            const TcPages second = tc_pages(table, kb_lo + 1, len, num_pages, err);
            tc_load_tile(k_tiles + TC_KV_BYTES, &map_k, second, kvh, KV, &tail.k_bar[1]);
        }
    }
    {
        const int r = tid >> 1;
        const bool ok = r < rows;
        copy_row_piece(smem + TC_OFF_Q, TC_Q_SLAB, r, (tid & 1) * (TC_DH / 16), TC_DH / 16,
                       q + ((size_t)(t_begin + r_base + (ok ? r : 0)) * H + h) * TC_DH, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tail.tmem_base;
    const unsigned tmem_row = tmem + ((unsigned)((warp & 3) * 32) << 16);      // this warp's 32 lanes
    const unsigned q_addr = smem_u32(smem + TC_OFF_Q), p_addr = smem_u32(smem + TC_OFF_P);
    constexpr unsigned IDESC_QK = instr_desc(TC_BM, TC_BN, 0);
    constexpr unsigned IDESC_PV = instr_desc(TC_BM, TC_DH, 1);
    constexpr int OW = TC_DH / 2;                                  // output elements per thread
    constexpr int SW = TC_BN / 2;                                  // scores per thread (32)

    // Four threads of four different warps share the side work, so that no warp falls far behind the others:
    // thread 0 issues Q K^T, thread 32 P V, thread 64 copies keys, thread 96 copies values.  The copying threads
    // look the pages up one block before they need them.
    const bool qk_thread = tid == 0, pv_thread = tid == 32, k_thread = tid == 64, v_thread = tid == 96;
    TcPages ahead;                                                 // k_thread: pages of block kb + 2; v_thread: of block kb + 1
    ahead.id[0] = ahead.id[1] = -1;
    if (k_thread && kb_lo + 1 < kb_hi) ahead = tc_pages(table, kb_lo + 2, len, num_pages, err);
    if (v_thread && kb_lo < kb_hi) ahead = tc_pages(table, kb_lo + 1, len, num_pages, err);

    // qk_thread: S[j & 1] = Q K^T for the j-th block of this tile, once its keys have arrived
    auto issue_qk = [&](int j) {
        if (!tc_mbar_wait(&tail.k_bar[j & 1], (unsigned)((j >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; }
        tc_fence_after();
        const unsigned k_addr = smem_u32(k_tiles + (j & 1) * TC_KV_BYTES);
#pragma unroll
        for (int i = 0; i < TC_DH / 16; i++) {
            unsigned qo = (unsigned)((i >> 2) * TC_Q_SLAB + (i & 3) * 32), ko = (unsigned)((i >> 2) * TC_KV_SLAB + (i & 3) * 32);
            umma_bf16(tmem + (j & 1) * TC_BN, smem_desc(q_addr + qo, 16, 1024), smem_desc(k_addr + ko, 16, 1024), IDESC_QK, i > 0);
        }
        umma_commit(&tail.s_bar);
    };
    if (qk_thread) issue_qk(0);

    float m = -FLT_MAX, l = 0.0f;                                  // m: in units of scaled log2 scores
    bool dead = false;
    int it = 0;                                                    // blocks done
    for (int kb = kb_lo; kb <= kb_hi; kb++, it++) {
        const int buf = it & 1;
        unsigned char* v_tile = v_tiles + buf * TC_KV_BYTES;
        // ---- S of this block is done (its key tile is free) ------------------------------------------------
        if (!tc_mbar_wait(&tail.s_bar, (unsigned)buf)) { atomicExch(err, 5); tail.dead = 1; }
        tc_fence_after();
        // the keys of the block after the next go into the tile that S of this block has just finished with
        if (k_thread && kb + 1 < kb_hi) {
            tc_load_tile(k_tiles + buf * TC_KV_BYTES, &map_k, ahead, kvh, KV, &tail.k_bar[buf]);
            if (kb + 2 < kb_hi) ahead = tc_pages(table, kb + 3, len, num_pages, err);
        }
        // ---- my 32 scores of the row: mask, maximum ------------------------------------------------------
        const int k0 = kb * TC_BN + half * SW;                     // my first key
        const bool edge = (kb * TC_BN + TC_BN - 1 > pos_first) || (window > 0 && kb * TC_BN < pos_last - window + 1);
        float s[SW];
        tmem_ld32(tmem_row + buf * TC_BN + half * SW, s);
        if (edge) {
#pragma unroll
            for (int i = 0; i < SW; i++) {
                int key = k0 + i;
                bool vis = key <= my_pos && (window <= 0 || key > my_pos - window);
                s[i] = vis ? s[i] : -FLT_MAX;
            }
        }
        float mx4[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};   // four chains instead of one of 32 steps
#pragma unroll
        for (int i = 0; i < SW; i++) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        mx = mx == -FLT_MAX ? -FLT_MAX : mx * scale_log2;          // scale > 0: the maximum of the scaled scores
        // every thread has read S; does any row have to raise its maximum?
        tc_fence_before();
        const bool raise = sync_or(mx > m + TC_LAZY || (m == -FLT_MAX && mx != -FLT_MAX));
        // a wait that ran out (this block's by any thread, thread 0's of the block before) is known to all here
        dead = tail.dead != 0;
        if (dead) break;
        // S of the next block goes into the other S buffer, which every thread has read by now.  It is started
        // only here, behind the block-wide barrier: every thread has then seen this block's phase of the S
        // barrier, so that barrier is never two phases ahead of a thread that waits on it by parity.
        if (qk_thread && kb < kb_hi) issue_qk(it + 1);
        // ---- P V of the block before is done: P, its value tile and the output are free -------------------
        if (it > 0) {
            if (!tc_mbar_wait(&tail.pv_bar, (unsigned)((it - 1) & 1))) { atomicExch(err, 5); tail.dead = 1; }
            tc_fence_after();
        }
        if (v_thread && kb < kb_hi) {
            tc_load_tile(v_tiles + (buf ^ 1) * TC_KV_BYTES, &map_v, ahead, kvh, KV, &tail.v_bar[buf ^ 1]);
            if (kb + 1 < kb_hi) ahead = tc_pages(table, kb + 2, len, num_pages, err);
        }
        if (raise) {
            // the row's two threads agree on its maximum: the second tells the first, the first answers
            if (half) tail.rowmax[row] = mx;
            __syncthreads();
            float m_new = 0.0f;
            if (!half) {
                m_new = fmaxf(m, fmaxf(mx, tail.rowmax[row]));
                tail.rowmax[row] = m_new;
            }
            __syncthreads();
            if (half) m_new = tail.rowmax[row];
            const float corr = m_new == m ? 1.0f : ((m == -FLT_MAX) ? 0.0f : ex2_approx(m - m_new));
            m = m_new;
            l *= corr;
            // the output so far, in tensor memory: the loads and stores are the whole warp's, so all its rows go along
            if (it > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int c = 0; c < OW / 32; c++) {
                    float ob[32];
                    tmem_ld32(tmem_row + TC_O_COL + half * OW + c * 32, ob);
#pragma unroll
                    for (int i = 0; i < 32; i++) ob[i] *= corr;
                    tmem_st32(tmem_row + TC_O_COL + half * OW + c * 32, ob);
                }
                tmem_st_wait();
            }
        }
        // ---- P = exp2(S * scale - m) as bfloat16 into the operand layout; sum --------------------------
        {
            const float neg_m = (m == -FLT_MAX) ? 0.0f : -m;
            unsigned char* p_row = smem + TC_OFF_P + row * 128;
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < SW / 8; c++) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    float x = s[c * 8 + e];
                    p[e] = (edge && x == -FLT_MAX) ? 0.0f : ex2_approx(fmaf(x, scale_log2, neg_m));
                    l4[e & 3] += p[e];
                }
                const int chunk = half * (SW / 8) + c;             // 16-byte chunk of the 64-key row
                *(uint4*)(p_row + ((chunk ^ (row & 7)) << 4)) =
                    make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        }
        // the values of this block have arrived (asked for a whole block ago)
        if (!tc_mbar_wait(&tail.v_bar[buf], (unsigned)((it >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; }
        if (kb * TC_BN + TC_BN > len) {
            // rows past the sequence's end hold whatever the pool holds there (or what the tile held before):
            // zero them, a weight of zero times not-a-number would still be not-a-number
            const int r = tid >> 2, first_bad = len - kb * TC_BN;
            if (r >= first_bad) {
#pragma unroll
                for (int sl = 0; sl < TC_SLABS; sl++)
#pragma unroll
                    for (int c = 0; c < 2; c++)
                        *(uint4*)(v_tile + sl * TC_KV_SLAB + r * 128 + (((tid & 3) * 2 + c) << 4)) = make_uint4(0, 0, 0, 0);
            }
        }
        // my part of P (and of the value tile) is written: tell the thread that issues P V and go on; nobody
        // waits here, the next block-wide barrier is the vote on the maximum of the next block
        fence_async_smem();
        tc_fence_before();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.p_bar)) : "memory");
        // ---- O += P V --------------------------------------------------------------------------------------
        if (pv_thread) {
            if (!tc_mbar_wait(&tail.p_bar, (unsigned)buf)) { atomicExch(err, 5); tail.dead = 1; }
            tc_fence_after();
            const unsigned v_addr = smem_u32(v_tile);
#pragma unroll
            for (int j = 0; j < TC_BN / 16; j++) {
                umma_bf16(tmem + TC_O_COL, smem_desc(p_addr + j * 32, 16, 1024),
                          smem_desc(v_addr + j * 16 * 128, TC_KV_SLAB, 1024), IDESC_PV, (it > 0 || j > 0) ? 1u : 0u);
            }
            umma_commit(&tail.pv_bar);
        }
    }
    // ---- the last product is done: out = O / l (l: both halves of the row) --------------------------------
    if (!dead && it > 0 && !tc_mbar_wait(&tail.pv_bar, (unsigned)((it - 1) & 1))) { atomicExch(err, 5); tail.dead = 1; }
    tc_fence_after();
    __syncthreads();
    dead = tail.dead != 0;
    if (half) tail.rowmax[row] = l;
    __syncthreads();
    if (!half) {
        l += tail.rowmax[row];
        tail.rowmax[row] = l;
    }
    __syncthreads();
    if (half) l = tail.rowmax[row];
    {
        // every lane of a warp takes part in the loads from tensor memory, whether its row is one of the tile's or not
        const bool mine = row < rows && !dead;
        const float inv = 1.0f / l;
        bf16* dst = out + ((size_t)(t_begin + r_base + (mine ? row : 0)) * H + h) * TC_DH + half * OW;
#pragma unroll
        for (int c = 0; c < OW / 32; c++) {
            float o[32];
            tmem_ld32(tmem_row + TC_O_COL + half * OW + c * 32, o);
            if (mine) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    w.x = pack_bf16(o[i] * inv, o[i + 1] * inv);
                    w.y = pack_bf16(o[i + 2] * inv, o[i + 3] * inv);
                    w.z = pack_bf16(o[i + 4] * inv, o[i + 5] * inv);
                    w.w = pack_bf16(o[i + 6] * inv, o[i + 7] * inv);
                    *(uint4*)(dst + c * 32 + i) = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// a pool [pages, KV, 32, Dh] of bfloat16 as a matrix [pages * KV * 32, Dh], copied in boxes of 32 rows x 64 elements
typedef CUresult (*tc_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int tc_pool_tensor_map(CUtensorMap* map, const void* pool, long long rows) {
    static tc_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !fn)
            RI_FAIL(-1, "attention_prefill_tc: the driver has no cuTensorMapEncodeTiled");
        encode = (tc_encode_tiled_fn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)TC_DH, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)TC_DH * 2};
    cuuint32_t box[2] = {64, TC_PAGE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RI_FAIL(-1, "attention_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
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
    RI_REQUIRE((long long)num_pages * KV * TC_PAGE < (1ll << 31), "attention_prefill_tc: a pool of %d pages", num_pages);
    CUtensorMap map_k, map_v;
    int rc = tc_pool_tensor_map(&map_k, k_pool, (long long)num_pages * KV * TC_PAGE);
    if (rc) return rc;
    rc = tc_pool_tensor_map(&map_v, v_pool, (long long)num_pages * KV * TC_PAGE);
    if (rc) return rc;
    attention_prefill_tc_kernel<<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(
        (const bf16*)q, map_k, map_v, (bf16*)out, page_table, seq_slot, seq_start, seq_len,
        H, KV, mpps, num_pages, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_prefill_tc");
    return 0;
}
