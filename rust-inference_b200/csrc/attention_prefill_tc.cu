// Prefill attention on the 5th-generation tensor cores (tcgen05) for bfloat16, head size 64 or 128.
//
// One block of 352 threads per SM.  A work item is two query tiles of 128 consecutive new tokens of one sequence
// and one head; the items are ordered (rows: the late ones, which see the most keys, first; sequence; head), and
// block c of G blocks takes item k G + c in its round k when k is even, item k G + G - 1 - c when k is odd, one
// after the other, so the block that drew the heaviest item of a round draws the lightest of the next.  The
// block's tensor memory, barriers and rings are set up once; buffers and barriers keep taking their turns across
// items (counted in blocks of keys), so the keys, values and queries of the next item are copied while the last
// blocks of the item at hand are worked on.
// Warps 0..3 own tile 0 (thread = row), warps 4..7 tile 1; one lane of warp 8 issues the tcgen05.mma of tile 0,
// one lane of warp 9 those of tile 1, one lane of warp 10 starts every TMA copy.  For every block of 64 keys
//   1. the keys and the values (two pages each) come from the paged cache by TMA tensor copies
//      (cp.async.bulk.tensor.2d, 128-byte swizzle: the layout the tensor core reads) into a ring of
//      TC_STAGES tiles, loaded once for both query tiles; a tile is refilled when a tcgen05.commit
//      behind its last reader has signalled k_empty / v_empty.  The first tile's rows end 128 positions
//      before the item's: it leaves out the blocks of keys past them (its issuing lane hands those stages
//      back as soon as they have landed).  The queries of an item come the same way (boxes of 128 rows);
//   2. S_t = Q_t K^T (M 128 queries, N 64 keys) goes into tensor memory.  S_t has two buffers, and the
//      product of block j + 2 is issued as soon as the tile's threads hold S_t of block j in their
//      registers: a message from the tensor core (tcgen05.commit -> mbarrier) takes longer to arrive
//      than a block's softmax, so the answer must be on its way two blocks ahead;
//   3. a thread reads its row of S_t (tcgen05.ld, 64 scores), and writes P_t = exp2(S_t * scale - m)
//      as bfloat16 into shared memory in the operand layout (two P buffers per tile, so that nobody
//      waits for the product that read the last one).  m is the row's running maximum, raised only
//      when some row of the warp (of the item's own rows) meets a score more than 2^8 above its own
//      (then the warp's rows take their true maxima and rescale their output in tensor memory with
//      tcgen05.ld / tcgen05.st); weights up to 2^8 are exact in float32 and as good as any in bfloat16.
//      No thread exchanges anything with another, and there is no block-wide barrier in the loop;
//   4. O_t += P_t V: tcgen05.mma with V read as an MN-major operand straight from the [key][element]
//      tile, accumulated in tensor memory over all blocks of the item.
// Everything is handed over through mbarriers:
//   s_full[t][b]  (tcgen05.commit)  S_t of a block is in tensor memory, in S buffer b
//   s_read[t][b]  (4 arrivals, one per warp)  the tile's threads hold it in registers: the buffer may be overwritten
//   p_ready[t][b] (4 arrivals)      the tile's threads have written P_t into P buffer b
//   pv_done[t][b] (tcgen05.commit)  O_t holds the block whose P_t was in buffer b: that buffer and O_t may be touched
//   k_full[s], v_full[s] (TMA)      a key / value tile has landed in stage s
//   k_empty[s], v_empty[s] (both issuing lanes: tcgen05.commit, or a plain arrival for a block left out)  stage s is free
//   q_full[t]  (TMA)                the item's queries of tile t have landed
//   q_empty[t] (tcgen05.commit)     the item's last product Q_t K^T is done: the next item's queries may come
//   o_free[t]  (4 arrivals)         the tile's threads hold the item's output: the next item's first product may overwrite O_t
// Every barrier belongs to one buffer; a barrier waited on by parity is never two phases ahead of a
// waiter, because its next phase needs something that waiter does after the wait.  Every wait is
// bounded by time and ends in an error code (5), not a hang: the thread that gave up says so in shared memory,
// the copying lane starts no further copy, the issuing lanes no further product, the rows' threads run through
// their blocks without waiting, and the block ends as usual (barrier, tensor memory given back) with a wrong
// result for its items.  -DTC_TEST_DROP_COPY_LEN=<n> (tests only; nothing in an ordinary build) leaves out one copy
// in sequences of exactly n keys, so that this path can be run.
// Tensor memory (512 columns): S_t buffer b at column (2 t + b) * 64, O_0 and O_1 at 256 and 384.
// Shared memory (224 KB at head size 128) leaves no room for slack: the dynamic shared memory must
// start on a multiple of 1024 bytes (the swizzle's period), else the kernel reports error 6.
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
#define TC_BM 128                       // queries per tile
#define TC_BN 64                        // keys per step
#define TC_SLABS (TC_DH / 64)           // 64-element (128-byte) slabs along the head
#define TC_Q_SLAB (TC_BM * 128)         // a slab of the query tile: 128 rows of 128 bytes
#define TC_KV_SLAB (TC_BN * 128)        // a slab of a key or value tile: 64 rows of 128 bytes
#define TC_Q_BYTES (TC_SLABS * TC_Q_SLAB)
#define TC_KV_BYTES (TC_SLABS * TC_KV_SLAB)
#define TC_P_BYTES (TC_BM * 128)        // P [128 x 64 keys]: one slab
#define TC_LAZY 8.0f                    // log2 of how far a score may exceed the running maximum

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
// the same load without the wait: the caller issues several and then tmem_ld_wait() once
__device__ __forceinline__ void tmem_ld32_start(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
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
// sm_100 arithmetic that halves the instruction count of the softmax: a maximum of three, and float32 pairs
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long r, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long fadd2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// The places in the pool of the two pages that hold keys 64 kb .. 64 kb + 63 (-1: the sequence has no such page,
// or the page lies wholly before key_lo, the first key any query of the block sees: a window group may have
// given such a page back already, so it is not looked up)
struct TcPages {
    int id[2];
};
__device__ __forceinline__ TcPages tc_pages(const int* __restrict__ table, int kb, int len, int key_lo, int num_pages, int* err) {
    TcPages r;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int pg = kb * (TC_BN / TC_PAGE) + j;
        int id = -1;
        if (pg * TC_PAGE < len && (pg + 1) * TC_PAGE > key_lo) {
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
// (`drop`: tests only, see TC_TEST_DROP_COPY_LEN: the first box is counted and not copied)
__device__ __forceinline__ void tc_load_tile(unsigned char* tile, const CUtensorMap* map, const TcPages& pg, int kvh, int KV,
                                             unsigned long long* bar, bool drop = false) {
    const int boxes = ((pg.id[0] >= 0) + (pg.id[1] >= 0)) * TC_SLABS;
    tc_expect_tx(bar, (unsigned)boxes * (TC_PAGE * 128));       // also completes the phase when there is nothing to copy
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (pg.id[j] < 0) continue;
        const int row = (pg.id[j] * KV + kvh) * TC_PAGE;
#pragma unroll
        for (int sl = 0; sl < TC_SLABS; sl++) {
            if (drop && j == 0 && sl == 0) continue;
            tc_tma_2d(tile + sl * TC_KV_SLAB + j * (TC_PAGE * 128), map, sl * 64, row, bar);
        }
    }
}

#define TC_TILES 2
#define TC_THREADS (32 * (4 * TC_TILES + TC_TILES + 1))
#define TC_Q_TILE_BYTES (TC_SLABS * TC_Q_SLAB)
#define TC_OFF_Q 0
#ifndef TC_STAGES
#define TC_STAGES (TC_DH == 128 ? 3 : 6)     // key and value tiles in flight or in use
#endif
#define TC_OFF_K (TC_OFF_Q + TC_TILES * TC_Q_TILE_BYTES)
#define TC_OFF_V (TC_OFF_K + TC_STAGES * TC_KV_BYTES)
#define TC_OFF_P (TC_OFF_V + TC_STAGES * TC_KV_BYTES)
#define TC_OFF_TAIL (TC_OFF_P + TC_TILES * 2 * TC_P_BYTES)      // two P buffers per tile
struct TcTail {
    unsigned long long s_full[2][2], s_read[2][2], p_ready[2][2], pv_done[2][2], k_full[TC_STAGES], v_full[TC_STAGES], k_empty[TC_STAGES], v_empty[TC_STAGES];
    unsigned long long q_full[2], q_empty[2], o_free[2];
    unsigned tmem_base;
    volatile int dead;
};
#define TC_SMEM_BYTES (TC_OFF_TAIL + 448)
#define TC_TMEM_COLS 512
#define TC_S_COL(t, b) (((t) * 2 + (b)) * TC_BN)       // two S buffers per tile
#define TC_O_COL(t) (4 * TC_BN + (t) * 128)

// One work item: 256 query rows (two tiles) of one sequence and one head.
struct TcItem {
    int h, kvh;
    int t_first;                 // the item's first row in q and out
    int len, rows, n_tiles;
    int pos_first, pos_last, key_lo, kb_lo;
    int n_blocks;                // blocks of 64 keys that the item's last row reaches
    int n_blocks_0;              // ... that the first tile's last row reaches (128 positions earlier)
    const int* table;
};
struct TcWork {
    const int* page_table;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_len;
    int seqs, H, KV, mpps, groups_max, n_items, window;
};
// The items in the order (group of rows: late ones, which see the most keys, first; sequence; head).  Block c of G
// takes item k G + c in its round k when k is even and item k G + G - 1 - c when k is odd, so the block that drew
// the heaviest item of one round draws the lightest of the next.  False: no item for this block in this round.
__device__ __forceinline__ bool tc_item(const TcWork& w, int k, TcItem& it) {
    const int G = (int)gridDim.x;
    const int id = (k & 1) ? k * G + G - 1 - (int)blockIdx.x : k * G + (int)blockIdx.x;
    if (id >= w.n_items) return false;
    const int per = w.seqs * w.H;
    const int g_rev = id / per, rem = id - g_rev * per;
    const int b = rem / w.H;
    it.h = rem - b * w.H;
    const int group = w.groups_max - 1 - g_rev;
    constexpr int ROWS = TC_TILES * TC_BM;
    const int t_begin = w.seq_start[b], n_new = w.seq_start[b + 1] - t_begin;
    if (group * ROWS >= n_new) return false;
    it.len = w.seq_len[b];
    const int r_base = group * ROWS;
    it.t_first = t_begin + r_base;
    it.rows = min(ROWS, n_new - r_base);
    it.n_tiles = it.rows > TC_BM ? 2 : 1;
    it.pos_first = it.len - n_new + r_base;
    it.pos_last = it.pos_first + it.rows - 1;
    it.key_lo = (w.window > 0 && it.pos_first - w.window + 1 > 0) ? it.pos_first - w.window + 1 : 0;
    it.kb_lo = it.key_lo / TC_BN;
    it.n_blocks = it.pos_last / TC_BN - it.kb_lo + 1;
    it.n_blocks_0 = it.n_tiles > 1 ? min(it.n_blocks, (it.pos_first + TC_BM - 1) / TC_BN - it.kb_lo + 1) : it.n_blocks;
    it.kvh = it.h / (w.H / w.KV);
    it.table = w.page_table + (size_t)w.seq_slot[b] * w.mpps;
    return true;
}
// blocks of keys that tile t of the item works on (the first tile leaves out those past its rows; a second tile
// without rows has none)
__device__ __forceinline__ int tc_tile_blocks(const TcItem& it, int t) {
    return t < it.n_tiles ? (t == 0 ? it.n_blocks_0 : it.n_blocks) : 0;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const TcWork work,
                             int num_pages, float scale_log2, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(err, 6);
        return;
    }
    TcTail& tail = *reinterpret_cast<TcTail*>(smem + TC_OFF_TAIL);
    const int H = work.H, KV = work.KV, window = work.window;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool mma_warp = warp >= 4 * TC_TILES && warp < 5 * TC_TILES, tma_warp = warp == 5 * TC_TILES;
    unsigned char* k_tiles = smem + TC_OFF_K;
    unsigned char* v_tiles = smem + TC_OFF_V;
    const int rounds = (work.n_items + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tail.tmem_base)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tma_warp && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_v) : "memory");
#pragma unroll
        for (int i = 0; i < 2; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.s_full[i][0])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.s_full[i][1])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.pv_done[i][0])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.pv_done[i][1])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.q_full[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.q_empty[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.o_free[i])), "r"(TC_BM / 32));
#pragma unroll
            for (int b2 = 0; b2 < 2; b2++) {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.p_ready[i][b2])), "r"(TC_BM / 32));
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.s_read[i][b2])), "r"(TC_BM / 32));
            }
        }
#pragma unroll
        for (int i = 0; i < TC_STAGES; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.k_full[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&tail.v_full[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.k_empty[i])), "r"(TC_TILES));    // both issuing lanes, always
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&tail.v_empty[i])), "r"(TC_TILES));
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        tail.dead = 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tail.tmem_base;
    constexpr unsigned IDESC_QK = instr_desc(TC_BM, TC_BN, 0);
    constexpr unsigned IDESC_PV = instr_desc(TC_BM, TC_DH, 1);

    int k_started = 0, v_started = 0, q_started = 0;     // copies that the copying lane has started: blocks of keys, of values, items' queries
    if (tma_warp) {
        if (lane == 0) {
            // ---- the copying lane: queries, keys and values of one item after the other, as buffers come free ----
            // After a wait has run out (here or anywhere in the block) this lane starts no further copy: the barrier of
            // a copy arrives once per phase, and behind a wait that was given up nothing says that the phase before has
            // ended (a second arrival in one phase is one more than the barrier was set up for).
            bool dead = false;
            auto wait = [&](unsigned long long* bar, unsigned parity) {
                if (!dead && !tc_mbar_wait(bar, parity)) { atomicExch(err, 5); tail.dead = 1; dead = true; }
                dead = dead || tail.dead != 0;
            };
            int kv_base = 0, n_it = 0;            // blocks of keys and items before the one at hand
            for (int k = 0; k < rounds && !dead; k++) {
                TcItem it;
                if (!tc_item(work, k, it)) continue;
                // both query tiles, once the products of the item before have read theirs (rows past the sequence's
                // belong to the next one or read as zeros past the last token: they are computed and never stored)
                auto load_q = [&]() {
#pragma unroll
                    for (int t = 0; t < TC_TILES; t++) {
                        if (n_it > 0) wait(&tail.q_empty[t], (unsigned)((n_it - 1) & 1));
                        if (dead) return;
                        tc_expect_tx(&tail.q_full[t], TC_Q_TILE_BYTES);
#pragma unroll
                        for (int sl = 0; sl < TC_SLABS; sl++)
                            tc_tma_2d(smem + TC_OFF_Q + t * TC_Q_TILE_BYTES + sl * TC_Q_SLAB, &map_q, it.h * TC_DH + sl * 64,
                                      it.t_first + t * TC_BM, &tail.q_full[t]);
                        q_started = n_it * TC_TILES + t + 1;
                    }
                };
                if (n_it == 0) load_q();
                // the queries of a later item wait for the last product Q K^T of the item before, which is also what
                // frees the key stage of that item's last block: they go in behind the keys that take that stage
                const int q_after = min(TC_STAGES - 1, it.n_blocks - 1);
                for (int j = 0; j < it.n_blocks && !dead; j++) {
                    const int gj = kv_base + j, buf = gj % TC_STAGES;
                    const unsigned parity = (unsigned)((gj / TC_STAGES - 1) & 1);
                    const TcPages pg = tc_pages(it.table, it.kb_lo + j, it.len, it.key_lo, num_pages, err);   // under the wait below
                    if (gj >= TC_STAGES) wait(&tail.k_empty[buf], parity);
                    if (dead) break;
#ifdef TC_TEST_DROP_COPY_LEN
                    // tests only: in a sequence of exactly this many keys the first copy of an item's first block of keys
                    // is left out, so that its barrier never completes and the waits behind it run out
                    const bool drop = it.len == TC_TEST_DROP_COPY_LEN && j == 0;
#else
                    const bool drop = false;
#endif
                    tc_load_tile(k_tiles + buf * TC_KV_BYTES, &map_k, pg, it.kvh, KV, &tail.k_full[buf], drop);
                    k_started = gj + 1;
                    if (n_it > 0 && j == q_after) load_q();
                    if (gj >= TC_STAGES) wait(&tail.v_empty[buf], parity);
                    if (dead) break;
                    tc_load_tile(v_tiles + buf * TC_KV_BYTES, &map_v, pg, it.kvh, KV, &tail.v_full[buf]);
                    v_started = gj + 1;
                }
                kv_base += it.n_blocks;
                n_it++;
            }
        }
    } else if (mma_warp) {
        const int t = warp - 4 * TC_TILES;                          // one issuing lane per query tile
        if (lane == 0) {
            // the operand descriptors, made once (a descriptor holds the address in units of 16 bytes)
            const unsigned long long q_base = smem_desc(smem_u32(smem + TC_OFF_Q + t * TC_Q_TILE_BYTES), 16, 1024);
            const unsigned long long k_base = smem_desc(smem_u32(k_tiles), 16, 1024);
            const unsigned long long p_base = smem_desc(smem_u32(smem + TC_OFF_P + t * 2 * TC_P_BYTES), 16, 1024);
            const unsigned long long v_base = smem_desc(smem_u32(v_tiles), TC_KV_SLAB, 1024);
            unsigned long long qd[TC_DH / 16], kd[TC_DH / 16], pd[TC_BN / 16], vd[TC_BN / 16];      // kd, vd: stage 0
#pragma unroll
            for (int i = 0; i < TC_DH / 16; i++) {
                qd[i] = q_base + (unsigned)(((i >> 2) * TC_Q_SLAB + (i & 3) * 32) >> 4);
                kd[i] = k_base + (unsigned)(((i >> 2) * TC_KV_SLAB + (i & 3) * 32) >> 4);
            }
#pragma unroll
            for (int i = 0; i < TC_BN / 16; i++) {
                pd[i] = p_base + (unsigned)((i * 32) >> 4);
                vd[i] = v_base + (unsigned)((i * 16 * 128) >> 4);
            }
            const unsigned o_col = tmem + TC_O_COL(t);
            bool dead = false;
            auto wait = [&](unsigned long long* bar, unsigned parity) {
                if (!dead && !tc_mbar_wait(bar, parity)) { atomicExch(err, 5); tail.dead = 1; dead = true; }
            };
            // c: blocks of keys this tile has worked on before the item at hand (S, P and their barriers take turns
            // by it); kv_base: blocks of keys of the items before (the stages take turns by it); n_it, n_mine: items
            // before, and those of them in which this tile had rows
            int c = 0, kv_base = 0, n_it = 0, n_mine = 0;
            for (int k = 0; k < rounds && !dead; k++) {
                TcItem it;
                if (!tc_item(work, k, it)) continue;
                const int my_blocks = tc_tile_blocks(it, t);
                wait(&tail.q_full[t], (unsigned)(n_it & 1));
                // S_t of the item's block jb = Q_t K^T into S buffer (c + jb) & 1, once the threads hold what that buffer
                // held two blocks earlier (of this item or of the one before) and the keys have landed
                auto issue_qk = [&](int jb) {
                    const int idx = c + jb, gj = kv_base + jb, st = gj % TC_STAGES;
                    if (idx >= 2) wait(&tail.s_read[t][idx & 1], (unsigned)(((idx - 2) >> 1) & 1));
                    wait(&tail.k_full[st], (unsigned)((gj / TC_STAGES) & 1));
                    tc_fence_after();
                    const unsigned long long off = (unsigned long long)(st * (TC_KV_BYTES >> 4));
                    const unsigned s_col = tmem + TC_S_COL(t, idx & 1);
#pragma unroll
                    for (int i = 0; i < TC_DH / 16; i++) umma_bf16(s_col, qd[i], kd[i] + off, IDESC_QK, i > 0);
                    umma_commit(&tail.s_full[t][idx & 1]);
                    umma_commit(&tail.k_empty[st]);                          // this tile is done with the keys of block jb
                    if (jb + 1 == my_blocks) umma_commit(&tail.q_empty[t]);  // ... and with the item's queries
                };
                if (my_blocks == 0) umma_commit(&tail.q_empty[t]);
                if (my_blocks > 0) issue_qk(0);
                if (my_blocks > 1) issue_qk(1);
                for (int j = 0; j < my_blocks && !dead; j++) {
                    const int idx = c + j, gj = kv_base + j, st = gj % TC_STAGES;
                    // as soon as the tile's threads hold S_t of block j in their registers, its buffer takes S_t of block
                    // j + 2: the tensor core's answer has two blocks' time to come back
                    if (j + 2 < my_blocks) issue_qk(j + 2);
                    // P_t of block j is written: O_t += P_t V
                    wait(&tail.p_ready[t][idx & 1], (unsigned)((idx >> 1) & 1));
                    wait(&tail.v_full[st], (unsigned)((gj / TC_STAGES) & 1));
                    // the first product of an item overwrites O_t: the threads must have read the item before out of it
                    if (j == 0 && n_mine > 0) wait(&tail.o_free[t], (unsigned)((n_mine - 1) & 1));
                    tc_fence_after();
                    {
                        const unsigned long long off = (unsigned long long)(st * (TC_KV_BYTES >> 4));
                        const unsigned long long poff = (unsigned long long)((idx & 1) * (TC_P_BYTES >> 4));
#pragma unroll
                        for (int i = 0; i < TC_BN / 16; i++) umma_bf16(o_col, pd[i] + poff, vd[i] + off, IDESC_PV, (j > 0 || i > 0) ? 1u : 0u);
                    }
                    umma_commit(&tail.pv_done[t][idx & 1]);
                    umma_commit(&tail.v_empty[st]);                           // this tile is done with the values of block j
                }
                // The blocks of keys that this tile leaves out: both tiles hand a stage back, so it does that once the
                // block has landed.  (Not earlier: before that the stage's barrier may still be in the phase of the block
                // that was there before, which the other tile may not have read yet.)
                for (int j = my_blocks; j < it.n_blocks && !dead; j++) {
                    const int gj = kv_base + j, st = gj % TC_STAGES;
                    wait(&tail.k_full[st], (unsigned)((gj / TC_STAGES) & 1));
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.k_empty[st])) : "memory");
                    wait(&tail.v_full[st], (unsigned)((gj / TC_STAGES) & 1));
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.v_empty[st])) : "memory");
                }
                c += my_blocks;
                kv_base += it.n_blocks;
                n_it++;
                n_mine += my_blocks > 0 ? 1 : 0;
            }
        }
    } else {
        // ---- a query row of tile t ------------------------------------------------------------------------------
        const int t = warp >> 2, row = tid & (TC_BM - 1);
        const unsigned tmem_row = tmem + ((unsigned)((warp & 3) * 32) << 16);
        unsigned char* p_rows = smem + TC_OFF_P + t * 2 * TC_P_BYTES + row * 128;
        bool dead = false;
        int c = 0, kv_base = 0;
        for (int k = 0; k < rounds; k++) {
            TcItem it;
            if (!tc_item(work, k, it)) continue;
            const int my_blocks = tc_tile_blocks(it, t);
            if (my_blocks == 0) {
                kv_base += it.n_blocks;
                continue;
            }
            const int len = it.len, kb_lo = it.kb_lo, key_lo = it.key_lo, pos_first = it.pos_first, pos_last = it.pos_last;
            const int my_pos = pos_first + t * TC_BM + row;
            const int tile_first = pos_first + t * TC_BM, tile_last = min(tile_first + TC_BM - 1, pos_last);
            const bool real_row = t * TC_BM + row < it.rows;
            float m = -FLT_MAX, l = 0.0f;
            for (int j = 0; j < my_blocks; j++) {
                const int kb = kb_lo + j, idx = c + j, gj = kv_base + j;
                if (!dead && !tc_mbar_wait(&tail.s_full[t][idx & 1], (unsigned)((idx >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; }
                dead = dead || tail.dead != 0;
                tc_fence_after();
                float s[TC_BN];
                {
                    unsigned a[32], c2[32];
                    tmem_ld32_start(tmem_row + TC_S_COL(t, idx & 1), a);
                    tmem_ld32_start(tmem_row + TC_S_COL(t, idx & 1) + 32, c2);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        s[i] = __uint_as_float(a[i]);
                        s[32 + i] = __uint_as_float(c2[i]);
                    }
                }
                // S_t is in my registers: the next S_t may be written
                tc_fence_before();
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.s_read[t][idx & 1])) : "memory");
                // a block of keys needs the mask if some query of this tile does not see all of it
                const bool edge = (kb * TC_BN + TC_BN - 1 > tile_first) || (window > 0 && kb * TC_BN < tile_last - window + 1);
                if (edge) {
#pragma unroll
                    for (int i = 0; i < TC_BN; i++) {
                        int key = kb * TC_BN + i;
                        bool vis = key <= my_pos && (window <= 0 || key > my_pos - window);
                        s[i] = vis ? s[i] : -FLT_MAX;
                    }
                }
                float mx4[4];                                         // four chains of three-way maxima
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) mx4[q4] = max3(s[q4 * 16], s[q4 * 16 + 1], s[q4 * 16 + 2]);
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {
#pragma unroll
                    for (int i = 3; i < 15; i += 2) mx4[q4] = max3(mx4[q4], s[q4 * 16 + i], s[q4 * 16 + i + 1]);
                    mx4[q4] = fmaxf(mx4[q4], s[q4 * 16 + 15]);
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                mx = mx == -FLT_MAX ? -FLT_MAX : mx * scale_log2;      // scale > 0
                unsigned char* p_row = p_rows + (idx & 1) * TC_P_BYTES;     // P_t has two buffers that take turns
                // (a row past the item's rows holds another sequence's query, or zeros: it has no say, so that a
                // sequence's bits do not depend on what stands behind it in the batch)
                const bool raise = real_row && (mx > m + TC_LAZY || (m == -FLT_MAX && mx != -FLT_MAX));
                if (__any_sync(0xffffffffu, raise)) {
                    // some row of this warp moves its maximum far: every row of the warp takes its true maximum
                    const float m_new = fmaxf(m, mx);
                    const float corr = m_new == m ? 1.0f : ((m == -FLT_MAX) ? 0.0f : ex2_approx(m - m_new));
                    m = m_new;
                    l *= corr;
                    if (j > 0) {
                        // the output is rescaled in tensor memory: P V of the block before must be done
                        if (!dead && !tc_mbar_wait(&tail.pv_done[t][(idx - 1) & 1], (unsigned)(((idx - 1) >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; dead = true; }
                        tc_fence_after();
#pragma unroll
                        for (int cc = 0; cc < TC_DH / 32; cc++) {
                            float ob[32];
                            tmem_ld32(tmem_row + TC_O_COL(t) + cc * 32, ob);
#pragma unroll
                            for (int i = 0; i < 32; i++) ob[i] *= corr;
                            tmem_st32(tmem_row + TC_O_COL(t) + cc * 32, ob);
                        }
                        tmem_st_wait();
                    }
                }
                // this P buffer was read by P V of the block before the last (of this item or the one before): long done, as a rule
                if (idx > 1) {
                    if (!dead && !tc_mbar_wait(&tail.pv_done[t][idx & 1], (unsigned)(((idx - 2) >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; dead = true; }
                }
                const float neg_m = (m == -FLT_MAX) ? 0.0f : -m;
                {
                    // pairs of float32 for the scaling and the sum.  A masked score is -FLT_MAX: times the (positive)
                    // scale and less any maximum it stays below every exponent that gives more than zero
                    const unsigned long long sc2 = pack2(scale_log2, scale_log2), nm2 = pack2(neg_m, neg_m);
                    unsigned long long l2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
#pragma unroll
                    for (int cc = 0; cc < TC_BN / 8; cc++) {
                        unsigned w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float x0, x1;
                            unpack2(ffma2(pack2(s[cc * 8 + 2 * e], s[cc * 8 + 2 * e + 1]), sc2, nm2), x0, x1);
                            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                            l2[e & 1] = fadd2(l2[e & 1], pack2(p0, p1));
                            w[e] = pack_bf16(p0, p1);
                        }
                        *(uint4*)(p_row + ((cc ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    float a0, a1, b0, b1;
                    unpack2(l2[0], a0, a1);
                    unpack2(l2[1], b0, b1);
                    l += (a0 + a1) + (b0 + b1);
                }
                const int st = gj % TC_STAGES;
                const unsigned st_parity = (unsigned)((gj / TC_STAGES) & 1);
                if (kb * TC_BN + TC_BN > len) {
                    // value rows past the sequence's end may hold anything: each tile's threads zero them before they say
                    // that P is written, so before their own tile's product (the tile has landed: the control lane waits
                    // for it before the product, but these writes must come before that too)
                    if (!dead && !tc_mbar_wait(&tail.v_full[st], st_parity)) { atomicExch(err, 5); tail.dead = 1; dead = true; }
                    unsigned char* v_tile = v_tiles + st * TC_KV_BYTES;
                    const int first_bad = len - kb * TC_BN;
                    for (int r = first_bad + (row >> 3); r < TC_BN; r += TC_BM / 8)
#pragma unroll
                        for (int sl = 0; sl < TC_SLABS; sl++)
                            *(uint4*)(v_tile + sl * TC_KV_SLAB + r * 128 + ((row & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                if (kb * TC_BN < key_lo) {
                    // value rows before the first key that any query of the item sees: their page may not have been
                    // copied at all (given back by a window group), so the stage may hold anything there, and P = 0
                    // times a NaN is a NaN: zeroed as above
                    if (!dead && !tc_mbar_wait(&tail.v_full[st], st_parity)) { atomicExch(err, 5); tail.dead = 1; dead = true; }
                    unsigned char* v_tile = v_tiles + st * TC_KV_BYTES;
                    const int head_bad = min(TC_BN, key_lo - kb * TC_BN);
                    for (int r = row >> 3; r < head_bad; r += TC_BM / 8)
#pragma unroll
                        for (int sl = 0; sl < TC_SLABS; sl++)
                            *(uint4*)(v_tile + sl * TC_KV_SLAB + r * 128 + ((row & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
                tc_fence_before();
                __syncwarp();                                            // one arrival per warp
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.p_ready[t][idx & 1])) : "memory");
            }
            // ---- out = O / l ----------------------------------------------------------------------------------------
            const int last = c + my_blocks - 1;
            if (!dead && !tc_mbar_wait(&tail.pv_done[t][last & 1], (unsigned)((last >> 1) & 1))) { atomicExch(err, 5); tail.dead = 1; dead = true; }
            tc_fence_after();
            const bool mine = real_row && !dead;
            const float inv = 1.0f / l;
            bf16* dst = out + ((size_t)(it.t_first + (mine ? t * TC_BM + row : 0)) * H + it.h) * TC_DH;
#pragma unroll
            for (int cc = 0; cc < TC_DH / 32; cc++) {
                float o[32];
                tmem_ld32(tmem_row + TC_O_COL(t) + cc * 32, o);        // the whole warp, whether the row is a query or not
                if (mine) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack_bf16(o[i] * inv, o[i + 1] * inv);
                        w.y = pack_bf16(o[i + 2] * inv, o[i + 3] * inv);
                        w.z = pack_bf16(o[i + 4] * inv, o[i + 5] * inv);
                        w.w = pack_bf16(o[i + 6] * inv, o[i + 7] * inv);
                        *(uint4*)(dst + cc * 32 + i) = w;
                    }
                }
            }
            // O_t is in my registers: the next item's first product may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&tail.o_free[t])) : "memory");
            c += my_blocks;
            kv_base += it.n_blocks;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tail.dead) {
        // Somebody gave up: before the block gives its shared memory back, the copying lane waits once more (each wait
        // with the same limit) for the copies it has started.
        if (tma_warp && lane == 0) {
            for (int g = k_started > TC_STAGES ? k_started - TC_STAGES : 0; g < k_started; g++) tc_mbar_wait(&tail.k_full[g % TC_STAGES], (unsigned)((g / TC_STAGES) & 1));
            for (int g = v_started > TC_STAGES ? v_started - TC_STAGES : 0; g < v_started; g++) tc_mbar_wait(&tail.v_full[g % TC_STAGES], (unsigned)((g / TC_STAGES) & 1));
            for (int g = q_started > TC_TILES ? q_started - TC_TILES : 0; g < q_started; g++) tc_mbar_wait(&tail.q_full[g % TC_TILES], (unsigned)((g / TC_TILES) & 1));
        }
        __syncthreads();
    }
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

// q [tokens, H, Dh] of bfloat16 as a matrix [tokens, H * Dh], copied in boxes of 128 rows x 64 elements (a slab of a
// query tile); rows past the last token read as zeros
static int tc_query_tensor_map(CUtensorMap* map, const void* q, long long tokens, int H) {
    static tc_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !fn)
            RI_FAIL(-1, "attention_prefill_tc: the driver has no cuTensorMapEncodeTiled");
        encode = (tc_encode_tiled_fn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)H * TC_DH, (cuuint64_t)tokens};
    cuuint64_t strides[1] = {(cuuint64_t)H * TC_DH * 2};
    cuuint32_t box[2] = {64, TC_BM};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RI_FAIL(-1, "attention_prefill_tc: cuTensorMapEncodeTiled of the queries failed with %d", (int)r);
    return 0;
}

extern "C" int ri_attention_prefill_tc_head_dim() { return TC_DH; }

// q, out [tokens, H, Dh] bf16; max_new = the most tokens one sequence brings in this step
extern "C" int ri_attention_prefill_tc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       const int* page_table, const int* seq_slot, const int* seq_start,
                                       const int* seq_len, int tokens, int seqs, int max_new, int H, int KV, int Dh, int mpps,
                                       int page_size, int num_pages, float scale, int window, int* err_flag,
                                       cudaStream_t stream) {
    if (seqs == 0 || max_new == 0 || tokens == 0) return 0;
    RI_REQUIRE(Dh == TC_DH, "attention_prefill_tc: built for head_dim %d, called with %d", TC_DH, Dh);
    RI_REQUIRE(page_size == TC_PAGE, "attention_prefill_tc: pages of %d tokens, this kernel needs %d", page_size, TC_PAGE);
    RI_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_prefill_tc: %d heads over %d kv heads", H, KV);
    RI_REQUIRE(tokens > 0 && max_new > 0 && max_new <= tokens, "attention_prefill_tc: %d tokens, at most %d of one sequence", tokens, max_new);
    RI_REQUIRE(window >= 0, "attention_prefill_tc: negative window");
    RI_REQUIRE(scale > 0.0f, "attention_prefill_tc: the score scale must be positive");
    RI_REQUIRE((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) == 0,
               "attention_prefill_tc: q, out and the pools must be 16-byte aligned");
    const int groups_max = (max_new + TC_TILES * TC_BM - 1) / (TC_TILES * TC_BM);
    const long long n_items = (long long)groups_max * seqs * H;
    RI_REQUIRE(n_items < (1ll << 30), "attention_prefill_tc: %lld work items", n_items);
    RI_REQUIRE((long long)num_pages * KV * TC_PAGE < (1ll << 31), "attention_prefill_tc: a pool of %d pages", num_pages);
    CUtensorMap map_q, map_k, map_v;
    int rc = tc_query_tensor_map(&map_q, q, tokens, H);
    if (rc) return rc;
    rc = tc_pool_tensor_map(&map_k, k_pool, (long long)num_pages * KV * TC_PAGE);
    if (rc) return rc;
    rc = tc_pool_tensor_map(&map_v, v_pool, (long long)num_pages * KV * TC_PAGE);
    if (rc) return rc;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES);
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_prefill_tc: %s", cudaGetErrorString(e));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    TcWork work;
    work.page_table = page_table;
    work.seq_slot = seq_slot;
    work.seq_start = seq_start;
    work.seq_len = seq_len;
    work.seqs = seqs;
    work.H = H;
    work.KV = KV;
    work.mpps = mpps;
    work.groups_max = groups_max;
    work.n_items = (int)n_items;
    work.window = window;
    // one block per SM (the kernel's shared memory allows no second), each taking its items one after the other
    const int blocks = n_items < sms ? (int)n_items : sms;
    attention_prefill_tc_kernel<<<blocks, TC_THREADS, TC_SMEM_BYTES, stream>>>(
        map_q, map_k, map_v, (bf16*)out, work, num_pages, scale * 1.4426950408889634f, err_flag);
    RI_CHECK_LAUNCH("attention_prefill_tc");
    return 0;
}
