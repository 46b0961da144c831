// Decode attention over the paged cache for bfloat16: one new token per sequence,
// the keys split into chunks, partial results merged afterwards.  Two kernels make the
// partial results: the streaming kernel further down (groups of up to 16 query heads,
// head sizes up to 128) and the one described here, which takes every other case, in
// chunks of 128 keys (four pages).
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
// keys 128c .. 128c+127), so with this kernel a sequence's result does not depend on
// the batch (with the streaming kernel it does, in its last bits: see there).
//
// Scratch memory: o_part [seqs, H, parts, Dh] and ml_part [seqs, H, parts, 2], float32,
// given by the caller, parts = ri_attention_decode_parts(max_chunks); this kernel uses
// the start of them, as [seqs, H, max_chunks, ...].
//
// Every wait on an mbarrier is bounded; if it runs out the kernel reports error 5
// through the error word and goes on (its output is then wrong, the context is not).
//
// Compile with -DRI_HEAD_DIM=<multiple of 16, at most 256>.  Page size is 32.
// Formula: thanhauco/rust-inference src/attention.rs:111-150.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <cuda.h>
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

// 16 bytes from global memory by an ordinary (coherent) load that is kept in L2 only.  Not ld.global.nc: what is read
// with it here, the newest key and the queries, was written by the kernel before this one while this kernel was
// already on the SMs (programmatic dependent launch), and a non-coherent load is only right for what nobody writes
// during the kernel's life; with rows that do not fill whole cache lines (head sizes other than 64 and 128) it
// was seen to return the line as it was before the write.
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// the same for 4 bytes, and for float data kept in L2 only (the merge reads every partial result once)
__device__ __forceinline__ unsigned ld_ca32(const void* p) {
    unsigned v;
    asm volatile("ld.global.ca.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cg_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
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
        page = key0 / AD_PAGE < mpps ? page_table[(size_t)slot * mpps + key0 / AD_PAGE] : -1;    // past the row: as unmapped
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

    bool waited = false, gave_up = false;
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
                kf[t][g] = (okr && d < AD_DH) ? ld_cg16(pk + d) : make_uint4(0, 0, 0, 0);
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
                qa[g] = (in && okA) ? ld_cg16(pa + d) : make_uint4(0, 0, 0, 0);
                qb[g] = (in && okB) ? ld_cg16(pb + d) : make_uint4(0, 0, 0, 0);
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
            if (valid_rows > 0 && !mbar_wait(&sm.bar[warp], 0)) {
                if (lane == 0) atomicExch(err, 5);
                gave_up = true;
            }
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
    // a warp whose wait ran out waits once more (with the same limit) for its copies before the block gives its
    // shared memory back
    if (gave_up) mbar_wait(&sm.bar[warp], 0);
}

// ---------------------------------------------------------------------------------------------
// The streaming kernel, for groups of at most 16 query heads and head sizes of 64 and 128.
//
// One block per SM, ADS_WARPS warps, and every warp works alone.  The pages that the step's
// queries see, of all sequences and kv heads, form one list (sequence by sequence, kv head by
// kv head, pages in rising order); it is cut into as many runs as the grid has warps, of
// lengths that differ by one page at most (and of at least ADS_MIN_PAGES pages), and a warp
// walks its run with the running maximum, sum and output of a flash decoder in its
// registers, so nothing is combined across warps, and with up to 32 sequences (their
// lengths in the warp's lanes) the block never synchronises; with more it does so once, at
// its start, for the table of the sequences' page counts in shared memory.  Every warp of
// the grid so has the same number of pages to read, whatever the batch and the lengths are.
// The keys and the values of a page are two tiles of a stream that runs through the warp's
// own ring of ADS_SLOTS shared-memory slots: one lane starts a TMA tensor copy
// (cp.async.bulk.tensor.2d, 128-byte swizzle, completion on the slot's mbarrier) per 64
// head elements of the tile, the warp waits for the oldest tile, reads it with ldmatrix
// (keys) or ldmatrix.trans (values) for mma.sync m16n8k16, and refills the slot with the
// tile ADS_SLOTS ahead - which may belong to the next (sequence, kv head) of the run, so
// the copies never stop.  A tile is one or two instructions to start, where a copy per row
// costs the warp a loop over its lanes; the swizzle makes the ldmatrix reads free of bank
// conflicts without padding.  With three slots of 8 KB for each of eight warps an SM has
// 192 KB on its way at all times.
//
// Where a run ends inside a (sequence, kv head), or passes from one to the next, the warp
// writes a partial result (maximum, sum, unnormalised output): piece i of a (sequence, kv
// head) comes from the i-th warp whose run touches it, at place i of that head's scratch
// rows (at most 2 max_chunks + 1 pieces, since a run has at least two pages), and the merge
// kernel, which computes the same cut from the same lengths, adds the pieces in that order.
// The cut depends on the whole batch: a sequence's result is the same from run to run, but
// its last bits may differ between batches (the pieces are other pieces).
//
// The running maximum is only raised when a page's maximum exceeds it by more than 2^8
// (the weights stay below 2^8, exact in float32 and as good as any in bfloat16), which
// saves rescaling the output on most pages.
// ---------------------------------------------------------------------------------------------
#define ADS_OK (AD_DH == 64 || AD_DH == 128)
#ifndef ADS_WARPS
#define ADS_WARPS 8
#endif
#define ADS_BOXES ((AD_DH + 63) / 64)                  // copies per tile: 64 head elements (128 bytes) x 32 rows each
#define ADS_BOX_BYTES (AD_PAGE * 128)
#define ADS_SLOT_BYTES (ADS_BOXES * ADS_BOX_BYTES)
#ifndef ADS_SLOTS
#define ADS_SLOTS_RAW ((208 * 1024) / (ADS_WARPS * ADS_SLOT_BYTES))
#define ADS_SLOTS (ADS_SLOTS_RAW > 6 ? 6 : ADS_SLOTS_RAW)
#endif
// a small batch has fewer runs of two pages than the grid has warps: then fewer warps per block (four, or two),
// each with a deeper ring, so that more of a run's tiles are on their way at once
#define ADS_SLOTS_FOR(warps) ((208 * 1024) / ((warps) * ADS_SLOT_BYTES) > 12 ? 12 : (208 * 1024) / ((warps) * ADS_SLOT_BYTES))
#define ADS_MAX_SEQS 1024                              // sequences of a step (their page counts stand in shared memory)
#define ADS_MIN_PAGES 2                                // a warp's run has at least this many pages
#define ADS_PARTS(max_chunks) (2 * (max_chunks) + 1)   // pieces of a (sequence, kv head) at most
#define ADS_SMEM_BYTES(warps, slots) ((size_t)(warps) * (slots) * ADS_SLOT_BYTES + (size_t)(warps) * (slots) * 8 + (ADS_MAX_SEQS + 1) * 4 + 1024)
#define ADS_LAZY 8.0f                                  // log2 of how far a page's maximum may exceed the running one

// where a warp stands in its run of pages
struct StreamCursor {
    int rem;           // pages of the run after the piece at hand
    int b, kvh;        // the piece at hand: of which sequence and kv head
    int seg, at;       // where the list has this (sequence, kv head), and where this piece of it
    int part;          // which of the (sequence, kv head)'s pieces it is (the cursor that computes keeps this)
    int len, first_key;
    int p, p_end;      // the page (index within the sequence) and the end of the piece
    int ids_base;      // lane l holds the pool index of page ids_base + l of the sequence
    int id_lane;
    int slot_row;      // the sequence's row of the page table
};

struct StreamArgs {
    const int* page_table;
    const int* seq_slot;
    const int* seq_len;
    int seqs, KV, mpps, num_pages, window, max_pages, parts;
    int* err;
};

__device__ __forceinline__ int warp_sum_int(int v) { return __reduce_add_sync(0xffffffffu, v); }

// the pages that the query of a sequence of `len` keys sees: [p_first, p_first + n)
__device__ __forceinline__ int stream_visible(int len, int window, int max_pages, int& first_key, int& p_first) {
    first_key = (window > 0 && len - window > 0) ? len - window : 0;
    p_first = first_key / AD_PAGE;
    int p_last = (len + AD_PAGE - 1) / AD_PAGE;
    p_last = p_last < max_pages ? p_last : max_pages;     // no partial result has a place beyond (the merge reports it)
    return p_last > p_first ? p_last - p_first : 0;
}
// How a list of `total` pages is cut into runs for `workers` warps: the first `more` runs have len + 1 pages, the
// others len, which together is the whole list; a list too short for runs of ADS_MIN_PAGES pages everywhere
// is cut into runs of that length, as many as it takes.
struct StreamCut {
    int len, more;
    __device__ __forceinline__ StreamCut(int total, int workers) {
        len = total / workers;
        more = total - len * workers;
        if (len < ADS_MIN_PAGES) {
            len = ADS_MIN_PAGES;
            more = 0;
        }
    }
    __device__ __forceinline__ int start(int w) const { return w * len + (w < more ? w : more); }     // of run w
    __device__ __forceinline__ int pages(int w) const { return len + (w < more ? 1 : 0); }
    __device__ __forceinline__ int owner(int u) const {                                                // the run that holds place u
        const int longs = more * (len + 1);
        return u < longs ? u / (len + 1) : more + (u - longs) / len;
    }
};

// The step's sequences as a warp's cursors see them: lengths, rows of the page table and the running count of
// visible pages.  SMALL (at most 32 sequences): lane b of the warp holds sequence b's, read once at the kernel's
// start and passed around by shuffles (every call is made by the whole warp); else the counts stand in shared
// memory and the rest is read from the step's tables.
template <bool SMALL>
struct SeqTable {
    const int* pre;                        // !SMALL: pre[b] = visible pages of the sequences before b, pre[seqs] = all
    const int* seq_len;
    const int* seq_slot;
    int seqs;
    int lane_through, lane_len, lane_slot; // SMALL
    __device__ __forceinline__ int through(int b) const {          // visible pages of sequences 0..b
        return SMALL ? __shfl_sync(0xffffffffu, lane_through, b) : pre[b + 1];
    }
    __device__ __forceinline__ int before(int b) const {
        if (!SMALL) return pre[b];
        const int v = __shfl_sync(0xffffffffu, lane_through, (b + 31) & 31);
        return b == 0 ? 0 : v;
    }
    __device__ __forceinline__ int all() const { return through(seqs - 1); }
    __device__ __forceinline__ int len(int b) const { return SMALL ? __shfl_sync(0xffffffffu, lane_len, b) : seq_len[b]; }
    __device__ __forceinline__ int slot(int b) const { return SMALL ? __shfl_sync(0xffffffffu, lane_slot, b) : seq_slot[b]; }
    // the sequence b with KV before(b) <= u < KV through(b), for a place u of the list
    __device__ __forceinline__ int find(int u, int KV) const {
        if (SMALL) return __popc(__ballot_sync(0xffffffffu, KV * lane_through <= u));     // lanes past the last sequence hold all()
        int lo = 0, hi = seqs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (KV * pre[mid] <= u) lo = mid; else hi = mid;
        }
        return lo;
    }
};

__device__ __forceinline__ void stream_load_ids(StreamCursor& c, const StreamArgs& a, int lane) {
    c.ids_base = c.p;
    int pg = c.p + lane;
    int id = (pg < c.p_end) ? (pg < a.mpps ? a.page_table[(size_t)c.slot_row * a.mpps + pg] : -1) : 0;
    if (id < 0 || id >= a.num_pages) {
        atomicExch(a.err, 4);
        id = 0;
    }
    c.id_lane = id;
}

// the piece of (c.b, c.kvh) that starts `off` pages into its visible pages and has at most `rem` pages;
// IDS: the cursor is the one that copies, so it needs the pages' places in the pool.
template <bool IDS, bool SMALL>
__device__ __forceinline__ void stream_piece(StreamCursor& c, const StreamArgs& a, const SeqTable<SMALL>& t, int off, int rem, const StreamCut& cut, int lane) {
    int p_first;
    c.len = t.len(c.b);
    const int n = stream_visible(c.len, a.window, a.max_pages, c.first_key, p_first);
    c.p = p_first + off;
    c.p_end = min(p_first + n, c.p + rem);
    c.rem = rem - (c.p_end - c.p);
    c.seg = a.KV * t.before(c.b) + c.kvh * n;
    c.at = c.seg + off;
    if (IDS) {
        c.slot_row = t.slot(c.b);
        stream_load_ids(c, a, lane);
    } else {
        c.part = cut.owner(c.at) - cut.owner(c.seg);         // (divisions: kept off the path to the first copies)
    }
}

// the first piece of the run [u, u + rem) of the list; false if the run is empty
template <bool IDS, bool SMALL>
__device__ __forceinline__ bool stream_seek(StreamCursor& c, const StreamArgs& a, const SeqTable<SMALL>& t, int u, int rem, const StreamCut& cut, int lane) {
    if (rem <= 0) return false;
    c.b = t.find(u, a.KV);
    const int r = u - a.KV * t.before(c.b), n = t.through(c.b) - t.before(c.b);
    c.kvh = r / n;
    stream_piece<IDS>(c, a, t, r - c.kvh * n, rem, cut, lane);
    return true;
}

// the next page of the run; false at its end
template <bool IDS, bool SMALL>
__device__ __forceinline__ bool stream_next(StreamCursor& c, const StreamArgs& a, const SeqTable<SMALL>& t, const StreamCut& cut, int lane) {
    if (++c.p < c.p_end) {
        if (IDS && c.p - c.ids_base == 32) stream_load_ids(c, a, lane);
        return true;
    }
    if (c.rem <= 0) return false;
    if (++c.kvh == a.KV) {                                    // pages are left, so a sequence with pages follows
        c.kvh = 0;
        do c.b++; while (c.b + 1 < a.seqs && t.through(c.b) == t.before(c.b));
    }
    stream_piece<IDS>(c, a, t, 0, c.rem, cut, lane);
    return true;
}

// one box of a tensor map into shared memory: x in elements (a multiple of 64 here, so of 16 bytes), y the row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

#if ADS_OK
template <int WARPS, int SLOTS, bool SMALL>
__global__ void __launch_bounds__(32 * WARPS, 1)
attention_decode_stream_kernel(const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_v, float* __restrict__ o_part,
                               float* __restrict__ ml_part, StreamArgs a, int H, float scale_log2) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    // the swizzle works on address bits 4..9: tiles start on multiples of 1024 bytes
    unsigned char* base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* ring = base + (size_t)warp * SLOTS * ADS_SLOT_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + (size_t)WARPS * SLOTS * ADS_SLOT_BYTES)
                               + warp * SLOTS;
    int* pre = reinterpret_cast<int*>(base + (size_t)WARPS * SLOTS * ADS_SLOT_BYTES + (size_t)WARPS * SLOTS * 8);
    const int G = H / a.KV;
    // the sequences' lengths and rows of the page table are tables of the step, not the work of the kernel before;
    // they are asked for first of all, so that they are on their way while the barriers are set up
    SeqTable<SMALL> tab;
    tab.pre = pre;
    tab.seq_len = a.seq_len;
    tab.seq_slot = a.seq_slot;
    tab.seqs = a.seqs;
    tab.lane_through = tab.lane_len = tab.lane_slot = 0;
    if (SMALL && lane < a.seqs) {
        tab.lane_len = a.seq_len[lane];
        tab.lane_slot = a.seq_slot[lane];
    }
    if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_v) : "memory");
#pragma unroll
        for (int s = 0; s < SLOTS; s++) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    if (SMALL) {
        int fk, pf;
        int v = lane < a.seqs ? stream_visible(tab.lane_len, a.window, a.max_pages, fk, pf) : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += up;
        }
        tab.lane_through = v;
    } else {
        for (int b = threadIdx.x; b < a.seqs; b += 32 * WARPS) {
            int fk, pf;
            pre[b + 1] = stream_visible(a.seq_len[b], a.window, a.max_pages, fk, pf);
        }
        __syncthreads();
        if (warp == 0) {
            int carry = 0;
            for (int b0 = 0; b0 < a.seqs; b0 += 32) {
                int v = b0 + lane < a.seqs ? pre[b0 + lane + 1] : 0;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += up;
                }
                if (b0 + lane < a.seqs) pre[b0 + lane + 1] = carry + v;
                carry += __shfl_sync(0xffffffffu, v, 31);
            }
            if (lane == 0) pre[0] = 0;
        }
        __syncthreads();
    }
    const int total = a.KV * tab.all(), workers = (int)gridDim.x * WARPS;
    const StreamCut cut(total, workers);
    const int my_run = blockIdx.x + gridDim.x * warp;        // neighbouring runs go to different SMs
    const int u0 = cut.start(my_run);

    StreamCursor ci, cc;                  // the page whose tiles are copied next, the page that is worked on
    bool more = u0 < total && stream_seek<true>(ci, a, tab, u0, min(cut.pages(my_run), total - u0), cut, lane);
    cc = ci;                              // (its part is computed below, once the first copies are on their way)
    bool live = more;
    int issue_v = 0;                      // 0: the keys of ci's page come next, 1: its values
    int in_flight = 0, slot_i = 0, slot_c = 0;
    unsigned phases = 0;
    bool dead = false;

    // starts the copies of the next tile of the stream into slot `slot_i`
    auto issue = [&]() {
        const int id = __shfl_sync(0xffffffffu, ci.id_lane, ci.p - ci.ids_base);
        if (lane == 0) {
            unsigned char* dst = ring + (size_t)slot_i * ADS_SLOT_BYTES;
            const int row = (id * a.KV + ci.kvh) * AD_PAGE;
            mbar_expect_tx(&bars[slot_i], ADS_SLOT_BYTES);
#pragma unroll
            for (int x = 0; x < ADS_BOXES; x++) {
#ifdef ADS_TEST_DROP_COPY_LEN
                // tests only: the first copy of the keys of page 0, kv head 0, of a sequence of exactly this many keys
                // is left out, so that its barrier never completes and the wait for it runs out
                if (ci.len == ADS_TEST_DROP_COPY_LEN && ci.p == 0 && ci.kvh == 0 && !issue_v && x == 0) continue;
#endif
                tma_load_2d(dst + x * ADS_BOX_BYTES, issue_v ? &map_v : &map_k, x * 64, row, &bars[slot_i]);
            }
        }
        slot_i = slot_i + 1 == SLOTS ? 0 : slot_i + 1;
        in_flight++;
        if (issue_v) more = stream_next<true>(ci, a, tab, cut, lane);
        issue_v ^= 1;
    };
    int gave_up_slot = 0;
    unsigned gave_up_parity = 0;
    auto wait_tile = [&]() {
        if (!dead && !ri_mbar_wait(&bars[slot_c], (phases >> slot_c) & 1u)) {
            if (lane == 0) atomicExch(a.err, 5);
            dead = true;
            gave_up_slot = slot_c;
            gave_up_parity = (phases >> slot_c) & 1u;
        }
        phases ^= 1u << slot_c;
    };
    auto release_tile = [&]() {
        __syncwarp();                     // every lane has read the tile
        slot_c = slot_c + 1 == SLOTS ? 0 : slot_c + 1;
        in_flight--;
        if (more && !dead) issue();
    };

    // The kernel before this one wrote the queries and the newest key and value (the last page of each
    // sequence); the pages before that one were written by earlier steps and may be copied at once.
#pragma unroll 1
    while (more && in_flight < SLOTS && (ci.p + 1) * AD_PAGE < ci.len) issue();
    // every block of this grid is on an SM from the start (one per SM), so the kernel after it (the merge: small
    // blocks that read the lengths and then wait) may come in at once
    if (live) cc.part = cut.owner(cc.at) - cut.owner(cc.seg);
    pdl_trigger();
    pdl_wait();
#pragma unroll 1
    while (more && in_flight < SLOTS) issue();

    float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.0f, 0.0f};
    float o[AD_DH / 8][4];
    unsigned qf[AD_DH / 16][4];
    bool fresh = true, new_item = true;   // the next page is the first of a piece (of another sequence or kv head)
    // this lane's corner of the 8x8 matrices that ldmatrix reads (rows of 128 bytes, 16-byte pieces swizzled by the row)
    const int k_row = (lane & 7) + ((lane >> 4) & 1) * 8, k_piece = (lane >> 3) & 1;
    const int v_row = (lane & 7) + ((lane >> 3) & 1) * 8, v_piece = lane >> 4;
#pragma unroll 1
    while (live) {
        if (new_item) {
            // ---- the piece's query fragments: rows quad and quad + 8 of the group --------------------------
            const bf16* pa = q + ((size_t)cc.b * H + cc.kvh * G + (quad < G ? quad : 0)) * AD_DH + qc * 2;
            const bf16* pb = q + ((size_t)cc.b * H + cc.kvh * G + (quad + 8 < G ? quad + 8 : 0)) * AD_DH + qc * 2;
#pragma unroll
            for (int ks = 0; ks < AD_DH / 16; ks++) {
                // (ordinary loads: the queries were written while this kernel was already on the SMs)
                qf[ks][0] = quad < G ? ld_ca32(pa + ks * 16) : 0u;
                qf[ks][1] = quad + 8 < G ? ld_ca32(pb + ks * 16) : 0u;
                qf[ks][2] = quad < G ? ld_ca32(pa + ks * 16 + 8) : 0u;
                qf[ks][3] = quad + 8 < G ? ld_ca32(pb + ks * 16 + 8) : 0u;
            }
            new_item = false;
        }
        if (fresh) {
#pragma unroll
            for (int t = 0; t < AD_DH / 8; t++)
#pragma unroll
                for (int e = 0; e < 4; e++) o[t][e] = 0.0f;
            m_run[0] = m_run[1] = -FLT_MAX;
            l_run[0] = l_run[1] = 0.0f;
            fresh = false;
        }
        const int key0 = cc.p * AD_PAGE;
        const int rows = min(AD_PAGE, cc.len - key0);
        // ---- S[16 rows, 32 keys] = Q K^T ----------------------------------------------------------------
        float s[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[t][e] = 0.0f;
        wait_tile();
        {
            const unsigned char* kt = ring + (size_t)slot_c * ADS_SLOT_BYTES + k_row * 128;
#pragma unroll
            for (int ks = 0; ks < AD_DH / 16; ks++) {
                const unsigned char* kb = kt + (ks / 4) * ADS_BOX_BYTES + ((((ks * 2 + k_piece) & 7) ^ (lane & 7)) << 4);
#pragma unroll
                for (int tp = 0; tp < 2; tp++) {              // keys 16 tp .. 16 tp + 15
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, kb + tp * 16 * 128);
                    mma_bf16(s[tp * 2], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma_bf16(s[tp * 2 + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
                }
            }
        }
        release_tile();
        // ---- mask (only the pages at the ends of the visible range need it), maximum, weights ---------------
        if (key0 < cc.first_key || rows < AD_PAGE) {
#pragma unroll
            for (int t = 0; t < 4; t++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    int key = key0 + t * 8 + qc * 2 + (e & 1);
                    if (key >= cc.len || key < cc.first_key) s[t][e] = -FLT_MAX;
                }
        }
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) mx[e >> 1] = fmaxf(mx[e >> 1], s[t][e]);
        bool raise = false;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            mx[r] = mx[r] == -FLT_MAX ? -FLT_MAX : mx[r] * scale_log2;      // the scale is positive
            raise = raise || mx[r] > m_run[r] + ADS_LAZY || m_run[r] == -FLT_MAX;
        }
        if (__any_sync(0xffffffffu, raise)) {
            // a row's maximum has moved far: every row takes its new maximum and the output is rescaled
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const float m_new = fmaxf(m_run[r], mx[r]);
                const float corr = ex2_fast(m_run[r] - m_new);   // 1 while nothing has been seen (both are -FLT_MAX)
                m_run[r] = m_new;
                l_run[r] *= corr;
#pragma unroll
                for (int t = 0; t < AD_DH / 8; t++) {
                    o[t][r * 2] *= corr;
                    o[t][r * 2 + 1] *= corr;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                // a masked score is -FLT_MAX: its weight underflows to zero against any maximum of a visible key
                float p = ex2_fast(fmaf(s[t][e], scale_log2, -m_run[e >> 1]));
                s[t][e] = p;
                l_run[e >> 1] += p;                       // this lane's columns; the quad is summed at the chunk's end
            }
        // ---- O[16, Dh] += P V ---------------------------------------------------------------------------
        wait_tile();
        {
            unsigned char* vt = ring + (size_t)slot_c * ADS_SLOT_BYTES;
            if (rows < AD_PAGE) {
                // rows past the sequence's end hold whatever the pool holds there: zero them (0 x NaN is NaN)
                if (lane >= rows)
#pragma unroll
                    for (int x = 0; x < ADS_BOXES; x++)
#pragma unroll
                        for (int c = 0; c < 8; c++) *(uint4*)(vt + x * ADS_BOX_BYTES + lane * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                __syncwarp();
            }
            const unsigned char* vl = vt + v_row * 128;
#pragma unroll
            for (int kk = 0; kk < 2; kk++) {           // 16 keys at a time
                unsigned a0 = pack_bf16(s[kk * 2][0], s[kk * 2][1]), a1 = pack_bf16(s[kk * 2][2], s[kk * 2][3]);
                unsigned a2 = pack_bf16(s[kk * 2 + 1][0], s[kk * 2 + 1][1]), a3 = pack_bf16(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
                for (int dp = 0; dp < AD_DH / 16; dp++) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3,
                                      vl + kk * 16 * 128 + (dp / 4) * ADS_BOX_BYTES + ((((dp * 2 + v_piece) & 7) ^ (lane & 7)) << 4));
                    mma_bf16(o[dp * 2], a0, a1, a2, a3, b0, b1);
                    mma_bf16(o[dp * 2 + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            if (rows < AD_PAGE) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the zeros, before the next copy into the slot
        }
        release_tile();
        // ---- the last page of a piece: write its partial result ------------------------------------------
        if (cc.p + 1 == cc.p_end) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
                const int row = quad + r * 8;
                if (row < G) {
                    const size_t at = ((size_t)cc.b * H + cc.kvh * G + row) * a.parts + cc.part;
                    float* dst = o_part + at * AD_DH + qc * 2;
#pragma unroll
                    for (int t = 0; t < AD_DH / 8; t++) *(float2*)(dst + t * 8) = make_float2(o[t][r * 2], o[t][r * 2 + 1]);
                    if (qc == 0) *(float2*)(ml_part + at * 2) = make_float2(m_run[r], l_run[r]);
                }
            }
            fresh = true;
            new_item = true;              // the next piece is of another sequence or kv head
        }
        live = stream_next<false>(cc, a, tab, cut, lane);
        if (dead) break;
    }
    if (dead) {
        // A warp that gave up has started no further copy; those it had started are waited for once more, each with
        // the same limit: a copy must not land in shared memory that the block has given back.
        ri_mbar_wait(&bars[gave_up_slot], gave_up_parity);
        for (; in_flight > 0; in_flight--) {
            ri_mbar_wait(&bars[slot_c], (phases >> slot_c) & 1u);
            phases ^= 1u << slot_c;
            slot_c = slot_c + 1 == SLOTS ? 0 : slot_c + 1;
        }
    }
}

// ---- tensor maps of the pools, made on the host -------------------------------------------------------
typedef CUresult (*ri_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// a pool [pages, KV, 32, Dh] of bfloat16 as a matrix [pages * KV * 32, Dh], copied in boxes of 32 rows x 64 elements
static int pool_tensor_map(CUtensorMap* map, const void* pool, long long rows) {
    static ri_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res);
        if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !fn)
            RI_FAIL(-1, "attention_decode: the driver has no cuTensorMapEncodeTiled");
        encode = (ri_encode_tiled_fn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)AD_DH, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)AD_DH * 2};
    cuuint32_t box[2] = {64, AD_PAGE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RI_FAIL(-1, "attention_decode: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}
#endif  // ADS_OK

// how the streaming kernel cut its list of pages (0 workers: the partial results are those of chunks of 128 keys)
struct MergeCut {
    int workers, seqs, KV, parts;
};

// out[b, h, :] = the partial results of the head's chunks (or pieces) added up.  The block's four warps each take
// a quarter of them (in rising order, four head elements per lane), then the four sums are added in
// warp order: the order of the additions depends on the partial results' number only.
__global__ void __launch_bounds__(AD_MERGE_THREADS)
attention_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                              bf16* __restrict__ out, const int* __restrict__ seq_len, int H, int max_chunks,
                              int window, MergeCut cut, int* __restrict__ err) {
    constexpr int MW = AD_MERGE_THREADS / 32;            // warps
    constexpr int PER = (AD_DH + 127) / 128;             // float4 per lane
    const int h = blockIdx.x, b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float s_w[AD_MERGE_TILE], s_red[MW], s_l[MW];
    __shared__ int s_cnt[2][MW];
    pdl_trigger();
    const int len = seq_len[b];                          // a table of the step, not the work of the kernel before
    const int first_key = (window > 0 && len - window > 0) ? len - window : 0;
    int c_lo = first_key / AD_CHUNK, c_hi = (len + AD_CHUNK - 1) / AD_CHUNK;           // [c_lo, c_hi)
    const bool too_long = c_hi > max_chunks;
    int stride = max_chunks;                             // partial results a head has room for
    if (too_long) {
        // the caller's scratch memory has no partial results for the keys past max_chunks * 128: they are left
        // out (nothing is read past the sequence's rows) and the mistake is reported
        c_hi = max_chunks;
        c_lo = c_lo < c_hi ? c_lo : c_hi;
    }
#if ADS_OK
    if (cut.workers > 0) {
        // the streaming kernel's cut, from the same lengths: the pages before this sequence's and all pages
        const int max_pages = max_chunks * (AD_CHUNK / AD_PAGE);
        int below = 0, all = 0;
        if (cut.seqs <= 32) {
            // every warp for itself: a lane per sequence, two additions across the warp
            int f2, p2;
            const int n = lane < cut.seqs ? stream_visible(seq_len[lane], window, max_pages, f2, p2) : 0;
            all = warp_sum_int(n);
            below = warp_sum_int(lane < b ? n : 0);
        } else {
            for (int s = threadIdx.x; s < cut.seqs; s += AD_MERGE_THREADS) {
                int f2, p2;
                const int n = stream_visible(seq_len[s], window, max_pages, f2, p2);
                all += n;
                below += s < b ? n : 0;
            }
            below = warp_sum_int(below);
            all = warp_sum_int(all);
            if (lane == 0) {
                s_cnt[0][warp] = below;
                s_cnt[1][warp] = all;
            }
            __syncthreads();
            below = all = 0;
#pragma unroll
            for (int w = 0; w < MW; w++) {
                below += s_cnt[0][w];
                all += s_cnt[1][w];
            }
        }
        int f2, p2;
        const int n = stream_visible(len, window, max_pages, f2, p2);
        const StreamCut runs(cut.KV * all, cut.workers);
        const int seg = cut.KV * below + (h / (H / cut.KV)) * n;
        c_lo = 0;
        c_hi = n > 0 ? runs.owner(seg + n - 1) - runs.owner(seg) + 1 : 0;
        stride = cut.parts;
    }
#endif
    pdl_wait();
    if (too_long && threadIdx.x == 0) atomicExch(err, 7);
    const float* ml = ml_part + ((size_t)b * H + h) * stride * 2;
    const float* op = o_part + ((size_t)b * H + h) * stride * AD_DH;
    __shared__ __align__(16) float s_acc[MW][AD_DH];
    // The partial outputs of this warp's first eight chunks are asked for at once, before the maxima (on which
    // their weights depend) are known: the kernel is a chain of trips to L2, and this takes one out of it.
    float4 first[8][PER];
    const int n0 = min(AD_MERGE_TILE, c_hi - c_lo);
    const int lo0 = n0 * warp / MW, hi0 = n0 * (warp + 1) / MW;
#pragma unroll
    for (int u = 0; u < 8; u++)
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int d = (j * 32 + lane) * 4;
            if (lo0 + u < hi0 && d < AD_DH) first[u][j] = ld_cg_f32x4(op + (size_t)(c_lo + lo0 + u) * AD_DH + d);
        }
    // the maximum over the visible chunks
    float M = -FLT_MAX;
    for (int c = c_lo + (int)threadIdx.x; c < c_hi; c += AD_MERGE_THREADS) M = fmaxf(M, ld_cg_f32(ml + c * 2));
    M = warp_max(M);
    if (lane == 0) s_red[warp] = M;
    __syncthreads();
    M = s_red[0];
#pragma unroll
    for (int w = 1; w < MW; w++) M = fmaxf(M, s_red[w]);
    float L = 0.0f;
    float4 acc[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) acc[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int t0 = c_lo; t0 < c_hi; t0 += AD_MERGE_TILE) {
        const int n = min(AD_MERGE_TILE, c_hi - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += AD_MERGE_THREADS) {
            float m = ld_cg_f32(ml + (t0 + i) * 2);
            s_w[i] = m == -FLT_MAX ? 0.0f : exp2f(m - M);
        }
        __syncthreads();
        // this warp's quarter of the tile
        const int lo = n * warp / MW, hi = n * (warp + 1) / MW;
        for (int i = lo + lane; i < hi; i += 32) L += ld_cg_f32(ml + (t0 + i) * 2 + 1) * s_w[i];
        // eight chunks' partial outputs are asked for before the first is added (the additions stay in rising order
        // of the chunks)
        for (int i0 = lo; i0 < hi; i0 += 8) {
            float4 v[8][PER];
            const bool have = t0 == c_lo && i0 == lo;             // the ones asked for at the top
#pragma unroll
            for (int u = 0; u < 8; u++)
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    const int d = (j * 32 + lane) * 4;
                    if (have) v[u][j] = first[u][j];
                    else if (i0 + u < hi && d < AD_DH) v[u][j] = ld_cg_f32x4(op + (size_t)(t0 + i0 + u) * AD_DH + d);
                }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (i0 + u >= hi) break;
                const float w = s_w[i0 + u];
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    const int d = (j * 32 + lane) * 4;
                    if (d < AD_DH) {
                        acc[j].x = fmaf(v[u][j].x, w, acc[j].x);
                        acc[j].y = fmaf(v[u][j].y, w, acc[j].y);
                        acc[j].z = fmaf(v[u][j].z, w, acc[j].z);
                        acc[j].w = fmaf(v[u][j].w, w, acc[j].w);
                    }
                }
            }
        }
    }
    L = warp_sum(L);
    if (lane == 0) s_l[warp] = L;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int d = (j * 32 + lane) * 4;
        if (d < AD_DH) *(float4*)&s_acc[warp][d] = acc[j];
    }
    __syncthreads();
    L = s_l[0];
#pragma unroll
    for (int w = 1; w < MW; w++) L += s_l[w];
    for (int d = threadIdx.x; d < AD_DH; d += AD_MERGE_THREADS) {
        float a = s_acc[0][d];
#pragma unroll
        for (int w = 1; w < MW; w++) a += s_acc[w][d];
        out[((size_t)b * H + h) * AD_DH + d] = __float2bfloat16_rn(L > 0.0f ? a / L : 0.0f);
    }
}

extern "C" int ri_attention_decode_head_dim() { return AD_DH; }
extern "C" int ri_attention_decode_chunk() { return AD_CHUNK; }

// shared memory of a launch with G query heads per kv head; on a device's first call the kernel's limit is set to
// the most any group size needs, so that no later call (of either entry point of this library) has to touch it
#define AD_MAX_DEVICES 64
static int decode_configure(int G, size_t* smem_out) {
    static bool configured[AD_MAX_DEVICES];
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode: cudaGetDevice: %s", cudaGetErrorString(e));
    RI_REQUIRE(device >= 0 && device < AD_MAX_DEVICES, "attention_decode: device %d", device);
    if (!configured[device]) {
        e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)decode_smem_bytes(AD_ROWS));
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode: shared memory limit: %s", cudaGetErrorString(e));
        configured[device] = true;
    }
    *smem_out = decode_smem_bytes(G < AD_ROWS ? G : AD_ROWS);
    return 0;
}

#if ADS_OK
template <int WARPS, int SLOTS, bool SMALL>
static int launch_stream_for(int blocks, cudaStream_t stream, const bf16* q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                         float* o_part, float* ml_part, StreamArgs a, int H, float scale_log2) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_stream_kernel<WARPS, SLOTS, SMALL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ADS_SMEM_BYTES(WARPS, SLOTS));
        if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode: shared memory limit: %s", cudaGetErrorString(e));
        configured = true;
    }
    ri_launch_pdl(attention_decode_stream_kernel<WARPS, SLOTS, SMALL>, dim3(blocks), dim3(32 * WARPS), ADS_SMEM_BYTES(WARPS, SLOTS),
                  stream, q, map_k, map_v, o_part, ml_part, a, H, scale_log2);
    RI_CHECK_LAUNCH("attention_decode_stream");
    return 0;
}
template <int WARPS, int SLOTS>
static int launch_stream(int blocks, cudaStream_t stream, const bf16* q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                         float* o_part, float* ml_part, StreamArgs a, int H, float scale_log2) {
    return a.seqs <= 32 ? launch_stream_for<WARPS, SLOTS, true>(blocks, stream, q, map_k, map_v, o_part, ml_part, a, H, scale_log2)
                        : launch_stream_for<WARPS, SLOTS, false>(blocks, stream, q, map_k, map_v, o_part, ml_part, a, H, scale_log2);
}
#endif

// how many partial results per (sequence, head) the scratch memory of ri_attention_decode must have room for
extern "C" int ri_attention_decode_parts(int max_chunks) {
#if ADS_OK && !defined(AD_NO_STREAM)
    return ADS_PARTS(max_chunks);
#else
    return max_chunks;
#endif
}

// q, out [seqs, H, Dh] bf16; o_part [seqs, H, parts, Dh] f32; ml_part [seqs, H, parts, 2] f32 with
// parts = ri_attention_decode_parts(max_chunks).  max_chunks * 128 must cover the longest sequence of the step.
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
#if ADS_OK && !defined(AD_NO_STREAM)
    if (H / KV <= AD_ROWS && scale > 0.0f && seqs <= ADS_MAX_SEQS) {
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        const int max_pages = max_chunks * (AD_CHUNK / AD_PAGE);
        RI_REQUIRE((long long)seqs * KV * max_pages < (1ll << 30), "attention_decode: %d sequences of up to %d pages", seqs, max_pages);
        RI_REQUIRE((long long)num_pages * KV * AD_PAGE < (1ll << 31), "attention_decode: a pool of %d pages", num_pages);
        CUtensorMap map_k, map_v;
        int rc_map = pool_tensor_map(&map_k, k_pool, (long long)num_pages * KV * AD_PAGE);
        if (rc_map) return rc_map;
        rc_map = pool_tensor_map(&map_v, v_pool, (long long)num_pages * KV * AD_PAGE);
        if (rc_map) return rc_map;
        StreamArgs a;
        a.page_table = page_table;
        a.seq_slot = seq_slot;
        a.seq_len = seq_len;
        a.seqs = seqs;
        a.KV = KV;
        a.mpps = mpps;
        a.num_pages = num_pages;
        a.max_pages = max_pages;
        a.parts = ADS_PARTS(max_chunks);
        a.window = window;
        a.err = err_flag;
        // the most runs of ADS_MIN_PAGES pages that the step can have: fewer blocks than SMs, or fewer warps per
        // block (each with a deeper ring), when they do not fill the grid
        const long long runs = ((long long)seqs * KV * max_pages + ADS_MIN_PAGES - 1) / ADS_MIN_PAGES;
        const int warps = runs <= (long long)sms * 2 ? 2 : (runs <= (long long)sms * 4 ? 4 : ADS_WARPS);
        const int blocks = (int)((runs + warps - 1) / warps < sms ? (runs + warps - 1) / warps : sms);
        const float scale_log2 = scale * 1.4426950408889634f;
        int rc;
        if (warps == 2)
            rc = launch_stream<2, ADS_SLOTS_FOR(2)>(blocks, stream, (const bf16*)q, map_k, map_v, o_part, ml_part, a, H, scale_log2);
        else if (warps == 4)
            rc = launch_stream<4, ADS_SLOTS_FOR(4)>(blocks, stream, (const bf16*)q, map_k, map_v, o_part, ml_part, a, H, scale_log2);
        else
            rc = launch_stream<ADS_WARPS, ADS_SLOTS>(blocks, stream, (const bf16*)q, map_k, map_v, o_part, ml_part, a, H, scale_log2);
        if (rc) return rc;
        MergeCut cut;
        cut.workers = blocks * warps;
        cut.seqs = seqs;
        cut.KV = KV;
        cut.parts = a.parts;
        ri_launch_pdl(attention_decode_merge_kernel, dim3(H, seqs), dim3(AD_MERGE_THREADS), 0, stream,
                      (const float*)o_part, (const float*)ml_part, (bf16*)out, seq_len, H, max_chunks, window, cut, err_flag);
        RI_CHECK_LAUNCH("attention_decode_merge");
        return 0;
    }
#endif
    size_t smem = 0;
    int rc = decode_configure(H / KV, &smem);
    if (rc) return rc;
    dim3 grid(max_chunks, KV, seqs);
    ri_launch_pdl(attention_decode_kernel, grid, dim3(32 * AD_WARPS), smem, stream,
                  (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, o_part, ml_part, page_table, seq_slot, seq_len,
                  H, KV, mpps, num_pages, max_chunks, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_decode");
    MergeCut chunks_of_128;
    chunks_of_128.workers = 0;
    chunks_of_128.seqs = seqs;
    chunks_of_128.KV = KV;
    chunks_of_128.parts = max_chunks;
    ri_launch_pdl(attention_decode_merge_kernel, dim3(H, seqs), dim3(AD_MERGE_THREADS), 0, stream,
                  (const float*)o_part, (const float*)ml_part, (bf16*)out, seq_len, H, max_chunks, window, chunks_of_128, err_flag);
    RI_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}
