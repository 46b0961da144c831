// The tiling of the decode-time linear (linear_skinny.cu), shared with the small kernels that run
// just before it and warm the L2 cache for it.
//
// A block of the linear owns SK_ROWS rows of W and all of K; each of its SK_WARPS warps takes a
// share of the row's stages of SK_STAGE_K k and keeps a ring of SK_STAGES of them in shared
// memory.  The ring of the blocks that are resident first (SK_MIN_BLOCKS per SM) is filled
// before the linear waits for its predecessor, so those bytes are on their way while the
// predecessor still runs.  Between the predecessor's end and the linear's start memory is idle:
// a kernel that runs in that gap can ask for the stages that those blocks will want NEXT
// (prefetch.global.L2, nothing is waited for and nothing is written), so that they are
// served from L2 when the linear asks.
#pragma once
#include "common.cuh"

#ifndef SK_WARPS
#define SK_WARPS 4
#endif
#define SK_ROWS 16
#ifndef SK_STAGE_K
#define SK_STAGE_K 256                       // k per stage
#endif
#ifndef SK_STAGES
#define SK_STAGES 2
#endif
#ifndef SK_MIN_BLOCKS
#define SK_MIN_BLOCKS 3
#endif
#ifndef SK_HINT_STAGES
#define SK_HINT_STAGES 1                     // stages per warp that a hint brings into L2
#endif
#ifndef SK_HINT_BLOCKS
#define SK_HINT_BLOCKS SK_MIN_BLOCKS         // blocks per SM whose rows a hint covers
#endif

// The weight matrix [rows, k] (bfloat16, rows of row_bytes) that a skinny linear reads next; base == nullptr: none.
struct WeightHint {
    const char* base;
    long long row_bytes;
    int rows;          // rows of the blocks that are resident first
    int stages;        // stages in a row
};

static inline WeightHint make_weight_hint(const void* w, int n, int k, int sms) {
    WeightHint h{nullptr, 0, 0, 0};
    if (!w || k % SK_STAGE_K || ((uintptr_t)w & 15)) return h;
    h.base = (const char*)w;
    h.row_bytes = (long long)k * 2;
    const long long first = (long long)sms * SK_HINT_BLOCKS * SK_ROWS;
    h.rows = (int)(first < n ? first : n);
    h.stages = k / SK_STAGE_K;
    return h;
}

#ifndef SK_HINT_LINE
#define SK_HINT_LINE 128                     // bytes asked for by one prefetch instruction
#endif

// Worker `worker` of `workers` threads asks for its share of the hinted bytes, a cache line per
// request (prefetch.global.L2: all lanes of a warp issue at once, where bulk prefetches of several
// lanes are issued one after another).
__device__ __forceinline__ void weight_hint_prefetch(const WeightHint& h, int worker, int workers) {
    if (!h.base) return;
    constexpr int STAGE_BYTES = SK_STAGE_K * 2;
    constexpr int LINES = SK_HINT_STAGES * STAGE_BYTES / SK_HINT_LINE;      // per row and warp
    const long long total = (long long)h.rows * SK_WARPS * LINES;
    for (long long i = worker; i < total; i += workers) {
        const int line = (int)(i % LINES);
        const int q = (int)((i / LINES) % SK_WARPS);
        const int row = (int)(i / (LINES * SK_WARPS));
        const int lo = (int)((long long)h.stages * q / SK_WARPS), hi = (int)((long long)h.stages * (q + 1) / SK_WARPS);
        const int s0 = lo + SK_STAGES;
        const int off = line * SK_HINT_LINE;                                // from the start of stage s0
        if (s0 * STAGE_BYTES + off < hi * STAGE_BYTES) {
            const char* p = h.base + (size_t)row * h.row_bytes + (size_t)s0 * STAGE_BYTES + off;
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p) : "memory");
        }
    }
}
