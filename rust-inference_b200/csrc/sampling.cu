// Next-token selection on the device: greedy, temperature, top-k, top-p and
// repetition penalty, with the meaning they have in thanhauco/rust-inference
// src/sampling.rs:73-140:
//
//   x_i = logit_i, and for tokens already in the context x_i / penalty if
//         x_i > 0 else x_i * penalty                                   (76-88)
//   temperature <= 0: the first index of the maximum                   (89-91, 132-140)
//   z_i = x_i / temperature; keep the top_k largest                    (93-98)
//   order the kept ones by falling z, equal z by rising index          (99)
//   p_i = exp(z_i - max) / sum                                         (101-104)
//   top_p < 1: keep the shortest prefix whose sum reaches top_p        (105-117)
//   draw: the first kept token, in that order, whose running sum of the
//         renormalised p exceeds the uniform number u                  (119-127)
//
// Nothing is sorted.  Each token gets the key (ordered bits of z_i, V-1-i), so
// that falling keys are exactly the reference's order, and a "prefix whose
// weight reaches a target" is found by a radix search over the key, 12 bits a
// pass, with weights summed as 64-bit integers (exp(z - max) * 2^40).  Integer
// sums make the result independent of the order of the additions: the same
// logits, options and u always give the same token.
//
// One block per row; rows are independent, so a sequence's draw does not depend
// on what it is batched with.
#include "common.cuh"
#include <float.h>

#define SP_THREADS 1024
#define SP_DIGIT 12
#define SP_BINS (1 << SP_DIGIT)
#define SP_IDX_BITS 24
#define SP_PASSES 5            // 5 * 12 = 60 >= 32 + 24 key bits
// The histogram of a pass is kept SP_SUBS times, one copy per residue of the lane number: logits crowd into few
// bins of the top digits (sign, exponent), and additions to one address of shared memory run one after another.
#ifndef SP_SUBS
#define SP_SUBS 4
#endif
#define SP_SMEM_BYTES (SP_SUBS * SP_BINS * 8)

typedef unsigned long long u64;

__device__ __forceinline__ unsigned ordered_bits(float z) {
    if (z != z) return 0u;                                   // NaN sorts last
    unsigned u = __float_as_uint(z);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowView {
    const float* logits;
    const unsigned char* seen;     // may be null
    float penalty;
    float temperature;
    int vocab;
    __device__ __forceinline__ float x(int i) const {
        float v = logits[i];
        if (seen && seen[i]) v = v > 0.0f ? v / penalty : v * penalty;
        return v;
    }
    __device__ __forceinline__ float z(int i) const { return x(i) / temperature; }
    __device__ __forceinline__ u64 key(int i, float zi) const {
        return ((u64)ordered_bits(zi) << SP_IDX_BITS) | (u64)((1u << SP_IDX_BITS) - 1u - (unsigned)i);
    }
};

__device__ u64 block_sum_u64(u64 v, u64* red) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        u64 t = lane < (blockDim.x >> 5) ? red[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// weight of token i: 1 when counting, exp(z - zmax) * 2^40 as an integer otherwise
__device__ __forceinline__ u64 weight_of(float zi, float zmax, int counting) {
    if (counting) return 1ull;
    return (u64)(expf(zi - zmax) * 1099511627776.0f);      // 2^40: exact scaling, sums stay below 2^64
}

// The largest key K (among tokens with key >= floor_key) such that the weight of
// all tokens with floor_key <= key and key >= K reaches `target`.  Returns 0 and
// sets *found = 0 when even all of them together stay below the target.
// `*reached` gets the weight of the tokens with key >= K.
__device__ u64 radix_select(const RowView& r, float zmax, int counting, u64 floor_key, u64 target, u64* bins,
                            u64* red, int* found, u64* reached) {
    __shared__ u64 s_prefix, s_remaining, s_above;
    __shared__ int s_found;
    if (threadIdx.x == 0) { s_prefix = 0; s_remaining = target; s_above = 0; s_found = 1; }
    __syncthreads();
    for (int pass = SP_PASSES - 1; pass >= 0; pass--) {
        int shift = pass * SP_DIGIT;
        for (int b = threadIdx.x; b < SP_SUBS * SP_BINS; b += blockDim.x) bins[b] = 0;
        __syncthreads();
        u64 prefix = s_prefix;
        u64* my_bins = bins + (threadIdx.x % SP_SUBS) * SP_BINS;
        for (int i = threadIdx.x; i < r.vocab; i += blockDim.x) {
            float zi = r.z(i);
            u64 k = r.key(i, zi);
            if (k < floor_key) continue;
            if (pass < SP_PASSES - 1 && (k >> (shift + SP_DIGIT)) != (prefix >> (shift + SP_DIGIT))) continue;
            u64 w = weight_of(zi, zmax, counting);
            if (w) atomicAdd(&my_bins[(unsigned)(k >> shift) & (SP_BINS - 1)], w);
        }
        __syncthreads();
        // the copies are added into the first (integer sums: the order does not matter)
        for (int b = threadIdx.x; b < SP_BINS; b += blockDim.x) {
            u64 t = bins[b];
#pragma unroll
            for (int c = 1; c < SP_SUBS; c++) t += bins[c * SP_BINS + b];
            bins[b] = t;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // lane l owns bins [128 l, 128 l + 127]; walk from the top bin down
            int lane = threadIdx.x;
            const int per = SP_BINS / 32;
            u64 mine = 0;
            for (int b = 0; b < per; b++) mine += bins[lane * per + b];
            // weight of all bins above this lane's range
            u64 above = 0;
            for (int l = 31; l > 0; l--) {
                u64 v = __shfl_sync(0xffffffffu, mine, l);
                if (lane < l) above += v;
            }
            u64 remaining = s_remaining;
            int owner = (above < remaining && above + mine >= remaining) ? 1 : 0;
            unsigned ballot = __ballot_sync(0xffffffffu, owner);
            if (ballot == 0) {
                if (lane == 0) s_found = 0;
            } else if (owner) {
                u64 acc = above;
                int chosen = lane * per;
                for (int b = per - 1; b >= 0; b--) {
                    u64 w = bins[lane * per + b];
                    if (acc + w >= remaining) { chosen = lane * per + b; break; }
                    acc += w;
                }
                s_prefix = prefix | ((u64)chosen << shift);
                s_remaining = remaining - acc;
                s_above += acc;
            }
        }
        __syncthreads();
        if (!s_found) break;
    }
    __syncthreads();
    int f = s_found;
    u64 K = f ? s_prefix : 0;
    __syncthreads();                 // every thread has its copies before the next call resets them
    *found = f;
    *reached = 0;
    if (f) {
        // exact weight of the tokens with floor_key <= key and key >= K
        u64 part = 0;
        for (int i = threadIdx.x; i < r.vocab; i += blockDim.x) {
            float zi = r.z(i);
            u64 k = r.key(i, zi);
            if (k >= floor_key && k >= K) part += weight_of(zi, zmax, counting);
        }
        *reached = block_sum_u64(part, red);
    }
    return K;
}

__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, const unsigned char* __restrict__ seen,
              const int* __restrict__ seen_rows, long long seen_stride, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ penalty,
              const float* __restrict__ uniform, int* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char sp_smem[];
    u64* bins = reinterpret_cast<u64*>(sp_smem);              // SP_SUBS copies of SP_BINS bins
    __shared__ u64 red[33];
    __shared__ float fred[33];
    __shared__ int ired[33];
    int row = blockIdx.x;
    RowView r;
    r.logits = logits + (size_t)row * row_stride;
    r.penalty = penalty ? penalty[row] : 1.0f;
    r.seen = (seen && r.penalty != 1.0f) ? seen + (size_t)(seen_rows ? seen_rows[row] : row) * seen_stride : nullptr;
    r.temperature = temperature[row];
    r.vocab = vocab;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // maximum of x and its first index (greedy answer; also the softmax shift)
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = r.x(i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { fred[warp] = best; ired[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (fred[w] > best || (fred[w] == best && ired[w] < bi)) { best = fred[w]; bi = ired[w]; }
        if (bi == 0x7fffffff) bi = 0;          // a row of NaN: the reference's loop also ends at index 0
        fred[32] = best;
        ired[32] = bi;
    }
    __syncthreads();
    best = fred[32];
    bi = ired[32];
    if (!(r.temperature > 0.0f)) {
        if (threadIdx.x == 0) out[row] = bi;
        return;
    }
    float zmax = best / r.temperature;

    int found;
    u64 reached;
    u64 floor_key = 0;
    int k = top_k ? top_k[row] : 0;
    if (k > 0 && k < vocab) {
        u64 K = radix_select(r, zmax, 1, 0, (u64)k, bins, red, &found, &reached);
        if (found) floor_key = K;
    }
    // total weight of the kept tokens
    u64 part = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float zi = r.z(i);
        if (r.key(i, zi) >= floor_key) part += weight_of(zi, zmax, 0);
    }
    u64 total = block_sum_u64(part, red);
    float tp = top_p ? top_p[row] : 1.0f;
    if (tp < 1.0f) {
        double want = (double)tp * (double)total;
        u64 target = (u64)want;
        if ((double)target < want) target += 1;           // ceil
        if (target < 1) target = 1;
        u64 K = radix_select(r, zmax, 0, floor_key, target, bins, red, &found, &reached);
        if (found) { floor_key = K; total = reached; }
    }
    double ru = (double)uniform[row] * (double)total;
    u64 target = (u64)ru + 1;                               // running sum > u * total
    if (target > total) target = total;
    u64 K = radix_select(r, zmax, 0, floor_key, target, bins, red, &found, &reached);
    if (threadIdx.x == 0) {
        int tok;
        if (found) tok = (int)(((1u << SP_IDX_BITS) - 1u) - (unsigned)(K & ((1u << SP_IDX_BITS) - 1u)));
        else tok = bi;                                      // cannot happen for total > 0; stay in range
        if (total == 0) tok = bi;
        out[row] = tok;
    }
}

// ---------------------------------------------------------------------------
// The same selection with several blocks per row, for large vocabularies: a row of 150,000 logits
// keeps one block busy for more than a millisecond.  The row is cut into slices, a block per slice
// and row; what the one-block kernel keeps in shared memory between its passes lies in global
// memory (SpRow, and a histogram of SP_BINS 64-bit sums per row), and every pass is a kernel of
// its own, so no block ever waits for another.  Sums are integers, so their order does not matter:
// the token is the one-block kernel's, bit for bit.
//
//   sp_max -> sp_begin -> [top-k: select] -> sp_total -> [top-p: select -> sp_total] -> select (the draw)
//   select = sp_select_begin -> SP_PASSES x (sp_hist -> sp_pick) -> sp_select_end
//
// These kernels are the form for batches too large for all their blocks to be on the device at once; smaller
// batches take sp_fused_kernel further down, the same passes in one launch.
// ---------------------------------------------------------------------------
#define SPW_THREADS 256
#define SPW_MAX_SLICES 64
enum { SP_MODE_TOPK = 0, SP_MODE_TOPP = 1, SP_MODE_DRAW = 2 };

struct __align__(16) SpRow {
    u64 floor_key;       // tokens with a smaller key are out (top-k, top-p)
    u64 total;           // weight of the tokens that are in
    u64 prefix, remaining, target;       // the radix search
    float best, zmax;    // maximum of x; of z
    int best_idx;        // first index of the maximum: the greedy answer
    int found, active, counting, done;
    int pad[5];
};

struct SpArgs {
    const float* logits;
    long long row_stride;
    const unsigned char* seen;
    const int* seen_rows;
    long long seen_stride;
    int vocab, slices, per_slice;
    const float* temperature;
    const int* top_k;
    const float* top_p;
    const float* penalty;
    const float* uniform;
    int* out;
    SpRow* st;           // [rows]
    u64* hist;           // [rows][SP_BINS]
    float* part_val;     // [rows][slices]
    int* part_idx;       // [rows][slices]
};

__device__ __forceinline__ RowView spw_row(const SpArgs& a, int row) {
    RowView r;
    r.logits = a.logits + (size_t)row * a.row_stride;
    r.penalty = a.penalty ? a.penalty[row] : 1.0f;
    r.seen = (a.seen && r.penalty != 1.0f) ? a.seen + (size_t)(a.seen_rows ? a.seen_rows[row] : row) * a.seen_stride : nullptr;
    r.temperature = a.temperature[row];
    r.vocab = a.vocab;
    return r;
}

// maximum of x over a slice, with the first index among equals
__global__ void __launch_bounds__(SPW_THREADS) sp_max_kernel(SpArgs a) {
    __shared__ float fred[SPW_THREADS / 32];
    __shared__ int ired[SPW_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y, s = blockIdx.x;
    const RowView r = spw_row(a, row);
    const int lo = s * a.per_slice, hi = min(a.vocab, lo + a.per_slice);
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
        float v = r.x(i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { fred[warp] = best; ired[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SPW_THREADS / 32; w++)
            if (fred[w] > best || (fred[w] == best && ired[w] < bi)) { best = fred[w]; bi = ired[w]; }
        a.part_val[(size_t)row * a.slices + s] = best;
        a.part_idx[(size_t)row * a.slices + s] = bi;
    }
}

// one block per row: the row's maximum from the slices', the greedy answer, a clean state and histogram
__global__ void __launch_bounds__(SPW_THREADS) sp_begin_kernel(SpArgs a) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    u64* hist = a.hist + (size_t)row * SP_BINS;
    for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS) hist[b] = 0;
    if (threadIdx.x == 0) {
        float best = -FLT_MAX;
        int bi = 0x7fffffff;
        for (int s = 0; s < a.slices; s++) {
            const float v = a.part_val[(size_t)row * a.slices + s];
            const int i = a.part_idx[(size_t)row * a.slices + s];
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
        if (bi == 0x7fffffff) bi = 0;          // a row of NaN: the reference's loop also ends at index 0
        SpRow& st = a.st[row];
        const float t = a.temperature[row];
        st.best = best;
        st.best_idx = bi;
        st.floor_key = 0;
        st.total = 0;
        st.done = !(t > 0.0f);
        st.zmax = st.done ? 0.0f : best / t;
        st.found = 0;
        st.active = 0;
        st.counting = 0;
        if (st.done) a.out[row] = bi;          // temperature <= 0: greedy
    }
}

// weight of the slice's tokens that are in, added to the row's total
__global__ void __launch_bounds__(SPW_THREADS) sp_total_kernel(SpArgs a) {
    __shared__ u64 red[33];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y, s = blockIdx.x;
    const SpRow& st = a.st[row];
    if (st.done) return;
    const RowView r = spw_row(a, row);
    const float zmax = st.zmax;
    const u64 floor_key = st.floor_key;
    const int lo = s * a.per_slice, hi = min(a.vocab, lo + a.per_slice);
    u64 part = 0;
    for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
        float zi = r.z(i);
        if (r.key(i, zi) >= floor_key) part += weight_of(zi, zmax, 0);
    }
    part = block_sum_u64(part, red);
    if (threadIdx.x == 0 && part) atomicAdd(&a.st[row].total, part);
}


// one thread per row: whether this search applies to the row, and its target
__global__ void sp_select_begin_kernel(SpArgs a, int mode, int rows) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    SpRow& st = a.st[row];
    st.active = 0;
    if (st.done) return;
    if (mode == SP_MODE_TOPK) {
        const int k = a.top_k ? a.top_k[row] : 0;
        if (k > 0 && k < a.vocab) {
            st.active = 1;
            st.counting = 1;
            st.target = (u64)k;
        }
    } else if (mode == SP_MODE_TOPP) {
        const float tp = a.top_p ? a.top_p[row] : 1.0f;
        if (tp < 1.0f) {
            const double want = (double)tp * (double)st.total;
            u64 target = (u64)want;
            if ((double)target < want) target += 1;           // ceil
            if (target < 1) target = 1;
            st.active = 1;
            st.counting = 0;
            st.target = target;
        }
    } else {
        const double ru = (double)a.uniform[row] * (double)st.total;
        u64 target = (u64)ru + 1;                             // running sum > u * total
        if (target > st.total) target = st.total;
        st.active = 1;
        st.counting = 0;
        st.target = target;
    }
    if (st.active) {
        st.prefix = 0;
        st.remaining = st.target;
        st.found = 1;
    }
}

// one digit of the search: the slice's histogram of that digit, added to the row's
__global__ void __launch_bounds__(SPW_THREADS) sp_hist_kernel(SpArgs a, int pass) {
    __shared__ u64 bins[SP_BINS];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y, s = blockIdx.x;
    const SpRow& st = a.st[row];
    if (!st.active || !st.found) return;
    const RowView r = spw_row(a, row);
    const float zmax = st.zmax;
    const u64 floor_key = st.floor_key, prefix = st.prefix;
    const int counting = st.counting, shift = pass * SP_DIGIT;
    for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS) bins[b] = 0;
    __syncthreads();
    const int lo = s * a.per_slice, hi = min(a.vocab, lo + a.per_slice);
    for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
        float zi = r.z(i);
        u64 k = r.key(i, zi);
        if (k < floor_key) continue;
        if (pass < SP_PASSES - 1 && (k >> (shift + SP_DIGIT)) != (prefix >> (shift + SP_DIGIT))) continue;
        u64 w = weight_of(zi, zmax, counting);
        if (w) atomicAdd(&bins[(unsigned)(k >> shift) & (SP_BINS - 1)], w);
    }
    __syncthreads();
    u64* hist = a.hist + (size_t)row * SP_BINS;
    for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS)
        if (bins[b]) atomicAdd(&hist[b], bins[b]);
}

// one block per row: the bin of this digit in which the target is reached; the histogram is left clean
__global__ void __launch_bounds__(SPW_THREADS) sp_pick_kernel(SpArgs a, int pass) {
    __shared__ u64 sh[SP_BINS];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    SpRow& st = a.st[row];
    __shared__ int go;                     // read once for the block: a lane below may clear `found`
    if (threadIdx.x == 0) go = st.active && st.found;
    __syncthreads();
    if (!go) return;
    // the histogram into shared memory, all threads side by side, and clean again for the next digit
    u64* hist = a.hist + (size_t)row * SP_BINS;
    for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS) {
        sh[b] = hist[b];
        hist[b] = 0;
    }
    __syncthreads();
    const int shift = pass * SP_DIGIT;
    if (threadIdx.x < 32) {
        // lane l owns bins [128 l, 128 l + 127]; walk from the top bin down
        const int lane = threadIdx.x;
        const int per = SP_BINS / 32;
        u64 mine = 0;
        for (int b = 0; b < per; b++) mine += sh[lane * per + b];
        u64 above = 0;                                        // weight of all bins above this lane's range
        for (int l = 31; l > 0; l--) {
            u64 v = __shfl_sync(0xffffffffu, mine, l);
            if (lane < l) above += v;
        }
        const u64 remaining = st.remaining, prefix = st.prefix;
        const int owner = (above < remaining && above + mine >= remaining) ? 1 : 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, owner);
        if (ballot == 0) {
            if (lane == 0) st.found = 0;
        } else if (owner) {
            u64 acc = above;
            int chosen = lane * per;
            for (int b = per - 1; b >= 0; b--) {
                u64 w = sh[lane * per + b];
                if (acc + w >= remaining) { chosen = lane * per + b; break; }
                acc += w;
            }
            st.prefix = prefix | ((u64)chosen << shift);
            st.remaining = remaining - acc;
        }
    }
}

// one thread per row: what the search found becomes the new floor (top-k, top-p) or the token (the draw)
__global__ void sp_select_end_kernel(SpArgs a, int mode, int rows) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    SpRow& st = a.st[row];
    if (st.done) return;
    if (mode == SP_MODE_DRAW) {
        int tok = st.best_idx;                                // cannot happen for total > 0; stay in range
        if (st.active && st.found && st.total != 0)
            tok = (int)(((1u << SP_IDX_BITS) - 1u) - (unsigned)(st.prefix & ((1u << SP_IDX_BITS) - 1u)));
        a.out[row] = tok;
        return;
    }
    if (st.active && st.found) st.floor_key = st.prefix;
    st.total = 0;                                             // the kernel after this one sums what is in now
}

// ---------------------------------------------------------------------------
// The same passes as one kernel.  The grid is (slices, rows) as above, launched cooperatively so that all blocks
// are on the device together, and the blocks of a row meet at a barrier of their own after every pass (an arrival
// counter per row that every block adds to and then polls; rows never wait for each other).  There is no row
// state in memory between the passes: after a barrier EVERY block of the row reads what the pass produced (the
// slices' maxima, a total, the row's histogram of 4,096 bins) and takes the row's small step itself, so all of
// them hold the same floor, prefix and remaining weight in registers and nobody waits for a leader.  The row's
// histogram has three copies that take turns: while a pass adds to one, the blocks clear the next, and the one
// before may still be read by a block that is late.  Sums are the same integers as in the other forms, so the
// token is the same bit for bit.  A pass costs about five trips to the L2 cache; a draw at a temperature is seven
// passes, a top-k or a top-p six more each.  Every wait is bounded by time (error 5, and the block returns).
//
// Scratch memory per row (SpFusedRow): zero at the start for `arrive` and `totals`: the launcher clears them.
// ---------------------------------------------------------------------------
#define SPF_TOTALS 4
struct __align__(16) SpFusedRow {
    unsigned arrive;
    unsigned pad[3];
    u64 totals[SPF_TOTALS];
};

struct SpFusedArgs {
    SpArgs a;
    SpFusedRow* rows;        // [rows]
    u64* hist3;              // [rows][3][SP_BINS]
    int* err;
};

// every block of the row has finished its pass and its writes are visible; false when the wait ran out
__device__ bool spf_barrier(unsigned* arrive, unsigned target, bool wait, int* err) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(arrive, 1u);
        int ok = 1;
        if (wait) {
            const unsigned long long start = ri_globaltimer();
            volatile unsigned* v = arrive;
            unsigned spins = 0;
            while (*v < target) {
                if ((++spins & 255u) == 0 && ri_globaltimer() - start > 4000000ull) {
                    atomicExch(err, 5);
                    ok = 0;
                    break;
                }
            }
            __threadfence();
        }
        s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
}

// the sum of `mine` over the lanes above this one, in five steps
__device__ __forceinline__ u64 spf_sum_above(u64 mine, int lane) {
    u64 suffix = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 v = __shfl_down_sync(0xffffffffu, suffix, o);
        if (lane + o < 32) suffix += v;
    }
    return suffix - mine;
}

__global__ void __launch_bounds__(SPW_THREADS) sp_fused_kernel(SpFusedArgs f, int use_top_k, int use_top_p) {
    __shared__ u64 bins[SP_BINS];
    __shared__ u64 red[33];
    __shared__ float fred[SPW_THREADS / 32];
    __shared__ int ired[SPW_THREADS / 32];
    __shared__ u64 s_prefix, s_remaining, s_group[32];
    __shared__ int s_found;
    const SpArgs& a = f.a;
    const int row = blockIdx.y, s = blockIdx.x, slices = a.slices;
    SpFusedRow* shared_row = f.rows + row;
    u64* hist3 = f.hist3 + (size_t)row * 3 * SP_BINS;
    const RowView r = spw_row(a, row);
    const int lo = s * a.per_slice, hi = min(a.vocab, lo + a.per_slice);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned barriers = 0;                 // barriers of this row so far
    int hp = 0, ti = 0;                    // histogram passes and total passes so far

    // this block's share of a copy of the row's histogram, cleared
    auto clear_share = [&](int copy) {
        u64* h = hist3 + (size_t)copy * SP_BINS;
        const int per = (SP_BINS + slices - 1) / slices;
        for (int b = s * per + threadIdx.x; b < min(SP_BINS, (s + 1) * per); b += SPW_THREADS) h[b] = 0;
    };

    // ---- the slice's maximum of x and its first index ----------------------------------------------------------
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
        float v = r.x(i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { fred[warp] = best; ired[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SPW_THREADS / 32; w++)
            if (fred[w] > best || (fred[w] == best && ired[w] < bi)) { best = fred[w]; bi = ired[w]; }
        a.part_val[(size_t)row * slices + s] = best;
        a.part_idx[(size_t)row * slices + s] = bi;
    }
    clear_share(0);
    if (!spf_barrier(&shared_row->arrive, ++barriers * (unsigned)slices, true, f.err)) return;
    // the row's maximum from the slices' (every block the same walk, in slice order)
    if (threadIdx.x == 0) {
        float rb = -FLT_MAX;
        int ri = 0x7fffffff;
        for (int q = 0; q < slices; q++) {
            const float v = __ldcg(a.part_val + (size_t)row * slices + q);
            const int i = __ldcg(a.part_idx + (size_t)row * slices + q);
            if (v > rb || (v == rb && i < ri)) { rb = v; ri = i; }
        }
        if (ri == 0x7fffffff) ri = 0;      // a row of NaN: the reference's loop also ends at index 0
        fred[0] = rb;
        ired[0] = ri;
    }
    __syncthreads();
    best = fred[0];
    bi = ired[0];
    __syncthreads();
    if (!(r.temperature > 0.0f)) {
        if (s == 0 && threadIdx.x == 0) a.out[row] = bi;       // greedy
        return;
    }
    const float zmax = best / r.temperature;
    u64 floor_key = 0, total = 0;

    // the weight of the tokens that are in: the slices' parts added in memory, read back by every block
    auto sum_total = [&]() -> bool {
        u64 part = 0;
        for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
            float zi = r.z(i);
            if (r.key(i, zi) >= floor_key) part += weight_of(zi, zmax, 0);
        }
        part = block_sum_u64(part, red);
        if (threadIdx.x == 0 && part) atomicAdd(&shared_row->totals[ti], part);
        if (!spf_barrier(&shared_row->arrive, ++barriers * (unsigned)slices, true, f.err)) return false;
        total = __ldcg(&shared_row->totals[ti]);
        ti++;
        return true;
    };
    // The radix search (see radix_select): the largest key K such that the tokens with floor_key <= key and key >= K
    // weigh `target` or more.  `last`: nobody but slice 0 needs the result of the last digit.
    auto select = [&](u64 target, int counting, bool last, u64* K, int* found_out) -> bool {
        u64 prefix = 0, remaining = target;
        int found = 1;
        for (int pass = SP_PASSES - 1; pass >= 0; pass--, hp++) {
            const int shift = pass * SP_DIGIT;
            u64* hist = hist3 + (size_t)(hp % 3) * SP_BINS;
            if (found && pass == SP_PASSES - 1) {
                // The top digit (sign, exponent, three bits of the mantissa): the tokens crowd into a few bins.  A
                // 64-bit addition to shared memory is a compare-and-swap loop that crawls when many threads want
                // one address, so a bin is kept as two 32-bit words: the low word is added with the old value
                // coming back (which tells whether this addition carried), the high word takes the carry along.
                unsigned* lo32 = reinterpret_cast<unsigned*>(bins);
                unsigned* hi32 = lo32 + SP_BINS;
                for (int b = threadIdx.x; b < 2 * SP_BINS; b += SPW_THREADS) lo32[b] = 0;
                __syncthreads();
                for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
                    float zi = r.z(i);
                    u64 k = r.key(i, zi);
                    if (k < floor_key) continue;
                    const u64 w = weight_of(zi, zmax, counting);
                    if (!w) continue;
                    const unsigned bin = (unsigned)(k >> shift) & (SP_BINS - 1);
                    const unsigned w_lo = (unsigned)w, w_hi = (unsigned)(w >> 32);
                    const unsigned old = atomicAdd(&lo32[bin], w_lo);
                    const unsigned carry = old + w_lo < old ? 1u : 0u;
                    if (w_hi + carry) atomicAdd(&hi32[bin], w_hi + carry);
                }
                __syncthreads();
                for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS) {
                    const u64 v = ((u64)hi32[b] << 32) + lo32[b];
                    if (v) atomicAdd(&hist[b], v);
                }
            } else if (found) {
                // a lower digit: only the tokens that share the digits found so far count, a handful as a rule;
                // they are added to the row's histogram directly
                for (int i = lo + threadIdx.x; i < hi; i += SPW_THREADS) {
                    float zi = r.z(i);
                    u64 k = r.key(i, zi);
                    if (k < floor_key) continue;
                    if ((k >> (shift + SP_DIGIT)) != (prefix >> (shift + SP_DIGIT))) continue;
                    u64 w = weight_of(zi, zmax, counting);
                    if (w) atomicAdd(&hist[(unsigned)(k >> shift) & (SP_BINS - 1)], w);
                }
            }
            clear_share((hp + 1) % 3);
            const bool waits = !(last && pass == 0) || s == 0;
            if (!spf_barrier(&shared_row->arrive, ++barriers * (unsigned)slices, waits, f.err)) return false;
            if (!waits) return true;                   // the last digit of the draw: slice 0 finishes alone
            if (found) {
                for (int b = threadIdx.x; b < SP_BINS; b += SPW_THREADS) bins[b] = __ldcg(hist + b);
                __syncthreads();
                // sums of the 32 groups of 128 bins: a warp takes four groups, its lanes stride through a group
                // (neighbouring lanes, neighbouring bins: no two lanes on one bank)
                {
                    const int per = SP_BINS / 32;
#pragma unroll
                    for (int q = 0; q < 32 / (SPW_THREADS / 32); q++) {
                        const int g = warp * (32 / (SPW_THREADS / 32)) + q;
                        u64 t = 0;
#pragma unroll
                        for (int j = 0; j < per / 32; j++) t += bins[g * per + j * 32 + lane];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                        if (lane == 0) s_group[g] = t;
                    }
                }
                __syncthreads();
                if (threadIdx.x < 32) {
                    // lane l stands for group l; from the top group down
                    const int per = SP_BINS / 32;
                    const u64 mine = s_group[lane];
                    const u64 above = spf_sum_above(mine, lane);
                    const int owner = (above < remaining && above + mine >= remaining) ? 1 : 0;
                    const unsigned ballot = __ballot_sync(0xffffffffu, owner);
                    if (ballot == 0) {
                        if (lane == 0) s_found = 0;
                    } else {
                        // inside the owning group the same once more: lane l holds bins 4 l .. 4 l + 3 of it
                        const int g = __ffs(ballot) - 1;
                        const u64 g_above = __shfl_sync(0xffffffffu, above, g);
                        u64 b4[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) b4[j] = bins[g * per + 4 * lane + j];
                        const u64 mine4 = (b4[0] + b4[1]) + (b4[2] + b4[3]);
                        const u64 above4 = g_above + spf_sum_above(mine4, lane);
                        if (above4 < remaining && above4 + mine4 >= remaining) {
                            u64 acc = above4;
                            int chosen = g * per + 4 * lane;
#pragma unroll
                            for (int j = 3; j >= 0; j--) {
                                if (acc + b4[j] >= remaining) { chosen = g * per + 4 * lane + j; break; }
                                acc += b4[j];
                            }
                            s_prefix = prefix | ((u64)chosen << shift);
                            s_remaining = remaining - acc;
                            s_found = 1;
                        }
                    }
                }
                __syncthreads();
                found = s_found;
                if (found) { prefix = s_prefix; remaining = s_remaining; }
                __syncthreads();
            }
        }
        *K = prefix;
        *found_out = found;
        return true;
    };

    u64 K;
    int found;
    const int k = (use_top_k && a.top_k) ? a.top_k[row] : 0;
    if (k > 0 && k < a.vocab) {
        if (!select((u64)k, 1, false, &K, &found)) return;
        if (found) floor_key = K;
    }
    if (!sum_total()) return;
    const float tp = (use_top_p && a.top_p) ? a.top_p[row] : 1.0f;
    if (tp < 1.0f) {
        const double want = (double)tp * (double)total;
        u64 target = (u64)want;
        if ((double)target < want) target += 1;           // ceil
        if (target < 1) target = 1;
        if (!select(target, 0, false, &K, &found)) return;
        if (found) floor_key = K;
        if (!sum_total()) return;
    }
    const double ru = (double)a.uniform[row] * (double)total;
    u64 target = (u64)ru + 1;                             // running sum > u * total
    if (target > total) target = total;
    if (!select(target, 0, true, &K, &found)) return;
    if (s == 0 && threadIdx.x == 0) {
        int tok = bi;                                     // cannot happen for total > 0; stay in range
        if (found && total != 0) tok = (int)(((1u << SP_IDX_BITS) - 1u) - (unsigned)(K & ((1u << SP_IDX_BITS) - 1u)));
        a.out[row] = tok;
    }
}

static size_t spw_align(size_t n) { return (n + 255) & ~(size_t)255; }
static int spw_slices(int vocab) {
    int s = (vocab + 2047) / 2048;
    return s < 1 ? 1 : (s > SPW_MAX_SLICES ? SPW_MAX_SLICES : s);
}

// bytes of scratch memory the several-blocks-per-row selection needs
extern "C" long long ri_sample_work_bytes(int rows, int vocab) {
    const int slices = spw_slices(vocab);
    return (long long)(spw_align((size_t)rows * sizeof(SpRow)) + spw_align((size_t)rows * SP_BINS * sizeof(u64)) +
                       2 * spw_align((size_t)rows * slices * 4) + spw_align((size_t)rows * sizeof(SpFusedRow)) +
                       spw_align((size_t)rows * 3 * SP_BINS * sizeof(u64)));
}

// how many blocks of the one-kernel form the device holds at once (0: it cannot be used)
static int spw_fused_capacity() {
    static int capacity = -1;
    if (capacity < 0) {
        int dev = 0, sms = 0, per_sm = 0, coop = 0;
        capacity = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sp_fused_kernel, SPW_THREADS, 0) == cudaSuccess)
            capacity = sms * per_sm;
    }
    return capacity;
}

static int launch_sample_wide(SpArgs a, int rows, void* work, int use_top_k, int use_top_p, int* err_flag, int one_kernel,
                              cudaStream_t stream) {
    unsigned char* w = (unsigned char*)work;
    a.slices = spw_slices(a.vocab);
    a.st = (SpRow*)w;
    w += spw_align((size_t)rows * sizeof(SpRow));
    a.hist = (u64*)w;
    w += spw_align((size_t)rows * SP_BINS * sizeof(u64));
    a.part_val = (float*)w;
    w += spw_align((size_t)rows * a.slices * 4);
    a.part_idx = (int*)w;
    w += spw_align((size_t)rows * a.slices * 4);
    SpFusedRow* fused_rows = (SpFusedRow*)w;
    w += spw_align((size_t)rows * sizeof(SpFusedRow));
    u64* hist3 = (u64*)w;
    use_top_k = use_top_k && a.top_k;
    use_top_p = use_top_p && a.top_p;
    if (one_kernel && err_flag && spw_fused_capacity() >= rows) {
        // all blocks must be on the device together: as many slices per row as that allows
        const int fit = spw_fused_capacity() / rows;
        if (a.slices > fit) a.slices = fit;
        a.per_slice = (a.vocab + a.slices - 1) / a.slices;
        cudaError_t e = cudaMemsetAsync(fused_rows, 0, (size_t)rows * sizeof(SpFusedRow), stream);
        if (e != cudaSuccess) RI_FAIL((int)e, "sample: %s", cudaGetErrorString(e));
        SpFusedArgs f;
        f.a = a;
        f.rows = fused_rows;
        f.hist3 = hist3;
        f.err = err_flag;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(a.slices, rows);
        cfg.blockDim = dim3(SPW_THREADS);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, sp_fused_kernel, f, use_top_k, use_top_p);
        if (e != cudaSuccess) RI_FAIL((int)e, "sample (one kernel): %s", cudaGetErrorString(e));
        return 0;
    }
    a.per_slice = (a.vocab + a.slices - 1) / a.slices;
    const dim3 wide(a.slices, rows), per_row(rows), few((rows + 127) / 128);
    auto select = [&](int mode) {
        ri_launch_pdl(sp_select_begin_kernel, few, dim3(128), 0, stream, a, mode, rows);
        for (int pass = SP_PASSES - 1; pass >= 0; pass--) {
            ri_launch_pdl(sp_hist_kernel, wide, dim3(SPW_THREADS), 0, stream, a, pass);
            ri_launch_pdl(sp_pick_kernel, per_row, dim3(SPW_THREADS), 0, stream, a, pass);
        }
        ri_launch_pdl(sp_select_end_kernel, few, dim3(128), 0, stream, a, mode, rows);
    };
    ri_launch_pdl(sp_max_kernel, wide, dim3(SPW_THREADS), 0, stream, a);
    ri_launch_pdl(sp_begin_kernel, per_row, dim3(SPW_THREADS), 0, stream, a);
    if (use_top_k) select(SP_MODE_TOPK);
    ri_launch_pdl(sp_total_kernel, wide, dim3(SPW_THREADS), 0, stream, a);
    if (use_top_p) {
        select(SP_MODE_TOPP);
        ri_launch_pdl(sp_total_kernel, wide, dim3(SPW_THREADS), 0, stream, a);
    }
    select(SP_MODE_DRAW);
    RI_CHECK_LAUNCH("sample (several blocks per row)");
    return 0;
}

extern "C" int ri_sample(const float* logits, long long row_stride, int rows, int vocab, const unsigned char* seen,
                         const int* seen_rows, long long seen_stride, const float* temperature, const int* top_k,
                         const float* top_p, const float* penalty, const float* uniform, int* out,
                         void* work, long long work_bytes, int use_top_k, int use_top_p, int* err_flag, int one_kernel,
                         cudaStream_t stream) {
    if (rows == 0) return 0;
    RI_REQUIRE(rows > 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    RI_REQUIRE(vocab <= (1 << SP_IDX_BITS), "sample: vocabulary %d exceeds the limit %d", vocab, 1 << SP_IDX_BITS);
    RI_REQUIRE(temperature && uniform && out, "sample: temperature, uniform and out are required");
    if (work) {
        // several blocks per row (the caller gives scratch memory for it): large vocabularies
        RI_REQUIRE(work_bytes >= ri_sample_work_bytes(rows, vocab), "sample: %lld bytes of scratch memory, %lld needed",
                   work_bytes, ri_sample_work_bytes(rows, vocab));
        RI_REQUIRE(rows <= 65535, "sample: %d rows", rows);
        SpArgs a{};
        a.logits = logits; a.row_stride = row_stride; a.seen = seen; a.seen_rows = seen_rows; a.seen_stride = seen_stride;
        a.vocab = vocab; a.temperature = temperature; a.top_k = top_k; a.top_p = top_p; a.penalty = penalty;
        a.uniform = uniform; a.out = out;
        return launch_sample_wide(a, rows, work, use_top_k, use_top_p, err_flag, one_kernel, stream);
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SP_SMEM_BYTES);
        if (e != cudaSuccess) RI_FAIL((int)e, "sample: shared memory limit: %s", cudaGetErrorString(e));
        configured = true;
    }
    sample_kernel<<<rows, SP_THREADS, SP_SMEM_BYTES, stream>>>(logits, row_stride, seen, seen_rows, seen_stride, vocab,
                                                   temperature, top_k, top_p, penalty, uniform, out);
    RI_CHECK_LAUNCH("sample");
    return 0;
}

// ---------------------------------------------------------------------------
// greedy only: first index of the row maximum (src/ops/reduce.rs:9-28)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(SP_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int* __restrict__ out) {
    __shared__ float fred[32];
    __shared__ int ired[32];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = x[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { fred[warp] = best; ired[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (fred[w] > best || (fred[w] == best && ired[w] < bi)) { best = fred[w]; bi = ired[w]; }
        out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Two stages for long rows: `slices` blocks per row each find the first maximum of their
// slice, a second kernel picks among the slices (lowest index on ties, so the result is the
// first maximum of the whole row).  part_val / part_idx: [rows, slices] scratch.
__global__ void __launch_bounds__(256)
argmax_slice_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int per_slice,
                    float* __restrict__ part_val, int* __restrict__ part_idx) {
    __shared__ float fred[8];
    __shared__ int ired[8];
    pdl_trigger();
    pdl_wait();
    const float* x = logits + (size_t)blockIdx.y * row_stride;
    int lo = blockIdx.x * per_slice, hi = min(vocab, lo + per_slice);
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = x[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { fred[warp] = best; ired[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (fred[w] > best || (fred[w] == best && ired[w] < bi)) { best = fred[w]; bi = ired[w]; }
        part_val[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best;
        part_idx[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = bi;
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int slices,
                                   int* __restrict__ out) {
    // one warp per row
    pdl_trigger();
    pdl_wait();
    int row = blockIdx.x, lane = threadIdx.x;
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int s = lane; s < slices; s += 32) {
        float v = part_val[(size_t)row * slices + s];
        int i = part_idx[(size_t)row * slices + s];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

extern "C" int ri_argmax_slices(int vocab) {
    int s = (vocab + 2047) / 2048;
    return s < 1 ? 1 : (s > 128 ? 128 : s);
}

// part_val, part_idx: [rows, ri_argmax_slices(vocab)] scratch (may be null when that is 1)
extern "C" int ri_argmax(const float* logits, long long row_stride, int rows, int vocab, int* out, float* part_val,
                         int* part_idx, cudaStream_t stream) {
    if (rows == 0) return 0;
    RI_REQUIRE(rows > 0 && vocab > 0, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
    int slices = ri_argmax_slices(vocab);
    if (slices == 1 || !part_val || !part_idx) {
        argmax_kernel<<<rows, SP_THREADS, 0, stream>>>(logits, row_stride, vocab, out);
        RI_CHECK_LAUNCH("argmax");
        return 0;
    }
    RI_REQUIRE(rows <= 65535, "argmax: at most 65535 rows");
    int per_slice = (vocab + slices - 1) / slices;
    ri_launch_pdl(argmax_slice_kernel, dim3(slices, rows), dim3(256), 0, stream, logits, row_stride, vocab, per_slice, part_val, part_idx);
    RI_CHECK_LAUNCH("argmax (slices)");
    ri_launch_pdl(argmax_pick_kernel, dim3(rows), dim3(32), 0, stream, (const float*)part_val, (const int*)part_idx, slices, out);
    RI_CHECK_LAUNCH("argmax (pick)");
    return 0;
}

// ---------------------------------------------------------------------------
// seen[row, token] = 1 for the given (row, token) pairs: the context of the
// repetition penalty, kept per sequence beside the cache.
// ---------------------------------------------------------------------------
__global__ void mark_seen_kernel(unsigned char* __restrict__ seen, long long seen_stride, const int* __restrict__ rows,
                                 const int* __restrict__ tokens, int n, int vocab) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int t = tokens[i];
    if (t >= 0 && t < vocab) seen[(size_t)rows[i] * seen_stride + t] = 1;
}

extern "C" int ri_mark_seen(unsigned char* seen, long long seen_stride, const int* rows, const int* tokens, int n,
                            int vocab, cudaStream_t stream) {
    if (n == 0) return 0;
    mark_seen_kernel<<<(n + 255) / 256, 256, 0, stream>>>(seen, seen_stride, rows, tokens, n, vocab);
    RI_CHECK_LAUNCH("mark_seen");
    return 0;
}
