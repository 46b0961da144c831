// Decode attention behind an entry point that allocates nothing: see attention_decode_noalloc.h
// for who needs that and for the rules.  The scratch memory is the file-scope array below; the
// kernels are attention_decode_kernel and attention_decode_merge_kernel of attention_decode.cu.
#include "attention_decode.cu"
#include "attention_decode_noalloc.h"

// Partial results of the key chunks.  In host code this name is only a handle for
// the runtime, not a device address: the address is asked for once per device
// (cudaGetSymbolAddress) and passed to the kernels.
static __device__ __align__(256) unsigned char ri_noalloc_scratch[RI_NOALLOC_SCRATCH_BYTES];

static float* g_scratch_addr[AD_MAX_DEVICES];      // per device, filled by the first call on it

static size_t round256(size_t n) { return (n + 255) & ~(size_t)255; }

extern "C" long long ri_attention_decode_noalloc_bytes(int seqs, int H, int Dh, int max_chunks) {
    if (seqs <= 0 || H <= 0 || Dh <= 0 || max_chunks <= 0) return 0;
    size_t o = (size_t)seqs * H * max_chunks * Dh * sizeof(float);
    size_t ml = (size_t)seqs * H * max_chunks * 2 * sizeof(float);
    return (long long)(round256(o) + round256(ml));
}

// once per device, with that device current
static int noalloc_setup(int device) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, ri_noalloc_scratch);
    if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    size_t unused = 0;
    int rc = decode_configure(AD_ROWS, &unused);     // the one place that sets the kernel's shared-memory limit
    if (rc) return rc;
    g_scratch_addr[device] = (float*)p;
    return 0;
}

extern "C" int ri_attention_decode_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                           const int* page_table, const int* seq_slot, const int* seq_len, int seqs,
                                           int H, int KV, int Dh, int mpps, int page_size, int num_pages,
                                           int max_chunks, float scale, int window, int* err_flag,
                                           cudaStream_t stream) {
    if (seqs == 0) return 0;
    RI_REQUIRE(q && k_pool && v_pool && out && page_table && seq_slot && seq_len && err_flag,
               "attention_decode_noalloc: a null pointer among the arguments");
    RI_REQUIRE(Dh == AD_DH, "attention_decode_noalloc: built for head_dim %d, called with %d", AD_DH, Dh);
    RI_REQUIRE(page_size == AD_PAGE, "attention_decode_noalloc: pages of %d tokens, this kernel needs %d", page_size, AD_PAGE);
    RI_REQUIRE(seqs > 0 && H > 0 && KV > 0 && H % KV == 0, "attention_decode_noalloc: %d sequences, %d heads over %d kv heads", seqs, H, KV);
    RI_REQUIRE(max_chunks > 0 && max_chunks <= 65535 && seqs <= 65535 && KV <= 65535 && H <= 65535, "attention_decode_noalloc: bad grid");
    RI_REQUIRE(mpps > 0 && num_pages > 0, "attention_decode_noalloc: a page table of %d columns over %d pages", mpps, num_pages);
    RI_REQUIRE(window >= 0, "attention_decode_noalloc: negative window");
    // the kernels read q in 16-byte pieces, the keys with 16-byte loads and the values by bulk copies
    RI_REQUIRE((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0,
               "attention_decode_noalloc: q and the pools must be 16-byte aligned");
    RI_REQUIRE(((uintptr_t)out & 1) == 0 && (((uintptr_t)page_table | (uintptr_t)seq_slot | (uintptr_t)seq_len | (uintptr_t)err_flag) & 3) == 0,
               "attention_decode_noalloc: out must be 2-byte aligned, the int32 arguments 4-byte aligned");
    long long need = ri_attention_decode_noalloc_bytes(seqs, H, Dh, max_chunks);
    RI_REQUIRE(need <= (long long)RI_NOALLOC_SCRATCH_BYTES,
               "attention_decode_noalloc: %d sequences x %d heads x %d chunks x head_dim %d need %lld bytes of scratch, "
               "the fixed array holds %u", seqs, H, max_chunks, Dh, need, (unsigned)RI_NOALLOC_SCRATCH_BYTES);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) RI_FAIL((int)e, "attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    RI_REQUIRE(device >= 0 && device < AD_MAX_DEVICES, "attention_decode_noalloc: device %d", device);
    if (!g_scratch_addr[device]) {
        int rc = noalloc_setup(device);
        if (rc) return rc;
    }
    float* o_part = g_scratch_addr[device];
    float* ml_part = (float*)((unsigned char*)o_part + round256((size_t)seqs * H * max_chunks * Dh * sizeof(float)));
    dim3 grid(max_chunks, KV, seqs);
    const int G = H / KV;
    attention_decode_kernel<<<grid, 32 * AD_WARPS, decode_smem_bytes(G < AD_ROWS ? G : AD_ROWS), stream>>>(
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, o_part, ml_part, page_table, seq_slot, seq_len, H, KV,
        mpps, num_pages, max_chunks, scale * 1.4426950408889634f, window, err_flag);
    RI_CHECK_LAUNCH("attention_decode_noalloc");
    MergeCut chunks_of_128;                    // the partial results are those of chunks of 128 keys
    chunks_of_128.workers = 0;
    chunks_of_128.seqs = seqs;
    chunks_of_128.KV = KV;
    chunks_of_128.parts = max_chunks;
    attention_decode_merge_kernel<<<dim3(H, seqs), AD_MERGE_THREADS, 0, stream>>>(
        o_part, ml_part, (bf16*)out, seq_len, H, max_chunks, window, chunks_of_128, err_flag);
    RI_CHECK_LAUNCH("attention_decode_noalloc (merge)");
    return 0;
}
