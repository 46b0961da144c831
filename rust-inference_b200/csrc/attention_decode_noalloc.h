// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in thanhauco/rust-inference: there every
// operation allocates its output and work buffers on the stream as it goes
// (src/cuda/buffer.rs:15-24).  It exists here for hosts that cannot do that
// around a call: code running inside a fixed memory budget that was handed out at
// start-up (a plug-in of a larger server, a real-time loop that may not block in
// the driver's allocator), or code that is not linked against torch and has no
// allocator of its own to ask.  Such a caller owns its inputs and outputs and
// nothing else.
//
// `ri_attention_decode_noalloc` computes what `ri_attention_decode` computes, with
// the same arguments but no scratch pointers: the partial results of the key
// chunks live in a fixed array inside the library, RI_NOALLOC_SCRATCH_BYTES of
// device memory that every GPU which loads the library holds until the process
// exits.  The call makes no cudaMalloc, cudaFree or other allocating call.
// It always runs the kernel with one block per chunk of 128 keys
// (attention_decode_kernel) and the merge kernel; `ri_attention_decode` takes its
// streaming kernel for groups of up to 16 query heads of size 64 or 128, so the
// two entry points agree within the rounding of bfloat16 weights, not bit for
// bit, and this one is the slower of the two in those cases.
//
// Limits and rules
//  * seqs * H * max_chunks * (head_dim + 2) * 4 bytes must fit in the array
//    (each of the two parts rounded up to 256 bytes); larger calls are refused with
//    an error code and a message (`ri_last_error`), nothing is launched.
//  * The first call on a device looks up the array's device address and sets the
//    kernel's shared-memory limit.  Make that first call outside of any stream
//    capture, and from one host thread: the set-up is not guarded against two
//    threads making a device's first call at the same time.
//  * Pointers are checked before anything is launched: none may be null, q and
//    the pools must be 16-byte aligned (the kernels read them in 16-byte pieces).
//  * max_chunks * 128 must cover the longest sequence.  A longer sequence is not
//    followed past the scratch memory: its keys beyond are left out and err_flag
//    is set to 7.
//  * All calls share the one array and it keeps what the last call left.  Nothing
//    in it has to start at zero: a call writes every partial result before it reads
//    it.  But two calls that overlap on the GPU (different streams, or graphs
//    replayed side by side) race on it; keep calls on one stream or order them with
//    events.
#pragma once
#include <cuda_runtime.h>

#define RI_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// q, out            [seqs, H, Dh] bfloat16 (device)
// k_pool, v_pool    [num_pages, KV, 32, Dh] bfloat16 (device)
// page_table        [slots, mpps] int32; seq_slot, seq_len [seqs] int32 (device)
// max_chunks * 128 must cover the longest sequence; scale multiplies q.k; window 0 = all keys
// err_flag          one int32 on the device, set to 4 if a page index is out of range, to 7 if a
//                   sequence is longer than max_chunks * 128
// Returns 0, or a non-zero code with the reason in ri_last_error().
int ri_attention_decode_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                const int* page_table, const int* seq_slot, const int* seq_len, int seqs, int H,
                                int KV, int Dh, int mpps, int page_size, int num_pages, int max_chunks, float scale,
                                int window, int* err_flag, cudaStream_t stream);

// bytes of the fixed array that a call of these sizes would use (to check beforehand)
long long ri_attention_decode_noalloc_bytes(int seqs, int H, int Dh, int max_chunks);

#ifdef __cplusplus
}
#endif
