// Split-key decode attention for callers that may not allocate.
//
// This entry point has no counterpart in vt-transformer: it exists for programs that embed the
// kernels and cannot call cudaMalloc (or anything that allocates, torch included) at the time they
// need attention -- a host application that gave all device memory to its own pool at start-up, a
// plug-in that runs under someone else's memory budget, a service loop in which the implicit
// synchronisation of an allocation is not acceptable.
//
// It computes single-token attention over the paged cache with the keys of each sequence cut into `n_splits`
// runs: `attention_mma_kernel<head_dim, 1>` (one warp a (sequence, KV head, run)) followed by
// `attention_combine_kernel`, which merges the runs; the same two kernels as the extension's `attention_mma`
// with n_splits > 1.  (Generation itself decodes with another kernel, `attention_decode_kernel`, which merges its
// runs inside thread-block clusters; this pair is the form whose scratch is one plain array.)  The partial results
// of the runs, which the ordinary entry point puts into scratch tensors that its caller allocates, go into a
// fixed array that is part of this library's device image instead:
//
//     VTB_NOALLOC_SCRATCH_FLOATS = 2,097,152 floats (8 MiB), held by every GPU that loads the
//     library, from load until the process exits.
//
// A call needs n_splits * n_seqs * heads * (head_dim + 2) floats of it and is refused (return 1,
// one line on stderr) if that is more than the array holds.  The caller passes inputs and outputs
// only; nothing is allocated or freed, by this function or by anything it calls.
//
// Set-up: the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
// that device current) and remembers it for the device; the first launch of the kernel on a device
// also sets its shared-memory attribute there.  Make that first call before any stream capture begins.
// First calls from two host threads at once are harmless (both look up the same address).
//
// Sharing: every call uses the same array and finds the last call's contents in it.  Nothing has to
// start at zero -- each (run, sequence, head) of a call writes its own partial result before the
// merge reads it -- so nothing is cleared.  Two calls that overlap on the GPU (different streams)
// would write the same scratch: that is a race; keep calls in one stream or order them yourself.
//
// Arguments are those of the ordinary entry point, as plain device pointers:
//   qkv         bfloat16 [n_seqs, qkv_stride], the queries in the first heads * head_dim columns
//   out         bfloat16 [n_seqs, heads * head_dim]
//   k_cache, v_cache  bfloat16 [n_pages, kv_heads, page_size, head_dim]
//   cu_q        int32 [n_seqs + 1] = 0, 1, ..., n_seqs (one new token a sequence)
//   q_start     int32 [n_seqs], position of each sequence's token (= keys cached before it)
//   block_table int32 [n_seqs, table_stride], page of every 16.. tokens of a sequence
//   window      keys a token sees (0: all);  scale: multiplier of q.k;  stream: a cudaStream_t
// Returns 0, or 1 (too large for the array), 2 (arguments the kernel does not take: a null pointer, head_dim
// not a multiple of 16 up to 128, more than 16 heads a KV head, page_size not a positive multiple of 16,
// n_splits outside 1..64, qkv_stride below heads * head_dim, table_stride or n_pages below 1; nothing is
// launched), 3 (a CUDA call failed; its message goes to stderr).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define VTB_NOALLOC_SCRATCH_FLOATS 2097152

__attribute__((visibility("default"))) int vtb_decode_attention_noalloc(
    const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache, const int* cu_q,
    const int* q_start, const int* block_table, int table_stride, int n_seqs, int n_pages, int heads, int kv_heads,
    int head_dim, int page_size, int window, float scale, int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
