// Launchers of the hand-written kernels.  Plain pointers and sizes; every launcher
// enqueues on `stream` and returns cudaGetLastError().  `status` points at two ints on
// the device (code, detail), see common.cuh; it may be null.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace vtb {

enum DType : int { kF32 = 0, kBF16 = 1 };

// out[t, :] = float(table[ids[t], :]).  hidden % 8 == 0.
cudaError_t launch_embedding(int table_dtype, const void* table, const int* ids, float* out, int n_tokens,
                             int hidden, int vocab, float scale, int* status, cudaStream_t stream);
// logits = cap * tanh(scale * logits / cap) in place; cap 0 applies the scale alone
cudaError_t launch_logits_scale_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream);

// For r in 0..n_rows: t = rows ? rows[r] : r; v = x[t] (+ delta[t], written back to x[t]);
// out[r] = weight * v * rsqrt(mean(v^2) + eps).  x float, weight float, delta/out of out_dtype.  Instead of
// delta: parts [n_parts, n_tokens, hidden] float, the unadded shares of a delta, added in the order of their index.
cudaError_t launch_rmsnorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                           const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                           int hidden, int* status, cudaStream_t stream);

// out[t, i] = silu(gate) * up.  interleave 0: gate = gu[t, i], up = gu[t, inter + i].  interleave 8: gate and up
// columns alternate in runs of 8 (g0..g7, u0..u7, g8.., ...): gate = gu[t, 16 (i / 8) + i % 8], up 8 further.
// inter % 8 == 0.
cudaError_t launch_silu_mul(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave,
                            cudaStream_t stream);

// Rotates q (in place) and k by the token's position and stores k and v into the pages.
// qkv [n_tokens, (heads + 2 kv_heads) * head_dim]; cos_sin [max_pos, head_dim / 2] of (cos, sin);
// k_cache, v_cache [pages, kv_heads, page_size, head_dim]; token_seq[t] < 0 marks padding.
// store == 0 rotates q only.
cudaError_t launch_rope_store(int dtype, void* qkv, const int* positions, const float2* cos_sin, int max_pos,
                              void* k_cache, void* v_cache, const int* token_seq, const int* block_table,
                              int table_stride, int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads,
                              int head_dim, int page_size, int rotate, int store, int* status, cudaStream_t stream);

// C[M, N] = A[M, K] W[N, K]^T (+ bias[N]) with 32-bit multiply-adds in a fixed order (no tensor cores).
// (in, out) dtypes: (float, float), (bfloat16, bfloat16), (bfloat16, float).  k % 4 == 0.
cudaError_t launch_gemm_simt(int in_dtype, int out_dtype, const void* a, const void* w, const float* bias, void* c,
                             int m, int n, int k, cudaStream_t stream);

// Attention of every token over the paged keys of its sequence, one warp for a (token, head).
// q is read from qkv [n_tokens, qkv_stride] at column head * head_dim; out [n_tokens, heads * head_dim].
// Token t at position p of sequence s sees keys j with max(0, p - window + 1) <= j <= p (window <= 0: all).
cudaError_t launch_attention_simt(int dtype, const void* qkv, int qkv_stride, void* out, const void* k_cache,
                                  const void* v_cache, const int* positions, const int* token_seq,
                                  const int* block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                                  int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                  int* status, cudaStream_t stream);

// out[M, N] = x[M, K] w[N, K]^T (+ bias) for M <= 64 rows of bfloat16 x: the weight-streaming kernel.
// out is bfloat16 or float.  k % 8 == 0.
cudaError_t launch_gemm_skinny(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n,
                               int k, cudaStream_t stream);

// out[M, N] = x[M, K] w[N, K]^T (+ bias) with tcgen05.mma fed by TMA, accumulators in tensor memory.
// bfloat16 x and w, out bfloat16 or float, any M and N, k % 8 == 0.  status receives kStatusWaitTimeout
// if a bounded wait inside the kernel runs out.  scratch (floats) and counters (ints, zero before the
// first launch; the kernel leaves them zero) let a small batch cut k over several CTAs; without them
// k is not cut.  Launches that share them must not overlap on the GPU.
// epilogue 0: out[M, N] = sums + bias.  epilogue 1 (bfloat16 out, no bias, N % 16 == 0): the rows of w are
// gate and up rows interleaved in runs of 8 (g0..g7, u0..u7, g8.., ...) and out[M, N / 2] = silu(gate) * up.
// epilogue 2 (float out, M <= 256): k is cut into gemm_tc_shares(M, N, K) shares and out[share, M, N] takes each
// share's sums as they are (the bias with share 0); the kernel that reads them adds them (launch_rmsnorm).
// NextProduct: the product that the stream runs after this one (its matrix [n, k] of bfloat16, which no kernel writes, and its
// epilogue).  A kernel that streams weights for a small batch asks the first `bytes` of what that product will read
// into L2 once its own last load is on its way, so that HBM has work between the two kernels.  A hint: it changes no result.
struct NextProduct {
    const void* w;
    int n, k, epilogue;
    long long bytes;
};
int gemm_tc_shares(int m, int n, int k);
cudaError_t launch_gemm_tc(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n, int k,
                           int epilogue, float* scratch, long long scratch_floats, int* counters, int n_counters,
                           int* status, cudaStream_t stream, const NextProduct* next = nullptr);
// The same product for many rows of x with a tile of 256 rows of x by `bn` (256 or 192) rows of w to a pair of CTAs
// (tcgen05.mma.cta_group::2): bfloat16 out, epilogue 0 (bias) or 1 (SiLU(gate) * up).
cudaError_t launch_gemm_tc_pair(const void* x, const void* w, const float* bias, void* out, int m, int n, int k, int epilogue,
                                int bn, float* scratch, long long scratch_floats, int* counters, int n_counters, int* status,
                                cudaStream_t stream);

// Tensor-core attention over the paged cache (bfloat16).  A tile is 16 * warps rows, row r being
// (token r / group, head r % group); `tiles` lists (sequence, first token) pairs, or is null when
// every sequence is one tile (single-token steps).  warps is 1 or 4.  With n_splits > 1 the keys of a
// tile are cut into n_splits runs whose partial results go to part_o [splits, tokens, heads, head_dim]
// and part_ml [splits, tokens, heads, 2] and are merged by a second kernel.
bool attention_mma_supports(int head_dim, int heads, int kv_heads, int warps);
cudaError_t launch_attention_mma(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                 const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                 const int* tiles, int n_tiles, int n_pages, int n_tokens, int heads, int kv_heads,
                                 int head_dim, int page_size, int window, float scale, int warps, int n_splits,
                                 float* part_o, float* part_ml, int* status, cudaStream_t stream);

// Attention of prompt portions on tcgen05 tensor cores with the scores in tensor memory (head size 128):
// tiles of 128 rows of (token, head of the group) as in launch_attention_mma with 8 warps.
bool attention_tc_supports(int head_dim, int heads, int kv_heads);
cudaError_t launch_attention_tc(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                const int* tiles, int n_tiles, int n_pages, int heads, int kv_heads, int head_dim,
                                int page_size, int window, float scale, int* status, cudaStream_t stream);

// Attention of single-token steps: every sequence brings tokens_per_tile = 16 / group tokens at most (one in a
// decode step).  Grid (sequences, kv_heads, n_splits), four warps a CTA.  With n_splits > 1 the runs' results
// pass through part_o [splits, tokens, heads, head_dim] and part_ml [splits, tokens, heads, 2], and
// counters [sequences * kv_heads] (zero before the first launch; left zero) tells the last CTA to merge.
// fuse_rope 1 (one token a sequence): q and k in qkv are still unrotated and the token's k and v are not in
// the cache; the kernel rotates q and k by cos_sin [max_pos, head_dim / 2] (null: no rotation) and, with
// store_kv, writes the token's k and v into their page: no rotation kernel has to run before it.  With fuse_rope,
// q, k and v may come as qkv_shares [n_shares, tokens, qkv_stride] float, the unadded shares of the product that
// made them (launch_gemm_tc, epilogue 2), instead of qkv: they are added where they are read.
// long_runs 1: the caller expects a warp to stream many blocks of keys (long contexts); head sizes 64 and 128 then
// fetch them as boxes of a tensor map, which arrive later than cp.async copies but cost far fewer instructions.
cudaError_t launch_attention_decode(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                    const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                    int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads, int head_dim,
                                    int page_size, int window, float scale, int n_splits, float* part_o, float* part_ml,
                                    int* counters, int fuse_rope, const float2* cos_sin, int max_pos, int store_kv,
                                    const float* qkv_shares, int n_shares, int long_runs, int run_blocks, int* status,
                                    cudaStream_t stream);

// out[r] = index of the largest logit of row r (the lowest index among equals).
cudaError_t launch_argmax(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream);

// Sampling of one token for each row of float logits [n_rows, vocab]:
// temperature[r] <= 0 or top_k[r] == 1: argmax.  Else p = softmax(logits / temperature) restricted to the
// top_k[r] largest (top_k <= 0: all) and then to the smallest set of largest p whose sum reaches top_p[r];
// the token is the first index, in index order, at which the running sum of the kept p exceeds u[r] * total.
cudaError_t launch_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                          const float* u, int* out, int n_rows, int vocab, cudaStream_t stream);

}  // namespace vtb
