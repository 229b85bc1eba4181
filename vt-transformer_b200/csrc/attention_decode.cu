// Attention of single-token steps over the paged cache on the tensor cores (bfloat16 in, 32-bit softmax and
// sums): the chain of vt-transformer's graph, scores = q k^T / sqrt(d), causal mask, softmax, P V
// (v1/models/qwen2-7b/inference_fp16.dag:307-318; v1/tensortype/cuda_tensor.cpp:761-773, 796-800, 869-881), for
// the query heads of one KV head at a time, with the keys of a sequence split over warps and CTAs.
#include "attention_decode.cuh"

namespace vtb {

cudaError_t launch_attention_decode(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                    const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                    int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads, int head_dim,
                                    int page_size, int window, float scale, int n_splits, float* part_o, float* part_ml,
                                    int* counters, int fuse_rope, const float2* cos_sin, int max_pos, int store_kv,
                                    const float* qkv_shares, int n_shares, int long_runs, int run_blocks, int* status,
                                    cudaStream_t stream) {
    if (n_seqs == 0 || n_tokens == 0) return cudaSuccess;
    if (!attention_mma_supports(head_dim, heads, kv_heads, 1) || page_size % 16 != 0) return cudaErrorInvalidValue;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 64) return cudaErrorInvalidValue;   // the merge keeps a weight a run in shared memory
    // up to 8 runs are the CTAs of a cluster and need no scratch; more, or any number where the caller gives scratch,
    // go through scratch and a counter
    if (n_splits > 8 && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return cudaErrorInvalidValue;
    const bool with_scratch = part_o != nullptr && part_ml != nullptr && counters != nullptr;
    const bool cluster = n_splits > 1 && n_splits <= 8 && !with_scratch;
    AttnParams p;
    p.cluster_merge = cluster ? 1 : 0;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.out = (__nv_bfloat16*)out;
    p.k_cache = (const __nv_bfloat16*)k_cache;
    p.v_cache = (const __nv_bfloat16*)v_cache;
    p.cu_q = cu_q;
    p.q_start = q_start;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.tiles = nullptr;
    p.n_pages = n_pages;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.page_size = page_size;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.tokens_per_tile = fuse_rope ? 1 : 16 / (heads / kv_heads);
    p.run_keys = long_runs ? 1 : 0;                  // the launcher of a head size with boxes sets the rows of a box
    p.n_splits = n_splits;
    p.run_blocks = run_blocks > 0 ? run_blocks : 0;
    p.part_o = part_o;
    p.part_ml = part_ml;
    p.n_tokens = n_tokens;
    p.status = status;
    p.fuse_rope = fuse_rope;
    p.cos_sin = cos_sin;
    p.max_pos = max_pos;
    p.store_kv = store_kv;
    p.k_out = (__nv_bfloat16*)const_cast<void*>(k_cache);
    p.v_out = (__nv_bfloat16*)const_cast<void*>(v_cache);
    if (qkv_shares != nullptr && (!fuse_rope || n_shares < 1 || n_shares > 8)) return cudaErrorInvalidValue;
    p.qkv_shares = qkv_shares;
    p.n_shares = n_shares;
    switch (head_dim) {
        case 16: return launch_decode_d<16>(p, n_seqs, counters, stream);
        case 32: return launch_decode_d<32>(p, n_seqs, counters, stream);
        case 48: return launch_decode_d<48>(p, n_seqs, counters, stream);
        case 64: return launch_decode_64_128(p, 64, n_seqs, counters, stream);
        case 80: return launch_decode_d<80>(p, n_seqs, counters, stream);
        case 96: return launch_decode_d<96>(p, n_seqs, counters, stream);
        case 112: return launch_decode_d<112>(p, n_seqs, counters, stream);
        case 128: return launch_decode_64_128(p, 128, n_seqs, counters, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace vtb
