// Attention over the paged cache, one warp for a (token, head): the plain kernel.
//
// It is the whole 32-bit path and the fallback of the bfloat16 path for head sizes the
// tensor-core kernels do not take.  What it computes is vt-transformer's chain
// scores = q k^T / sqrt(d) (v1/tensortype/cuda_tensor.cpp:730,761-773), causal mask
// (v1/tensortype/cuda_kernels/causal_mask.cu:69-84), softmax (cuda_tensor.cpp:796-800),
// P V (cuda_tensor.cpp:869-881), with the KV head of a query head being head / group
// (v1/tensortype/cuda_kernels/transpose_0213.cu:93-105) -- but without the [heads, T, F]
// score tensor, the repeated heads or the dense copy of the cache: the keys are read where
// they lie in their pages, one after the other in the order of their positions, with a
// running maximum and sum in 32-bit.  The result for a token depends on its own keys only.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int kMaxPerLane = 8;   // head_dim <= 256
}

template <typename T>
__global__ void __launch_bounds__(128)
attention_simt_kernel(const T* __restrict__ qkv, int qkv_stride, T* __restrict__ out, const T* __restrict__ k_cache,
                      const T* __restrict__ v_cache, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ block_table, int table_stride,
                      int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads, int head_dim, int page_size,
                      int window, float scale, int* status) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= (long long)n_tokens * heads) return;
    const int t = (int)(pair / heads), h = (int)(pair % heads);
    const int seq = token_seq[t];
    T* o = out + (size_t)t * heads * head_dim + (size_t)h * head_dim;
    if (seq < 0) {   // padding
        for (int i = lane; i < head_dim; i += 32) o[i] = from_float<T>(0.f);
        return;
    }
    if (seq >= n_seqs) {
        if (lane == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    const int pos = positions[t];
    const int kvh = h / (heads / kv_heads);
    const int* table = block_table + (size_t)seq * table_stride;

    float q[kMaxPerLane], acc[kMaxPerLane];
    const T* qp = qkv + (size_t)t * qkv_stride + (size_t)h * head_dim;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int i = lane + 32 * r;
        q[r] = (i < head_dim) ? to_float(qp[i]) : 0.f;
        acc[r] = 0.f;
    }
    float mx = -INFINITY, sum = 0.f;
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    for (int j = first; j <= pos; ++j) {
        const int page = table[j / page_size];
        if (page < 0 || page >= n_pages) {
            if (lane == 0) set_status(status, kStatusBadPage, page);
            continue;
        }
        const size_t base = (((size_t)page * kv_heads + kvh) * page_size + (j % page_size)) * head_dim;
        float part = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            if (i < head_dim) part = fmaf(q[r], to_float(k_cache[base + i]), part);
        }
        const float s = warp_sum(part) * scale;
        const float new_mx = fmaxf(mx, s);
        const float corr = expf(mx - new_mx);   // 0 at the first key (mx = -inf)
        const float p = expf(s - new_mx);
        sum = sum * corr + p;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            if (i < head_dim) acc[r] = acc[r] * corr + p * to_float(v_cache[base + i]);
        }
        mx = new_mx;
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int i = lane + 32 * r;
        if (i < head_dim) o[i] = from_float<T>(acc[r] * inv);
    }
}

cudaError_t launch_attention_simt(int dtype, const void* qkv, int qkv_stride, void* out, const void* k_cache,
                                  const void* v_cache, const int* positions, const int* token_seq,
                                  const int* block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                                  int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                  int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (head_dim > 32 * kMaxPerLane) return cudaErrorInvalidValue;
    const long long pairs = (long long)n_tokens * heads;
    const int blocks = (int)((pairs + 3) / 4);
    if (dtype == kBF16)
        return launch(attention_simt_kernel<__nv_bfloat16>, blocks, 128, 0, stream,
            (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, positions, token_seq, block_table, table_stride, n_seqs, n_pages, n_tokens,
            heads, kv_heads, head_dim, page_size, window, scale, status);
    return launch(attention_simt_kernel<float>, blocks, 128, 0, stream,
            (const float*)qkv, qkv_stride, (float*)out, (const float*)k_cache, (const float*)v_cache, positions,
            token_seq, block_table, table_stride, n_seqs, n_pages, n_tokens, heads, kv_heads, head_dim, page_size,
            window, scale, status);
}

}  // namespace vtb
