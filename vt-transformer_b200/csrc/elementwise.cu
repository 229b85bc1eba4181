// Embedding, RMS norm with the residual sum, SiLU * up, rotation with the cache store.
//
// Formulas after vt-transformer's kernels: v1/tensortype/cuda_kernels/rmsnorm.cu:20-47
// (w * x * rsqrt(mean(x^2) + eps), all in 32-bit, one rounding),
// v1/tensortype/cuda_kernels/rotary_embed.cu:19-29 (pairs (i, i + d/2)),
// v1/tensortype/cuda_kernels/silu_product.cu:15-17 (act / (1 + exp(-act)) * in),
// v1/tensortype/host_tensor.cpp:189-198 (the embedding is a copy of rows).
// The launch shapes are this engine's: one block a token, 16-byte accesses, the residual
// sum folded into the norm, and the keys and values written straight into their pages.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

// ------------------------------------------------------------------------- embedding

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, float scale, int* status) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && id >= vocab) set_status(status, kStatusBadTokenId, id);
        // a negative id marks a padding token: its row is zero
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            Vec8<float>::store(o + i, z);
        }
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float f[8];
        Vec8<T>::load(row + i, f);
        if (scale != 1.0f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= scale;
        }
        Vec8<float>::store(o + i, f);
    }
}

cudaError_t launch_embedding(int table_dtype, const void* table, const int* ids, float* out, int n_tokens,
                             int hidden, int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    int threads = min(256, max(32, ((hidden / 8 + 31) / 32) * 32));
    if (table_dtype == kBF16)
        return launch(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab, scale, status);
    return launch(embedding_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab, scale, status);
}

// ------------------------------------------------------------------------- logits: scale and soft cap

// logits = cap * tanh(scale * logits / cap) in place (cap 0: the scale alone), 32-bit.
__global__ void logits_scale_cap_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
    pdl_launch();
    pdl_wait();
    const float inv = cap > 0.f ? 1.f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = logits[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv);
        logits[i] = v;
    }
}

cudaError_t launch_logits_scale_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int blocks = (int)min((n + 255) / 256, (long long)148 * 8);
    return launch(logits_scale_cap_kernel, blocks, 256, 0, stream, logits, n, scale, cap);
}

// ------------------------------------------------------------------------- rmsnorm

// One block a row.  Pass 1 forms v = x (+ delta) in 32-bit, writes it back when there is a
// delta, and sums v^2; pass 2 reads v again (its own writes) and scales it.  The sum's order
// depends on hidden and the block size only, never on the batch.  The delta may also come as `n_parts` 32-bit
// shares [n_parts, n_tokens, hidden] (a matrix product whose inner dimension was cut over CTAs leaves its shares
// unadded): they are added here in the order of their index.
template <typename T>
__global__ void rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ parts,
                               int n_parts, const float* __restrict__ weight, float eps, T* __restrict__ out,
                               const int* __restrict__ rows, int n_tokens, int hidden, int* status) {
    __shared__ float scratch[32];
    pdl_launch();
    // the norm's weight and the list of rows are written by no kernel of the step: they are read before the wait
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float w_first[8];
    if ((int)threadIdx.x * 8 < hidden) Vec8<float>::load(weight + threadIdx.x * 8, w_first);
    pdl_wait();
    T* o = out + (size_t)r * hidden;
    if (t < 0 || t >= n_tokens) {
        if (threadIdx.x == 0) set_status(status, kStatusBadRow, t);
        return;
    }
    float* xr = x + (size_t)t * hidden;
    const T* dr = delta ? delta + (size_t)t * hidden : nullptr;
    const float* pr = parts ? parts + (size_t)t * hidden : nullptr;
    const size_t stride = (size_t)n_tokens * hidden;
    // v = x (+ delta, or + the shares in the order of their index) for the eight values at i
    auto row_values = [&](int i, float (&v)[8]) {
        Vec8<float>::load(xr + i, v);
        if (dr) {
            float d[8];
            Vec8<T>::load(dr + i, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += d[j];
        } else if (pr) {
#pragma unroll 4
            for (int q = 0; q < n_parts; ++q) {
                float d[8];
                Vec8<float>::load(pr + i + q * stride, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += d[j];
            }
        }
    };
    const int first = threadIdx.x * 8;
    const bool once = hidden <= (int)blockDim.x * 8;      // a thread has all its values at once: they stay in registers
    float keep[8];
    float ss = 0.f;
    for (int i = first; i < hidden; i += blockDim.x * 8) {
        float v[8];
        row_values(i, v);
        if (dr || pr) Vec8<float>::store(xr + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ss += v[j] * v[j];
            keep[j] = v[j];
        }
    }
    const float total = block_sum(ss, scratch);
    const float rs = rsqrtf(total / (float)hidden + eps);
    for (int i = first; i < hidden; i += blockDim.x * 8) {
        float v[8], w[8], y[8];
        if (once) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = keep[j];
        } else {
            Vec8<float>::load(xr + i, v);       // its own writes, or x as it was
        }
        if (i == first) {
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = w_first[j];
        } else {
            Vec8<float>::load(weight + i, w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = w[j] * v[j] * rs;
        Vec8<T>::store(o + i, y);
    }
}

cudaError_t launch_rmsnorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                           const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                           int hidden, int* status, cudaStream_t stream) {
    if (delta != nullptr && parts != nullptr) return cudaErrorInvalidValue;
    if (n_rows == 0) return cudaSuccess;
    int threads = min(512, max(32, ((hidden / 8 + 31) / 32) * 32));
    if (out_dtype == kBF16)
        return launch(rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, x, (const __nv_bfloat16*)delta, parts, n_parts, weight, eps,
                      (__nv_bfloat16*)out, rows, n_tokens, hidden, status);
    return launch(rmsnorm_kernel<float>, n_rows, threads, 0, stream, x, (const float*)delta, parts, n_parts, weight, eps, (float*)out, rows, n_tokens,
                  hidden, status);
}

// ------------------------------------------------------------------------- silu * up

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int n_tokens, int inter, int interleave) {
    pdl_launch();
    pdl_wait();
    const int per_row = inter / 8;
    const size_t total = (size_t)n_tokens * per_row;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / per_row);
        const int i = (int)(e % per_row) * 8;
        float g[8], u[8], y[8];
        const T* row = gu + (size_t)t * 2 * inter;
        Vec8<T>::load(row + (interleave ? 2 * i : i), g);
        Vec8<T>::load(row + (interleave ? 2 * i + 8 : inter + i), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = g[j] / (1.f + expf(-g[j])) * u[j];
        Vec8<T>::store(out + (size_t)t * inter + i, y);
    }
}

cudaError_t launch_silu_mul(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave,
                            cudaStream_t stream) {
    if (interleave != 0 && interleave != 8) return cudaErrorInvalidValue;
    const size_t total = (size_t)n_tokens * (inter / 8);
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const int blocks = (int)min((size_t)148 * 16, (total + threads - 1) / threads);
    if (dtype == kBF16)
        return launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens, inter, interleave);
    return launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (const float*)gu, (float*)out, n_tokens, inter, interleave);
}

// ------------------------------------------------------------------------- rotation + cache store

// One block a token.  The angle's cos and sin come from a table of float pairs built on the
// host as vt-transformer builds its own (v1/tensortype/common.cpp:6-24); the rotation is done
// in 32-bit with one rounding.  Keys are rotated on their way into the page, values are copied.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float2* __restrict__ cos_sin, int max_pos, T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, const int* __restrict__ token_seq,
                                  const int* __restrict__ block_table, int table_stride, int n_seqs, int n_pages,
                                  int heads, int kv_heads, int head_dim, int page_size, int rotate, int store,
                                  int* status) {
    // Positions, sequences and block tables are the step's own inputs, there before its first kernel starts: they are
    // read while the kernel before this one may still run; qkv, which that kernel writes, waits.  (Every thread
    // waits before it leaves: a kernel all of whose blocks left early would be done before the one before it.)
    pdl_launch();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool seq_ok = seq >= 0 && seq < n_seqs;
    const int pos = seq_ok ? positions[t] : 0;
    const bool pos_ok = pos >= 0 && (!rotate || pos < max_pos);
    const int page = (store && seq_ok && pos_ok) ? block_table[(size_t)seq * table_stride + pos / page_size] : 0;
    pdl_wait();
    if (seq < 0) return;  // padding
    if (!seq_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    if (!pos_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPosition, pos);
        return;
    }
    const int half = head_dim / 2;
    const int q_dim = heads * head_dim, kv_dim = kv_heads * head_dim;
    T* row = qkv + (size_t)t * (q_dim + 2 * kv_dim);
    const float2* cs = cos_sin + (size_t)pos * half;

    size_t page_base = 0;
    int slot = 0;
    if (store) {
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0) set_status(status, kStatusBadPage, page);
            store = 0;
        }
        page_base = (size_t)page * kv_heads * page_size * head_dim;
        slot = pos % page_size;
    }

    // eight pairs (i, i + half) at a time: 16- or 32-byte loads and stores (head_dim is a multiple of 16)
    auto rotate8 = [&](const T* src, T* dst, int i) {
        float a[8], b[8];
        Vec8<T>::load(src + i, a);
        Vec8<T>::load(src + i + half, b);
        if (rotate) {
            float c[16];
            Vec8<float>::load(reinterpret_cast<const float*>(cs + i), *reinterpret_cast<float(*)[8]>(c));
            Vec8<float>::load(reinterpret_cast<const float*>(cs + i) + 8, *reinterpret_cast<float(*)[8]>(c + 8));
            float ra[8], rb[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ra[j] = a[j] * c[2 * j] - b[j] * c[2 * j + 1];
                rb[j] = b[j] * c[2 * j] + a[j] * c[2 * j + 1];
            }
            Vec8<T>::store(dst + i, ra);
            Vec8<T>::store(dst + i + half, rb);
        } else {
            Vec8<T>::store(dst + i, a);
            Vec8<T>::store(dst + i + half, b);
        }
    };
    const int half8 = half / 8;
    // queries: rotate in place
    if (rotate) {
        for (int e = threadIdx.x; e < heads * half8; e += blockDim.x) {
            T* p = row + (e / half8) * head_dim;
            rotate8(p, p, (e % half8) * 8);
        }
    }
    if (!store) return;
    // keys: rotate into the page
    for (int e = threadIdx.x; e < kv_heads * half8; e += blockDim.x) {
        const int h = e / half8;
        rotate8(row + q_dim + h * head_dim, k_cache + page_base + ((size_t)h * page_size + slot) * head_dim, (e % half8) * 8);
    }
    // values: copy into the page
    for (int e = threadIdx.x; e < kv_dim / 8; e += blockDim.x) {
        const int h = (e * 8) / head_dim, i = (e * 8) % head_dim;
        float v[8];
        Vec8<T>::load(row + q_dim + kv_dim + e * 8, v);
        Vec8<T>::store(v_cache + page_base + ((size_t)h * page_size + slot) * head_dim + i, v);
    }
}

cudaError_t launch_rope_store(int dtype, void* qkv, const int* positions, const float2* cos_sin, int max_pos,
                              void* k_cache, void* v_cache, const int* token_seq, const int* block_table,
                              int table_stride, int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads,
                              int head_dim, int page_size, int rotate, int store, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (head_dim % 16 != 0) return cudaErrorInvalidValue;       // eight pairs (i, i + head_dim / 2) a thread
    const int work = max(heads * head_dim / 16, kv_heads * head_dim / 8);
    const int threads = min(512, max(32, ((work + 31) / 32) * 32));
    if (dtype == kBF16)
        return launch(rope_store_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream,
            (__nv_bfloat16*)qkv, positions, cos_sin, max_pos, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, token_seq,
            block_table, table_stride, n_seqs, n_pages, heads, kv_heads, head_dim, page_size, rotate, store, status);
    return launch(rope_store_kernel<float>, n_tokens, threads, 0, stream,
            (float*)qkv, positions, cos_sin, max_pos, (float*)k_cache, (float*)v_cache, token_seq, block_table,
            table_stride, n_seqs, n_pages, heads, kv_heads, head_dim, page_size, rotate, store, status);
}

}  // namespace vtb
