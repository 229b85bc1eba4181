// Greedy, temperature, top-k and top-p sampling over 32-bit logits, one block a row.
//
// vt-transformer samples with an argmax (v1/tensortype/cuda_kernels/easy_sampling.cu:141-169)
// and with "top 3": logits / temperature, the three largest, softmax over those, one uniform
// number (easy_sampling.cu:32-104).  Its front end's parameters are temperature, top_k and
// top_p (sglfront/sglfront/core.py:6-17).  This kernel does the general form: the kept set is
// the top_k largest logits (equal values at the edge are all kept), cut further to the
// smallest set of largest probabilities whose sum reaches top_p; the token is drawn from the
// softmax over the kept set by walking the vocabulary in index order.  top_k = 3 gives the
// distribution of the reference's sampler.  Sums are kept in 64-bit so that the draw agrees
// with a host implementation on the same logits and the same uniform number.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float, larger key
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// All threads get the block's sum.  `sh` holds 32 doubles.
__device__ __forceinline__ double block_sum_d(double v, double* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_d(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double r = (lane < (kThreads >> 5)) ? sh[lane] : 0.0;
    return warp_sum_d(r);
}

// Largest value and its lowest index over the block.
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* shv, int* shi) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { shv[warp] = v; shi[warp] = idx; }
    __syncthreads();
    v = (lane < (kThreads >> 5)) ? shv[lane] : -INFINITY;
    idx = (lane < (kThreads >> 5)) ? shi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

__device__ __forceinline__ void thread_argmax(const float* l, int vocab, float& best, int& bi) {
    best = -INFINITY;
    bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += kThreads) {
        const float v = l[i];
        if (v > best) { best = v; bi = i; }   // ascending i: the first of equals stays
    }
}

}  // namespace

__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float shv[32];
    __shared__ int shi[32];
    pdl_launch();
    pdl_wait();
    const float* l = logits + (size_t)blockIdx.x * vocab;
    float best;
    int bi;
    thread_argmax(l, vocab, best, bi);
    block_argmax(best, bi, shv, shi);
    if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ u, int* __restrict__ out, int vocab) {
    __shared__ float shv[32];
    __shared__ int shi[32];
    __shared__ double shd[32];
    __shared__ double warp_prefix[32];
    pdl_launch();
    pdl_wait();
    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * vocab;
    const float temp = temperature[row];
    const int k = top_k[row];
    const float p_keep = top_p[row];

    float best;
    int bi;
    thread_argmax(l, vocab, best, bi);
    block_argmax(best, bi, shv, shi);
    if (bi == 0x7fffffff) bi = 0;
    if (!(temp > 0.f) || k == 1) {
        if (threadIdx.x == 0) out[row] = bi;
        return;
    }
    const float inv_t = 1.f / temp;
    const float top = best;

    // the k-th largest key, bit by bit from the top: the largest key with count(key >= it) >= k
    uint32_t low_key = 0;
    if (k > 0 && k < vocab) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            double cnt = 0.0;
            for (int i = threadIdx.x; i < vocab; i += kThreads) cnt += (order_key(l[i]) >= cand) ? 1.0 : 0.0;
            cnt = block_sum_d(cnt, shd);
            if (cnt >= (double)k) prefix = cand;
        }
        low_key = prefix;
    }
    // top-p: the largest key whose tail of probabilities still sums to top_p of the kept total
    if (p_keep < 1.f) {
        double total = 0.0;
        for (int i = threadIdx.x; i < vocab; i += kThreads)
            if (order_key(l[i]) >= low_key) total += (double)expf((l[i] - top) * inv_t);
        total = block_sum_d(total, shd);
        const double need = (double)p_keep * total;
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            const uint32_t thr = cand > low_key ? cand : low_key;
            double s = 0.0;
            for (int i = threadIdx.x; i < vocab; i += kThreads)
                if (order_key(l[i]) >= thr) s += (double)expf((l[i] - top) * inv_t);
            s = block_sum_d(s, shd);
            if (s >= need) prefix = cand;
        }
        if (prefix > low_key) low_key = prefix;
    }

    // the draw: each thread owns a run of consecutive indices
    const int chunk = (vocab + kThreads - 1) / kThreads;
    const int begin = min(vocab, threadIdx.x * chunk), end = min(vocab, begin + chunk);
    double local = 0.0;
    for (int i = begin; i < end; ++i)
        if (order_key(l[i]) >= low_key) local += (double)expf((l[i] - top) * inv_t);
    // exclusive prefix of `local` over the threads, in thread (= index) order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double other = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += other;
    }
    __syncthreads();
    if (lane == 31) shd[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        double w = shd[lane];
        double wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double other = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += other;
        }
        warp_prefix[lane] = wi - w;
        if (lane == 31) shd[0] = wi;   // the total
    }
    if (threadIdx.x == 0) out[row] = bi;   // stands if rounding leaves no thread with the target
    __syncthreads();
    const double total = shd[0];
    const double before = warp_prefix[warp] + (incl - local);
    const double target = (double)u[row] * total;
    if (before <= target && target < before + local) {
        double run = before;
        int pick = -1;
        for (int i = begin; i < end; ++i) {
            if (order_key(l[i]) >= low_key) {
                run += (double)expf((l[i] - top) * inv_t);
                if (run > target) { pick = i; break; }
                pick = i;   // the last kept index of the run, should rounding end the walk early
            }
        }
        if (pick >= 0) out[row] = pick;
    }
}

cudaError_t launch_argmax(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows == 0) return cudaSuccess;
    return launch(argmax_kernel, n_rows, kThreads, 0, stream, logits, out, vocab);
}

cudaError_t launch_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                          const float* u, int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows == 0) return cudaSuccess;
    return launch(sample_kernel, n_rows, kThreads, 0, stream, logits, temperature, top_k, top_p, u, out, vocab);
}

}  // namespace vtb
