// Greedy, temperature, top-k and top-p sampling over 32-bit logits, one block a row.
//
// vt-transformer samples with an argmax (v1/tensortype/cuda_kernels/easy_sampling.cu:141-169)
// and with "top 3": logits / temperature, the three largest, softmax over those, one uniform
// number (easy_sampling.cu:32-104).  Its front end's parameters are temperature, top_k and
// top_p (sglfront/sglfront/core.py:6-17).  This kernel does the general form: the kept set is
// the top_k largest logits (equal values at the edge are all kept), cut further to the
// smallest set of largest probabilities whose sum reaches top_p; the token is drawn from the
// softmax over the kept set by walking the vocabulary in index order.  top_k = 3 gives the
// distribution of the reference's sampler.  The sums that decide the kept set are integer sums (fixed point), the
// sums of the draw 64-bit: the draw agrees with a host implementation on the same logits and the same uniform
// number, and does not change from run to run.  How the row is gone through is told above `sample_kernel`.
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

// Calls f(value, index, valid) for a thread's share of a row, every thread of the block the same number of times
// (f may hold warp-wide operations): after the row's first values up to a 16-byte boundary, four values a load and
// four loads on their way at a time, the threads of a warp side by side.  A thread's valid indices ascend.
template <typename F>
__device__ __forceinline__ void for_each_of_row(const float* l, int vocab, F f) {
    const int head = min(vocab, (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(l) & 15)) & 15u) >> 2));
    {
        const bool valid = (int)threadIdx.x < head;
        f(valid ? l[threadIdx.x] : 0.f, (int)threadIdx.x, valid);
    }
    const float4* l4 = reinterpret_cast<const float4*>(l + head);
    const int n4 = (vocab - head) >> 2;
    for (int base = 0; base < n4; base += 4 * kThreads) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * kThreads + threadIdx.x;
            v[u] = i < n4 ? l4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * kThreads + threadIdx.x;
            const bool valid = i < n4;
            const int at = head + (i << 2);
            f(v[u].x, at, valid);
            f(v[u].y, at + 1, valid);
            f(v[u].z, at + 2, valid);
            f(v[u].w, at + 3, valid);
        }
    }
    for (int base = head + (n4 << 2); base < vocab; base += kThreads) {
        const int j = base + threadIdx.x;
        const bool valid = j < vocab;
        f(valid ? l[j] : 0.f, j, valid);
    }
}

// The largest of a thread's share of a row and its (lowest) index: the first of equals stays.
__device__ __forceinline__ void thread_argmax(const float* l, int vocab, float& best, int& bi) {
    float b = -INFINITY;
    int at = 0x7fffffff;
    for_each_of_row(l, vocab, [&](float v, int i, bool valid) {
        if (valid && v > b) { b = v; at = i; }
    });
    best = b;
    bi = at;
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

// ---- thresholds and the draw ----------------------------------------------------------------------------
//
// Both thresholds are keys (order_key of a logit): the k-th largest key, and the largest key whose tail of
// probabilities sums to top_p of the kept total.  Probabilities enter these sums as integers: 2^x of a row's values
// (32-bit expf of (v - max) / temperature, at most 1) times 2^(3 b), b chosen so that a whole row's sum of one
// b-bit limb fits 32 bits.  Integer sums do not depend on the order in which threads add, so the kept set is the same
// from run to run, and 32-bit shared-memory atomics take them (64-bit ones are many times slower).
//
// A pass over the row builds histograms over the keys' top 11 bits (counts; probabilities as three limbs).  The
// bucket in which the threshold lies is then known, and with it the number of keys from that bucket upward.  Up to
// kCap of them are gathered into shared memory and everything else (the k-th key, the top_p cut, the draw in index
// order) happens there, a candidate a thread.  More than that (a top_k beyond kCap, top_p over a flat row, many equal
// values at the edge) takes the general way: the remaining digits by further passes, and a draw over the whole row.

constexpr int kBins = 2048;          // histogram over a key's top 11 bits
constexpr int kCap = 1024;           // candidates finished in shared memory, one a thread

struct SampleShared {
    union {
        struct {
            unsigned int count[kBins];
            unsigned int limb[3][kBins];
        } hist;                                             // 32 KB
        struct {
            float value[kCap];
            int index[kCap];
            unsigned int key[kCap];                         // in index order from here on
            int sorted_index[kCap];
            unsigned long long weight[kCap];
        } cand;                                             // 24 KB
    };
    unsigned long long scan[33];
    double dsum[32];
    double warp_prefix[32];
    float shv[32];
    int shi[32];
    unsigned long long out_above, out_inside;
    int out_bin;
    int n_cand;
    unsigned int pick_key;
    int pick_index;
};

// Inclusive suffix sum over the block's threads (this thread and all after it); every thread calls.
__device__ __forceinline__ unsigned long long block_suffix(unsigned long long v, unsigned long long* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long other = __shfl_down_sync(0xffffffffu, v, o);
        if (lane + o < 32) v += other;
    }
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    unsigned long long later = 0;
    for (int w = warp + 1; w < (kThreads >> 5); ++w) later += sh[w];
    return v + later;
}

// The last bin b of `bins` (two a thread) with weight(bins >= b) >= need; leaves the bin, the weight of the bins above
// it and the bin's own weight in shared memory (bin 0 if no bin reaches `need`).  weight_of(bin) reads a bin.
template <typename W>
__device__ __forceinline__ void find_bin(SampleShared& sh, unsigned long long need, int bins, W weight_of) {
    const int b0 = 2 * threadIdx.x, b1 = b0 + 1;
    const unsigned long long w0 = b0 < bins ? weight_of(b0) : 0ull, w1 = b1 < bins ? weight_of(b1) : 0ull;
    const unsigned long long from0 = block_suffix(w0 + w1, sh.scan);       // weight(bins >= b0)
    const unsigned long long from1 = from0 - w0, from2 = from1 - w1;
    if (threadIdx.x == 0) {
        sh.out_bin = 0;
        sh.out_above = from1;
        sh.out_inside = w0;
    }
    __syncthreads();
    if (from1 >= need && from2 < need && b1 < bins) {
        sh.out_bin = b1;
        sh.out_above = from2;
        sh.out_inside = w1;
    } else if (from0 >= need && from1 < need && b0 > 0 && b0 < bins) {
        sh.out_bin = b0;
        sh.out_above = from1;
        sh.out_inside = w0;
    }
    __syncthreads();
}

// Adds a weight to the histogram(s) at a digit: counts, or the three limbs of a probability.  A thread adds up runs of
// equal digits by itself before it touches shared memory.
struct RunAdder {
    int cur = -1;
    unsigned int n = 0;
    unsigned long long w = 0;
    __device__ __forceinline__ void flush(SampleShared& sh, bool weights, int limb_bits) {
        if (cur < 0) return;
        if (n) atomicAdd(&sh.hist.count[cur], n);
        if (weights && w) {
            const unsigned int mask = (1u << limb_bits) - 1;
            // a run's sum of limbs may exceed a limb: each part is carried into the next histogram by value
            atomicAdd(&sh.hist.limb[0][cur], (unsigned int)(w & mask));
            atomicAdd(&sh.hist.limb[1][cur], (unsigned int)((w >> limb_bits) & mask));
            atomicAdd(&sh.hist.limb[2][cur], (unsigned int)(w >> (2 * limb_bits)));
        }
        n = 0;
        w = 0;
    }
    __device__ __forceinline__ void add(SampleShared& sh, int digit, unsigned long long weight, bool weights, int limb_bits) {
        if (digit != cur) {
            flush(sh, weights, limb_bits);
            cur = digit;
        }
        ++n;
        w += weight;
    }
};

__device__ __forceinline__ unsigned long long bin_weight(const SampleShared& sh, int b, int limb_bits) {
    return (unsigned long long)sh.hist.limb[0][b] + ((unsigned long long)sh.hist.limb[1][b] << limb_bits) +
           ((unsigned long long)sh.hist.limb[2][b] << (2 * limb_bits));
}

__device__ __forceinline__ void clear_hist(SampleShared& sh) {
    for (int i = threadIdx.x; i < 4 * kBins; i += kThreads) (&sh.hist.count[0])[i] = 0u;
    __syncthreads();
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ u, int* __restrict__ out, int vocab) {
    __shared__ SampleShared sh;
    pdl_launch();
    pdl_wait();
    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * vocab;
    const float temp = temperature[row];
    const int k = top_k[row];
    const float p_keep = top_p[row];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float best;
    int bi;
    thread_argmax(l, vocab, best, bi);
    block_argmax(best, bi, sh.shv, sh.shi);
    if (bi == 0x7fffffff) bi = 0;
    if (!(temp > 0.f) || k == 1) {
        if (threadIdx.x == 0) out[row] = bi;
        return;
    }
    const float inv_t = 1.f / temp;
    const float top = best;
    const bool by_count = k > 0 && k < vocab, by_mass = p_keep < 1.f;

    // probabilities as integers: three limbs of `limb_bits` bits
    int vocab_bits = 0;
    while ((1ll << vocab_bits) < (long long)vocab) ++vocab_bits;
    const int limb_bits = max(4, min(14, 32 - vocab_bits));
    const float fixed_one = __uint_as_float((uint32_t)(127 + 3 * limb_bits) << 23);     // 2^(3 limb_bits)
    auto fixed = [&](float v) -> unsigned long long { return __float2ull_rz(expf((v - top) * inv_t) * fixed_one); };

    uint32_t low_key = 0;            // keys from here on are kept
    bool drawn = false;
    if (by_count || by_mass) {
        // ---- the first digit of the threshold(s): histograms over the top 11 bits of every key ------------------
        const bool weights = by_mass && !by_count;      // with top_k the kept total is known only after its cut
        clear_hist(sh);
        {
            RunAdder run;
            for_each_of_row(l, vocab, [&](float v, int, bool valid) {
                if (valid) run.add(sh, (int)(order_key(v) >> 21), weights ? fixed(v) : 0ull, weights, limb_bits);
            });
            run.flush(sh, weights, limb_bits);
        }
        __syncthreads();
        unsigned long long need_mass = 0;
        if (by_count) {
            find_bin(sh, (unsigned long long)k, kBins, [&](int b) { return (unsigned long long)sh.hist.count[b]; });
        } else {
            const unsigned long long total = block_suffix(bin_weight(sh, 2 * threadIdx.x, limb_bits) +
                                                          bin_weight(sh, 2 * threadIdx.x + 1, limb_bits), sh.scan);
            __syncthreads();
            if (threadIdx.x == 0) sh.out_above = total;
            __syncthreads();
            const double need = (double)p_keep * (double)sh.out_above;
            need_mass = need <= 1.0 ? 1ull : (unsigned long long)ceil(need);      // (top_p of 0 keeps the largest)
            find_bin(sh, need_mass, kBins, [&](int b) { return bin_weight(sh, b, limb_bits); });
        }
        const int bin1 = sh.out_bin;
        const unsigned long long above1 = sh.out_above;
        // how many keys lie in this bucket or above it
        const unsigned long long from_bin =
            block_suffix((2 * threadIdx.x >= bin1 ? sh.hist.count[2 * threadIdx.x] : 0u) +
                         (unsigned long long)(2 * threadIdx.x + 1 >= bin1 ? sh.hist.count[2 * threadIdx.x + 1] : 0u), sh.scan);
        __syncthreads();
        if (threadIdx.x == 0) sh.n_cand = (int)min(from_bin, (unsigned long long)(kCap + 1));
        __syncthreads();
        const int n_from_bin = sh.n_cand;
        __syncthreads();

        if (n_from_bin <= kCap) {
            // ---- few candidates: gather them, and finish in shared memory --------------------------------------
            const uint32_t from_key = (uint32_t)bin1 << 21;
            if (threadIdx.x == 0) sh.n_cand = 0;
            __syncthreads();                                   // (the histograms are not read again)
            for_each_of_row(l, vocab, [&](float v, int i, bool valid) {
                if (valid && order_key(v) >= from_key) {
                    const int slot = atomicAdd(&sh.n_cand, 1);
                    if (slot < kCap) {
                        sh.cand.value[slot] = v;
                        sh.cand.index[slot] = i;
                    }
                }
            });
            __syncthreads();
            const int n = min(sh.n_cand, kCap);
            const int t = threadIdx.x;
            // in index order (the slots were handed out in no order)
            float my_v = 0.f;
            int my_i = 0, pos = 0;
            if (t < n) {
                my_v = sh.cand.value[t];
                my_i = sh.cand.index[t];
                for (int j = 0; j < n; ++j) pos += sh.cand.index[j] < my_i ? 1 : 0;
            }
            __syncthreads();
            if (t < n) {
                sh.cand.key[pos] = order_key(my_v);
                sh.cand.sorted_index[pos] = my_i;
                sh.cand.weight[pos] = fixed(my_v);
            }
            __syncthreads();
            const uint32_t key = t < n ? sh.cand.key[t] : 0u;
            const unsigned long long w = t < n ? sh.cand.weight[t] : 0ull;
            bool kept = t < n;
            if (by_count) {
                // kept by top_k: fewer than k keys are greater (values equal to the k-th are all kept); the keys above
                // the bucket are all among the candidates
                int greater = 0;
                for (int j = 0; j < n; ++j) greater += sh.cand.key[j] > key ? 1 : 0;
                kept = kept && greater < k;
            }
            if (by_mass) {
                // the kept total: of the candidates kept by top_k, or (without top_k) of the whole row
                unsigned long long total;
                if (by_count) {
                    total = block_suffix(kept ? w : 0ull, sh.scan);
                    __syncthreads();
                    if (threadIdx.x == 0) sh.out_above = total;
                    __syncthreads();
                    total = sh.out_above;
                    const double need = (double)p_keep * (double)total;
                    need_mass = need <= 1.0 ? 1ull : (unsigned long long)ceil(need);      // (top_p of 0 keeps the largest)
                }
                // the largest key whose tail reaches the need
                if (by_count) {
                    __syncthreads();
                    sh.cand.value[t] = kept ? 1.f : 0.f;       // (the values are no longer needed: kept flags)
                    __syncthreads();
                }
                unsigned long long tail = 0;
                if (kept)
                    for (int j = 0; j < n; ++j)
                        if (sh.cand.key[j] >= key && (!by_count || sh.cand.value[j] != 0.f)) tail += sh.cand.weight[j];
                if (threadIdx.x == 0) sh.pick_key = 0u;
                __syncthreads();
                if (kept && tail >= need_mass) atomicMax(&sh.pick_key, key);
                __syncthreads();
                kept = kept && key >= sh.pick_key;
            }
            // the draw: the first candidate, in index order, at which the running sum of the kept weights exceeds
            // u times their total
            const unsigned long long mine = kept ? w : 0ull;
            const unsigned long long from_me = block_suffix(mine, sh.scan);      // this one and all after it
            __syncthreads();
            if (threadIdx.x == 0) {
                sh.out_above = from_me;                                          // the total
                sh.pick_index = bi;                                              // stands if nothing is kept
            }
            __syncthreads();
            const unsigned long long total = sh.out_above;
            const unsigned long long upto_me = total - from_me + mine;           // the running sum with this one
            const double target_real = (double)u[row] * (double)total;
            const unsigned long long target = target_real <= 0.0 ? 0ull : (unsigned long long)target_real;   // floor
            if (kept && mine > 0 && upto_me > target && upto_me - mine <= target) sh.pick_index = sh.cand.sorted_index[t];
            __syncthreads();
            if (threadIdx.x == 0) out[row] = sh.pick_index;
            drawn = true;
        } else {
            // ---- the general way: the thresholds' other digits by further passes over the row -------------------
            // A threshold is found digit by digit (11, 11 and 10 bits); `restrict_from`: keys below it take no part.
            auto rest_of_key = [&](uint32_t prefix, unsigned long long above, unsigned long long need, bool weighted,
                                   uint32_t restrict_from) -> uint32_t {
                for (int pass = 1; pass < 3; ++pass) {
                    const int shift = pass == 1 ? 10 : 0, bits = pass == 1 ? 11 : 10;
                    clear_hist(sh);
                    RunAdder run;
                    for_each_of_row(l, vocab, [&](float v, int, bool valid) {
                        const uint32_t key = order_key(v);
                        if (valid && key >= restrict_from && (key >> (shift + bits)) == (prefix >> (shift + bits)))
                            run.add(sh, (int)((key >> shift) & ((1u << bits) - 1)), weighted ? fixed(v) : 0ull, weighted, limb_bits);
                    });
                    run.flush(sh, weighted, limb_bits);
                    __syncthreads();
                    const unsigned long long need_here = need > above ? need - above : 0ull;
                    if (weighted) find_bin(sh, need_here, 1 << bits, [&](int b) { return bin_weight(sh, b, limb_bits); });
                    else find_bin(sh, need_here, 1 << bits, [&](int b) { return (unsigned long long)sh.hist.count[b]; });
                    prefix |= (uint32_t)sh.out_bin << shift;
                    above += sh.out_above;
                    __syncthreads();
                }
                return prefix;
            };
            if (by_count) {
                low_key = rest_of_key((uint32_t)bin1 << 21, above1, (unsigned long long)k, false, 0u);
                if (by_mass) {
                    // the first digit again, now with the probabilities of the keys that top_k kept
                    clear_hist(sh);
                    RunAdder run;
                    for_each_of_row(l, vocab, [&](float v, int, bool valid) {
                        const uint32_t key = order_key(v);
                        if (valid && key >= low_key) run.add(sh, (int)(key >> 21), fixed(v), true, limb_bits);
                    });
                    run.flush(sh, true, limb_bits);
                    __syncthreads();
                    const unsigned long long total = block_suffix(bin_weight(sh, 2 * threadIdx.x, limb_bits) +
                                                                  bin_weight(sh, 2 * threadIdx.x + 1, limb_bits), sh.scan);
                    __syncthreads();
                    if (threadIdx.x == 0) sh.out_above = total;
                    __syncthreads();
                    const double need = (double)p_keep * (double)sh.out_above;
                    need_mass = need <= 1.0 ? 1ull : (unsigned long long)ceil(need);      // (top_p of 0 keeps the largest)
                    find_bin(sh, need_mass, kBins, [&](int b) { return bin_weight(sh, b, limb_bits); });
                    const uint32_t first = (uint32_t)sh.out_bin << 21;
                    const unsigned long long above = sh.out_above;
                    __syncthreads();
                    const uint32_t cut = rest_of_key(first, above, need_mass, true, low_key);
                    if (cut > low_key) low_key = cut;
                }
            } else {
                low_key = rest_of_key((uint32_t)bin1 << 21, above1, need_mass, true, 0u);
            }
        }
    }
    if (drawn) return;

    // ---- the draw over the whole row ----------------------------------------------------------------------
    // A warp owns a run of consecutive indices (a multiple of 128), its lanes side by side: the warps' sums and their
    // running total in index order; then the run in which the target falls is cut into 32 pieces, a warp each, and
    // the warp whose piece holds the target walks it, 32 indices at a time with a running sum over its lanes.
    auto weight = [&](float v) -> double { return order_key(v) >= low_key ? (double)expf((v - top) * inv_t) : 0.0; };
    const bool row_aligned = (reinterpret_cast<uintptr_t>(l) & 15) == 0;
    auto sum_of = [&](int begin, int end) -> double {
        double local = 0.0;
        int base = begin;
        if (row_aligned && (begin & 3) == 0) {
            // four values a load, four loads (512 indices a warp) on their way at a time
            for (; base + 512 <= end; base += 512) {
                float4 v[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) v[r] = *reinterpret_cast<const float4*>(l + base + 128 * r + 4 * lane);
#pragma unroll
                for (int r = 0; r < 4; ++r) local += (weight(v[r].x) + weight(v[r].y)) + (weight(v[r].z) + weight(v[r].w));
            }
        }
        for (; base < end; base += 128) {
            float v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) v[r] = (base + 32 * r + lane < end) ? l[base + 32 * r + lane] : -INFINITY;
#pragma unroll
            for (int r = 0; r < 4; ++r) local += (base + 32 * r + lane < end) ? weight(v[r]) : 0.0;
        }
        return warp_sum_d(local);
    };
    // exclusive prefix over the warps' sums, in warp order; returns this warp's, leaves the total in dsum[0]
    auto prefix_of_warps = [&](double mine) -> double {
        __syncthreads();
        if (lane == 0) sh.dsum[warp] = mine;
        __syncthreads();
        if (warp == 0) {
            const double w = sh.dsum[lane];
            double wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double other = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += other;
            }
            sh.warp_prefix[lane] = wi - w;
            if (lane == 31) sh.dsum[0] = wi;
        }
        __syncthreads();
        return sh.warp_prefix[warp];
    };
    const int per_warp = ((vocab + 4 * kThreads - 1) / (4 * kThreads)) * 128;
    const int begin = min(vocab, warp * per_warp), end = min(vocab, begin + per_warp);
    const double mine = sum_of(begin, end);
    const double before = prefix_of_warps(mine);
    const double total = sh.dsum[0];
    const double target = (double)u[row] * total;
    if (threadIdx.x == 0) {
        out[row] = bi;              // stands if rounding leaves no run with the target
        sh.pick_index = -1;
    }
    __syncthreads();
    if (lane == 0 && before <= target && target < before + mine) {
        sh.pick_index = warp;
        sh.dsum[1] = before;
    }
    __syncthreads();
    const int owner = sh.pick_index;
    if (owner < 0) return;
    const double before_run = sh.dsum[1];
    const int run_begin = min(vocab, owner * per_warp), run_end = min(vocab, run_begin + per_warp);
    const int piece = ((run_end - run_begin + 32 * 32 - 1) / (32 * 32)) * 32;          // a multiple of 32 indices a warp
    const int p_begin = min(run_end, run_begin + warp * piece), p_end = min(run_end, p_begin + piece);
    const double p_mine = sum_of(p_begin, p_end);
    const double p_before = before_run + prefix_of_warps(p_mine);
    if (p_before <= target && target < p_before + p_mine) {
        double run = p_before;
        int pick = -1;
        for (int base = p_begin; base < p_end; base += 32) {
            const double w = (base + lane < p_end) ? weight(l[base + lane]) : 0.0;
            double incl = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double other = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += other;
            }
            // the first lane at which the running sum exceeds the target; and the last kept index so far, should
            // rounding end the walk early
            const unsigned over = __ballot_sync(0xffffffffu, w > 0.0 && run + incl > target);
            const unsigned kept = __ballot_sync(0xffffffffu, w > 0.0);
            if (over) {
                pick = base + __ffs(over) - 1;
                break;
            }
            if (kept) pick = base + 31 - __clz(kept);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0 && pick >= 0) out[row] = pick;
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
