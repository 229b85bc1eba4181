// Attention of prompt portions over the paged cache on the 5th-generation tensor cores (head size 128).
//
// The computation is the chain of vt-transformer's graph (scores = q k^T / sqrt(d), causal mask, softmax,
// P V: v1/models/qwen2-7b/inference_fp16.dag:307-318) done block by block with a running maximum and sum,
// as in attention_mma.cu; here both products run as tcgen05.mma with their results in tensor memory:
//
//   tile   128 rows, a row being (token, head of the KV group): a key is fetched once for the whole group
//   block  128 keys = 8 runs of 16 keys, each run inside one page; TMA brings a run of K and of V as two
//          boxes of 64 dims (128-byte rows, 128-byte swizzle); runs beyond the last key are zero-filled
//   S      = Q K^T: A = Q (K-major), B = K block (K-major, N = 128 keys), accumulator [128 x 128] floats in
//          tensor memory, double-buffered so that S of the next block is computed under the softmax
//   P      four warps, one row a thread: tcgen05.ld of the row of S, scale, mask, running maximum, 2^x,
//          sum; P rounded to bfloat16 and written into shared memory in the swizzled K-major layout
//   PV     = P V: A = P (K-major over keys), B = V block as it lies ([key][dim]: MN-major), [128 x 128]
//          floats in tensor memory; the softmax warps add it to their registers: O = (O + PV) * correction
//
// Warp 0 loads (one thread), warp 1 issues the MMAs (one thread), warps 2..5 do the softmax and keep O.
// Every wait on a barrier is bounded; a wait that runs out sets the status word and the CTA winds down.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tc_common.cuh"

namespace vtb {

namespace {

constexpr int TQ = 128;              // rows of a tile
constexpr int TK = 128;              // keys of a block
constexpr int HALF_BYTES = 128 * 128;   // 128 rows of 128 bytes (64 bfloat16): 16 KB
constexpr int RUN_BYTES = 16 * 128;     // 16 keys of a run in one half
constexpr int ATC_THREADS = 192;

struct AttnTcParams {
    const __nv_bfloat16* qkv;
    int qkv_stride;
    __nv_bfloat16* out;
    const int* cu_q;
    const int* q_start;
    const int* block_table;
    int table_stride;
    const int2* tiles;
    int n_pages, heads, kv_heads, page_size, window;
    float scale_log2;
    int tokens_per_tile;
    int cache_rows;          // pages * kv_heads * page_size: a row index beyond it makes TMA fill zeros
    int* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Largest raw score of a row of S (128 columns of tensor memory at s_addr).  MASKED: keys this row does not
// see (beyond its position, or before its window) count as -infinity.
template <bool MASKED>
__device__ __forceinline__ float row_max(uint32_t s_addr, int kb, int pos, int window, bool valid) {
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
    for (int c0 = 0; c0 < TK; c0 += 32) {
        uint32_t raw[32];
        tc_ld32(s_addr + c0, raw);
        if (MASKED) {
            // keys [lo, hi) of this chunk are seen
            const int hi = valid ? min(32, pos - (kb + c0) + 1) : 0;
            const int lo = (window > 0) ? max(0, pos - window + 1 - (kb + c0)) : 0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                mx[i & 3] = fmaxf(mx[i & 3], (i >= lo && i < hi) ? __uint_as_float(raw[i]) : -INFINITY);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(raw[i]));
        }
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

// P = 2^(raw * scale - base) of a row, rounded to bfloat16 and written into the row's 16-byte pieces of the
// swizzled K-major P tile; returns the sum of the row (of the unrounded values).
template <bool MASKED>
__device__ __forceinline__ float write_p(uint32_t s_addr, unsigned char* p_s, int r, int kb, int pos, int window,
                                         bool valid, float scale_log2, float base) {
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int c0 = 0; c0 < TK; c0 += 32) {
        uint32_t raw[32];
        tc_ld32(s_addr + c0, raw);
        const int hi = valid ? min(32, pos - (kb + c0) + 1) : 0;
        const int lo = (window > 0) ? max(0, pos - window + 1 - (kb + c0)) : 0;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float pv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pv[e] = ex2(fmaf(__uint_as_float(raw[i + e]), scale_log2, -base));
                if (MASKED) pv[e] = (i + e >= lo && i + e < hi) ? pv[e] : 0.f;
            }
            sum[(i >> 1) & 3] += pv[0] + pv[1];
            __nv_bfloat162 b = __floats2bfloat162_rn(pv[0], pv[1]);
            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        // 32 keys = four 16-byte pieces of this row of P
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int c = (c0 >> 3) + q4;              // piece index among the 16 of the row
            *reinterpret_cast<uint4*>(p_s + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
                make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
    }
    return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

template <int D>
__global__ void __launch_bounds__(ATC_THREADS)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const AttnTcParams p) {
    static_assert(D == 128, "built for head size 128");
    constexpr int HALVES = D / 64;
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;      // Q, a stage of K, a stage of V
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + TILE_BYTES;               // [2][TILE_BYTES]
    unsigned char* v_s = k_s + 2 * TILE_BYTES;           // [2][TILE_BYTES]
    unsigned char* p_s = v_s + 2 * TILE_BYTES;           // [2 halves of 64 keys][16 KB]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * HALF_BYTES);
    uint64_t *k_full = bars, *k_empty = bars + 2, *v_full = bars + 4, *v_empty = bars + 6, *s_full = bars + 8,
             *s_empty = bars + 10, *p_full = bars + 12, *pv_full = bars + 13, *q_full = bars + 14;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 4);
        }
        mbar_init(p_full, 4);
        mbar_init(pv_full, 1);
        mbar_init(q_full, 4);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;          // columns 0..127 and 128..255: S (two buffers); 256..383: P V
    pdl_launch();
    pdl_wait();                                 // q, and the keys and values of this step, come from kernels before

    const int kvh = blockIdx.y;
    const int2 tl = p.tiles[blockIdx.x];
    const int seq = tl.x, tok0 = tl.y;
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    const int group = p.heads / p.kv_heads;
    const int rows_valid = max(0, ntok) * group;
    const int start = p.q_start[seq];
    const int pos_lo = start + tok0, pos_hi = pos_lo + max(1, ntok) - 1;
    int key_lo = (p.window > 0) ? max(0, pos_lo - p.window + 1) : 0;
    key_lo = key_lo / TK * TK;
    const int key_hi = pos_hi + 1;
    const int nb = (ntok > 0) ? (key_hi - key_lo + TK - 1) / TK : 0;
    bool timed_out = false;

    if (warp == 0) {
        if (lane == 0 && nb > 0) {
            const int* table = p.block_table + (size_t)seq * p.table_stride;
            for (int j = 0; j < nb && !timed_out; ++j) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1)) { timed_out = true; break; }
                int rows[TK / 16];
#pragma unroll
                for (int run = 0; run < TK / 16; ++run) {
                    const int key = key_lo + j * TK + run * 16;
                    int row = p.cache_rows;                      // outside the cache: the box is filled with zeros
                    if (key < key_hi) {
                        const int page = table[key / p.page_size];
                        // a page behind a window may be gone already; its keys are masked
                        if (page >= 0 && page < p.n_pages) row = (page * p.kv_heads + kvh) * p.page_size + key % p.page_size;
                    }
                    rows[run] = row;
                }
                mbar_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
                for (int run = 0; run < TK / 16; ++run)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(k_s + st * TILE_BYTES + h * HALF_BYTES + run * RUN_BYTES, &map_k, h * 64, rows[run], &k_full[st]);
                if (j >= 2 && !mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1)) { timed_out = true; break; }
                mbar_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
                for (int run = 0; run < TK / 16; ++run)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(v_s + st * TILE_BYTES + h * HALF_BYTES + run * RUN_BYTES, &map_v, h * 64, rows[run], &v_full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nb > 0) {
            const uint32_t idesc_s = instr_desc(TQ, TK), idesc_pv = instr_desc(TQ, D, true);
            auto issue_s = [&](int j) -> bool {
                const int st = j & 1;
                if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
                if (j >= 2 && !mbar_wait(&s_empty[st], ((j >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)     // 16 dims = 32 bytes further along the swizzled rows
                        tc_mma(tmem + (uint32_t)(st * TK), smem_desc(q_s + h * HALF_BYTES) + 2 * kk,
                               smem_desc(k_s + st * TILE_BYTES + h * HALF_BYTES) + 2 * kk, idesc_s, (h | kk) ? 1u : 0u);
                tc_commit(&k_empty[st]);
                tc_commit(&s_full[st]);
                return true;
            };
            if (!mbar_wait(q_full, 0)) timed_out = true;
            tc_fence_after();
            if (!timed_out && !issue_s(0)) timed_out = true;
            for (int j = 0; j < nb && !timed_out; ++j) {
                if (j + 1 < nb && !issue_s(j + 1)) { timed_out = true; break; }
                const int st = j & 1;
                if (!mbar_wait(p_full, j & 1) || !mbar_wait(&v_full[st], (j >> 1) & 1)) { timed_out = true; break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < TK / 16; ++ks)   // 16 keys: A 32 bytes along P's rows, B 16 rows of V further
                    tc_mma(tmem + 2 * TK, smem_desc(p_s + (ks >> 2) * HALF_BYTES) + 2 * (ks & 3),
                           smem_desc_lbo(v_s + st * TILE_BYTES + ks * RUN_BYTES, HALF_BYTES), idesc_pv, ks ? 1u : 0u);
                tc_commit(&v_empty[st]);
                tc_commit(pv_full);
            }
        }
    } else {
        // ---- softmax warps: thread = row of the tile ---------------------------------------------------
        const int qd = warp & 3;
        const int r = qd * 32 + lane;
        const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
        const bool valid = r < rows_valid;
        const int tk = valid ? r / group : 0;
        const int tok = q_begin + tok0 + tk;
        const int pos = pos_lo + tk;
        const int head = kvh * group + (valid ? r % group : 0);
        if (nb > 0) {
            // Q row into shared memory, K-major with the 128-byte swizzle: 16-byte piece c of a 128-byte row
            // goes to piece c ^ (row % 8)
            const uint4* src = reinterpret_cast<const uint4*>(p.qkv + (size_t)tok * p.qkv_stride + (size_t)head * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(q_s + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        float o[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < nb && !timed_out; ++j) {
            const int st = j & 1;
            if (!mbar_wait(&s_full[st], (j >> 1) & 1)) { timed_out = true; break; }
            tc_fence_after();
            const int kb = key_lo + j * TK;
            // a block all of whose keys every row of the tile sees needs no mask
            const bool open = (kb + TK - 1 <= pos_lo) && (p.window <= 0 || kb > pos_hi - p.window);
            const uint32_t s_addr = tmem + lane_base + (uint32_t)(st * TK);
            const float raw_max = open ? row_max<false>(s_addr, kb, pos, p.window, valid)
                                       : row_max<true>(s_addr, kb, pos, p.window, valid);
            const float mx = fmaxf(m, raw_max * p.scale_log2);          // the scale is positive
            const float corr = (mx == -INFINITY) ? 1.f : ex2(m - mx);
            const float base = (mx == -INFINITY) ? 0.f : mx;
            m = mx;
            if (j > 0) {
                // the product of the block before: O = (O + P V) * correction.  Its MMAs have read P, too.
                if (!mbar_wait(pv_full, (j - 1) & 1)) { timed_out = true; break; }
                tc_fence_after();
                const bool rescale = __any_sync(0xffffffffu, corr != 1.f);
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t raw[32];
                    tc_ld32(tmem + lane_base + 2 * TK + c0, raw);
                    if (rescale) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[c0 + i] = (o[c0 + i] + __uint_as_float(raw[i])) * corr;
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[c0 + i] += __uint_as_float(raw[i]);
                    }
                }
            }
            const float lsum = open ? write_p<false>(s_addr, p_s, r, kb, pos, p.window, valid, p.scale_log2, base)
                                    : write_p<true>(s_addr, p_s, r, kb, pos, p.window, valid, p.scale_log2, base);
            l = l * corr + lsum;
            if (j == nb - 1) {
                // The last run of 16 keys may reach beyond the last key, into rows of the page that hold
                // whatever was there before.  Their P is 0, but 0 times a stale NaN or infinity is not:
                // those rows of V are cleared before the product reads them.
                const int first = key_hi - kb, last = min(TK, (first + 15) / 16 * 16);
                if (first < last) {
                    if (!mbar_wait(&v_full[st], (j >> 1) & 1)) { timed_out = true; break; }
                    for (int idx = threadIdx.x - 64; idx < (last - first) * HALVES * 8; idx += 128) {
                        const int row = first + idx / (HALVES * 8), piece = idx % (HALVES * 8);
                        *reinterpret_cast<uint4*>(v_s + st * TILE_BYTES + (piece >> 3) * HALF_BYTES + row * 128 + ((piece & 7) << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            // S has been read and P is written: tell the MMA warp
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_empty[st]);
                mbar_arrive(p_full);
            }
        }
        if (nb > 0 && !timed_out) {
            if (!mbar_wait(pv_full, (nb - 1) & 1)) timed_out = true;
            tc_fence_after();
            if (!timed_out) {
                // the loads of tensor memory are warp-wide: rows without a query take part and store nothing
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = p.out + ((size_t)tok * p.heads + head) * D;
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t raw[32];
                    tc_ld32(tmem + lane_base + 2 * TK + c0, raw);
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            hp[e] = __floats2bfloat162_rn((o[c0 + i + 2 * e] + __uint_as_float(raw[i + 2 * e])) * inv,
                                                          (o[c0 + i + 2 * e + 1] + __uint_as_float(raw[i + 2 * e + 1])) * inv);
                        if (valid) *reinterpret_cast<uint4*>(dst + c0 + i) = u;
                    }
                }
            }
        }
    }
    __syncwarp();
    if (timed_out && p.status) set_status(p.status, kStatusWaitTimeout, blockIdx.x);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
    }
}

}  // namespace

bool attention_tc_supports(int head_dim, int heads, int kv_heads) {
    return head_dim == 128 && kv_heads > 0 && heads % kv_heads == 0 && heads / kv_heads <= TQ;
}

cudaError_t launch_attention_tc(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                const int* tiles, int n_tiles, int n_pages, int heads, int kv_heads, int head_dim,
                                int page_size, int window, float scale, int* status, cudaStream_t stream) {
    if (n_tiles == 0) return cudaSuccess;
    if (!attention_tc_supports(head_dim, heads, kv_heads) || page_size % 16 != 0 || tiles == nullptr) return cudaErrorInvalidValue;
    const long long cache_rows = (long long)n_pages * kv_heads * page_size;
    if (cache_rows >= (1LL << 31) - 16) return cudaErrorInvalidValue;
    CUtensorMap map_k, map_v;
    if (!make_map(&map_k, k_cache, cache_rows, head_dim, 16) || !make_map(&map_v, v_cache, cache_rows, head_dim, 16))
        return cudaErrorInvalidValue;
    AttnTcParams p;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.out = (__nv_bfloat16*)out;
    p.cu_q = cu_q;
    p.q_start = q_start;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.tiles = (const int2*)tiles;
    p.n_pages = n_pages;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.page_size = page_size;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.tokens_per_tile = TQ / (heads / kv_heads);
    p.cache_rows = (int)cache_rows;
    p.status = status;
    constexpr int smem = (2 + 2 * 2 * 2 + 2) * HALF_BYTES + 1024 + 256;     // Q, K x2, V x2 (two halves each), P
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    return launch(attention_tc_kernel<128>, dim3(n_tiles, kv_heads, 1), dim3(ATC_THREADS, 1, 1), smem, stream, map_k, map_v, p);
}

}  // namespace vtb
