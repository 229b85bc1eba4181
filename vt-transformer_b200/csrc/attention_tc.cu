// Attention of prompt portions over the paged cache on the 5th-generation tensor cores (head sizes 64 and 128).
//
// The computation is the chain of vt-transformer's graph (scores = q k^T / sqrt(d), causal mask, softmax,
// P V: v1/models/qwen2-7b/inference_fp16.dag:307-318) done block by block with a running maximum and sum,
// as in attention_mma.cu; here both products run as tcgen05.mma with their results in tensor memory:
//
//   tile   128 rows, a row being (token, head of the KV group): a key is fetched once for the whole group
//   block  128 keys in runs of 16, 32, 64 or 128 keys (the largest that divides the page size), each run
//          inside one page; TMA brings a run of K and of V as two boxes of 64 dims (128-byte rows, 128-byte
//          swizzle); runs beyond the last key are zero-filled.  The TMA unit takes a box in some tens of
//          cycles whatever its size: pages of 16 keys hold this kernel to about half of what pages of 64 allow
//   S      = Q K^T: A = Q (K-major), B = K block (K-major, N = 128 keys), accumulator [128 x 128] floats in
//          tensor memory; two buffers, one for the even and one for the odd blocks
//   P      two groups of four warps, one for the even and one for the odd blocks, a thread a row: the row of S
//          into registers (four tcgen05.ld on their way together), mask, maximum, scale, 2^x, sum; P rounded to
//          bfloat16 and stored (tcgen05.st) over the first 64 columns of S: it is the A operand of the next
//          product.  The half of P over the first 64 keys is announced by itself, so that its product with V
//          runs while the warps still compute the other half
//   PV     O += P V: A = P in tensor memory, B = V block as it lies ([key][dim]: MN-major); each group has
//          its own accumulator O [128 x 128] and its own running maximum and sum, which meet at the end
//
// While one group works on the scores of its block, the tensor cores compute the other group's products.
// The maximum a group scales by is raised only when the true maximum has moved by more than 2^8 (P stays
// below 2^8, exact in the 32-bit sum and with the same relative rounding in bfloat16); raising it means
// multiplying O in tensor memory by the correction, which then happens in few blocks only.
//
// Warp 0 loads (one thread), warp 1 issues the MMAs (one thread), warps 2..5 and 6..9 are the two groups.
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
constexpr int STEP_BYTES = 16 * 128;    // the 16 keys of one MMA in one half
constexpr int ATC_THREADS = 320;        // loader, MMA issuer, two groups of four softmax warps
constexpr float RAISE = 8.f;            // the scaling maximum follows the true one when it is this far behind (log2)

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
    int run_keys;            // keys of a run: 16, 32, 64 or 128, a divisor of the page size
    int cache_rows;          // pages * kv_heads * page_size: a row index beyond it makes TMA fill zeros
    int* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// The 128 scores of a row of S from tensor memory into registers: four loads on their way together, one wait.
#define VTB_TC_LD32_ASYNC(taddr, r, o)                                                                                   \
    asm volatile(                                                                                                        \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"                 \
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"                                     \
        : "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]),   \
          "=r"(r[o + 7]), "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]),              \
          "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15]), "=r"(r[o + 16]), "=r"(r[o + 17]), "=r"(r[o + 18]),           \
          "=r"(r[o + 19]), "=r"(r[o + 20]), "=r"(r[o + 21]), "=r"(r[o + 22]), "=r"(r[o + 23]), "=r"(r[o + 24]),           \
          "=r"(r[o + 25]), "=r"(r[o + 26]), "=r"(r[o + 27]), "=r"(r[o + 28]), "=r"(r[o + 29]), "=r"(r[o + 30]),           \
          "=r"(r[o + 31])                                                                                                \
        : "r"(taddr))

__device__ __forceinline__ void load_row(uint32_t s_addr, uint32_t (&raw)[TK]) {
    VTB_TC_LD32_ASYNC(s_addr, raw, 0);
    VTB_TC_LD32_ASYNC(s_addr + 32, raw, 32);
    VTB_TC_LD32_ASYNC(s_addr + 64, raw, 64);
    VTB_TC_LD32_ASYNC(s_addr + 96, raw, 96);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Largest raw score of a row (its 128 scores in registers; kb: their first key).  MASKED: keys [lo, hi) of the
// block are seen by this row; the others count as -infinity.
template <bool MASKED>
__device__ __forceinline__ float row_max(const uint32_t (&raw)[TK], int lo, int hi) {
    float mx[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) mx[c] = -INFINITY;
#pragma unroll
    for (int i = 0; i < TK; i += 2) {
        const float a = (!MASKED || (i >= lo && i < hi)) ? __uint_as_float(raw[i]) : -INFINITY;
        const float b = (!MASKED || (i + 1 >= lo && i + 1 < hi)) ? __uint_as_float(raw[i + 1]) : -INFINITY;
        mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], a, b);
    }
    return fmaxf(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], max3(mx[5], mx[6], mx[7])));
}

// P = 2^(raw * scale - base) of half a row (the 64 keys from H * 64 on), rounded to bfloat16 and stored over 32 of the
// first 64 columns of the row of S (two keys a column); adds the unrounded values to `sum`.  Two values at a time
// where the hardware has an instruction for two (the scaling, the sum, the rounding); 2^x comes from the
// special-function unit.  (A quarter or a half of the 2^x as a polynomial on the FMA pipe instead was slower, and
// so was the kernel with no 2^x at all no faster: what the kernel waits for is the tensor pipe's queue, which one
// thread feeds, and the traffic of tensor memory, not these warps' arithmetic.)
template <bool MASKED, int H>
__device__ __forceinline__ void write_p_half(const uint32_t (&raw)[TK], uint32_t s_addr, int lo, int hi, float scale_log2, float base,
                                             float2 (&sum)[2]) {
    const float2 sc = make_float2(scale_log2, scale_log2), nb = make_float2(-base, -base);
#pragma unroll
    for (int c0 = H * 64; c0 < H * 64 + 64; c0 += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c0 + i]), __uint_as_float(raw[c0 + i + 1])), sc, nb);
            float2 pv = make_float2(ex2(x.x), ex2(x.y));
            if (MASKED) {
                pv.x = (c0 + i >= lo && c0 + i < hi) ? pv.x : 0.f;
                pv.y = (c0 + i + 1 >= lo && c0 + i + 1 < hi) ? pv.y : 0.f;
            }
            sum[(i >> 1) & 1] = __fadd2_rn(sum[(i >> 1) & 1], pv);
            __nv_bfloat162 b = __floats2bfloat162_rn(pv.x, pv.y);
            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        tc_st16(s_addr + (c0 >> 1), pk);
    }
}

template <int D>
__global__ void __launch_bounds__(ATC_THREADS)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const AttnTcParams p) {
    static_assert(D == 64 || D == 128, "built for head sizes 64 and 128");
    constexpr int HALVES = D / 64;
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;      // Q, a stage of K, a stage of V
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + TILE_BYTES;               // [2][TILE_BYTES]
    unsigned char* v_s = k_s + 2 * TILE_BYTES;           // [2][TILE_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * TILE_BYTES);
    // s_full[b]: S of a block with parity b is there (and its stage of K free); p_full[2 b + h]: half h of its P is
    // stored; o_done[b]: its product with V is done (and its stage of V free)
    uint64_t *k_full = bars, *v_full = bars + 2, *s_full = bars + 4, *p_full = bars + 6, *o_done = bars + 10,
             *q_full = bars + 12, *pair = bars + 13;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
    float* xch = reinterpret_cast<float*>(bars + 20);     // [2 groups][128 rows][maximum, sum]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // what the step's own inputs say about this tile (they are there before the step's first kernel starts)
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
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[2 * i], 4);
            mbar_init(&p_full[2 * i + 1], 4);
            mbar_init(&o_done[i], 1);
        }
        mbar_init(q_full, 8);
        for (int i = 0; i < 4; ++i) mbar_init(&pair[i], 2);
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
    // columns 0..127 and 128..255: S of the even and of the odd blocks (P over their first 64);
    // 256..383 and 384..511: O of the even and of the odd blocks
    const uint32_t tmem = *tmem_slot;
    pdl_launch();
    pdl_wait();                                 // q, and the keys and values of this step, come from kernels before

    bool timed_out = false;

    if (warp == 0) {
        if (nb > 0) {
            // Lane `run` looks up the page of its run of keys and issues the run's boxes; lane 0 waits
            // for the stage and announces the bytes.  The block table is read one block ahead of its use.
            const int* table = p.block_table + (size_t)seq * p.table_stride;
            auto row_of = [&](int j) -> int {
                const int key = key_lo + j * TK + (lane & 7) * p.run_keys;
                int row = p.cache_rows;                      // outside the cache: the box is filled with zeros
                if (j < nb && key < key_hi && (lane & 7) * p.run_keys < TK) {
                    const int page = table[key / p.page_size];
                    // a page behind a window may be gone already; its keys are masked
                    if (page >= 0 && page < p.n_pages) row = (page * p.kv_heads + kvh) * p.page_size + key % p.page_size;
                }
                return row;
            };
            // K or V of block j into its stage (j % 2), once the product that read the stage before is done
            auto load = [&](int j, int row, const CUtensorMap* map, unsigned char* base, uint64_t* full, uint64_t* empty) -> bool {
                const int st = j & 1;
                int ok = 1;
                if (lane == 0) {
                    if (j >= 2 && !mbar_wait(&empty[st], ((j >> 1) & 1) ^ 1)) ok = 0;
                    if (ok) mbar_expect_tx(&full[st], TILE_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) return false;
                if (lane * p.run_keys < TK) {
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(base + st * TILE_BYTES + h * HALF_BYTES + lane * p.run_keys * 128, map, h * 64, row, &full[st]);
                }
                return true;
            };
            // in the order in which the products want them: K0, K1, V0, K2, V1, ...
            int row_cur = row_of(0), row_next = row_of(1);
            if (!load(0, row_cur, &map_k, k_s, k_full, s_full)) timed_out = true;
            for (int j = 0; j < nb && !timed_out; ++j) {
                const int row_after = row_of(j + 2);
                if (j + 1 < nb && !load(j + 1, row_next, &map_k, k_s, k_full, s_full)) { timed_out = true; break; }
                if (!load(j, row_cur, &map_v, v_s, v_full, o_done)) timed_out = true;
                row_cur = row_next;
                row_next = row_after;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nb > 0) {
            const uint32_t idesc_s = instr_desc(TQ, TK), idesc_pv = instr_desc(TQ, D, true);
            // descriptors of the tiles' first bytes; a tile further on adds its distance / 16 to the address field
            const uint64_t desc_q = smem_desc(q_s), desc_k = smem_desc(k_s), desc_v = smem_desc_lbo(v_s, HALF_BYTES);
            auto issue_s = [&](int j, bool keys_there) -> bool {
                const int st = j & 1;
                if (!keys_there) {
                    if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
                    tc_fence_after();
                }
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)     // 16 dims = 32 bytes further along the swizzled rows
                        tc_mma(tmem + (uint32_t)(st * TK), desc_q + (uint64_t)((h * HALF_BYTES >> 4) + 2 * kk),
                               desc_k + (uint64_t)(((st * TILE_BYTES + h * HALF_BYTES) >> 4) + 2 * kk), idesc_s, (h | kk) ? 1u : 0u);
                tc_commit(&s_full[st]);
                return true;
            };
            if (!mbar_wait(q_full, 0)) timed_out = true;
            tc_fence_after();
            if (!timed_out && !issue_s(0, false)) timed_out = true;
            if (!timed_out && nb > 1 && !issue_s(1, false)) timed_out = true;
            for (int j = 0; j < nb && !timed_out; ++j) {
                const int st = j & 1;
                // (the barriers whose turn came long ago first: the keys of the block after next, this block's values)
                if (j + 2 < nb && !mbar_wait(&k_full[st], ((j + 2) >> 1) & 1)) { timed_out = true; break; }
                // the product over the first 64 keys runs while the softmax warps still write the P of the other 64
                if (!mbar_wait(&v_full[st], (j >> 1) & 1)) { timed_out = true; break; }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (!mbar_wait(&p_full[2 * st + h], (j >> 1) & 1)) { timed_out = true; break; }
                    tc_fence_after();
#pragma unroll
                    for (int ks = h * 4; ks < h * 4 + 4; ++ks)   // 16 keys: 8 columns of P, 16 rows of V further
                        tc_mma_ta(tmem + 2 * TK + st * D, tmem + (uint32_t)(st * TK + ks * 8),
                                  desc_v + (uint64_t)((st * TILE_BYTES + ks * STEP_BYTES) >> 4), idesc_pv, (j >= 2 || ks) ? 1u : 0u);
                }
                if (timed_out) break;
                tc_commit(&o_done[st]);
                // the scores of the group's next block go where this P lies: the tensor cores run the
                // products in the order in which they were issued
                if (j + 2 < nb && !issue_s(j + 2, true)) { timed_out = true; break; }
            }
        }
    } else {
        // ---- softmax warps: group g has the blocks g, g + 2, ...; a thread a row ---------------------------
        const int qd = warp & 3;
        const int g = (warp - 2) >> 2;
        const int r = qd * 32 + lane;
        const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
        const bool valid = r < rows_valid;
        const int tk = valid ? r / group : 0;
        const int tok = q_begin + tok0 + tk;
        const int pos = pos_lo + tk;
        const int head = kvh * group + (valid ? r % group : 0);
        if (nb > 0) {
            // half a Q row into shared memory, K-major with the 128-byte swizzle: 16-byte piece c of a 128-byte
            // row goes to piece c ^ (row % 8)
            const uint4* src = reinterpret_cast<const uint4*>(p.qkv + (size_t)tok * p.qkv_stride + (size_t)head * D + g * (D / 2));
#pragma unroll
            for (int c = 0; c < D / 16; ++c) {
                const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
                const int piece = g * (D / 16) + c;          // the row's 16-byte piece: 8 pieces a half of 64 dims
                *reinterpret_cast<uint4*>(q_s + (piece >> 3) * HALF_BYTES + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        const uint32_t s_addr = tmem + lane_base + (uint32_t)(g * TK);
        const uint32_t o_addr = tmem + lane_base + (uint32_t)(2 * TK + g * D);
        float m = -INFINITY, l = 0.f;       // the maximum P is scaled by (in log2 units), and the sum at that scale
        for (int j = g; j < nb && !timed_out; j += 2) {
            const int u = j >> 1;           // the group's u-th block
            if (!mbar_wait(&s_full[g], u & 1)) { timed_out = true; break; }
            tc_fence_after();
            const int kb = key_lo + j * TK;
            // a block all of whose keys every row of the tile sees needs no mask
            const bool open = (kb + TK - 1 <= pos_lo) && (p.window <= 0 || kb > pos_hi - p.window);
            uint32_t raw[TK];
            load_row(s_addr, raw);
            // keys [lo, hi) of the block are seen by this row
            const int hi = valid ? pos - kb + 1 : 0;
            const int lo = (p.window > 0) ? pos - p.window + 1 - kb : 0;
            const float raw_max = open ? row_max<false>(raw, lo, hi) : row_max<true>(raw, lo, hi);
            const float mx = fmaxf(m, raw_max * p.scale_log2);          // the scale is positive
            // a row that has seen no key yet takes the maximum as it is: its O is still zero
            const bool raise = (m != -INFINITY) && (mx > m + RAISE);
            if (__any_sync(0xffffffffu, raise)) {
                // O of this group, as the product of its block before left it, times 2^(old - new maximum)
                if (!mbar_wait(&o_done[g], (u - 1) & 1)) { timed_out = true; break; }
                tc_fence_after();
                const float corr = raise ? ex2(m - mx) : 1.f;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t raw[32];
                    tc_ld32(o_addr + c0, raw);
#pragma unroll
                    for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * corr);
                    tc_st32(o_addr + c0, raw);
                }
                l *= corr;
                if (raise) m = mx;
            }
            if (m == -INFINITY) m = mx;
            const float base = (m == -INFINITY) ? 0.f : m;
            if (j == nb - 1) {
                // The last run of keys may reach beyond the last key, into rows of the page that hold
                // whatever was there before.  Their P is 0, but 0 times a stale NaN or infinity is not:
                // those rows of V are cleared before the product reads them.
                const int first = key_hi - kb, last = min(TK, (first + p.run_keys - 1) / p.run_keys * p.run_keys);
                if (first < last) {
                    if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1)) { timed_out = true; break; }
                    for (int idx = r; idx < (last - first) * HALVES * 8; idx += 128) {
                        const int row = first + idx / (HALVES * 8), piece = idx % (HALVES * 8);
                        *reinterpret_cast<uint4*>(v_s + (j & 1) * TILE_BYTES + (piece >> 3) * HALF_BYTES + row * 128 + ((piece & 7) << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
            }
            float2 sum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            if (open) write_p_half<false, 0>(raw, s_addr, lo, hi, p.scale_log2, base, sum);
            else write_p_half<true, 0>(raw, s_addr, lo, hi, p.scale_log2, base, sum);
            // half of P is in tensor memory: tell the MMA warp
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[2 * g]);
            if (open) write_p_half<false, 1>(raw, s_addr, lo, hi, p.scale_log2, base, sum);
            else write_p_half<true, 1>(raw, s_addr, lo, hi, p.scale_log2, base, sum);
            l += (sum[0].x + sum[0].y) + (sum[1].x + sum[1].y);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[2 * g + 1]);
        }
        if (nb > 0 && !timed_out) {
            // the two groups' maxima and sums of the row meet; each thread then writes 64 dims of it
            xch[(g * 128 + r) * 2] = m;
            xch[(g * 128 + r) * 2 + 1] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(&pair[qd]);
            if (!mbar_wait(&pair[qd], 0)) timed_out = true;
            const int n_even = (nb + 1) >> 1, n_odd = nb >> 1;
            if (!timed_out && !mbar_wait(&o_done[0], (n_even - 1) & 1)) timed_out = true;
            if (!timed_out && n_odd > 0 && !mbar_wait(&o_done[1], (n_odd - 1) & 1)) timed_out = true;
            tc_fence_after();
            if (!timed_out) {
                const float m_other = xch[((g ^ 1) * 128 + r) * 2], l_other = xch[((g ^ 1) * 128 + r) * 2 + 1];
                const float m_all = fmaxf(m, m_other);
                const float w_mine = (m == -INFINITY) ? 0.f : ex2(m - m_all);
                const float w_other = (m_other == -INFINITY) ? 0.f : ex2(m_other - m_all);
                const float sum = l * w_mine + l_other * w_other;
                const float inv = sum > 0.f ? 1.f / sum : 0.f;
                const float w_even = (g == 0 ? w_mine : w_other) * inv, w_odd = (g == 0 ? w_other : w_mine) * inv;
                __nv_bfloat16* dst = p.out + ((size_t)tok * p.heads + head) * D + g * (D / 2);
                // the loads of tensor memory are warp-wide: rows without a query take part and store nothing
#pragma unroll 1
                for (int c0 = 0; c0 < D / 2; c0 += 32) {
                    uint32_t even[32], odd[32];
                    tc_ld32(tmem + lane_base + 2 * TK + g * (D / 2) + c0, even);
                    if (n_odd > 0) {
                        tc_ld32(tmem + lane_base + 2 * TK + D + g * (D / 2) + c0, odd);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) odd[i] = 0u;
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u4;
                        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&u4);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            hp[e] = __floats2bfloat162_rn(
                                __uint_as_float(even[i + 2 * e]) * w_even + __uint_as_float(odd[i + 2 * e]) * w_odd,
                                __uint_as_float(even[i + 2 * e + 1]) * w_even + __uint_as_float(odd[i + 2 * e + 1]) * w_odd);
                        if (valid) *reinterpret_cast<uint4*>(dst + c0 + i) = u4;
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
    return (head_dim == 128 || head_dim == 64) && kv_heads > 0 && heads % kv_heads == 0 && heads / kv_heads <= TQ;
}

cudaError_t launch_attention_tc(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                const int* tiles, int n_tiles, int n_pages, int heads, int kv_heads, int head_dim,
                                int page_size, int window, float scale, int* status, cudaStream_t stream) {
    if (n_tiles == 0) return cudaSuccess;
    if (!attention_tc_supports(head_dim, heads, kv_heads) || page_size % 16 != 0 || tiles == nullptr) return cudaErrorInvalidValue;
    const long long cache_rows = (long long)n_pages * kv_heads * page_size;
    if (cache_rows >= (1LL << 31) - 256) return cudaErrorInvalidValue;
    CUtensorMap map_k, map_v;
    const int run_keys = page_size % 128 == 0 ? 128 : page_size % 64 == 0 ? 64 : page_size % 32 == 0 ? 32 : 16;
    if (!make_map(&map_k, k_cache, cache_rows, head_dim, run_keys) || !make_map(&map_v, v_cache, cache_rows, head_dim, run_keys))
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
    p.run_keys = run_keys;
    p.status = status;
    // Q, two stages of K and of V (HALVES halves of 16 KB each), barriers, the exchange; never so little that two CTAs
    // would fit an SM: each takes all of its tensor memory
    const int halves = head_dim / 64;
    const int smem = max((1 + 2 * 2) * halves * HALF_BYTES + 1024 + 256 + 2 * 128 * 2 * 4, 120 * 1024);
    auto kernel = head_dim == 128 ? attention_tc_kernel<128> : attention_tc_kernel<64>;
    static std::atomic<unsigned long long> configured[2] = {{0}, {0}};
    cudaError_t e = allow_dynamic_smem(kernel, smem, configured[halves - 1]);
    if (e != cudaSuccess) return e;
    return launch(kernel, dim3(n_tiles, kv_heads, 1), dim3(ATC_THREADS, 1, 1), smem, stream, map_k, map_v, p);
}

}  // namespace vtb
