// out = x w^T (+ bias) on the 5th-generation tensor cores: TMA -> shared memory -> tcgen05.mma ->
// tensor memory -> registers -> global memory.  bfloat16 operands, 32-bit accumulation, one
// rounding at the end (the bias is added in 32-bit before it).
//
// vt-transformer calls cuBLASLt for these products and adds the bias in a second pass that rounds
// again (v1/tensortype/cuda_kernels/lt_sgemm.cu:55-126, v1/tensortype/cuda_tensor.cpp:544-563).
// Here both x [M, K] and w [N, K] are K-major, so either can be the 128-row operand of the MMA:
//   * many rows of x (prompt portions): a tile is 128 rows of x by BN rows of w, D[token, feature];
//   * few rows of x (decode): "swapped": a tile is 128 rows of w by all rows of x (BN = 16..64),
//     D[feature, token], so a weight is read once and the small batch rides along.  A matrix with
//     fewer tiles than SMs has its k range cut over several CTAs (grid z) so that one wave of CTAs
//     covers the machine; each CTA leaves its share in a scratch buffer and counts itself in; the
//     CTA that arrives last adds the shares in rank order and stores (no CTA waits for another).
//
// The kernel is persistent: one CTA an SM, each taking tiles in turn.  Warp 0 issues the TMA loads
// (one elected thread), warp 1 owns the tensor memory and issues the MMAs (one elected thread), warps
// 2..5 read the accumulator back (tcgen05.ld, each warp its quarter of the 128 lanes) and store.  A
// ring of STAGES stages of 64 k (128-byte rows, 128-byte swizzle) lies between loads and MMAs, with a
// full and an empty mbarrier a stage, and runs on across tiles.  The accumulator is double-buffered
// in tensor memory, so the epilogue of a tile runs under the MMAs of the next one.
// TMA fills what lies outside a matrix with zeros, so any M, N and K (K % 8 == 0) is taken.
// Every wait on a barrier is bounded by a clock limit; a wait that runs out records it in the status
// word and the CTA winds down: tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "look_ahead.cuh"
#include "tc_common.cuh"

namespace vtb {

namespace {

constexpr int BM = 128;                  // rows of the 128-lane operand in a tile
constexpr int BK = 64;                   // k in a stage: 64 bfloat16 = one 128-byte swizzled row
constexpr int A_STAGE = BM * BK * 2;     // 16 KB
constexpr int THREADS = 192;
// BN: rows of the other operand in a tile (columns of the accumulator).  SWAP: the 128-row operand is w.
template <int BN, int STAGES, bool SWAP, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const float* __restrict__ bias, TOut* __restrict__ out, int rows_a, int rows_b, int k, int ldo, int n_full,
               int s_tail, float* __restrict__ scratch, int* __restrict__ counters, int* status,
               const __grid_constant__ CUtensorMap map_ahead, const AheadTiles ahead) {
    constexpr int B_STAGE = BN * BK * 2;
    constexpr int COLS = BN < 32 ? 32 : BN;          // tensor-memory columns of an accumulator
    constexpr int ALLOC = 2 * COLS <= 64 ? 64 : 2 * COLS <= 128 ? 128 : 2 * COLS <= 256 ? 256 : 512;   // a power of two
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_s = smem;
    unsigned char* b_s = smem + STAGES * A_STAGE;
    uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * B_STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]: the MMAs of a unit are done, its accumulator is whole
    uint64_t* acc_empty = acc_full + 2;        // [2]: the epilogue has read the accumulator, it may be overwritten
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a_tiles = (rows_a + BM - 1) / BM, b_tiles = (rows_b + BN - 1) / BN;
    // Units of work: the first n_full tiles whole, every tile after them cut into s_tail shares of k.
    const int units = n_full + (a_tiles * b_tiles - n_full) * s_tail;
    const int nkb_all = (k + BK - 1) / BK;
    auto unit_of = [&](int u, int& tile, int& krank, int& ks) {
        if (u < n_full) { tile = u; krank = 0; ks = 1; }
        else { const int t = u - n_full; tile = n_full + t / s_tail; krank = t % s_tail; ks = s_tail; }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);       // one arrival from each epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(ALLOC));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;
    // Barriers and tensor memory are set up.  The kernels before this one in the stream may still be
    // running (programmatic dependent launch): nothing they write may be read, and nothing they read may
    // be written, before pdl_wait.  The weights are written by no kernel, so the loader starts to fetch
    // the first stages of the weight operand at once; x, the bias and all stores wait.
    pdl_launch();

    // A CTA takes the units blockIdx.x, blockIdx.x + gridDim.x, ...  A unit is (tile of the 128-row operand,
    // tile of the other operand, share of k), the first index running fastest: CTAs that run together
    // share the other operand's tile, which is then fetched from HBM once and found in L2 after.
    if (warp == 0) {
        if (lane == 0) {
            int kit = 0;                               // k-blocks loaded so far, over all units: ring position
            bool waited = false;
            for (int u = blockIdx.x; u < units && !timed_out; u += gridDim.x) {
                int tile, krank, ks;
                unit_of(u, tile, krank, ks);
                const int a_row0 = (tile % a_tiles) * BM, b_row0 = (tile / a_tiles) * BN;
                const int kb0 = (int)((long long)krank * nkb_all / ks), kb1 = (int)((long long)(krank + 1) * nkb_all / ks);
                int kb = kb0;
                if (!waited) {
                    // first unit: the weight halves of the first stages go out before the wait
                    const int early = min(STAGES, kb1 - kb0);
                    for (int i = 0; i < early; ++i) {
                        mbar_expect_tx(&full[i], A_STAGE + B_STAGE);
                        if (SWAP) tma_load_2d(a_s + i * A_STAGE, &map_a, (kb0 + i) * BK, a_row0, &full[i]);
                        else tma_load_2d(b_s + i * B_STAGE, &map_b, (kb0 + i) * BK, b_row0, &full[i]);
                    }
                    pdl_wait();
                    waited = true;
                    for (int i = 0; i < early; ++i) {
                        if (SWAP) tma_load_2d(b_s + i * B_STAGE, &map_b, (kb0 + i) * BK, b_row0, &full[i]);
                        else tma_load_2d(a_s + i * A_STAGE, &map_a, (kb0 + i) * BK, a_row0, &full[i]);
                    }
                    kb += early;
                    kit += early;
                }
                for (; kb < kb1; ++kb, ++kit) {
                    const int s = kit % STAGES;
                    if (kit >= STAGES && !mbar_wait(&empty[s], ((kit / STAGES) & 1) ^ 1)) { timed_out = true; break; }
                    mbar_expect_tx(&full[s], A_STAGE + B_STAGE);
                    tma_load_2d(a_s + s * A_STAGE, &map_a, kb * BK, a_row0, &full[s]);
                    tma_load_2d(b_s + s * B_STAGE, &map_b, kb * BK, b_row0, &full[s]);
                }
            }
            // This CTA's last load is on its way: from here to the first loads of the next kernel (the last MMAs, the
            // epilogue, the end of the grid, the next kernel's set-up and its wait for x) HBM would have nothing to do.
            // The weights of the product that runs next are written by no kernel: the first k-blocks of its first
            // units are asked into L2 now.
            for (int u = blockIdx.x; u < ahead.units && ahead.depth > 0; u += gridDim.x) {
                int bx, by;
                for (int i = 0; i < ahead.depth && ahead_box(ahead, u, i, bx, by); ++i) ahead_prefetch(&map_ahead, bx, by);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BM, BN);
            int kit = 0, ui = 0;
            for (int u = blockIdx.x; u < units && !timed_out; u += gridDim.x, ++ui) {
                int tile, krank, ks;
                unit_of(u, tile, krank, ks);
                const int kb0 = (int)((long long)krank * nkb_all / ks), kb1 = (int)((long long)(krank + 1) * nkb_all / ks);
                const int buf = ui & 1;
                // the accumulator of two units ago must have been read
                if (ui >= 2 && !mbar_wait(&acc_empty[buf], ((ui >> 1) & 1) ^ 1)) { timed_out = true; break; }
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(buf * COLS);
                for (int kb = kb0; kb < kb1; ++kb, ++kit) {
                    const int s = kit % STAGES;
                    if (!mbar_wait(&full[s], (kit / STAGES) & 1)) { timed_out = true; break; }
                    tc_fence_after();
                    const uint64_t ad = smem_desc(a_s + s * A_STAGE), bd = smem_desc(b_s + s * B_STAGE);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)   // 16 k = 32 bytes further along the swizzled row
                        tc_mma(acc, ad + 2 * kk, bd + 2 * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);                  // the stage is free when these MMAs have read it
                }
                tc_commit(&acc_full[buf]);                 // the accumulator is whole when all MMAs are done
            }
        }
    }
    __syncwarp();
    pdl_wait();    // every thread waits before it stores or leaves (the loader did so above already)

    // ---- epilogue: warps 2..5, each its quarter of the lanes --------------------------------------
    if (warp >= 2) {
        const int q = warp & 3;
        const int r = q * 32 + lane;                   // lane of the accumulator = row of the 128-row operand
        int ui = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++ui) {
            int tile, krank, ksplit;
            unit_of(u, tile, krank, ksplit);
            const int a_row0 = (tile % a_tiles) * BM, b_row0 = (tile / a_tiles) * BN;
            const int cut = tile - n_full;              // index among the tiles that are cut
            const int buf = ui & 1;
            bool ok = !timed_out && mbar_wait(&acc_full[buf], (ui >> 1) & 1);
            if (!ok) timed_out = true;
            tc_fence_after();
            float* mine = (EPI == 2) ? nullptr : scratch + ((size_t)cut * ksplit + krank) * (BN * BM);   // this unit's share [BN][128]
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (ok) {
                    uint32_t raw[16];
                    tc_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * COLS + c0), raw);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(raw[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
                if (c0 + 16 >= BN) {
                    // the last columns are in registers: the MMA warp may overwrite this accumulator
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                }
                if (EPI == 2) {
                    // this share of k as it is, into out[share]: the kernel that reads the result adds the shares
                    if (ok)
                        emit16<SWAP, 0, TOut>(v, r, a_row0, b_row0, c0, rows_a, rows_b, krank == 0 ? bias : nullptr,
                                              out + (size_t)krank * rows_b * ldo, ldo);
                    continue;
                }
                if (ksplit > 1) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (c0 + i) * BM + r, v[i]);
                    continue;
                }
                emit16<SWAP, EPI, TOut>(v, r, a_row0, b_row0, c0, rows_a, rows_b, bias, out, ldo);
            }
            if (EPI != 2 && ksplit > 1) {
                // count this unit in; the one that finds all others counted adds the shares and stores
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (threadIdx.x == 64) *last_flag = (atomicAdd(&counters[cut], 1) == ksplit - 1) ? 1 : 0;
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                const bool last = *last_flag != 0;
                asm volatile("bar.sync 1, 128;\n" ::: "memory");   // all have read the flag before it is written again
                if (last) {
                    __threadfence();
                    const float* all = scratch + (size_t)cut * ksplit * (BN * BM);
                    const bool live = (a_row0 + r) < rows_a;
                    // 16 columns at a time, all their loads in flight together; ranks added in order
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (b_row0 + c0 >= rows_b) break;
                        float sum[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) sum[i] = 0.f;
                        if (live) {
#pragma unroll 4
                            for (int rk = 0; rk < ksplit; ++rk) {
                                const float* src = all + ((size_t)rk * BN + c0) * BM + r;
#pragma unroll
                                for (int i = 0; i < 16; ++i) sum[i] += __ldcg(src + i * BM);
                            }
                        }
                        emit16<SWAP, EPI, TOut>(sum, r, a_row0, b_row0, c0, rows_a, rows_b, bias, out, ldo);
                    }
                    if (threadIdx.x == 64) counters[cut] = 0;       // ready for the next launch
                }
            }
        }
    }
    if (timed_out && status) set_status(status, kStatusWaitTimeout, blockIdx.x);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(ALLOC));
    }
}

// ---- host side ------------------------------------------------------------------------------------

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

template <int BN, int STAGES, bool SWAP, int EPI, typename TOut>
cudaError_t launch_cfg(const void* a, int rows_a, const void* b, int rows_b, int k, const float* bias, TOut* out, int ldo,
                       int n_full, int s_tail, float* scratch, int* counters, int* status, cudaStream_t stream,
                       const NextProduct* next) {
    CUtensorMap map_a, map_b, map_ahead;
    if (!make_map(&map_a, a, rows_a, k, BM) || !make_map(&map_b, b, rows_b, k, BN)) return cudaErrorInvalidValue;
    AheadTiles ahead = {1, 0, 1, 1, 0};
    if (!SWAP || !look_ahead(next, rows_b, &map_ahead, &ahead)) map_ahead = map_a;
    constexpr int smem = STAGES * (A_STAGE + BN * BK * 2) + 1024 + 256;
    static std::atomic<unsigned long long> configured{0};
    cudaError_t e = allow_dynamic_smem(gemm_tc_kernel<BN, STAGES, SWAP, EPI, TOut>, smem, configured);
    if (e != cudaSuccess) return e;
    const int tiles = ((rows_a + BM - 1) / BM) * ((rows_b + BN - 1) / BN);
    const int units = n_full + (tiles - n_full) * s_tail;
    return launch(gemm_tc_kernel<BN, STAGES, SWAP, EPI, TOut>, dim3(units < sm_count() ? units : sm_count(), 1, 1),
                  dim3(THREADS, 1, 1), smem, stream, map_a, map_b, bias, out, rows_a, rows_b, k, ldo, n_full, s_tail, scratch,
                  counters, status, map_ahead, ahead);
}

// Into how many shares k is cut when w is the 128-row operand (small batches).  One CTA fits an SM, so the
// CTAs run in waves of one an SM; k is cut over s CTAs so that the last wave is full, counting a fixed cost
// a CTA (set-up, filling the ring, the merge) as a few k-blocks: least waves * (k-blocks a CTA + cost).
int small_batch_ksplit(int n, int k, int bn, bool have_scratch, long long scratch_floats, int n_counters) {
    const int sms = sm_count();
    const int tiles = (n + BM - 1) / BM, nkb = (k + BK - 1) / BK;
    int ksplit = 1;
    long best = -1;
    for (int s = 1; s <= 16; ++s) {
        if (s > 1 && (nkb / s < 4 || s > nkb || !have_scratch || tiles > n_counters ||
                      (long long)tiles * s * bn * BM > scratch_floats))
            break;
        const long waves = (tiles * s + sms - 1) / sms;
        const long cost = waves * ((nkb + s - 1) / s + 6 + (s > 1 ? 2 : 0));
        if (best < 0 || cost < best) {
            best = cost;
            ksplit = s;
        }
    }
    return ksplit;
}

// Which operand has the 128 rows, for up to 256 rows of x.  Swapped (w has them) every weight is streamed once and
// the batch rides along as columns; its epilogue then holds a feature a thread and writes the batch's rows with a
// stride, which costs more the wider the batch is.  Measured on a B200 (products alone, from cold caches): up to 32
// rows swapped always wins; beyond, it wins only where the weights are large enough that streaming them is the
// whole cost (from about 64 MB; the product with SiLU(gate) * up, whose swapped epilogue pairs rows across
// lanes, from 100 MB and up to 64 rows).  Shares left unadded for the norm (EPI 2) exist swapped only.
template <int EPI>
bool swapped_for(int m, int n, int k) {
    if (m > 256) return false;
    if (EPI == 2 || m <= 32) return true;
    const long long weight_bytes = (long long)n * k * 2;
    if (EPI == 1) return m <= 64 && weight_bytes >= (100LL << 20);
    return weight_bytes >= (64LL << 20);
}

template <int EPI, typename TOut>
cudaError_t launch_typed(const void* x, const void* w, const float* bias, TOut* out, int m, int n, int k, float* scratch,
                         long long scratch_floats, int* counters, int n_counters, int* status, cudaStream_t stream,
                         const NextProduct* next) {
    if (swapped_for<EPI>(m, n, k)) {
        // swapped: w is the 128-row operand and every weight is streamed once; the batch rides along as 16 to 256
        // columns.  (At 256 columns a k-block's MMAs take about as long as its 16 KB of weights take to arrive.)
        const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)));
        const bool have_scratch = scratch != nullptr && counters != nullptr;
        const int ksplit = (EPI == 2) ? gemm_tc_shares(m, n, k)
                                      : small_batch_ksplit(n, k, bn, have_scratch, scratch_floats, n_counters);
        if (bn == 16) return launch_cfg<16, 8, true, EPI, TOut>(w, n, x, m, k, bias, out, EPI == 1 ? n / 2 : n, 0, ksplit, scratch, counters, status, stream, next);
        if (bn == 32) return launch_cfg<32, 8, true, EPI, TOut>(w, n, x, m, k, bias, out, EPI == 1 ? n / 2 : n, 0, ksplit, scratch, counters, status, stream, next);
        if (bn == 64) return launch_cfg<64, 8, true, EPI, TOut>(w, n, x, m, k, bias, out, EPI == 1 ? n / 2 : n, 0, ksplit, scratch, counters, status, stream, next);
        if (bn == 128) return launch_cfg<128, 6, true, EPI, TOut>(w, n, x, m, k, bias, out, EPI == 1 ? n / 2 : n, 0, ksplit, scratch, counters, status, stream, next);
        return launch_cfg<256, 4, true, EPI, TOut>(w, n, x, m, k, bias, out, EPI == 1 ? n / 2 : n, 0, ksplit, scratch, counters, status, stream, next);
    }
    if constexpr (EPI == 2) {
        return cudaErrorInvalidValue;     // shares are left unadded for small batches only
    } else {
        // x is the 128-row operand: tiles of 128 tokens by 256 (or 128) features, one an SM at a time.  With fewer
        // tiles than SMs and a long k, every tile is cut into shares of k so that more SMs work.  (Cutting the
        // tiles of the last, partial round of a larger product was tried and lost: merging the shares of a
        // 128x256 tile costs the CTA that does it more than the shorter round saves.)
        const int sms = sm_count();
        const bool wide = !(n <= 128 || m <= 128);
        // The width of a tile: 256 features, or fewer where that makes the rounds of one tile an SM come out
        // better (n = 3584 and 2,048 tokens: 224 tiles of 256 features are 1.5 rounds and take the time of 2;
        // 288 tiles of 208 are 1.95 rounds of narrower tiles; a few hundred tokens: tiles of 160 or 128 features,
        // so that most SMs have one: 640 tokens by 3584 x 18944 in 109 us where tiles of 192 took 165).  Cost of a
        // width: rounds * (width + a fixed part for the 128-row operand of every k-block).
        int bn = wide ? 256 : 128;
        // a small product (a wide batch of a small model: 256 rows by a matrix of a megabyte or two) has a dozen tiles
        // of 128 x 192: tiles of 64 features give four times the CTAs, each done in a quarter of the time
        const long tiles_128 = (long)((m + BM - 1) / BM) * ((n + 127) / 128);
        if (tiles_128 * 2 <= sms) {
            bn = 64;
        } else if (wide) {
            long best = -1;
            for (int cand : {256, 240, 224, 208, 192, 160, 128}) {
                const long t = (long)((m + BM - 1) / BM) * ((n + cand - 1) / cand);
                const long cost = ((t + sms - 1) / sms) * (cand + 24);
                if (best < 0 || cost < best) {
                    best = cost;
                    bn = cand;
                }
            }
        }
        const int tiles = ((m + BM - 1) / BM) * ((n + bn - 1) / bn), nkb = (k + BK - 1) / BK;
        int rem = tiles % sms, n_full = tiles - rem, s_tail = 1;
        if (tiles < sms && scratch != nullptr && counters != nullptr && rem <= n_counters) {
            double best = 1.0;
            for (int s = 2; s <= 4; ++s) {
                // a share must be long enough to pay for the merge of the shares
                if (nkb / s < 48 || (long long)rem * s * bn * BM > scratch_floats) break;
                const double cost = (double)((rem * s + sms - 1) / sms) / s + 0.04;
                if (cost < best) {
                    best = cost;
                    s_tail = s;
                }
            }
        }
        if (s_tail == 1) n_full = tiles;
        const int ldo = EPI == 1 ? n / 2 : n;
        switch (bn) {
            case 256: return launch_cfg<256, 4, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 240: return launch_cfg<240, 4, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 224: return launch_cfg<224, 5, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 208: return launch_cfg<208, 5, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 192: return launch_cfg<192, 5, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 160: return launch_cfg<160, 5, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
            case 128: if (wide) return launch_cfg<128, 6, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
        }
        if (bn == 64) return launch_cfg<64, 8, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
        return launch_cfg<128, 4, false, EPI, TOut>(x, m, w, n, k, bias, out, ldo, n_full, s_tail, scratch, counters, status, stream, next);
    }
}

}  // namespace

// How the product that runs next over the same m rows will cut its weights, if it runs with w as the 128-row operand;
// false if there is nothing to ask for.  (It stands on the workspace that the engine gives every product; where the
// next launch decides otherwise, other boxes of the same matrix are asked for and nothing else changes.)
bool look_ahead(const NextProduct* next, int m, CUtensorMap* map, AheadTiles* tiles) {
    if (next == nullptr || next->w == nullptr || next->bytes < A_STAGE || next->k % 8 != 0 || next->k < 8 || next->n < 1 ||
        ((uintptr_t)next->w & 15) != 0)
        return false;
    const int n = next->n, k = next->k;
    const bool swapped = next->epilogue == 2 ? swapped_for<2>(m, n, k)
                         : next->epilogue == 1 ? swapped_for<1>(m, n, k) : swapped_for<0>(m, n, k);
    if (!swapped) return false;
    const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)));
    const int ks = next->epilogue == 2 ? gemm_tc_shares(m, n, k) : small_batch_ksplit(n, k, bn, true, 8LL << 20, 4096);
    tiles->a_tiles = (n + BM - 1) / BM;
    tiles->s_tail = ks;
    tiles->nkb = (k + BK - 1) / BK;
    const int sms = sm_count();
    tiles->units = tiles->a_tiles * ks < sms ? tiles->a_tiles * ks : sms;
    const long long boxes = next->bytes / A_STAGE;
    const long long depth = (boxes + tiles->units - 1) / tiles->units, longest = tiles->nkb / ks + 1;
    tiles->depth = (int)(depth < longest ? depth : longest);
    return make_map(map, next->w, n, k, BM);
}

int gemm_tc_shares(int m, int n, int k) {
    const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)));
    return small_batch_ksplit(n, k, bn, true, 1LL << 60, 1 << 30);
}

// Whether a product goes to the kernel that gives a tile to a pair of CTAs (gemm_tc_pair.cu).  Measured on a B200
// against the kernel of this file: it wins by 5 to 13 % where every pair has a tile of 256 x 256 to begin with and k is
// long enough that the ring, not the first fill and the last epilogue, is the time (7B: every product from 1,536
// rows on, the feed-forward's from 512; 1.5B: the feed-forward's from 1,024 rows, by 1 to 7 %); with k = 896 or fewer
// tiles than pairs it is level or loses.
static bool pair_for(int m, int n, int k) {
    if (k < 1536 || m <= 256) return false;
    const long pair_tiles = (long)((m + 255) / 256) * ((n + 255) / 256);
    // a long inner dimension under a few hundred rows (the feed-forward's second product of a short portion): the pairs
    // take it with k in two shares, 76 to 92 us where the kernel of one CTA a tile takes 97 to 104 (272 to 512 rows by
    // 3584 x 18944); with more tiles than half the pairs there are no shares and the kernel of one CTA a tile is ahead again
    if (k >= 8192 && 4 * pair_tiles <= sm_count()) return true;
    if (m < 512) return false;
    return pair_tiles * 2 >= sm_count();
}

cudaError_t launch_gemm_tc(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n, int k,
                           int epilogue, float* scratch, long long scratch_floats, int* counters, int n_counters,
                           int* status, cudaStream_t stream, const NextProduct* next) {
    if (m == 0 || n == 0) return cudaSuccess;
    if (k % 8 != 0 || k < 8) return cudaErrorInvalidValue;
    if (out_dtype == kBF16 && (epilogue == 0 || epilogue == 1) && pair_for(m, n, k))
        return launch_gemm_tc_pair(x, w, bias, out, m, n, k, epilogue, 0, scratch, scratch_floats, counters, n_counters, status, stream);
    if (epilogue == 1) {
        if (n % 16 != 0 || bias != nullptr || out_dtype != kBF16) return cudaErrorInvalidValue;
        return launch_typed<1, __nv_bfloat16>(x, w, nullptr, (__nv_bfloat16*)out, m, n, k, scratch, scratch_floats,
                                              counters, n_counters, status, stream, next);
    }
    if (epilogue == 2) {
        if (out_dtype != kF32 || m > 256) return cudaErrorInvalidValue;
        return launch_typed<2, float>(x, w, bias, (float*)out, m, n, k, nullptr, 0, nullptr, 0, status, stream, next);
    }
    if (epilogue != 0) return cudaErrorInvalidValue;
    if (out_dtype == kBF16)
        return launch_typed<0, __nv_bfloat16>(x, w, bias, (__nv_bfloat16*)out, m, n, k, scratch, scratch_floats, counters,
                                              n_counters, status, stream, next);
    if (out_dtype == kF32)
        return launch_typed<0, float>(x, w, bias, (float*)out, m, n, k, scratch, scratch_floats, counters, n_counters,
                                      status, stream, next);
    return cudaErrorInvalidValue;
}

}  // namespace vtb
