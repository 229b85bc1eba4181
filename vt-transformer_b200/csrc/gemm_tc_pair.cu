// out = x w^T (+ bias, or SiLU(gate) * up) for many rows of x, a tile to a PAIR of CTAs: tcgen05.mma.cta_group::2.
//
// The kernel of gemm_tc.cu gives a tile of 128 rows of x by 256 rows of w to one CTA; every k-block of 64 it brings
// 16 KB of x and 32 KB of w from L2 for 524 cycles of MMAs, and the products stand at 74 to 81 % of the tensor
// pipe.  Here two CTAs on neighbouring SMs (a cluster of two) share a tile of 256 rows of x by BN rows of w: each
// loads its own 128 rows of x and HALF of the rows of w (loads of its own: no multicast), and one thread of the
// first CTA issues MMAs that read both CTAs' shared memory and write both CTAs' tensor memory (each CTA ends up with
// its 128 rows by all BN columns).  A k-block then costs a CTA 16 + 16 KB, so the ring is six stages deep where it
// was four, and L2 delivers a third less.
//
// What crosses between the two CTAs, and how:
//   full[s]      lives in the first CTA.  It arms it for the bytes of both CTAs' loads; the second CTA's TMA loads
//                complete on it too (cp.async.bulk.tensor ... cta_group::2 with the barrier's address in the first
//                CTA, from mapa).
//   empty[s]     one in each CTA; the MMA thread's commit arrives on both (tcgen05.commit ... multicast::cluster).
//   acc_full[b]  one in each CTA, both signalled by the commit after a tile's last MMA.
//   acc_empty[b] lives in the first CTA; the four epilogue warps of each CTA arrive on it (a remote arrive from the
//                second CTA), eight arrivals a phase.
// The rest is the structure of gemm_tc.cu: persistent pairs taking tiles in turn, warp 0 loads, warp 1 owns the
// tensor memory (and, in the first CTA, issues the MMAs), warps 2..5 are the epilogue under the next tile's MMAs;
// every wait is bounded.  The two CTAs meet at a cluster barrier after set-up and before they free their tensor
// memory: neither may leave while the other's MMAs or loads still name its memory.
#include <cuda.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tc_common.cuh"

namespace vtb {

namespace {

constexpr int PBM = 128;                 // rows of x a CTA holds of the pair's 256
constexpr int PBK = 64;
constexpr int PA_STAGE = PBM * PBK * 2;  // 16 KB
constexpr int PTHREADS = 192;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of the same place in CTA `rank`
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(local), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// a box of a tensor map into this CTA's shared memory, its bytes counted on a barrier that may lie in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            smem_u32(smem)),
        "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives, when the MMAs issued so far are done, on the barrier at this place in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
                     smem_u32(bar)),
                 "h"(both)
                 : "memory");
}

template <int BN, int STAGES, int EPI, typename TOut>
__global__ void __launch_bounds__(PTHREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const float* __restrict__ bias, TOut* __restrict__ out, int rows_a, int rows_b, int k, int ldo, int n_full, int s_tail, int cols_first,
                    float* __restrict__ scratch, int* __restrict__ counters, int* status) {
    static_assert(BN % 32 == 0 && BN <= 256, "each CTA holds half of the tile's rows of w, in whole swizzle groups");
    constexpr int BH = BN / 2;                       // rows of w a CTA loads
    constexpr int B_STAGE = BH * PBK * 2;
    constexpr int COLS = BN;                         // tensor-memory columns of an accumulator
    constexpr int ALLOC = 2 * COLS <= 256 ? 256 : 512;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_s = smem;
    unsigned char* b_s = smem + STAGES * PA_STAGE;
    uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * B_STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();            // 0: the CTA that issues the MMAs
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int a_tiles = (rows_a + 2 * PBM - 1) / (2 * PBM), b_tiles = (rows_b + BN - 1) / BN;
    const int tiles = a_tiles * b_tiles;
    const int nkb = (k + PBK - 1) / PBK;
    // A unit is (tile, share of k).  The first n_full tiles are units by themselves; the k-blocks of each tile after
    // them are cut into s_tail shares, units of their own (share by share over those tiles).  Two uses: few tiles and a
    // long k (n_full = 0: every tile in two shares, for twice the pairs), and the tiles of a last, partial round
    // (n_full = the whole rounds' tiles: the few tiles left over are cut over the pairs that would stand idle).
    const int tail = tiles - n_full;
    const int units = n_full + tail * s_tail;
    // The tiles in the order in which pairs that run together take them: down the rows of x first (they share a tile
    // of w, and x, if it fits L2, stays there), or across the rows of w first (for an x larger than L2 and a smaller w).
    auto a_of = [&](int t) { return cols_first ? t / b_tiles : t % a_tiles; };
    auto b_of = [&](int t) { return cols_first ? t % b_tiles : t / a_tiles; };
    auto unit_of = [&](int u, int& t, int& krank, int& ks) {
        if (u < n_full) {
            t = u;
            krank = 0;
            ks = 1;
        } else {
            t = n_full + (u - n_full) % tail;
            krank = (u - n_full) / tail;
            ks = s_tail;
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);                  // the first CTA's arrival with the bytes to expect
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);             // four epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(ALLOC));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                              // both CTAs' barriers and tensor memory are there
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            int kit = 0;
            bool waited = false;
            for (int u = pair; u < units && !timed_out; u += n_pairs) {
                int t, krank, ksplit;
                unit_of(u, t, krank, ksplit);
                const int kb0 = (int)((long long)krank * nkb / ksplit), kb1 = (int)((long long)(krank + 1) * nkb / ksplit);
                const int a_row0 = a_of(t) * 2 * PBM + (int)rank * PBM, b_row0 = b_of(t) * BN + (int)rank * BH;
                for (int kb = kb0; kb < kb1; ++kb, ++kit) {
                    const int s = kit % STAGES;
                    if (kit >= STAGES && !mbar_wait(&empty[s], ((kit / STAGES) & 1) ^ 1)) { timed_out = true; break; }
                    const uint32_t bar = in_cta(smem_u32(&full[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * (PA_STAGE + B_STAGE));
                    // the weights are written by no kernel: they go out before the dependency wait
                    tma_load_2d_pair(b_s + s * B_STAGE, &map_b, kb * PBK, b_row0, bar);
                    if (!waited) {
                        pdl_wait();
                        waited = true;
                    }
                    tma_load_2d_pair(a_s + s * PA_STAGE, &map_a, kb * PBK, a_row0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc(2 * PBM, BN);
            int kit = 0, ui = 0;
            for (int u = pair; u < units && !timed_out; u += n_pairs, ++ui) {
                int t, krank, ksplit;
                unit_of(u, t, krank, ksplit);
                const int kb0 = (int)((long long)krank * nkb / ksplit), kb1 = (int)((long long)(krank + 1) * nkb / ksplit);
                const int buf = ui & 1;
                if (ui >= 2 && !mbar_wait(&acc_empty[buf], ((ui >> 1) & 1) ^ 1)) { timed_out = true; break; }
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(buf * COLS);
                for (int kb = kb0; kb < kb1; ++kb, ++kit) {
                    const int s = kit % STAGES;
                    if (!mbar_wait(&full[s], (kit / STAGES) & 1)) { timed_out = true; break; }
                    tc_fence_after();
                    const uint64_t ad = smem_desc(a_s + s * PA_STAGE), bd = smem_desc(b_s + s * B_STAGE);
#pragma unroll
                    for (int kk = 0; kk < PBK / 16; ++kk)
                        tc_mma_pair(acc, ad + 2 * kk, bd + 2 * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                    tc_commit_pair(&empty[s]);
                }
                tc_commit_pair(&acc_full[buf]);
            }
        }
    }
    __syncwarp();
    pdl_wait();

    if (warp >= 2) {
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t acc_empty_first = in_cta(smem_u32(&acc_empty[0]), 0);
        int ui = 0;
        for (int u = pair; u < units; u += n_pairs, ++ui) {
            int t, krank, ksplit;
            unit_of(u, t, krank, ksplit);
            const int cut = t - n_full;                 // index among the tiles that are cut
            const int a_row0 = a_of(t) * 2 * PBM + (int)rank * PBM, b_row0 = b_of(t) * BN;
            const int buf = ui & 1;
            bool ok = !timed_out && mbar_wait(&acc_full[buf], (ui >> 1) & 1);
            if (!ok) timed_out = true;
            tc_fence_after();
            // a share of k: this CTA's 128 rows of it as 32-bit [row][column] in scratch memory
            float* mine = ksplit > 1 ? scratch + (((size_t)cut * ksplit + krank) * 2 + rank) * (size_t)(BN * PBM) : nullptr;
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
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(acc_empty_first + (uint32_t)(buf * 8));
                }
                if (ksplit > 1) {
#pragma unroll
                    for (int i = 0; i < 16; i += 4)
                        __stcg(reinterpret_cast<float4*>(mine + (size_t)r * BN + c0 + i), make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));
                    continue;
                }
                emit16<false, EPI, TOut>(v, r, a_row0, b_row0, c0, rows_a, rows_b, bias, out, ldo);
            }
            if (ksplit > 1) {
                // count this share in (a counter a tile and CTA of the pair: each CTA has its own 128 rows); the one
                // that finds all others counted adds the shares, in their order, and stores.  Nobody waits.
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (threadIdx.x == 64) *last_flag = (atomicAdd(&counters[2 * cut + (int)rank], 1) == ksplit - 1) ? 1 : 0;
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                const bool last = *last_flag != 0;
                asm volatile("bar.sync 1, 128;\n" ::: "memory");   // all have read the flag before it is written again
                if (last) {
                    __threadfence();
                    const float* all = scratch + ((size_t)cut * ksplit * 2 + rank) * (size_t)(BN * PBM);
                    const bool live = (a_row0 + r) < rows_a;
                    // a row a thread, 32 columns at a time: 16-byte loads, those of all shares on their way together
                    // (a share is [row][column]: with one value a load the merge took longer than the share's products)
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        if (b_row0 + c0 >= rows_b) break;
                        float sum[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) sum[i] = 0.f;
                        if (live) {
#pragma unroll 4
                            for (int rk = 0; rk < ksplit; ++rk) {
                                const float4* src = reinterpret_cast<const float4*>(all + (size_t)rk * 2 * (BN * PBM) + (size_t)r * BN + c0);
                                float4 part[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) part[i] = __ldcg(src + i);
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    sum[4 * i] += part[i].x;
                                    sum[4 * i + 1] += part[i].y;
                                    sum[4 * i + 2] += part[i].z;
                                    sum[4 * i + 3] += part[i].w;
                                }
                            }
                        }
                        emit16<false, EPI, TOut>(*reinterpret_cast<float(*)[16]>(&sum[0]), r, a_row0, b_row0, c0, rows_a, rows_b, bias, out, ldo);
                        if (c0 + 16 < BN)
                            emit16<false, EPI, TOut>(*reinterpret_cast<float(*)[16]>(&sum[16]), r, a_row0, b_row0, c0 + 16, rows_a, rows_b, bias, out, ldo);
                    }
                    if (threadIdx.x == 64) counters[2 * cut + (int)rank] = 0;     // ready for the next launch
                }
            }
        }
    }
    if (timed_out && status) set_status(status, kStatusWaitTimeout, blockIdx.x);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                              // neither CTA's memory is named by the other any more
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(ALLOC));
    }
}

template <int BN, int STAGES, int EPI, typename TOut>
cudaError_t launch_pair_cfg(const void* x, int m, const void* w, int n, int k, const float* bias, TOut* out, int ldo,
                            float* scratch, long long scratch_floats, int* counters, int n_counters, int* status,
                            cudaStream_t stream) {
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, x, m, k, PBM) || !make_map(&map_b, w, n, k, BN / 2)) return cudaErrorInvalidValue;
    constexpr int smem = STAGES * (PA_STAGE + (BN / 2) * PBK * 2) + 1024 + 256;      // (barriers, the slot, the flag: 17 words of 8 bytes at most)
    static std::atomic<unsigned long long> configured{0};
    cudaError_t e = allow_dynamic_smem(gemm_tc_pair_kernel<BN, STAGES, EPI, TOut>, smem, configured);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const int tiles = ((m + 2 * PBM - 1) / (2 * PBM)) * ((n + BN - 1) / BN);
    // Half as many tiles as pairs of SMs, or fewer, and a long k: k in two shares, so that twice the pairs work.  Measured
    // on a B200 (3584 features, k = 18944): 256 to 512 rows 67 to 78 us with two shares against 96 to 98 without; three
    // shares in two rounds (640 and 768 rows) lost to no shares at all, and so did two shares of a short k (3584: a
    // share's trip through scratch memory costs about as much as 60 k-blocks).  Two shares also add up to the same
    // number in either order.
    // More tiles than pairs, a long k, and a last round that at most half the pairs would take: its tiles are cut
    // into up to four shares each (added in their order), as many as make units for the idle pairs.
    int n_full = tiles, s_tail = 1;
    const int all_pairs = sms / 2, nkb = (k + PBK - 1) / PBK;
    const bool may_cut = nkb >= 128 && scratch != nullptr && counters != nullptr;
    if (may_cut && 2 * tiles <= all_pairs && 2 * tiles <= n_counters && (long long)tiles * 2 * 2 * BN * PBM <= scratch_floats) {
        n_full = 0;
        s_tail = 2;
    } else if (may_cut && tiles > all_pairs) {
        const int rem = tiles % all_pairs;
        if (rem > 0 && 2 * rem <= all_pairs) {
            int s = all_pairs / rem;
            if (s > 4) s = 4;
            while (s > 1 && nkb / s < 32) --s;
            if (s > 1 && 2 * rem <= n_counters && (long long)rem * s * 2 * BN * PBM <= scratch_floats) {
                n_full = tiles - rem;
                s_tail = s;
            }
        }
    }
    const int units = n_full + (tiles - n_full) * s_tail;
    const int pairs = units < all_pairs ? units : all_pairs;
    // x larger than half of L2 and w smaller than x: across the rows of w first (8,192 rows of k = 18944 are 310 MB; with
    // the rows of x first they would come from HBM again for every column of tiles)
    int l2 = 0;
    if (cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess || l2 <= 0) l2 = 64 << 20;
    const long long x_bytes = (long long)m * k * 2, w_bytes = (long long)n * k * 2;
    const int cols_first = (x_bytes > l2 / 2 && w_bytes < x_bytes) ? 1 : 0;
    return launch(gemm_tc_pair_kernel<BN, STAGES, EPI, TOut>, dim3(2 * pairs, 1, 1), dim3(PTHREADS, 1, 1), smem, stream, dim3(2, 1, 1),
                  map_a, map_b, bias, out, m, n, k, ldo, n_full, s_tail, cols_first, scratch, counters, status);
}

}  // namespace

// bfloat16 out [m, n] (epilogue 0, with bias) or [m, n / 2] (epilogue 1: SiLU(gate) * up over rows of w interleaved
// in runs of 8).  `bn`: rows of w in a tile: 256, 224 or 192; 0: the one whose rounds of one tile a pair come out best.
cudaError_t launch_gemm_tc_pair(const void* x, const void* w, const float* bias, void* out, int m, int n, int k, int epilogue,
                                int bn, float* scratch, long long scratch_floats, int* counters, int n_counters, int* status,
                                cudaStream_t stream) {
    if (m == 0 || n == 0) return cudaSuccess;
    if (k % 8 != 0 || k < 8) return cudaErrorInvalidValue;
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    if (bn == 0) {
        // rounds of one tile a pair, times the width of a tile and a fixed part for the 128 rows of x of every
        // k-block; a narrower tile also has a little less of the tensor pipe (measured: 192 is a fifth slower a column)
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        const int pairs = sms / 2;
        const int nkb = (k + PBK - 1) / PBK;
        double best = -1.0;
        for (int cand : {256, 224}) {
            const long t = (long)((m + 2 * PBM - 1) / (2 * PBM)) * ((n + cand - 1) / cand);
            const long rem = t % pairs;
            // a last round that at most half the pairs would take is cut into shares of k where k is long (launch_pair_cfg)
            double rounds = (double)(t / pairs);
            if (rem > 0) rounds += (t > pairs && 2 * rem <= pairs && nkb >= 128 && scratch != nullptr) ? 0.4 : 1.0;
            const double cost = rounds * (cand + 32 + (256 - cand) / 2);
            if (best < 0 || cost < best) {
                best = cost;
                bn = cand;
            }
        }
    }
    if (epilogue == 1) {
        if (n % 16 != 0 || bias != nullptr) return cudaErrorInvalidValue;
        if (bn == 192) return launch_pair_cfg<192, 7, 1, __nv_bfloat16>(x, m, w, n, k, nullptr, o, n / 2, scratch, scratch_floats, counters, n_counters, status, stream);
        if (bn == 224) return launch_pair_cfg<224, 6, 1, __nv_bfloat16>(x, m, w, n, k, nullptr, o, n / 2, scratch, scratch_floats, counters, n_counters, status, stream);
        return launch_pair_cfg<256, 6, 1, __nv_bfloat16>(x, m, w, n, k, nullptr, o, n / 2, scratch, scratch_floats, counters, n_counters, status, stream);
    }
    if (epilogue != 0) return cudaErrorInvalidValue;
    if (bn == 192) return launch_pair_cfg<192, 7, 0, __nv_bfloat16>(x, m, w, n, k, bias, o, n, scratch, scratch_floats, counters, n_counters, status, stream);
    if (bn == 224) return launch_pair_cfg<224, 6, 0, __nv_bfloat16>(x, m, w, n, k, bias, o, n, scratch, scratch_floats, counters, n_counters, status, stream);
    return launch_pair_cfg<256, 6, 0, __nv_bfloat16>(x, m, w, n, k, bias, o, n, scratch, scratch_floats, counters, n_counters, status, stream);
}

}  // namespace vtb
