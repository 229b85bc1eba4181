// The kernel of single-token attention and its launchers by head size: included by the files that instantiate
// it (attention_decode.cu: the head sizes without tensor-map boxes; attention_decode_boxes.cu: 64 and 128).
#pragma once

#include <cooperative_groups.h>

#include <cstring>

#include "attention_mma.cuh"
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace vtb {

// head sizes 64 and 128, compiled in a file of their own (attention_decode_boxes.cu)
cudaError_t launch_decode_64_128(const AttnParams& p, int head_dim, int n_seqs, int* counters, cudaStream_t stream);

namespace {

// ---- single-token steps -----------------------------------------------------------------------------
// A CTA of four (or three) warps serves one (sequence, KV head, run of keys).  The run's blocks of 32 keys go
// to the warps in turn; each warp streams its blocks through its own two-stage ring (cp.async, or tensor-map
// boxes counted into an mbarrier) and keeps a running maximum, sum and output for the up to 16 rows (token,
// head of the group).  The warps' results are merged in shared memory.  With more than one run a sequence
// (n_splits > 1): up to 8 runs are the CTAs of a cluster and merge through distributed shared memory; with more
// the CTA leaves its merged result in scratch and counts itself in, and the CTA that arrives last merges the
// runs and stores, so there is no second kernel and no CTA waits for another.
constexpr int DKB = 16;    // keys in a warp's block
constexpr int DHALVES = DKB / 16;   // runs of 16 keys in a block: each lies in one page
constexpr int DFULL = (1 << DHALVES) - 1;
constexpr int DWARPS_MAX = 8;     // most warps of a CTA
constexpr int DSTAGES_MAX = 4;    // most stages of a warp's ring
// Head sizes of whole 128-byte lines (64, 128): a block's keys and values can come as boxes of a tensor map, one
// request of the copy engine for 16 or 32 rows of 128 bytes where the other head sizes issue a 16-byte cp.async
// a lane and piece (whose issue rate, not the memory, bounded the kernel).  A box lands with the 128-byte swizzle:
// piece c of row r at piece c ^ (r % 8), so that ldmatrix finds eight rows' pieces in eight different banks
// without padding.
constexpr bool decode_by_boxes(int d) { return d % 64 == 0; }
constexpr int DTILE = DKB * 128;   // bytes of a box-loaded tile: DKB rows of 64 values
// bytes of the stages of a warp's ring, keys and values
constexpr int decode_warp_bytes(int d, bool boxes, int stages) {
    return boxes ? stages * 2 * (d / 64) * DTILE : stages * 2 * DKB * (d + 8) * 2;
}

//
// NARROW (at most 8 rows, that is one token of a group of up to 8 heads): the products are taken the other way
// round, scores as K (16 keys) by q^T (8 rows) and the output as V^T (16 of d) by P^T (8 rows), so that the eight
// columns of a tensor-core product hold the rows and none of its sixteen lines stay empty: half the products, half
// the exponentials and half the registers of the output.
//
// BOXES: see decode_by_boxes.  A box takes longer to arrive than a cp.async; it pays where a warp has many blocks
// to stream (long contexts), not where it has three.
template <int D, int W, int S, bool NARROW, bool BOXES>
__global__ void __launch_bounds__(W * 32)
attention_decode_kernel(const AttnParams p, int* __restrict__ counters, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v) {
    static_assert(!BOXES || decode_by_boxes(D), "boxes are rows of whole 128-byte lines");
    constexpr int LD = D + 8;                                 // row length without boxes: padded against bank conflicts
    static_assert(S >= 2 && S <= DSTAGES_MAX && W <= DWARPS_MAX, "a barrier a warp and stage");
    constexpr int WARP_BYTES = decode_warp_bytes(D, BOXES, S);   // K and V, S stages
    constexpr int STAGE_BYTES = WARP_BYTES / S;                  // with boxes: [K tiles of 64 d][V tiles of 64 d]
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    // swizzled tiles start on a 1,024-byte boundary
    unsigned char* smem_raw = BOXES ? reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023) : smem_dyn;
    __shared__ int last_flag;
    __shared__ __align__(8) uint64_t arrived[DWARPS_MAX][DSTAGES_MAX];      // with boxes: a warp's stage has arrived
    __shared__ float2 cs_row[D / 2];                                        // the rotation's (cos, sin) of the step's token
    // The kernels before this one in the stream may still be running (programmatic dependent launch).  What
    // the step's description says (lengths, block tables: copied from the host before the step's first kernel)
    // and the keys and values of earlier steps may be read at once; q, and a key or value written in this
    // step, only after pdl_wait.
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    if constexpr (BOXES) {
        if (threadIdx.x == 0) {                                // the maps' descriptors on their way before the first box
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
        }
    }
    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ntok = min(p.tokens_per_tile, q_len);
    if (ntok <= 0) {                                           // padding: a sequence without tokens
        pdl_wait();
        return;
    }
    const int group = p.heads / p.kv_heads;
    const int rows_valid = ntok * group;
    const int start = p.q_start[seq];
    const int pos_lo = start, pos_hi = start + ntok - 1;
    int key_lo = (p.window > 0) ? max(0, pos_lo - p.window + 1) : 0;
    key_lo = key_lo / DKB * DKB;
    const int key_hi = pos_hi + 1;
    const int nblk = (key_hi - key_lo + DKB - 1) / DKB;
    // The runs of this sequence: n_splits equal ones, or, with run_blocks, as many as make runs of about that many
    // blocks (between two thirds and one and a half of it), so that sequences of different lengths give CTAs of
    // like work; the CTAs beyond them have no keys.
    int runs = p.n_splits;
    if (p.run_blocks > 0) runs = min(p.n_splits, max(1, (nblk + p.run_blocks / 2) / p.run_blocks));
    const bool idle = split >= runs;
    if (idle && !p.cluster_merge) {                            // nobody waits for this CTA
        pdl_wait();
        return;
    }
    const int blk0 = idle ? 0 : (int)((long long)split * nblk / runs), blk1 = idle ? 0 : (int)((long long)(split + 1) * nblk / runs);
    const bool alone = p.n_splits == 1 || (!p.cluster_merge && runs == 1);   // this CTA's result is the sequence's

    unsigned char* wbase = smem_raw + (size_t)warp * WARP_BYTES;
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(wbase);                 // without boxes: [S][DKB][LD]
    __nv_bfloat16* vs = ks + S * DKB * LD;
    // the 16-byte piece c (d 8 c .. 8 c + 7) of row r of a stage's keys or values
    auto kpiece = [&](int stage, int r, int c) -> __nv_bfloat16* {
        if constexpr (BOXES)
            return reinterpret_cast<__nv_bfloat16*>(wbase + stage * STAGE_BYTES + (c >> 3) * DTILE + r * 128 + (((c & 7) ^ (r & 7)) << 4));
        else
            return ks + ((size_t)stage * DKB + r) * LD + c * 8;
    };
    auto vpiece = [&](int stage, int r, int c) -> __nv_bfloat16* {
        if constexpr (BOXES)
            return reinterpret_cast<__nv_bfloat16*>(wbase + stage * STAGE_BYTES + (D / 64 + (c >> 3)) * DTILE + r * 128 +
                                                    (((c & 7) ^ (r & 7)) << 4));
        else
            return vs + ((size_t)stage * DKB + r) * LD + c * 8;
    };
    if constexpr (BOXES) {
        if (lane == 0) {
#pragma unroll
            for (int st = 0; st < S; ++st) mbar_init(&arrived[warp][st], 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        __syncwarp();
    }

    int row[2], pos[2], tok[2], head[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row[i] = gq + 8 * i;
        valid[i] = row[i] < rows_valid;
        const int tk = valid[i] ? row[i] / group : 0;
        tok[i] = q_begin + tk;
        pos[i] = pos_lo + tk;
        head[i] = kvh * group + (valid[i] ? row[i] % group : 0);
    }
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    // the page and the place in it of a key: by shift and mask where a page holds a power of two of tokens
    const int pshift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
    auto page_index = [&](int key) -> int { return pshift >= 0 ? key >> pshift : key / p.page_size; };
    auto in_page = [&](int key) -> int { return pshift >= 0 ? key & (p.page_size - 1) : key % p.page_size; };
    // the pages of a block's runs of 16 keys (-1: none); looked up a block ahead of the block's loads
    auto pages_of = [&](int blk, int (&pg)[DHALVES]) {
#pragma unroll
        for (int h = 0; h < DHALVES; ++h) {
            const int key = key_lo + blk * DKB + 16 * h;
            pg[h] = (blk < blk1 && key < key_hi) ? table[page_index(key)] : -1;
        }
    };
    // Sends for a block's keys and values; the answer says which halves of 16 keys were asked for (bit h).
    auto load_block = [&](int blk, int stage, const int (&pg)[DHALVES]) -> int {
        const int kb = key_lo + blk * DKB;
        if constexpr (BOXES) {
            const int br = p.run_keys;               // rows of a box: the block's, or 16 where a page is no multiple of the block
            int asked = 0;
#pragma unroll
            for (int h = 0; h < DHALVES; ++h)
                if (kb + 16 * h < key_hi && pg[h] >= 0 && pg[h] < p.n_pages) asked |= 1 << h;
            if (br == DKB) asked = (asked & 1) ? DFULL : 0;   // one page holds the block: its first run decides
            if (lane == 0) {
                uint64_t* bar = &arrived[warp][stage];
                const int boxes = br == DKB ? (asked ? 1 : 0) : __popc(asked);
                if (boxes == 0) {
                    mbar_arrive(bar);
                } else {
                    mbar_expect_tx(bar, (uint32_t)(boxes * 2 * (D / 64) * br * 128));
                    for (int h = 0; h < DKB / br; ++h) {
                        if (!(asked >> (h * (br / 16)) & 1)) continue;
                        const int key = kb + h * br;
                        const int y = (pg[h * (br / 16)] * p.kv_heads + kvh) * p.page_size + in_page(key);
                        unsigned char* dst = wbase + stage * STAGE_BYTES + h * br * 128;
#pragma unroll
                        for (int t = 0; t < D / 64; ++t) {
                            tma_load_2d(dst + t * DTILE, &map_k, t * 64, y, bar);
                            tma_load_2d(dst + (D / 64 + t) * DTILE, &map_v, t * 64, y, bar);
                        }
                    }
                }
            }
            return asked;
        }
        constexpr int CHUNKS = D / 8;
        size_t base[DHALVES];
        bool okp[DHALVES];
        bool all_ok = true;
#pragma unroll
        for (int h = 0; h < DHALVES; ++h) {
            const int key = kb + 16 * h;
            okp[h] = key < key_hi && pg[h] >= 0 && pg[h] < p.n_pages;
            base[h] = okp[h] ? (((size_t)pg[h] * p.kv_heads + kvh) * p.page_size + in_page(key)) * D : 0;
            all_ok = all_ok && okp[h];
        }
        if constexpr (32 % CHUNKS == 0) {
            // A whole block of a head size whose rows are a power of two long: the lane's first row and its piece
            // of it are found once; every further copy lies a constant number of bytes from them.
            if (all_ok && kb + DKB <= key_hi) {
                constexpr int RPI = 32 / CHUNKS;         // rows that the warp's lanes cover in one turn
                const int r0 = lane / CHUNKS, piece = lane % CHUNKS;
                const unsigned ks0 = (unsigned)__cvta_generic_to_shared(ks + ((size_t)stage * DKB + r0) * LD + piece * 8);
                const unsigned vs0 = (unsigned)__cvta_generic_to_shared(vs + ((size_t)stage * DKB + r0) * LD + piece * 8);
#pragma unroll
                for (int h = 0; h < DHALVES; ++h) {
                    const __nv_bfloat16* kg0 = p.k_cache + base[h] + (size_t)r0 * D + piece * 8;
                    const __nv_bfloat16* vg0 = p.v_cache + base[h] + (size_t)r0 * D + piece * 8;
#pragma unroll
                    for (int i = 0; i < 16 / RPI; ++i) {
                        const int r = 16 * h + i * RPI;  // rows below the lane's first
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(ks0 + r * LD * 2), "l"(kg0 + i * RPI * D));
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vs0 + r * LD * 2), "l"(vg0 + i * RPI * D));
                    }
                }
                return DFULL;
            }
        }
        for (int c = lane; c < DKB * CHUNKS; c += 32) {
            const int r = c / CHUNKS, piece = c % CHUNKS;
            const int h = r >> 4;
            const bool ok = okp[h] && (kb + r) < key_hi;
            const size_t off = base[h] + (size_t)(r & 15) * D + piece * 8;
            cp_async16(ks + ((size_t)stage * DKB + r) * LD + piece * 8, p.k_cache + (ok ? off : 0), ok);
            cp_async16(vs + ((size_t)stage * DKB + r) * LD + piece * 8, p.v_cache + (ok ? off : 0), ok);
        }
        return DFULL;                                // rows that were not asked for are filled with zeros
    };

    const int first = blk0 + warp;
    // The warp's ring: block j of the warp (first + j W) lies in stage j % S.  Before the loop the first S - 1 blocks
    // are sent for, and every turn of the loop sends for the block S - 1 turns ahead, so that S - 1 blocks are on
    // their way while one is worked on.  A block of earlier steps' keys may be sent for before the dependency wait;
    // the block with the step's own token only if this kernel itself puts the token there (otherwise another kernel
    // of the step may still be writing it): the early blocks are a prefix of the warp's blocks.
    auto early_ok = [&](int blk) -> bool {
        const int kb_ = key_lo + blk * DKB;
        return blk < blk1 && (!(pos_lo >= kb_ && pos_lo < kb_ + DKB) || (p.fuse_rope && p.store_kv));
    };
    unsigned asked_bits = 0;                          // which runs of 16 keys of a stage's block were asked for
    auto set_asked = [&](int stage, int a) {
        asked_bits = (asked_bits & ~((unsigned)DFULL << (stage * DHALVES))) | ((unsigned)a << (stage * DHALVES));
    };
    int pg_pro[S - 1][DHALVES], pg_next[DHALVES];
#pragma unroll
    for (int j = 0; j < S - 1; ++j) pages_of(first + j * W, pg_pro[j]);
    pages_of(first + (S - 1) * W, pg_next);
    // The rotation table is written by no kernel and the token's position is in the step's description: its row is
    // fetched before the wait (one token a sequence, q as unadded shares: the barrier behind their sum publishes it).
    const bool cs_staged = p.fuse_rope && p.cos_sin != nullptr && p.qkv_shares != nullptr && ntok == 1 && pos_lo < p.max_pos;
    if (cs_staged) {
        for (int i = threadIdx.x; i < D / 2; i += W * 32) cs_row[i] = p.cos_sin[(size_t)pos_lo * (D / 2) + i];
    }
    int sent = 0;                                     // blocks of the prologue sent for before the wait
#pragma unroll
    for (int j = 0; j < S - 1; ++j) {
        if (sent == j && early_ok(first + j * W)) {
            set_asked(j, load_block(first + j * W, j, pg_pro[j]));
            if constexpr (!BOXES) cp_async_commit();
            sent = j + 1;
        }
    }
    pdl_wait();
#pragma unroll
    for (int j = 0; j < S - 1; ++j) {
        if (j >= sent) {
            if (first + j * W < blk1) set_asked(j, load_block(first + j * W, j, pg_pro[j]));
            if constexpr (!BOXES) cp_async_commit();  // a group a block of the prologue, empty where there is no block
        }
    }
    uint32_t qf[D / 16][4];
    // With q, k and v as unadded shares (one token a sequence): this CTA's part of the token's row, that is its
    // group's heads of q, then its head of k and of v, is added once, share by share, and kept as bfloat16 in the
    // shared memory that later takes the merged result.
    __nv_bfloat16* own = reinterpret_cast<__nv_bfloat16*>(smem_raw + (size_t)W * WARP_BYTES);     // [group + 2][D]
    if (p.qkv_shares != nullptr) {
        const size_t share_stride = (size_t)p.n_tokens * p.qkv_stride;
        const float* row0 = p.qkv_shares + (size_t)q_begin * p.qkv_stride;
        for (int e = threadIdx.x; e < (group + 2) * (D / 2); e += W * 32) {
            const int j = e / (D / 2), d2 = (e % (D / 2)) * 2;
            const int col = (j < group ? (kvh * group + j) : (j == group ? p.heads + kvh : p.heads + p.kv_heads + kvh)) * D + d2;
            float2 v[8];                       // all shares' loads in flight together; added in order
#pragma unroll
            for (int q = 0; q < 8; ++q)
                v[q] = (q < p.n_shares) ? __ldcg(reinterpret_cast<const float2*>(row0 + q * share_stride + col)) : make_float2(0.f, 0.f);
            float2 acc = v[0];
#pragma unroll
            for (int q = 1; q < 8; ++q) {
                acc.x += v[q].x;
                acc.y += v[q].y;
            }
            *reinterpret_cast<uint32_t*>(own + j * D + d2) = pack_bf16(acc.x, acc.y);
        }
        __syncthreads();
    }
    // two neighbouring values of q: row `t` of qkv, head `h`, at `d`
    auto pair_at = [&](int t, int h, int d) -> uint32_t {
        if (p.qkv_shares != nullptr) return *reinterpret_cast<const uint32_t*>(own + (h - kvh * group) * D + d);
        return *reinterpret_cast<const uint32_t*>(p.qkv + (size_t)t * p.qkv_stride + (size_t)h * D + d);
    };
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int ks_ = 0; ks_ < D / 16; ++ks_) {
            qf[ks_][i] = valid[i] ? pair_at(tok[i], head[i], ks_ * 16 + 2 * tq) : 0u;
            qf[ks_][i + 2] = valid[i] ? pair_at(tok[i], head[i], ks_ * 16 + 8 + 2 * tq) : 0u;
        }
    }
    if (p.fuse_rope && p.cos_sin != nullptr) {
        // rotate q in registers: the 8-wide chunk u of the first half pairs with chunk u + D / 16 (pairs (i, i + D/2),
        // v1/tensortype/cuda_kernels/rotary_embed.cu:19-29); 32-bit arithmetic, one rounding, as the separate kernel does
        constexpr int HC = D / 16;             // 8-wide chunks in half a head
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;
            if (pos[i] >= p.max_pos) {
                if (tq == 0) set_status(p.status, kStatusBadPosition, pos[i]);
                continue;
            }
            const float2* cs = cs_staged ? cs_row : p.cos_sin + (size_t)pos[i] * (D / 2);
#pragma unroll
            for (int u = 0; u < HC; ++u) {
                const int v = u + HC;
                uint32_t& xa = qf[u / 2][(u % 2) * 2 + i];
                uint32_t& ya = qf[v / 2][(v % 2) * 2 + i];
                const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xa));
                const float2 y = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&ya));
                const float2 c0 = cs[u * 8 + 2 * tq], c1 = cs[u * 8 + 2 * tq + 1];
                xa = pack_bf16(x.x * c0.x - y.x * c0.y, x.y * c1.x - y.y * c1.y);
                ya = pack_bf16(y.x * c0.x + x.x * c0.y, y.y * c1.x + x.y * c1.y);
            }
        }
    }
    // The output: rows gq and gq + 8 by eight of d a tile; NARROW: d gq and gq + 8 of sixteen a tile by rows 2 tq and
    // 2 tq + 1.  Maximum and sum: of rows gq and gq + 8; NARROW: of rows 2 tq and 2 tq + 1.
    constexpr int OT = NARROW ? D / 16 : D / 8;
    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    // NARROW: the lane's two rows, 2 tq and 2 tq + 1
    bool nvalid[2];
    int npos[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        nvalid[c] = 2 * tq + c < rows_valid;
        npos[c] = pos_lo + (nvalid[c] ? (2 * tq + c) / group : 0);
    }

    int stage = 0, phase = 0;
    for (int blk = first; blk < blk1; blk += W) {
        const int kb = key_lo + blk * DKB;
        {
            const int nb = blk + (S - 1) * W, ns = stage == 0 ? S - 1 : stage - 1;   // the stage worked on a turn ago
            if (nb < blk1) set_asked(ns, load_block(nb, ns, pg_next));
            if constexpr (!BOXES) cp_async_commit();   // a group a turn, empty where there was nothing to send for
            pages_of(nb + W, pg_next);                 // for the next turn; the answer comes under this block's work
            if constexpr (!BOXES) cp_async_wait<S - 1>();
        }
        if constexpr (BOXES) {
            if (!mbar_wait(&arrived[warp][stage], phase)) {         // the clock limit ran out: give up, say so
                if (lane == 0) set_status(p.status, kStatusWaitTimeout, blk);
                break;
            }
            // Rows that no box brought, and rows of a box behind the last key, hold what the memory held; a weight of
            // zero times that may be no number: their values are cleared.
            const int have = (asked_bits >> (stage * DHALVES)) & DFULL;
            if (have != DFULL || kb + DKB > key_hi) {
                for (int r = 0; r < DKB; ++r) {
                    if ((have >> (r >> 4) & 1) && kb + r < key_hi) continue;
                    if (lane < D / 8) *reinterpret_cast<uint4*>(vpiece(stage, r, lane)) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // before a later box lands on these rows
            }
        }
        __syncwarp();
        if (p.fuse_rope && p.store_kv && pos_lo >= kb && pos_lo < kb + DKB) {
            // the step's own token lies in this block: its k (rotated) and v come from qkv and go into the
            // block in shared memory and into their page.  (A run of a layer that only reads another run's
            // cache finds the token's k and v there already.)
            const int r = pos_lo - kb;
            const int kcol = (p.heads + kvh) * D, vcol = kcol + p.kv_heads * D;
            auto value_at = [&](int col) -> __nv_bfloat16 {       // col: from the start of the token's k
                if (p.qkv_shares != nullptr) return own[group * D + (col < kcol + D ? col - kcol : D + col - vcol)];
                return p.qkv[(size_t)q_begin * p.qkv_stride + col];
            };
            auto ksm = [&](int d) -> __nv_bfloat16& { return kpiece(stage, r, d >> 3)[d & 7]; };
            auto vsm = [&](int d) -> __nv_bfloat16& { return vpiece(stage, r, d >> 3)[d & 7]; };
            __nv_bfloat16 *kg = nullptr, *vg = nullptr;
            {
                const int page = table[pos_lo / p.page_size];
                if (page >= 0 && page < p.n_pages) {
                    const size_t off = (((size_t)page * p.kv_heads + kvh) * p.page_size + pos_lo % p.page_size) * D;
                    kg = p.k_out + off;
                    vg = p.v_out + off;
                } else if (lane == 0) {
                    set_status(p.status, kStatusBadPage, page);
                }
            }
            const bool rot = p.cos_sin != nullptr && pos_lo < p.max_pos;
            const float2* cs = cs_staged ? cs_row : p.cos_sin + (size_t)(rot ? pos_lo : 0) * (D / 2);
            for (int i = lane; i < D / 2; i += 32) {
                __nv_bfloat16 ka = value_at(kcol + i), kb2 = value_at(kcol + i + D / 2);
                const float a = __bfloat162float(ka), b = __bfloat162float(kb2);
                if (rot) {
                    const float2 c = cs[i];
                    ka = __float2bfloat16_rn(a * c.x - b * c.y);
                    kb2 = __float2bfloat16_rn(b * c.x + a * c.y);
                }
                ksm(i) = ka;
                ksm(i + D / 2) = kb2;
                if (kg) { kg[i] = ka; kg[i + D / 2] = kb2; }
            }
            for (int i = lane; i < D; i += 32) {
                const __nv_bfloat16 vv = value_at(vcol + i);
                vsm(i) = vv;
                if (vg) vg[i] = vv;
            }
            __syncwarp();
            if constexpr (BOXES) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        if constexpr (NARROW) {
            const int mat = lane >> 3, r8 = lane & 7;
            float st[DKB / 16][4];                 // keys gq and gq + 8 of a tile of 16 by rows 2 tq and 2 tq + 1
#pragma unroll
            for (int kt = 0; kt < DKB / 16; ++kt) st[kt][0] = st[kt][1] = st[kt][2] = st[kt][3] = 0.f;
#pragma unroll
            for (int ks_ = 0; ks_ < D / 16; ++ks_) {
#pragma unroll
                for (int kt = 0; kt < DKB / 16; ++kt) {
                    // four 8x8 pieces of K: (keys 0..7, d 0..7), (keys 8..15, d 0..7), (keys 0..7, d 8..15), (keys 8..15, d 8..15)
                    uint32_t kf[4];
                    ldmatrix_x4(kf, kpiece(stage, kt * 16 + (mat & 1) * 8 + r8, ks_ * 2 + (mat >> 1)));
                    mma_bf16(st[kt], kf, qf[ks_][0], qf[ks_][2]);
                }
            }
            float mnew[2] = {mrow[0], mrow[1]};
            // a block all of whose keys every token sees needs no comparison of positions (rows beyond the valid
            // ones hold q = 0 and are never stored: they may run along)
            const bool open = (kb + DKB - 1 <= pos_lo) && (p.window <= 0 || kb > pos_hi - p.window);
            if (open) {
#pragma unroll
                for (int kt = 0; kt < DKB / 16; ++kt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        st[kt][e] *= p.scale_log2;
                        mnew[e & 1] = fmaxf(mnew[e & 1], st[kt][e]);
                    }
                }
            } else {
#pragma unroll
                for (int kt = 0; kt < DKB / 16; ++kt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = e & 1;
                        const int key = kb + kt * 16 + gq + (e >> 1) * 8;
                        const bool see = nvalid[c] && key <= npos[c] && (p.window <= 0 || key > npos[c] - p.window);
                        st[kt][e] = see ? st[kt][e] * p.scale_log2 : -INFINITY;
                        mnew[c] = fmaxf(mnew[c], st[kt][e]);
                    }
                }
            }
            float corr[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                mnew[c] = fmaxf(mnew[c], __shfl_xor_sync(0xffffffffu, mnew[c], 4));
                mnew[c] = fmaxf(mnew[c], __shfl_xor_sync(0xffffffffu, mnew[c], 8));
                mnew[c] = fmaxf(mnew[c], __shfl_xor_sync(0xffffffffu, mnew[c], 16));
                corr[c] = (mnew[c] == -INFINITY) ? 1.f : fast_exp2(mrow[c] - mnew[c]);
                mrow[c] = mnew[c];
                lrow[c] *= corr[c];
            }
            const float base2[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};
#pragma unroll
            for (int kt = 0; kt < DKB / 16; ++kt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = fast_exp2(st[kt][e] - base2[e & 1]);
                    st[kt][e] = pv;
                    lrow[e & 1] += pv;
                }
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // no maximum moved: nothing to rescale
#pragma unroll
                for (int i = 0; i < OT; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[1];
                    o[i][2] *= corr[0]; o[i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kt = 0; kt < DKB / 16; ++kt) {
                // P^T of the tile's 16 keys as the second operand: the lane's (key gq, rows 2 tq, 2 tq + 1) becomes
                // (row gq, keys 2 tq, 2 tq + 1) by a transposition within the warp
                const uint32_t pb0 = movmatrix_trans(pack_bf16(st[kt][0], st[kt][1]));
                const uint32_t pb1 = movmatrix_trans(pack_bf16(st[kt][2], st[kt][3]));
#pragma unroll
                for (int dt = 0; dt < D / 16; ++dt) {
                    // V^T: (d 0..7, keys 0..7), (d 8..15, keys 0..7), (d 0..7, keys 8..15), (d 8..15, keys 8..15)
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vpiece(stage, kt * 16 + (mat >> 1) * 8 + r8, dt * 2 + (mat & 1)));
                    mma_bf16(o[dt], vf, pb0, pb1);
                }
            }
        } else {
            float s[DKB / 8][4];
#pragma unroll
            for (int j = 0; j < DKB / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks_ = 0; ks_ < D / 16; ++ks_) {
#pragma unroll
                for (int j = 0; j < DKB / 8; j += 2) {
                    // four 8x8 pieces of K: (keys of tile j, d 0..7), (tile j, d 8..15), (tile j+1, d 0..7), (tile j+1, d 8..15)
                    uint32_t kf[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4(kf, kpiece(stage, (j + (mat >> 1)) * 8 + r, ks_ * 2 + (mat & 1)));
                    mma_bf16(s[j], qf[ks_], kf[0], kf[1]);
                    mma_bf16(s[j + 1], qf[ks_], kf[2], kf[3]);
                }
            }
            float mnew[2] = {mrow[0], mrow[1]};
            // a block all of whose keys every token of the tile sees needs no comparison of positions
            const bool open = (kb + DKB - 1 <= pos_lo) && (p.window <= 0 || kb > pos_hi - p.window);
            if (open) {
#pragma unroll
                for (int j = 0; j < DKB / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[j][e] = valid[e >> 1] ? s[j][e] * p.scale_log2 : -INFINITY;
                        mnew[e >> 1] = fmaxf(mnew[e >> 1], s[j][e]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < DKB / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const int key = kb + j * 8 + 2 * tq + (e & 1);
                        const bool see = valid[i] && key <= pos[i] && (p.window <= 0 || key > pos[i] - p.window);
                        s[j][e] = see ? s[j][e] * p.scale_log2 : -INFINITY;
                        mnew[i] = fmaxf(mnew[i], s[j][e]);
                    }
                }
            }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 1));
                mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 2));
                corr[i] = (mnew[i] == -INFINITY) ? 1.f : fast_exp2(mrow[i] - mnew[i]);
                mrow[i] = mnew[i];
                lrow[i] *= corr[i];
            }
            const float base2[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};
#pragma unroll
            for (int j = 0; j < DKB / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = fast_exp2(s[j][e] - base2[e >> 1]);
                    s[j][e] = pv;
                    lrow[e >> 1] += pv;
                }
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // no maximum moved: nothing to rescale
#pragma unroll
                for (int i = 0; i < D / 8; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[0];
                    o[i][2] *= corr[1]; o[i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < DKB / 16; ++kk) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < D / 16; ++dn) {
                    uint32_t vf[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4_trans(vf, vpiece(stage, kk * 16 + (mat & 1) * 8 + r, dn * 2 + (mat >> 1)));
                    mma_bf16(o[2 * dn], pf, vf[0], vf[1]);
                    mma_bf16(o[2 * dn + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncwarp();
        if (++stage == S) {
            stage = 0;
            phase ^= 1;
        }
    }
    if constexpr (!BOXES) cp_async_wait<0>();         // (only empty groups are left)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if constexpr (NARROW) {
            lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 4);
            lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 8);
            lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 16);
        } else {
            lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
            lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
        }
    }
    // each warp leaves (output [16][D], maximum [16], sum [16]) at the start of its own buffers
    float* wo = reinterpret_cast<float*>(wbase);
    float* wm = wo + 16 * D;
    float* wl = wm + 16;
    if constexpr (NARROW) {
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) wo[(2 * tq + (e & 1)) * D + dt * 16 + gq + (e >> 1) * 8] = o[dt][e];
        }
        if (gq < 2) {                              // rows 0..7 from the lanes of gq 0; rows 8..15 are empty
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                wm[8 * gq + 2 * tq + c] = gq == 0 ? mrow[c] : -INFINITY;
                wl[8 * gq + 2 * tq + c] = gq == 0 ? lrow[c] : 0.f;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt)
                *reinterpret_cast<float2*>(wo + row[i] * D + dt * 8 + 2 * tq) = make_float2(o[dt][2 * i], o[dt][2 * i + 1]);
            if (tq == 0) {
                wm[row[i]] = mrow[i];
                wl[row[i]] = lrow[i];
            }
        }
    }
    __syncthreads();
    // merge the warps: first one weight a (row, warp), the row's maximum and its sum; then every thread takes
    // elements (row, d) of the [16][D] output
    const int tile = seq * p.kv_heads + kvh;
    float* res = reinterpret_cast<float*>(smem_raw + (size_t)W * WARP_BYTES);   // [16][D], then maxima [16], sums [16]
    float* wwgt = res + 16 * D + 32;                                            // [16][W] weights, then [16][8] for the runs
    if (threadIdx.x < 16) {
        const int r = threadIdx.x;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const float* b = reinterpret_cast<const float*>(smem_raw + (size_t)w * WARP_BYTES);
            if (b[16 * D + 16 + r] > 0.f) mx = fmaxf(mx, b[16 * D + r]);
        }
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const float* b = reinterpret_cast<const float*>(smem_raw + (size_t)w * WARP_BYTES);
            const float l = b[16 * D + 16 + r];
            const float wg = (l > 0.f) ? fast_exp2(b[16 * D + r] - mx) : 0.f;
            wwgt[r * W + w] = wg;
            tot += l * wg;
        }
        res[16 * D + r] = mx;
        res[16 * D + 16 + r] = tot;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 16 * D; e += W * 32) {
        const int r = e / D, d = e % D;
        if (r >= rows_valid) continue;
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w)
            acc += reinterpret_cast<const float*>(smem_raw + (size_t)w * WARP_BYTES)[e] * wwgt[r * W + w];
        const float mx = res[16 * D + r], tot = res[16 * D + 16 + r];
        const int t = q_begin + r / group, h = kvh * group + r % group;
        if (alone) {
            p.out[((size_t)t * p.heads + h) * D + d] = __float2bfloat16_rn(tot > 0.f ? acc / tot : 0.f);
        } else if (p.cluster_merge) {
            res[e] = acc;
        } else {
            const size_t idx = ((size_t)split * p.n_tokens + t) * p.heads + h;
            __stcg(p.part_o + idx * D + d, acc);
            if (d == 0) {
                __stcg(p.part_ml + idx * 2, mx);
                __stcg(p.part_ml + idx * 2 + 1, tot);
            }
        }
    }
    if (alone) return;
    if (p.cluster_merge) {
        // the runs are the CTAs of one cluster: each takes a share of the elements and reads every
        // CTA's result through distributed shared memory, runs added in rank order
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int ranks = (int)cluster.num_blocks(), me = (int)cluster.block_rank();
        // one weight a (row, run) and the row's sum, from the runs' maxima and sums (all read at once) ...
        float* rwgt = wwgt + 16 * W;             // [16][8]
        float* rtot = rwgt + 16 * 8;             // [16]
        if (threadIdx.x < 16) {
            const int r = threadIdx.x;
            float m[8], l[8];
#pragma unroll
            for (int rk = 0; rk < 8; ++rk) {
                const float* o_r = cluster.map_shared_rank(res, rk < ranks ? rk : me);
                m[rk] = o_r[16 * D + r];
                l[rk] = rk < ranks ? o_r[16 * D + 16 + r] : 0.f;
            }
            float mx = -INFINITY;
#pragma unroll
            for (int rk = 0; rk < 8; ++rk)
                if (l[rk] > 0.f) mx = fmaxf(mx, m[rk]);
            float tot = 0.f;
#pragma unroll
            for (int rk = 0; rk < 8; ++rk) {
                const float wg = (l[rk] > 0.f) ? fast_exp2(m[rk] - mx) : 0.f;
                rwgt[r * 8 + rk] = wg;
                tot += l[rk] * wg;
            }
            rtot[r] = tot;
        }
        __syncthreads();
        // ... then this CTA's share of the elements, the runs added in rank order
        for (int e = me * W * 32 + threadIdx.x; e < 16 * D; e += ranks * W * 32) {
            const int r = e / D, d = e % D;
            if (r >= rows_valid) continue;
            float v[8];
#pragma unroll
            for (int rk = 0; rk < 8; ++rk) v[rk] = rk < ranks ? cluster.map_shared_rank(res, rk)[e] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int rk = 0; rk < 8; ++rk) acc += v[rk] * rwgt[r * 8 + rk];
            const float tot = rtot[r];
            const int t = q_begin + r / group, h = kvh * group + r % group;
            p.out[((size_t)t * p.heads + h) * D + d] = __float2bfloat16_rn(tot > 0.f ? acc / tot : 0.f);
        }
        cluster.sync();    // nobody leaves while its shared memory is still being read
        return;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_flag = (atomicAdd(&counters[tile], 1) == runs - 1) ? 1 : 0;
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    // The last CTA merges the runs.  First the maxima and sums of all (row, run), loaded side by side and
    // turned into one weight a (row, run) in shared memory; then the outputs, runs added in order.
    constexpr int MAXS = 64;
    float* wgt = reinterpret_cast<float*>(smem_raw);            // [16][MAXS] weights, then [16] totals
    float* tot_s = wgt + 16 * MAXS;
    const size_t stride = (size_t)p.n_tokens * p.heads;
    for (int e = threadIdx.x; e < 16 * runs; e += W * 32) {
        const int r = e / runs, sp = e % runs;
        float m = -INFINITY, l = 0.f;
        if (r < rows_valid) {
            const size_t idx = sp * stride + (size_t)(q_begin + r / group) * p.heads + kvh * group + r % group;
            m = __ldcg(p.part_ml + idx * 2);
            l = __ldcg(p.part_ml + idx * 2 + 1);
        }
        wgt[r * MAXS + sp] = (l > 0.f) ? m : -INFINITY;      // for now the maximum (or -inf for an empty run)
        wgt[16 * MAXS + 16 + r * MAXS + sp] = l;               // and the sum, behind the totals
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        const int r = threadIdx.x;
        float mx = -INFINITY;
        for (int sp = 0; sp < runs; ++sp) mx = fmaxf(mx, wgt[r * MAXS + sp]);
        float tot = 0.f;
        for (int sp = 0; sp < runs; ++sp) {
            const float m = wgt[r * MAXS + sp];
            const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
            wgt[r * MAXS + sp] = w;
            tot += wgt[16 * MAXS + 16 + r * MAXS + sp] * w;
        }
        tot_s[r] = tot;
    }
    __syncthreads();
    // four dims of a row a thread (the rows that hold a query only), the runs' parts added in order, eight 16-byte
    // loads on their way at a time: with one value a load and the rows without a query gone through as well, a
    // single long sequence (64 runs) spent more time here than on its keys
    for (int e = threadIdx.x; e < rows_valid * (D / 4); e += W * 32) {
        const int r = e / (D / 4), d = (e % (D / 4)) * 4;
        const size_t idx0 = (size_t)(q_begin + r / group) * p.heads + kvh * group + r % group;
        const float* src = p.part_o + idx0 * D + d;
        const float* w_r = wgt + r * MAXS;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = 0;
        for (; sp + 8 <= runs; sp += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + i) * stride * D));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float w = w_r[sp + i];
                acc.x += v[i].x * w;
                acc.y += v[i].y * w;
                acc.z += v[i].z * w;
                acc.w += v[i].w * w;
            }
        }
        for (; sp < runs; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * stride * D));
            const float w = w_r[sp];
            acc.x += v.x * w;
            acc.y += v.y * w;
            acc.z += v.z * w;
            acc.w += v.w * w;
        }
        const float tot = tot_s[r];
        // (a / tot as before, not a * (1 / tot): the same bits as the merge inside a cluster gives)
        __nv_bfloat162 lo = __floats2bfloat162_rn(tot > 0.f ? acc.x / tot : 0.f, tot > 0.f ? acc.y / tot : 0.f);
        __nv_bfloat162 hi = __floats2bfloat162_rn(tot > 0.f ? acc.z / tot : 0.f, tot > 0.f ? acc.w / tot : 0.f);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + idx0 * D + d) = packed;
    }
    if (threadIdx.x == 0) counters[tile] = 0;
}

template <int D, int W, int S, bool NARROW, bool BOXES>
cudaError_t launch_decode_n(AttnParams p, int n_seqs, int* counters, cudaStream_t stream) {
    constexpr int WARP_BYTES = decode_warp_bytes(D, BOXES, S);
    // with boxes 1,024 bytes more: the swizzled tiles start on such a boundary
    constexpr int smem = W * WARP_BYTES + (16 * D + 32 + 16 * W + 16 * 8 + 16) * 4 + (BOXES ? 1024 : 0);
    static_assert(WARP_BYTES >= (16 * D + 32) * 4, "a warp's buffers must hold its merged result");
    static_assert(W * WARP_BYTES >= (2 * 16 * 64 + 16) * 4, "the merge of the runs needs its weights");
    CUtensorMap map_k, map_v;
    memset(&map_k, 0, sizeof(map_k));
    memset(&map_v, 0, sizeof(map_v));
    if constexpr (BOXES) {
        // the caches as matrices [pages * kv_heads * page_size, D]; a box never crosses a page
        p.run_keys = p.page_size % DKB == 0 ? DKB : 16;
        const long long rows = (long long)p.n_pages * p.kv_heads * p.page_size;
        if (!make_map(&map_k, p.k_cache, rows, D, p.run_keys) || !make_map(&map_v, p.v_cache, rows, D, p.run_keys))
            return cudaErrorInvalidValue;
    }
    static std::atomic<unsigned long long> configured{0};
    cudaError_t e = allow_dynamic_smem(attention_decode_kernel<D, W, S, NARROW, BOXES>, smem, configured);
    if (e != cudaSuccess) return e;
    return launch(attention_decode_kernel<D, W, S, NARROW, BOXES>, dim3(n_seqs, p.kv_heads, p.n_splits), dim3(W * 32, 1, 1), smem, stream,
                  dim3(1, 1, p.cluster_merge ? p.n_splits : 1), p, counters, map_k, map_v);
}

template <int D, int W, int S>
cudaError_t launch_decode_w(const AttnParams& p, int n_seqs, int* counters, cudaStream_t stream) {
    const bool narrow = p.tokens_per_tile * (p.heads / p.kv_heads) <= 8;
    if constexpr (decode_by_boxes(D)) {
        if (p.run_keys != 0)                       // the caller expects long runs of keys a warp
            return narrow ? launch_decode_n<D, W, S, true, true>(p, n_seqs, counters, stream)
                          : launch_decode_n<D, W, S, false, true>(p, n_seqs, counters, stream);
    }
    return narrow ? launch_decode_n<D, W, S, true, false>(p, n_seqs, counters, stream)
                  : launch_decode_n<D, W, S, false, false>(p, n_seqs, counters, stream);
}

// The shape of a CTA: warps and stages of a warp's ring.  The ring's bytes bound both: W * S blocks of keys and
// values fit an SM once (8 x 2 or 4 x 4 at head size 128) or, for two CTAs an SM, half as many each (6 x 2 or
// 3 x 4).  With more CTAs than SMs the kernel runs the shape of which two fit an SM (head sizes 64 and 128): the
// CTAs then need not run in rounds of one an SM, whose last round is partly empty.
inline int decode_shape() {
    static int shape = -1;
    if (shape < 0) {
        const char* v = std::getenv("VTB200_DECODE_SHAPE");     // "deep": fewer warps with deeper rings (for measurements)
        shape = (v != nullptr && v[0] == 'd') ? 1 : 0;
    }
    return shape;
}

template <int D>
cudaError_t launch_decode_d(const AttnParams& p, int n_seqs, int* counters, cudaStream_t stream) {
    if constexpr (D == 128 || D == 64) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 0;
        const bool two = sms > 0 && (long long)n_seqs * p.kv_heads * p.n_splits > sms;
        if (decode_shape() == 1)
            return two ? launch_decode_w<D, 3, 4>(p, n_seqs, counters, stream) : launch_decode_w<D, 4, 4>(p, n_seqs, counters, stream);
        return two ? launch_decode_w<D, 6, 2>(p, n_seqs, counters, stream) : launch_decode_w<D, 8, 2>(p, n_seqs, counters, stream);
    }
    return launch_decode_w<D, 8, 2>(p, n_seqs, counters, stream);
}

}  // namespace

}  // namespace vtb
