// Attention over the paged cache on the tensor cores (bfloat16 in, 32-bit softmax and sums).
//
// What it computes is the chain of vt-transformer's graph, scores = q k^T / sqrt(d), causal mask,
// softmax, P V (v1/models/qwen2-7b/inference_fp16.dag:307-318; v1/tensortype/cuda_tensor.cpp:761-773,
// 796-800, 869-881), for the query heads of one KV head at a time (head / group,
// v1/tensortype/cuda_kernels/transpose_0213.cu:93-105).  How it computes it is this engine's: one
// pass over the keys with a running maximum and sum, keys and values read from their pages through
// the block table, the heads of a group packed into the rows of one tile so that a key is fetched
// once for all of them, and for single-token steps the keys split over several CTAs whose partial
// results a second kernel merges.  The [heads, T, F] score tensor, the mask tensor and the repeated
// heads of the reference are never formed.
//
// A tile is 16 * WARPS rows; row r is (token r / group, head r % group) of its tile.  Keys come in
// blocks of 64 through a two-stage cp.async pipeline; a run of 16 keys never crosses a page
// (page_size % 16 == 0).  S = Q K^T and O += P V are mma.sync m16n8k16 (P rounded to bfloat16).
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"
#include "attention_mma.cuh"
#include "launch.cuh"

namespace cg = cooperative_groups;

namespace vtb {

namespace {

template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_mma_kernel(const AttnParams p) {
    constexpr int LD = D + 8;                 // padded row: conflict-free fragment loads, 16-byte aligned rows
    constexpr int THREADS = WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][KB][LD]
    __nv_bfloat16* vs = ks + 2 * KB * LD;                             // [2][KB][LD]

    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int kvh = blockIdx.y, split = blockIdx.z;
    int seq, tok0;
    if (p.tiles) {
        const int2 t = p.tiles[blockIdx.x];
        seq = t.x;
        tok0 = t.y;
    } else {
        seq = blockIdx.x;
        tok0 = 0;
    }
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    if (ntok <= 0) return;
    const int group = p.heads / p.kv_heads;
    const int rows_valid = ntok * group;
    const int start = p.q_start[seq];
    const int pos_lo = start + tok0, pos_hi = pos_lo + ntok - 1;
    int key_lo = (p.window > 0) ? max(0, pos_lo - p.window + 1) : 0;
    key_lo = key_lo / KB * KB;
    const int key_hi = pos_hi + 1;
    const int nblk = (key_hi - key_lo + KB - 1) / KB;
    const int per_split = (nblk + p.n_splits - 1) / p.n_splits;
    const int blk0 = split * per_split, blk1 = min(nblk, blk0 + per_split);

    // the two rows of this thread
    int row[2], pos[2], tok[2], head[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row[i] = warp * 16 + gq + 8 * i;
        valid[i] = row[i] < rows_valid;
        const int tk = valid[i] ? row[i] / group : 0;
        tok[i] = q_begin + tok0 + tk;
        pos[i] = pos_lo + tk;
        head[i] = kvh * group + (valid[i] ? row[i] % group : 0);
    }

    // Q fragments
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __nv_bfloat16* qp = p.qkv + (size_t)tok[i] * p.qkv_stride + (size_t)head[i] * D;
#pragma unroll
        for (int ks_ = 0; ks_ < D / 16; ++ks_) {
            qf[ks_][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + ks_ * 16 + 2 * tq) : 0u;
            qf[ks_][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + ks_ * 16 + 8 + 2 * tq) : 0u;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    const int* table = p.block_table + (size_t)seq * p.table_stride;
    auto load_block = [&](int blk, int stage) {
        const int kb = key_lo + blk * KB;
        constexpr int CHUNKS = D / 8;          // 16-byte pieces in a row
        // the block's four runs of 16 keys lie in one page each: their bases once, then plain offsets
        static_assert(KB == 64, "four runs of 16 keys");
        size_t base[4];
        bool okp[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const int key = kb + 16 * h;
            okp[h] = key < key_hi;
            base[h] = 0;
            if (okp[h]) {
                const int page = table[key / p.page_size];
                // a page behind a window may be gone already; its keys are masked below
                if (page < 0 || page >= p.n_pages) okp[h] = false;
                else base[h] = (((size_t)page * p.kv_heads + kvh) * p.page_size + key % p.page_size) * D;
            }
        }
        for (int c = threadIdx.x; c < KB * CHUNKS; c += THREADS) {
            const int r = c / CHUNKS, piece = c % CHUNKS;
            const int h = r >> 4;                  // selected without indexing, so the bases stay in registers
            const size_t bh = h == 0 ? base[0] : h == 1 ? base[1] : h == 2 ? base[2] : base[3];
            const bool oh = h == 0 ? okp[0] : h == 1 ? okp[1] : h == 2 ? okp[2] : okp[3];
            const bool ok = oh && (kb + r) < key_hi;
            const size_t off = ok ? bh + (size_t)(r & 15) * D + piece * 8 : 0;
            cp_async16(ks + ((size_t)stage * KB + r) * LD + piece * 8, p.k_cache + off, ok);
            cp_async16(vs + ((size_t)stage * KB + r) * LD + piece * 8, p.v_cache + off, ok);
        }
    };

    if (blk0 < blk1) {
        load_block(blk0, 0);
        cp_async_commit();
    }
    for (int blk = blk0; blk < blk1; ++blk) {
        const int stage = (blk - blk0) & 1;
        if (blk + 1 < blk1) {
            load_block(blk + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* kst = ks + (size_t)stage * KB * LD;
        const __nv_bfloat16* vst = vs + (size_t)stage * KB * LD;
        const int kb = key_lo + blk * KB;

        // S = Q K^T
        float s[KB / 8][4];
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks_ = 0; ks_ < D / 16; ++ks_) {
#pragma unroll
            for (int j = 0; j < KB / 8; j += 2) {
                // four 8x8 pieces of K: (keys of tile j, d 0..7), (tile j, d 8..15), (tile j+1, d 0..7), (tile j+1, d 8..15)
                uint32_t kf[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(kf, kst + (size_t)((j + (mat >> 1)) * 8 + r) * LD + ks_ * 16 + (mat & 1) * 8);
                mma_bf16(s[j], qf[ks_], kf[0], kf[1]);
                mma_bf16(s[j + 1], qf[ks_], kf[2], kf[3]);
            }
        }
        // mask, running maximum and sum (log2 domain)
        float mnew[2] = {mrow[0], mrow[1]};
        // a block all of whose keys every row of the tile sees needs no mask
        const bool open = (kb + KB - 1 <= pos_lo) && (p.window <= 0 || kb > pos_hi - p.window);
        if (open) {
#pragma unroll
            for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] *= p.scale_log2;
                    mnew[e >> 1] = fmaxf(mnew[e >> 1], s[j][e]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < KB / 8; ++j) {
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
        const float base[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = fast_exp2(s[j][e] - base[e >> 1]);   // 2^(-inf) = 0 for masked keys
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
        // O += P V
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                uint32_t vf[4];
                const int mat = lane >> 3, r = lane & 7;
                const __nv_bfloat16* vp = vst + (size_t)(kk * 16 + (mat & 1) * 8 + r) * LD + dn * 16 + (mat >> 1) * 8;
                ldmatrix_x4_trans(vf, vp);
                mma_bf16(o[2 * dn], pf, vf[0], vf[1]);
                mma_bf16(o[2 * dn + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();
    }

    // epilogue
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
    }
    if (p.n_splits == 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;
            const float inv = lrow[i] > 0.f ? 1.f / lrow[i] : 0.f;
            __nv_bfloat16* op = p.out + (size_t)tok[i] * p.heads * D + (size_t)head[i] * D;
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt) {
                const uint32_t v = pack_bf16(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
                *reinterpret_cast<uint32_t*>(op + dt * 8 + 2 * tq) = v;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!valid[i]) continue;
            const size_t idx = ((size_t)split * p.n_tokens + tok[i]) * p.heads + head[i];
            float* op = p.part_o + idx * D;
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt)
                *reinterpret_cast<float2*>(op + dt * 8 + 2 * tq) = make_float2(o[dt][2 * i], o[dt][2 * i + 1]);
            if (tq == 0) {
                p.part_ml[idx * 2] = mrow[i];
                p.part_ml[idx * 2 + 1] = lrow[i];
            }
        }
    }
}

// Merges the partial results of the splits: one warp for a (token, head).
template <int D>
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out, int n_tokens, int heads, int n_splits) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (pair >= (long long)n_tokens * heads) return;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) {
        const float l = part_ml[((size_t)s * n_tokens * heads + pair) * 2 + 1];
        if (l > 0.f) mx = fmaxf(mx, part_ml[((size_t)s * n_tokens * heads + pair) * 2]);
    }
    float total = 0.f;
    float acc[D / 32 + 1];
#pragma unroll
    for (int r = 0; r < D / 32 + 1; ++r) acc[r] = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const size_t idx = (size_t)s * n_tokens * heads + pair;
        const float l = part_ml[idx * 2 + 1];
        if (!(l > 0.f)) continue;
        const float w = exp2f(part_ml[idx * 2] - mx);
        total += l * w;
#pragma unroll
        for (int r = 0; r < D / 32 + 1; ++r) {
            const int d = lane + 32 * r;
            if (d < D) acc[r] += part_o[idx * D + d] * w;
        }
    }
    const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
    for (int r = 0; r < D / 32 + 1; ++r) {
        const int d = lane + 32 * r;
        if (d < D) out[(size_t)pair * D + d] = __float2bfloat16_rn(acc[r] * inv);
    }
}

template <int D, int WARPS>
cudaError_t launch_one(const AttnParams& p, int n_tiles, cudaStream_t stream) {
    constexpr int smem = 2 * 2 * KB * (D + 8) * (int)sizeof(__nv_bfloat16);
    static std::atomic<unsigned long long> configured{0};
    cudaError_t e = allow_dynamic_smem(attention_mma_kernel<D, WARPS>, smem, configured);
    if (e != cudaSuccess) return e;
    dim3 grid(n_tiles, p.kv_heads, p.n_splits);
    e = launch(attention_mma_kernel<D, WARPS>, grid, WARPS * 32, smem, stream, p);
    if (e != cudaSuccess) return e;
    if (p.n_splits > 1) {
        const long long pairs = (long long)p.n_tokens * p.heads;
        e = launch(attention_combine_kernel<D>, (int)((pairs + 3) / 4), 128, 0, stream, (const float*)p.part_o,
                   (const float*)p.part_ml, p.out, p.n_tokens, p.heads, p.n_splits);
    }
    return e;
}

template <int D>
cudaError_t launch_d(const AttnParams& p, int warps, int n_tiles, cudaStream_t stream) {
    if (warps == 1) return launch_one<D, 1>(p, n_tiles, stream);
    if (warps == 8) return launch_one<D, 8>(p, n_tiles, stream);
    return launch_one<D, 4>(p, n_tiles, stream);
}

}  // namespace

bool attention_mma_supports(int head_dim, int heads, int kv_heads, int warps) {
    if (head_dim % 16 != 0 || head_dim > 128 || head_dim < 16) return false;
    if (warps != 1 && warps != 4 && warps != 8) return false;
    return heads / kv_heads <= 16 * warps;
}

cudaError_t launch_attention_mma(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                 const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                 const int* tiles, int n_tiles, int n_pages, int n_tokens, int heads, int kv_heads,
                                 int head_dim, int page_size, int window, float scale, int warps, int n_splits,
                                 float* part_o, float* part_ml, int* status, cudaStream_t stream) {
    if (n_tiles == 0 || n_tokens == 0) return cudaSuccess;
    if (!attention_mma_supports(head_dim, heads, kv_heads, warps) || page_size % 16 != 0) return cudaErrorInvalidValue;
    if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return cudaErrorInvalidValue;
    AttnParams p;
    p.cluster_merge = 0;
    p.fuse_rope = 0;
    p.cos_sin = nullptr;
    p.max_pos = 0;
    p.store_kv = 0;
    p.k_out = nullptr;
    p.v_out = nullptr;
    p.qkv_shares = nullptr;
    p.n_shares = 0;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.out = (__nv_bfloat16*)out;
    p.k_cache = (const __nv_bfloat16*)k_cache;
    p.v_cache = (const __nv_bfloat16*)v_cache;
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
    p.tokens_per_tile = (16 * warps) / (heads / kv_heads);
    p.n_splits = n_splits < 1 ? 1 : n_splits;
    p.run_blocks = 0;
    p.part_o = part_o;
    p.part_ml = part_ml;
    p.n_tokens = n_tokens;
    p.status = status;
    switch (head_dim) {
        case 16: return launch_d<16>(p, warps, n_tiles, stream);
        case 32: return launch_d<32>(p, warps, n_tiles, stream);
        case 48: return launch_d<48>(p, warps, n_tiles, stream);
        case 64: return launch_d<64>(p, warps, n_tiles, stream);
        case 80: return launch_d<80>(p, warps, n_tiles, stream);
        case 96: return launch_d<96>(p, warps, n_tiles, stream);
        case 112: return launch_d<112>(p, warps, n_tiles, stream);
        case 128: return launch_d<128>(p, warps, n_tiles, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace vtb
