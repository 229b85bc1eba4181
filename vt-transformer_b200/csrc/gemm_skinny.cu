// out[M, N] = x[M, K] w[N, K]^T (+ bias) for a few rows of x (M <= 64): the decode step's
// projections, where every weight is read once from HBM and the time is the time of that read.
//
// vt-transformer sends these products to cuBLASLt one by one, for the logits even one row at a
// time (v1/tensortype/cuda_tensor.cpp:544-552, 946-992).  This kernel is shaped for the read
// instead: a CTA owns 16 rows of w and streams them from end to end with 16-byte loads that go
// straight into the A operand of mma.sync m16n8k16 (w is the 16-row operand, the few rows of x
// the 8-column one); its 8 warps take the 32-wide k-blocks in turn, so the CTA reads consecutive
// memory, and their partial sums meet in shared memory.  Which k of a block goes to which slot
// of the operand does not matter for a dot product, as long as w and x agree: a thread's 8
// consecutive elements serve two MMAs, and x is loaded the same way.
//
// A matrix with few rows (the o and down projections: 224 tiles of 16 rows for 148 SMs) would
// leave most of the machine without loads in flight, so its k range is cut over the CTAs of a
// thread-block cluster (up to 8); each CTA sums its share, and the shares are added in rank
// order through distributed shared memory: no scratch in global memory, no atomics, the same
// sum whatever the timing.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace cg = cooperative_groups;

namespace vtb {

namespace {

constexpr int WARPS = 8;
constexpr int UNROLL = 4;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int NT, typename TOut>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ bias, TOut* __restrict__ out, int m, int n, int k) {
    __shared__ float red[WARPS][NT][16][8 + 1];
    __shared__ float tile[NT * 128];
    pdl_launch();
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), csize = cluster.num_blocks();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.y * 16;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool ok0 = r0 < n, ok1 = r1 < n;
    const __nv_bfloat16* w0 = w + (size_t)(ok0 ? r0 : 0) * k + 8 * t;
    const __nv_bfloat16* w1 = w + (size_t)(ok1 ? r1 : 0) * k + 8 * t;
    const __nv_bfloat16* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = (j * 8 + g) < m;
        xr[j] = x + (size_t)(xok[j] ? j * 8 + g : 0) * k + 8 * t;
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    const int nkb_all = (k + 31) / 32;
    const int per_cta = (nkb_all + (int)csize - 1) / (int)csize;
    const int kb_begin = (int)rank * per_cta;
    const int nkb = min(nkb_all, kb_begin + per_cta);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int kb = kb_begin + warp; kb < nkb; kb += WARPS * UNROLL) {
        uint4 a[UNROLL], b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kk = (kb + u * WARPS) * 32;
            // k % 8 == 0: a thread's piece lies inside or outside as a whole
            const bool in = (kb + u * WARPS) < nkb && kk + 8 * t + 8 <= k;
            a[u] = (in && ok0) ? load_stream(reinterpret_cast<const uint4*>(w0 + kk)) : zero;
            b[u] = (in && ok1) ? load_stream(reinterpret_cast<const uint4*>(w1 + kk)) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kk = (kb + u * WARPS) * 32;
            const bool in = (kb + u * WARPS) < nkb && kk + 8 * t + 8 <= k;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 xv = (in && xok[j]) ? __ldg(reinterpret_cast<const uint4*>(xr[j] + kk)) : zero;
                mma_bf16(acc[j], a[u].x, b[u].x, a[u].y, b[u].y, xv.x, xv.y);
                mma_bf16(acc[j], a[u].z, b[u].z, a[u].w, b[u].w, xv.z, xv.w);
            }
        }
    }
    // acc[j][0..1]: (w row g, x rows j*8 + 2t, +1); acc[j][2..3]: (w row g + 8, same x rows)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][j][g][2 * t] = acc[j][0];
        red[warp][j][g][2 * t + 1] = acc[j][1];
        red[warp][j][g + 8][2 * t] = acc[j][2];
        red[warp][j][g + 8][2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    // this CTA's share of every output of the tile: e = (j, x column, w row)
    for (int e = threadIdx.x; e < NT * 128; e += WARPS * 32) {
        const int row = e & 15, col = (e >> 4) & 7, j = e >> 7;
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) s += red[wv][j][row][col];
        tile[e] = s;
    }
    cluster.sync();
    // the CTAs of the cluster share out the outputs; each adds the shares in rank order
    for (int e = (int)rank * (WARPS * 32) + threadIdx.x; e < NT * 128; e += (int)csize * WARPS * 32) {
        const int row = e & 15, col = (e >> 4) & 7, j = e >> 7;
        const int mm = j * 8 + col, nn = n0 + row;
        if (mm >= m || nn >= n) continue;
        float s = 0.f;
        for (unsigned r = 0; r < csize; ++r) s += cluster.map_shared_rank(tile, r)[e];
        if (bias) s += bias[nn];
        out[(size_t)mm * n + nn] = from_float<TOut>(s);
    }
    cluster.sync();   // nobody leaves while its shared memory is still being read
}

template <int NT, typename TOut>
cudaError_t launch_nt(const __nv_bfloat16* x, const __nv_bfloat16* w, const float* bias, TOut* out, int m, int n, int k,
                      int ksplit, cudaStream_t stream) {
    return launch(gemm_skinny_kernel<NT, TOut>, dim3(ksplit, (n + 15) / 16, 1), dim3(WARPS * 32, 1, 1), 0, stream,
                  dim3(ksplit, 1, 1), x, w, bias, out, m, n, k);
}

template <typename TOut>
cudaError_t launch_t(const __nv_bfloat16* x, const __nv_bfloat16* w, const float* bias, TOut* out, int m, int n, int k,
                     cudaStream_t stream) {
    // enough CTAs to keep loads in flight on all 148 SMs: cut k over a cluster when the rows are few,
    // but leave every warp at least one unrolled round of k-blocks
    const int tiles = (n + 15) / 16, nkb = (k + 31) / 32;
    int ksplit = 1;
    while (ksplit < 8 && tiles * ksplit < 1184 && nkb / (ksplit * 2) >= WARPS * UNROLL / 2) ksplit *= 2;
    if (m <= 8) return launch_nt<1, TOut>(x, w, bias, out, m, n, k, ksplit, stream);
    if (m <= 16) return launch_nt<2, TOut>(x, w, bias, out, m, n, k, ksplit, stream);
    if (m <= 32) return launch_nt<4, TOut>(x, w, bias, out, m, n, k, ksplit, stream);
    if (m <= 64) return launch_nt<8, TOut>(x, w, bias, out, m, n, k, ksplit, stream);
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_gemm_skinny(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n,
                               int k, cudaStream_t stream) {
    if (m == 0 || n == 0) return cudaSuccess;
    if (k % 8 != 0) return cudaErrorInvalidValue;
    if (out_dtype == kBF16)
        return launch_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)out, m, n, k, stream);
    if (out_dtype == kF32)
        return launch_t<float>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (float*)out, m, n, k, stream);
    return cudaErrorInvalidValue;
}

}  // namespace vtb
