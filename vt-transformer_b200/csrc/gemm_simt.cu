// C[M, N] = A[M, K] W[N, K]^T (+ bias) with 32-bit multiply-adds: FFMA only, no tensor cores,
// no TF32.  Operands are float, or bfloat16 widened exactly on the way in.
//
// vt-transformer sends its 32-bit products to cuBLASLt and lets it pick tensor operations
// (v1/tensortype/cuda_kernels/lt_sgemm.cu:53-54), so it has no verified 32-bit run.  With float
// operands this kernel is the engine's 32-bit path: every output element is the sum over
// k = 0, 1, 2, ... in that order, whatever M is and whatever else is in the batch, so logits
// agree bit for bit however the tokens are cut into steps.  With bfloat16 operands it is the
// plain twin of the tensor-core products.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;
}

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ a, const TA* __restrict__ w, const float* __restrict__ bias,
                 TC* __restrict__ c, int m, int n, int k) {
    pdl_launch();
    pdl_wait();
    __shared__ __align__(16) float as[BK][BM + PAD];
    __shared__ __align__(16) float ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;   // loader: row of the tile, 4 consecutive k
    const int ty = tid >> 4, tx = tid & 15;          // compute: rows ty*4.., cols tx*4..
    float acc[4][4] = {};

    const bool a_ok = (m0 + lrow) < m, w_ok = (n0 + lrow) < n;
    const TA* ap = a + (size_t)(m0 + lrow) * k + lk;
    const TA* wp = w + (size_t)(n0 + lrow) * k + lk;

    for (int k0 = 0; k0 < k; k0 += BK) {
        float4 av = make_float4(0.f, 0.f, 0.f, 0.f), wv = av;
        if (k0 + lk < k) {   // k % 4 == 0, so the four elements are inside or outside together
            if (a_ok) av = load4<TA>(ap + k0);
            if (w_ok) wv = load4<TA>(wp + k0);
        }
        as[lk + 0][lrow] = av.x; as[lk + 1][lrow] = av.y; as[lk + 2][lrow] = av.z; as[lk + 3][lrow] = av.w;
        ws[lk + 0][lrow] = wv.x; ws[lk + 1][lrow] = wv.y; ws[lk + 2][lrow] = wv.z; ws[lk + 3][lrow] = wv.w;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 x = *reinterpret_cast<const float4*>(&as[kk][ty * 4]);
            const float4 y = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
            const float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xs[i], ys[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = m0 + ty * 4 + i;
        if (row >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + tx * 4 + j;
            if (col < n) c[(size_t)row * n + col] = from_float<TC>(acc[i][j] + (bias ? bias[col] : 0.f));
        }
    }
}

cudaError_t launch_gemm_simt(int in_dtype, int out_dtype, const void* a, const void* w, const float* bias, void* c,
                             int m, int n, int k, cudaStream_t stream) {
    if (m == 0 || n == 0) return cudaSuccess;
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    if (in_dtype == kF32 && out_dtype == kF32)
        return launch(gemm_simt_kernel<float, float>, grid, 256, 0, stream, (const float*)a, (const float*)w, bias, (float*)c, m, n, k);
    if (in_dtype == kBF16 && out_dtype == kBF16)
        return launch(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream,
            (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)c, m, n, k);
    if (in_dtype == kBF16 && out_dtype == kF32)
        return launch(gemm_simt_kernel<__nv_bfloat16, float>, grid, 256, 0, stream,
            (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, bias, (float*)c, m, n, k);
    return cudaErrorInvalidValue;
}

}  // namespace vtb
