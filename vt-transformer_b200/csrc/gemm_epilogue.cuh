// The epilogue of the tcgen05 products: what becomes of 16 finished sums of one accumulator lane (bias, or
// SiLU(gate) * up, rounding, store).  Shared by gemm_tc.cu (one CTA a tile) and gemm_tc_pair.cu (a pair of CTAs a tile).
#pragma once

#include "common.cuh"

namespace vtb {

namespace {

template <typename T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// Writes 16 finished sums of one accumulator lane: columns c0 .. c0 + 15 of lane r of the tile.
// EPI 0: out = sum + bias.  EPI 1 (gate and up rows of w interleaved in runs of 8: g0..g7, u0..u7,
// g8.., ...): out[token, 8 j + i] = silu(sum of row 16 j + i) * (sum of row 16 j + 8 + i), in 32-bit,
// silu(z) = z / (1 + exp(-z)) (v1/tensortype/cuda_kernels/silu_product.cu:15-17); out has half the
// columns.  Every lane of a warp must call it (the swapped form trades values between lanes).
template <bool SWAP, int EPI, typename TOut>
__device__ __forceinline__ void emit16(float (&v)[16], int r, int a_row0, int b_row0, int c0, int rows_a, int rows_b,
                                       const float* __restrict__ bias, TOut* __restrict__ out, int ldo) {
    if (SWAP) {
        const int n = a_row0 + r;                  // feature (row of w)
        if (EPI == 1) {
            const bool gate = (r & 8) == 0;
            const int f = ((n >> 4) << 3) + (n & 7);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
                const int m = b_row0 + c0 + i;     // token
                if (gate && n < rows_a && m < rows_b)
                    out[(size_t)m * ldo + f] = from_float<TOut>(v[i] / (1.f + expf(-v[i])) * other);
            }
        } else if (n < rows_a) {
            const float b = bias ? bias[n] : 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int m = b_row0 + c0 + i;
                if (m < rows_b) out[(size_t)m * ldo + n] = from_float<TOut>(v[i] + b);
            }
        }
    } else {
        const int m = a_row0 + r;                  // token
        if (m >= rows_a) return;
        const int n0 = b_row0 + c0;                // feature of v[0]
        if (EPI == 1) {
            if (n0 + 16 > rows_b) return;          // rows of w come in whole runs of 16
            float act[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) act[j] = v[j] / (1.f + expf(-v[j])) * v[8 + j];
            TOut* o = out + (size_t)m * ldo + (n0 >> 1);
            if ((ldo & 7) == 0) {
                store8<TOut>(o, act);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = from_float<TOut>(act[j]);
            }
            return;
        }
        TOut* o = out + (size_t)m * ldo + n0;
        if (bias) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] += (n0 + i < rows_b) ? bias[n0 + i] : 0.f;
        }
        if ((ldo & 7) == 0 && n0 + 16 <= rows_b) {
            store8<TOut>(o, v);
            store8<TOut>(o + 8, v + 8);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (n0 + i < rows_b) o[i] = from_float<TOut>(v[i]);
        }
    }
}

}  // namespace

}  // namespace vtb
