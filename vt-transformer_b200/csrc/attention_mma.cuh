// What the tensor-core attention kernels over the paged cache share: asynchronous copies, the mma.sync
// and ldmatrix forms, and the description of a launch.  Used by attention_mma.cu (prompt portions) and
// attention_decode.cu (single-token steps).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace vtb {

struct AttnParams {
    const __nv_bfloat16* qkv;
    int qkv_stride;
    __nv_bfloat16* out;
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    const int* cu_q;
    const int* q_start;
    const int* block_table;
    int table_stride;
    const int2* tiles;      // (sequence, first token of the tile among the sequence's new tokens); null: tile = sequence
    int n_pages, heads, kv_heads, page_size, window;
    float scale_log2;       // scale * log2(e)
    int tokens_per_tile;
    int run_keys;              // single-token steps, head sizes 64 and 128: rows of a box of the keys' and values' tensor maps
    int n_splits;
    // single-token steps: blocks of keys that a run is to hold; a sequence then takes about (its blocks / run_blocks)
    // of the n_splits CTAs, the others stay idle.  0: every sequence is cut into n_splits equal runs.
    int run_blocks;
    float* part_o;          // [splits, tokens, heads, D] unnormalised sums, when n_splits > 1
    float* part_ml;         // [splits, tokens, heads, 2] running maximum (log2 domain) and sum
    int n_tokens;
    int* status;
    int cluster_merge;      // 1: the runs of a sequence are the CTAs of a cluster and merge through their shared memory
    // single-token steps may rotate q and k and store k and v themselves (no separate kernel before them)
    int fuse_rope;          // 1: q and k in qkv are not rotated yet and the token's k and v are not in the cache yet
    const float2* cos_sin;  // [max_pos, D / 2] (cos, sin), or null: no rotation
    int max_pos;
    int store_kv;           // 1: write the token's k and v into their page
    __nv_bfloat16* k_out;   // the cache again, writable
    __nv_bfloat16* v_out;
    // single-token steps may also take q, k and v as the unadded 32-bit shares [n_shares, tokens, qkv_stride] that
    // the product before them left (its inner dimension cut over CTAs): they are added, in order, where they are read
    const float* qkv_shares;
    int n_shares;
};

namespace {

constexpr int KB = 64;   // keys in a block

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}

// the 8x8 matrix of 16-bit values that the warp holds (lane 4 r + c: row r, columns 2 c and 2 c + 1), transposed
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}

// 2^x, the hardware approximation (2 ulp); exp2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


}  // namespace

}  // namespace vtb
