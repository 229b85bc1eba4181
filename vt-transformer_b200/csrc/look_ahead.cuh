// Asking for the weights of the product that runs next, ahead of its kernel.
//
// The weights are written by no kernel, so a kernel of the step may ask for them into L2 while HBM has little to do: a
// product that streams weights does so when its last load is on its way.  What is asked for are boxes of 64 k by 128
// rows, the first `depth` k-blocks of each of the first units of the next product's kernel (gemm_tc.cu, w as the
// 128-row operand), which is what that kernel loads first.
#pragma once
#include <cuda.h>

#include "kernels.h"

namespace vtb {

struct AheadTiles {
    int a_tiles, units, s_tail, nkb, depth;    // tiles of 128 rows, each in s_tail shares of nkb k-blocks
};

// How the product `next` will cut its weights when it runs over m rows; false if there is nothing to ask for
// (no hint, or it will not run with w as the 128-row operand).  Defined in gemm_tc.cu.
bool look_ahead(const NextProduct* next, int m, CUtensorMap* map, AheadTiles* tiles);

// Box i of unit u: its coordinates in the matrix (k, row); false beyond the unit's share of k.
__device__ __forceinline__ bool ahead_box(const AheadTiles& t, int u, int i, int& x, int& y) {
    const int tile = u / t.s_tail, krank = u % t.s_tail;
    const int kb0 = (int)((long long)krank * t.nkb / t.s_tail), kb1 = (int)((long long)(krank + 1) * t.nkb / t.s_tail);
    x = (kb0 + i) * 64;
    y = (tile % t.a_tiles) * 128;
    return kb0 + i < kb1;
}

__device__ __forceinline__ void ahead_prefetch(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n" ::"l"(map), "r"(x), "r"(y) : "memory");
}

}  // namespace vtb
