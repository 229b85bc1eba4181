// The one entry point that allocates nothing: see attention_noalloc.h.
#include "attention_noalloc.h"

#include <atomic>
#include <cstdio>

#include "kernels.h"

namespace {

// The scratch of the split-key kernel, in the library's device image.  In host code this name is a
// host-side stand-in, not a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float vtb_noalloc_scratch[VTB_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
std::atomic<float*> g_scratch[kMaxDevices] = {};   // device address of the array, by device, once looked up

}  // namespace

extern "C" int vtb_decode_attention_noalloc(const void* qkv, int qkv_stride, void* out, const void* k_cache,
                                            const void* v_cache, const int* cu_q, const int* q_start,
                                            const int* block_table, int table_stride, int n_seqs, int n_pages,
                                            int heads, int kv_heads, int head_dim, int page_size, int window,
                                            float scale, int n_splits, void* stream) {
    if (n_seqs <= 0) return 0;
    if (qkv == nullptr || out == nullptr || k_cache == nullptr || v_cache == nullptr || cu_q == nullptr ||
        q_start == nullptr || block_table == nullptr) {
        std::fprintf(stderr, "vtb_decode_attention_noalloc: a null pointer among the inputs and outputs\n");
        return 2;
    }
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || n_splits < 1 || n_splits > 64 || page_size < 16 ||
        page_size % 16 != 0 || table_stride < 1 || n_pages < 1 || !vtb::attention_mma_supports(head_dim, heads, kv_heads, 1) ||
        (long long)qkv_stride < (long long)heads * head_dim) {
        std::fprintf(stderr, "vtb_decode_attention_noalloc: unsupported arguments (heads %d, kv_heads %d, head_dim %d, "
                             "page_size %d, n_splits %d, qkv_stride %d, table_stride %d, n_pages %d)\n",
                     heads, kv_heads, head_dim, page_size, n_splits, qkv_stride, table_stride, n_pages);
        return 2;
    }
    const long long need = (long long)n_splits * n_seqs * heads * (head_dim + 2);
    if (need > (long long)VTB_NOALLOC_SCRATCH_FLOATS) {
        std::fprintf(stderr, "vtb_decode_attention_noalloc: %lld floats of scratch needed (n_splits %d x n_seqs %d x "
                             "heads %d x (head_dim %d + 2)), the fixed array holds %d\n",
                     need, n_splits, n_seqs, heads, head_dim, VTB_NOALLOC_SCRATCH_FLOATS);
        return 1;
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        std::fprintf(stderr, "vtb_decode_attention_noalloc: cudaGetDevice: %s\n", cudaGetErrorString(e));
        return 3;
    }
    float* part_o = g_scratch[device].load(std::memory_order_acquire);
    if (part_o == nullptr) {
        // first call on this device (it is the current one): the array's address on this device
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, vtb_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            std::fprintf(stderr, "vtb_decode_attention_noalloc: cudaGetSymbolAddress: %s\n", cudaGetErrorString(e));
            return 3;
        }
        g_scratch[device].store(ptr, std::memory_order_release);
        part_o = ptr;
    }
    float* part_ml = part_o + (size_t)n_splits * n_seqs * heads * head_dim;
    e = vtb::launch_attention_mma(qkv, qkv_stride, out, k_cache, v_cache, cu_q, q_start, block_table, table_stride,
                                  /*tiles=*/nullptr, /*n_tiles=*/n_seqs, n_pages, /*n_tokens=*/n_seqs, heads, kv_heads,
                                  head_dim, page_size, window, scale, /*warps=*/1, n_splits, part_o, part_ml,
                                  /*status=*/nullptr, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        std::fprintf(stderr, "vtb_decode_attention_noalloc: launch: %s\n", cudaGetErrorString(e));
        return 3;
    }
    return 0;
}
