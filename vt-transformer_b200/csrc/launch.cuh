// Launch helper: cudaLaunchKernelEx with programmatic stream serialization (the kernel may start
// before the one in front of it has ended; it waits at its `pdl_wait`), and a cluster shape if asked.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

namespace vtb {

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = std::getenv("VTB200_PDL");   // VTB200_PDL=0 switches the overlap off (for measurements)
        on = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// A kernel's limit of dynamic shared memory is an attribute of the kernel on one device.  `done` is the caller's
// static flag word, one bit a device: the attribute is set at the kernel's first launch on each device.  Setting it
// twice is harmless, so two host threads that both find the bit clear may both set it.
template <typename K>
cudaError_t allow_dynamic_smem(K kernel, int bytes, std::atomic<unsigned long long>& done) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = 1ull << (device & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done.fetch_or(bit, std::memory_order_release);
    return cudaSuccess;
}

template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                   Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return launch(kernel, grid, block, smem, stream, dim3(1, 1, 1), args...);
}

}  // namespace vtb
