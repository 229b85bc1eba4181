// Single-token attention at head sizes 64 and 128: the two sizes whose keys and values can also come as boxes of a
// tensor map, and so have twice the variants; a file of their own so that they compile beside the other sizes.
#include "attention_decode.cuh"

namespace vtb {

cudaError_t launch_decode_64_128(const AttnParams& p, int head_dim, int n_seqs, int* counters, cudaStream_t stream) {
    if (head_dim == 64) return launch_decode_d<64>(p, n_seqs, counters, stream);
    if (head_dim == 128) return launch_decode_d<128>(p, n_seqs, counters, stream);
    return cudaErrorInvalidValue;
}

}  // namespace vtb
