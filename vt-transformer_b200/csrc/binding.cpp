// Python bindings of the kernels: tensors in, checks of device, dtype, shape and layout,
// then the plain-pointer launchers of kernels.h on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels.h"

namespace {

using torch::Tensor;

int dtype_code(const Tensor& t, const char* name) {
    if (t.scalar_type() == torch::kFloat32) return vtb::kF32;
    if (t.scalar_type() == torch::kBFloat16) return vtb::kBF16;
    TORCH_CHECK(false, name, ": dtype must be float32 or bfloat16, found ", t.scalar_type());
}

void check_cuda(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, ": must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.is_contiguous(), name, ": must be contiguous");
}

void check_i32(const Tensor& t, const char* name) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == torch::kInt32, name, ": must be int32");
}

void check_f32(const Tensor& t, const char* name) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, ": must be float32");
}

void check_launch(cudaError_t e, const char* what) {
    TORCH_CHECK(e == cudaSuccess, what, ": launch failed: ", cudaGetErrorString(e));
}

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

int* status_ptr(const c10::optional<Tensor>& status) {
    if (!status.has_value()) return nullptr;
    check_i32(*status, "status");
    TORCH_CHECK(status->numel() >= 2, "status: needs two ints");
    return status->data_ptr<int>();
}

void embedding(const Tensor& table, const Tensor& ids, Tensor& out, c10::optional<Tensor> status, double scale) {
    check_cuda(table, "table"); check_i32(ids, "ids"); check_f32(out, "out");
    TORCH_CHECK(table.dim() == 2 && out.dim() == 2, "embedding: table and out must be 2-d");
    const int hidden = table.size(1);
    TORCH_CHECK(hidden % 8 == 0, "embedding: hidden size ", hidden, " must be a multiple of 8");
    TORCH_CHECK(out.size(1) == hidden && out.size(0) == ids.numel(), "embedding: out must be [tokens, hidden]");
    c10::cuda::CUDAGuard guard(table.device());
    check_launch(vtb::launch_embedding(dtype_code(table, "table"), table.data_ptr(), ids.data_ptr<int>(),
                                       out.data_ptr<float>(), ids.numel(), hidden, table.size(0), (float)scale,
                                       status_ptr(status), stream_of(table)), "embedding");
}

void logits_scale_cap(Tensor& logits, double scale, double cap) {
    check_f32(logits, "logits");
    TORCH_CHECK(logits.is_contiguous(), "logits_scale_cap: logits must be contiguous");
    TORCH_CHECK(cap >= 0.0, "logits_scale_cap: the cap must not be negative");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_logits_scale_cap(logits.data_ptr<float>(), logits.numel(), (float)scale, (float)cap,
                                              stream_of(logits)), "logits_scale_cap");
}

void rmsnorm(Tensor& x, c10::optional<Tensor> delta, const Tensor& weight, double eps, Tensor& out,
             c10::optional<Tensor> rows, c10::optional<Tensor> status) {
    check_f32(x, "x"); check_f32(weight, "weight"); check_cuda(out, "out");
    TORCH_CHECK(x.dim() == 2 && out.dim() == 2, "rmsnorm: x and out must be 2-d");
    const int hidden = x.size(1);
    TORCH_CHECK(hidden % 8 == 0, "rmsnorm: hidden size ", hidden, " must be a multiple of 8");
    TORCH_CHECK(weight.numel() == hidden && out.size(1) == hidden, "rmsnorm: weight and out must match hidden size");
    const int code = dtype_code(out, "out");
    const void* dp = nullptr;
    const float* pp = nullptr;
    int n_parts = 0;
    if (delta.has_value() && delta->dim() == 3) {
        // the unadded shares of a matrix product: [shares, tokens, hidden] in 32-bit
        check_f32(*delta, "delta");
        TORCH_CHECK(delta->size(1) == x.size(0) && delta->size(2) == hidden && delta->size(0) >= 1,
                    "rmsnorm: shares of a delta must be [shares, tokens, hidden]");
        pp = delta->data_ptr<float>();
        n_parts = delta->size(0);
    } else if (delta.has_value()) {
        check_cuda(*delta, "delta");
        TORCH_CHECK(delta->scalar_type() == out.scalar_type(), "rmsnorm: delta and out must have one dtype");
        TORCH_CHECK(delta->sizes() == x.sizes(), "rmsnorm: delta must have the shape of x");
        dp = delta->data_ptr();
    }
    const int* rp = nullptr;
    int n_rows = x.size(0);
    if (rows.has_value()) {
        check_i32(*rows, "rows");
        rp = rows->data_ptr<int>();
        n_rows = rows->numel();
    }
    TORCH_CHECK(out.size(0) == n_rows, "rmsnorm: out must have one row for each normed row");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_rmsnorm(code, x.data_ptr<float>(), dp, pp, n_parts, weight.data_ptr<float>(), (float)eps,
                                     out.data_ptr(), rp, n_rows, x.size(0), hidden, status_ptr(status),
                                     stream_of(x)), "rmsnorm");
}

void silu_mul(const Tensor& gu, Tensor& out, int64_t interleave) {
    check_cuda(gu, "gu"); check_cuda(out, "out");
    TORCH_CHECK(gu.dim() == 2 && out.dim() == 2 && gu.size(1) == 2 * out.size(1) && gu.size(0) == out.size(0),
                "silu_mul: gu must be [tokens, 2 * inter] and out [tokens, inter]");
    TORCH_CHECK(gu.scalar_type() == out.scalar_type(), "silu_mul: one dtype");
    TORCH_CHECK(out.size(1) % 8 == 0, "silu_mul: intermediate size ", out.size(1), " must be a multiple of 8");
    c10::cuda::CUDAGuard guard(gu.device());
    TORCH_CHECK(interleave == 0 || interleave == 8, "silu_mul: interleave must be 0 or 8");
    check_launch(vtb::launch_silu_mul(dtype_code(gu, "gu"), gu.data_ptr(), out.data_ptr(), gu.size(0), out.size(1),
                                      interleave, stream_of(gu)), "silu_mul");
}

void check_cache(const Tensor& k_cache, const Tensor& v_cache, const Tensor& ref, int kv_heads, int head_dim) {
    check_cuda(k_cache, "k_cache"); check_cuda(v_cache, "v_cache");
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.sizes() == v_cache.sizes(),
                "cache: k and v must be [pages, kv_heads, page_size, head_dim]");
    TORCH_CHECK(k_cache.size(1) == kv_heads && k_cache.size(3) == head_dim, "cache: kv_heads or head_dim differ");
    TORCH_CHECK(k_cache.scalar_type() == ref.scalar_type() && v_cache.scalar_type() == ref.scalar_type(),
                "cache: dtype differs from the activations'");
}

void rope_store(Tensor& qkv, const Tensor& positions, c10::optional<Tensor> cos_sin, Tensor& k_cache, Tensor& v_cache,
                const Tensor& token_seq, const Tensor& block_table, int64_t heads, int64_t kv_heads, int64_t head_dim,
                bool store, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_i32(positions, "positions"); check_i32(token_seq, "token_seq");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (heads + 2 * kv_heads) * head_dim,
                "rope_store: qkv must be [tokens, (heads + 2 kv_heads) * head_dim]");
    TORCH_CHECK(head_dim % 2 == 0, "rope_store: head_dim must be even");
    const int n = qkv.size(0);
    TORCH_CHECK(positions.numel() == n && token_seq.numel() == n, "rope_store: one position and sequence a token");
    TORCH_CHECK(block_table.dim() == 2, "rope_store: block_table must be [sequences, stride]");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    const float2* cs = nullptr;
    int max_pos = 0;
    if (cos_sin.has_value()) {
        check_f32(*cos_sin, "cos_sin");
        TORCH_CHECK(cos_sin->dim() == 3 && cos_sin->size(1) == head_dim / 2 && cos_sin->size(2) == 2,
                    "rope_store: cos_sin must be [positions, head_dim / 2, 2]");
        cs = reinterpret_cast<const float2*>(cos_sin->data_ptr<float>());
        max_pos = cos_sin->size(0);
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_rope_store(dtype_code(qkv, "qkv"), qkv.data_ptr(), positions.data_ptr<int>(), cs, max_pos,
                                        k_cache.data_ptr(), v_cache.data_ptr(), token_seq.data_ptr<int>(),
                                        block_table.data_ptr<int>(), block_table.size(1), block_table.size(0),
                                        k_cache.size(0), n, heads, kv_heads, head_dim, k_cache.size(2),
                                        cs != nullptr, store, status_ptr(status), stream_of(qkv)), "rope_store");
}

void gemm_simt(const Tensor& a, const Tensor& w, c10::optional<Tensor> bias, Tensor& c) {
    check_cuda(a, "a"); check_cuda(w, "w"); check_cuda(c, "c");
    TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && c.dim() == 2, "gemm_simt: 2-d tensors");
    TORCH_CHECK(a.scalar_type() == w.scalar_type(), "gemm_simt: a and w must have one dtype");
    const int in_code = dtype_code(a, "a"), out_code = dtype_code(c, "c");
    TORCH_CHECK(out_code == vtb::kF32 || out_code == in_code, "gemm_simt: out must be float32 or the dtype of a");
    const int m = a.size(0), k = a.size(1), n = w.size(0);
    TORCH_CHECK(w.size(1) == k && c.size(0) == m && c.size(1) == n, "gemm_simt: shapes [m,k] x [n,k] -> [m,n]");
    TORCH_CHECK(k % 8 == 0, "gemm_simt: inner size ", k, " must be a multiple of 8");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_simt: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(a.device());
    check_launch(vtb::launch_gemm_simt(in_code, out_code, a.data_ptr(), w.data_ptr(), bp, c.data_ptr(), m, n, k,
                                       stream_of(a)), "gemm_simt");
}

void gemm_skinny(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16,
                "gemm_skinny: x and w must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_skinny: 2-d tensors");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(w.size(1) == k && out.size(0) == m && out.size(1) == n, "gemm_skinny: shapes [m,k] x [n,k] -> [m,n]");
    TORCH_CHECK(m <= 64, "gemm_skinny: at most 64 rows, found ", m);
    TORCH_CHECK(k % 8 == 0, "gemm_skinny: inner size ", k, " must be a multiple of 8");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_skinny: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_skinny(dtype_code(out, "out"), x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k,
                                         stream_of(x)), "gemm_skinny");
}

// The hint of a product that runs next (kernels.h: NextProduct), from the arguments that carry it.
vtb::NextProduct next_product(const Tensor& like, const c10::optional<Tensor>& next_w, int64_t next_epilogue, int64_t next_bytes,
                              const char* who) {
    vtb::NextProduct next = {nullptr, 0, 0, 0, 0};
    if (next_w.has_value() && next_bytes > 0) {
        TORCH_CHECK(next_w->is_cuda() && next_w->scalar_type() == torch::kBFloat16 && next_w->dim() == 2 && next_w->is_contiguous() &&
                        next_w->device() == like.device() && next_epilogue >= 0 && next_epilogue <= 2,
                    who, ": next_w must be a contiguous bfloat16 matrix on the same device, next_epilogue 0, 1 or 2");
        next = {next_w->data_ptr(), (int)next_w->size(0), (int)next_w->size(1), (int)next_epilogue, (long long)next_bytes};
    }
    return next;
}

void gemm_tc(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out, c10::optional<Tensor> status,
             c10::optional<Tensor> scratch, c10::optional<Tensor> counters, int64_t epilogue, c10::optional<Tensor> next_w,
             int64_t next_epilogue, int64_t next_bytes) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16, "gemm_tc: x and w must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2, "gemm_tc: x and w must be 2-d");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(epilogue >= 0 && epilogue <= 2, "gemm_tc: epilogue must be 0 (bias), 1 (silu(gate) * up) or 2 (unadded shares)");
    if (epilogue == 2) {
        TORCH_CHECK(w.size(1) == k && out.dim() == 3 && out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
                        out.size(0) == vtb::gemm_tc_shares(m, n, k) && out.size(1) == m && out.size(2) == n,
                    "gemm_tc: the shares of k go to a float32 out [gemm_tc_shares(m, n, k), m, n]");
    } else {
        TORCH_CHECK(w.size(1) == k && out.dim() == 2 && out.size(0) == m && out.size(1) == (epilogue == 1 ? n / 2 : n),
                    "gemm_tc: shapes [m,k] x [n,k] -> [m,n] (or [m,n/2] with the silu epilogue)");
    }
    TORCH_CHECK(epilogue != 1 || (n % 16 == 0 && !bias.has_value() && out.scalar_type() == torch::kBFloat16),
                "gemm_tc: the silu epilogue takes n % 16 == 0, no bias and a bfloat16 out");
    TORCH_CHECK(k % 8 == 0, "gemm_tc: inner size ", k, " must be a multiple of 8 (TMA rows start on 16-byte boundaries)");
    TORCH_CHECK(((uintptr_t)x.data_ptr() & 15) == 0 && ((uintptr_t)w.data_ptr() & 15) == 0,
                "gemm_tc: x and w must start on 16-byte boundaries");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_tc: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    float* sp = nullptr;
    int* cp = nullptr;
    long long sn = 0;
    int cn = 0;
    if (scratch.has_value() && counters.has_value()) {
        check_f32(*scratch, "scratch"); check_i32(*counters, "counters");
        sp = scratch->data_ptr<float>();
        sn = scratch->numel();
        cp = counters->data_ptr<int>();
        cn = counters->numel();
    }
    const vtb::NextProduct next = next_product(x, next_w, next_epilogue, next_bytes, "gemm_tc");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_tc(dtype_code(out, "out"), x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k,
                                     (int)epilogue, sp, sn, cp, cn, status_ptr(status), stream_of(x),
                                     next.w != nullptr ? &next : nullptr), "gemm_tc");
}

void gemm_tc_pair(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out, int64_t epilogue, int64_t bn,
                  c10::optional<Tensor> status, c10::optional<Tensor> scratch, c10::optional<Tensor> counters) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "gemm_tc_pair: x, w and out must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_tc_pair: x, w and out must be 2-d");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(epilogue == 0 || epilogue == 1, "gemm_tc_pair: epilogue must be 0 (bias) or 1 (silu(gate) * up)");
    TORCH_CHECK(bn == 0 || bn == 256 || bn == 224 || bn == 192, "gemm_tc_pair: tiles of 256, 224 or 192 rows of w (0: chosen by the sizes)");
    TORCH_CHECK(w.size(1) == k && out.size(0) == m && out.size(1) == (epilogue == 1 ? n / 2 : n),
                "gemm_tc_pair: shapes [m,k] x [n,k] -> [m,n] (or [m,n/2] with the silu epilogue)");
    TORCH_CHECK(epilogue != 1 || (n % 16 == 0 && !bias.has_value()), "gemm_tc_pair: the silu epilogue takes n % 16 == 0 and no bias");
    TORCH_CHECK(k % 8 == 0, "gemm_tc_pair: inner size ", k, " must be a multiple of 8 (TMA rows start on 16-byte boundaries)");
    TORCH_CHECK(((uintptr_t)x.data_ptr() & 15) == 0 && ((uintptr_t)w.data_ptr() & 15) == 0,
                "gemm_tc_pair: x and w must start on 16-byte boundaries");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_tc_pair: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    // scratch and counters (zeroed once; the kernel leaves them zero): with them, k is cut over pairs where the tiles are few
    float* sp = nullptr;
    int* cp = nullptr;
    long long scratch_floats = 0;
    int n_counters = 0;
    if (scratch.has_value() && counters.has_value()) {
        check_f32(*scratch, "scratch");
        check_cuda(*counters, "counters");
        TORCH_CHECK(counters->scalar_type() == torch::kInt32 && counters->is_contiguous(), "gemm_tc_pair: counters must be contiguous int32");
        sp = scratch->data_ptr<float>();
        scratch_floats = scratch->numel();
        cp = counters->data_ptr<int>();
        n_counters = (int)counters->numel();
    }
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_tc_pair(x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k, (int)epilogue, (int)bn, sp,
                                          scratch_floats, cp, n_counters, status_ptr(status), stream_of(x)), "gemm_tc_pair");
}

bool attention_mma_supports(int64_t head_dim, int64_t heads, int64_t kv_heads, int64_t warps) {
    return vtb::attention_mma_supports(head_dim, heads, kv_heads, warps);
}

void attention_mma(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                   const Tensor& q_start, const Tensor& block_table, c10::optional<Tensor> tiles, int64_t heads,
                   int64_t kv_heads, int64_t head_dim, int64_t window, double scale, int64_t warps, int64_t n_splits,
                   c10::optional<Tensor> part_o, c10::optional<Tensor> part_ml, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_mma: bfloat16 only");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention_mma: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention_mma: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0, "attention_mma: heads must be a multiple of kv_heads");
    TORCH_CHECK(vtb::attention_mma_supports(head_dim, heads, kv_heads, warps),
                "attention_mma: head_dim ", head_dim, " with ", heads / kv_heads, " heads in a group and ", warps,
                " warps is not supported (head_dim a multiple of 16 up to 128, group <= 16 * warps)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_mma: page size must be a multiple of 16");
    const int n_seqs = cu_q.numel() - 1;
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_mma: one q_start and one block-table row for each sequence");
    const int* tp = nullptr;
    int n_tiles = n_seqs;
    if (tiles.has_value()) {
        check_i32(*tiles, "tiles");
        TORCH_CHECK(tiles->dim() == 2 && tiles->size(1) == 2, "attention_mma: tiles must be [n, 2]");
        tp = tiles->data_ptr<int>();
        n_tiles = tiles->size(0);
    }
    float *po = nullptr, *pm = nullptr;
    const int n_tokens = qkv.size(0);
    if (n_splits > 1) {
        TORCH_CHECK(part_o.has_value() && part_ml.has_value(), "attention_mma: splits need scratch tensors");
        check_f32(*part_o, "part_o"); check_f32(*part_ml, "part_ml");
        TORCH_CHECK(part_o->numel() >= n_splits * n_tokens * heads * head_dim &&
                        part_ml->numel() >= n_splits * n_tokens * heads * 2, "attention_mma: scratch too small");
        po = part_o->data_ptr<float>();
        pm = part_ml->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_mma(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                           v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                           block_table.data_ptr<int>(), block_table.size(1), tp, n_tiles,
                                           k_cache.size(0), n_tokens, heads, kv_heads, head_dim, k_cache.size(2), window,
                                           (float)scale, warps, n_splits, po, pm, status_ptr(status), stream_of(qkv)),
                 "attention_mma");
}

bool attention_tc_supports(int64_t head_dim, int64_t heads, int64_t kv_heads) {
    return vtb::attention_tc_supports(head_dim, heads, kv_heads);
}

void attention_tc(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                  const Tensor& q_start, const Tensor& block_table, const Tensor& tiles, int64_t heads, int64_t kv_heads,
                  int64_t head_dim, int64_t window, double scale, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table"); check_i32(tiles, "tiles");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_tc: bfloat16 only");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim && qkv.size(1) % 8 == 0 && qkv.is_contiguous(),
                "attention_tc: qkv must hold the queries first, rows a multiple of 16 bytes");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim && out.is_contiguous(),
                "attention_tc: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0 && vtb::attention_tc_supports(head_dim, heads, kv_heads),
                "attention_tc: head_dim ", head_dim, " with ", heads / std::max<int64_t>(kv_heads, 1),
                " heads in a group is not supported (head_dim 128, group <= 128)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_tc: page size must be a multiple of 16");
    TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous() &&
                    reinterpret_cast<uintptr_t>(k_cache.data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(v_cache.data_ptr()) % 16 == 0,
                "attention_tc: the caches must be dense and 16-byte aligned");
    const int n_seqs = cu_q.numel() - 1;
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_tc: one q_start and one block-table row for each sequence");
    TORCH_CHECK(tiles.dim() == 2 && tiles.size(1) == 2, "attention_tc: tiles must be [n, 2]");
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_tc(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                          block_table.data_ptr<int>(), block_table.size(1), tiles.data_ptr<int>(),
                                          tiles.size(0), k_cache.size(0), heads, kv_heads, head_dim, k_cache.size(2),
                                          window, (float)scale, status_ptr(status), stream_of(qkv)),
                 "attention_tc");
}

void attention_decode(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                      const Tensor& q_start, const Tensor& block_table, int64_t heads, int64_t kv_heads, int64_t head_dim,
                      int64_t window, double scale, int64_t n_splits, c10::optional<Tensor> part_o,
                      c10::optional<Tensor> part_ml, c10::optional<Tensor> counters, bool fuse_rope,
                      c10::optional<Tensor> cos_sin, bool store_kv, c10::optional<Tensor> status,
                      c10::optional<Tensor> qkv_shares, bool long_runs, int64_t run_blocks) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_decode: bfloat16 only");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention_decode: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention_decode: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0 && vtb::attention_mma_supports(head_dim, heads, kv_heads, 1),
                "attention_decode: head_dim ", head_dim, " with ", heads / std::max<int64_t>(kv_heads, 1),
                " heads in a group is not supported (head_dim a multiple of 16 up to 128, group <= 16)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_decode: page size must be a multiple of 16");
    const int n_seqs = cu_q.numel() - 1, n_tokens = qkv.size(0);
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_decode: one q_start and one block-table row for each sequence");
    float *po = nullptr, *pm = nullptr;
    int* pc = nullptr;
    if (n_splits > 8 || part_o.has_value()) {
        TORCH_CHECK(part_o.has_value() && part_ml.has_value() && counters.has_value(),
                    "attention_decode: more than 8 runs need scratch tensors and counters");
        check_f32(*part_o, "part_o"); check_f32(*part_ml, "part_ml"); check_i32(*counters, "counters");
        TORCH_CHECK(part_o->numel() >= n_splits * n_tokens * heads * head_dim &&
                        part_ml->numel() >= n_splits * n_tokens * heads * 2 && counters->numel() >= n_seqs * kv_heads,
                    "attention_decode: scratch too small");
        po = part_o->data_ptr<float>();
        pm = part_ml->data_ptr<float>();
        pc = counters->data_ptr<int>();
    }
    const float2* cs = nullptr;
    int max_pos = 0;
    if (cos_sin.has_value()) {
        check_f32(*cos_sin, "cos_sin");
        TORCH_CHECK(cos_sin->dim() == 3 && cos_sin->size(1) == head_dim / 2 && cos_sin->size(2) == 2,
                    "attention_decode: cos_sin must be [positions, head_dim / 2, 2]");
        cs = reinterpret_cast<const float2*>(cos_sin->data_ptr<float>());
        max_pos = cos_sin->size(0);
    }
    if (fuse_rope) {
        TORCH_CHECK(n_tokens == n_seqs, "attention_decode: the fused rotation takes one token a sequence");
        TORCH_CHECK(qkv.size(1) == (heads + 2 * kv_heads) * head_dim, "attention_decode: qkv must hold q, k and v");
    }
    const float* shp = nullptr;
    int n_shares = 0;
    if (qkv_shares.has_value()) {
        check_f32(*qkv_shares, "qkv_shares");
        TORCH_CHECK(fuse_rope && qkv_shares->dim() == 3 && qkv_shares->size(1) == n_tokens && qkv_shares->size(2) == qkv.size(1) &&
                        qkv_shares->is_contiguous() && qkv_shares->size(0) >= 1 && qkv.size(1) % 2 == 0,
                    "attention_decode: shares of qkv must be [shares, tokens, width of qkv] float, with the fused rotation");
        shp = qkv_shares->data_ptr<float>();
        n_shares = qkv_shares->size(0);
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_decode(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                              v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                              block_table.data_ptr<int>(), block_table.size(1), n_seqs, k_cache.size(0),
                                              n_tokens, heads, kv_heads, head_dim, k_cache.size(2), window, (float)scale,
                                              n_splits, po, pm, pc, fuse_rope ? 1 : 0, cs, max_pos, store_kv ? 1 : 0,
                                              shp, n_shares, long_runs ? 1 : 0, (int)run_blocks, status_ptr(status),
                                              stream_of(qkv)), "attention_decode");
}

void attention_simt(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache,
                    const Tensor& positions, const Tensor& token_seq, const Tensor& block_table, int64_t heads,
                    int64_t kv_heads, int64_t head_dim, int64_t window, double scale, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(positions, "positions");
    check_i32(token_seq, "token_seq"); check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(out.scalar_type() == qkv.scalar_type(), "attention: one dtype");
    TORCH_CHECK(head_dim <= 256, "attention: head_dim ", head_dim, " is above 256");
    TORCH_CHECK(heads % kv_heads == 0, "attention: heads must be a multiple of kv_heads");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    const int n = qkv.size(0);
    TORCH_CHECK(positions.numel() == n && token_seq.numel() == n, "attention: one position and sequence a token");
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_simt(dtype_code(qkv, "qkv"), qkv.data_ptr(), qkv.size(1), out.data_ptr(),
                                            k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr<int>(),
                                            token_seq.data_ptr<int>(), block_table.data_ptr<int>(),
                                            block_table.size(1), block_table.size(0), k_cache.size(0), n, heads,
                                            kv_heads, head_dim, k_cache.size(2), window, (float)scale,
                                            status_ptr(status), stream_of(qkv)), "attention_simt");
}

void argmax(const Tensor& logits, Tensor& out) {
    check_f32(logits, "logits"); check_i32(out, "out");
    TORCH_CHECK(logits.dim() == 2 && out.numel() == logits.size(0), "argmax: logits [rows, vocab], out [rows]");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_argmax(logits.data_ptr<float>(), out.data_ptr<int>(), logits.size(0), logits.size(1),
                                    stream_of(logits)), "argmax");
}

void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p, const Tensor& u,
            Tensor& out) {
    check_f32(logits, "logits"); check_f32(temperature, "temperature"); check_i32(top_k, "top_k");
    check_f32(top_p, "top_p"); check_f32(u, "u"); check_i32(out, "out");
    const int rows = logits.size(0);
    TORCH_CHECK(logits.dim() == 2 && temperature.numel() == rows && top_k.numel() == rows && top_p.numel() == rows &&
                    u.numel() == rows && out.numel() == rows,
                "sample: one parameter of each kind for each row of logits");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_sample(logits.data_ptr<float>(), temperature.data_ptr<float>(), top_k.data_ptr<int>(),
                                    top_p.data_ptr<float>(), u.data_ptr<float>(), out.data_ptr<int>(), rows,
                                    logits.size(1), stream_of(logits)), "sample");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    namespace py = pybind11;
    m.def("embedding", &embedding, py::arg("table"), py::arg("ids"), py::arg("out"), py::arg("status") = py::none(),
          py::arg("scale") = 1.0);
    m.def("logits_scale_cap", &logits_scale_cap, py::arg("logits"), py::arg("scale"), py::arg("cap"));
    m.def("rmsnorm", &rmsnorm, py::arg("x"), py::arg("delta"), py::arg("weight"), py::arg("eps"), py::arg("out"),
          py::arg("rows") = py::none(), py::arg("status") = py::none());
    m.def("silu_mul", &silu_mul, py::arg("gu"), py::arg("out"), py::arg("interleave") = 0);
    m.def("rope_store", &rope_store, py::arg("qkv"), py::arg("positions"), py::arg("cos_sin"), py::arg("k_cache"),
          py::arg("v_cache"), py::arg("token_seq"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("store"), py::arg("status") = py::none());
    m.def("gemm_simt", &gemm_simt, py::arg("a"), py::arg("w"), py::arg("bias"), py::arg("c"));
    m.def("attention_simt", &attention_simt, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("positions"), py::arg("token_seq"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("status") = py::none());
    m.def("gemm_skinny", &gemm_skinny, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"));
    m.def("gemm_tc", &gemm_tc, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"), py::arg("status") = py::none(),
          py::arg("scratch") = py::none(), py::arg("counters") = py::none(), py::arg("epilogue") = 0,
          py::arg("next_w") = py::none(), py::arg("next_epilogue") = 0, py::arg("next_bytes") = 0);
    m.def("gemm_tc_pair", &gemm_tc_pair, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"), py::arg("epilogue") = 0,
          py::arg("bn") = 256, py::arg("status") = py::none(), py::arg("scratch") = py::none(), py::arg("counters") = py::none());
    m.def("gemm_tc_shares", [](int64_t m, int64_t n, int64_t k) { return (int64_t)vtb::gemm_tc_shares(m, n, k); });
    m.def("attention_mma_supports", &attention_mma_supports);
    m.def("attention_mma", &attention_mma, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("tiles"), py::arg("heads"),
          py::arg("kv_heads"), py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("warps"),
          py::arg("n_splits"), py::arg("part_o") = py::none(), py::arg("part_ml") = py::none(),
          py::arg("status") = py::none());
    m.def("attention_tc_supports", &attention_tc_supports);
    m.def("attention_tc", &attention_tc, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("tiles"), py::arg("heads"),
          py::arg("kv_heads"), py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("status") = py::none());
    m.def("attention_decode", &attention_decode, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("n_splits"), py::arg("part_o") = py::none(),
          py::arg("part_ml") = py::none(), py::arg("counters") = py::none(), py::arg("fuse_rope") = false,
          py::arg("cos_sin") = py::none(), py::arg("store_kv") = false, py::arg("status") = py::none(),
          py::arg("qkv_shares") = py::none(), py::arg("long_runs") = false, py::arg("run_blocks") = 0);
    m.def("argmax", &argmax, py::arg("logits"), py::arg("out"));
    m.def("sample", &sample, py::arg("logits"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"),
          py::arg("u"), py::arg("out"));
}
