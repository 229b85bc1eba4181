"""Makes tests/golden/reference_kernels.npz from vt-transformer's own CUDA kernels, compiled unchanged for sm_100
and run once on a B200 on small seeded inputs (float instantiations):

    v1/tensortype/cuda_kernels/rmsnorm.cu        kr_rmsnorm<float>
    v1/tensortype/cuda_kernels/rotary_embed.cu   kr_rotary_embed<float>
    v1/tensortype/cuda_kernels/silu_product.cu   kr_silu_product<float>
    v1/tensortype/cuda_kernels/causal_mask.cu    kr_causal_mask<float>
    v1/tensortype/cuda_kernels/easy_sampling.cu  kr_sampling_top1<float>, kr_sampling_top3<float>

Usage (needs a CUDA device): python tests/golden/make_kernel_golden.py <path to the vt-transformer checkout>

The five files are given to nvcc as they are, with a few lines of extern "C" wrappers (below) that call their
launchers on the default stream.  Inputs and outputs are stored as they went in and came out.  tests/test_plain.py
compares the plain implementation's rms_norm, rotate, the activation of swiglu, the mask rule of attention and
the samplers with them: these are the formulas that otherwise rest on a reading of the source.
"""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

WRAP = r"""
#include "cuda_kernels.hpp"
using namespace vt::cuda;
extern "C" {
int g_rmsnorm(const float* x, const float* w, float* out, float* norm2, size_t batch, size_t dim, float eps) {
    int r = kr_rmsnorm<float>(x, w, out, norm2, batch, dim, eps, 0); cudaDeviceSynchronize(); return r; }
int g_rotary(const float* in, const float* cos_sin, const int* pos, float* out, size_t bs, size_t hnum, size_t len, size_t dims) {
    int r = kr_rotary_embed<float>(in, cos_sin, pos, out, bs, hnum, len, dims, 0); cudaDeviceSynchronize(); return r; }
int g_silu_product(const float* act, const float* in, float* out, size_t n) {
    int r = kr_silu_product<float>(act, in, out, n, 0); cudaDeviceSynchronize(); return r; }
int g_causal_mask(const int* mask, float* out, size_t batch, size_t new_tokens, size_t full_tokens) {
    int r = kr_causal_mask<float>(mask, out, batch, new_tokens, full_tokens, 0); cudaDeviceSynchronize(); return r; }
int g_top1(const float* logits, int* out, size_t batch, size_t vocab) {
    int r = kr_sampling_top1<float>(logits, out, batch, vocab, 0); cudaDeviceSynchronize(); return r; }
int g_top3(const float* logits, int* out, size_t batch, size_t vocab, float temperature, float randx) {
    int r = kr_sampling_top3<float>(logits, out, batch, vocab, temperature, randx, 0); cudaDeviceSynchronize(); return r; }
}
"""
FILES = ["rmsnorm.cu", "rotary_embed.cu", "silu_product.cu", "causal_mask.cu", "easy_sampling.cu"]


def main():
    import torch
    ref = sys.argv[1]
    # the checkout, or the folder baseline/build_reference.sh made, which holds the checkout's v1/ as src/
    v1 = os.path.join(ref, "v1") if os.path.isdir(os.path.join(ref, "v1")) else os.path.join(ref, "src")
    ck = os.path.join(v1, "tensortype", "cuda_kernels")
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "wrap.cu"), "w") as f:
            f.write(WRAP)
        lib_path = os.path.join(tmp, "libgolden.so")
        subprocess.check_call(["nvcc", "-std=c++17", "-O3", "-gencode", "arch=compute_100,code=sm_100", "-shared",
                               "-Xcompiler", "-fPIC", "-I", ck, "-I", "/usr/include/x86_64-linux-gnu",
                               os.path.join(tmp, "wrap.cu"), *[os.path.join(ck, f) for f in FILES], "-o", lib_path])
        lib = ctypes.CDLL(lib_path)
        dev = "cuda:0"
        g = torch.Generator().manual_seed(2024)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        Z = ctypes.c_size_t

        # RMS norm: dim must be a multiple of 256 (rmsnorm.cu:57-60)
        for n, (batch, dim, eps) in enumerate([(5, 512, 1e-6), (3, 768, 1e-5)]):
            x = (torch.randn(batch, dim, generator=g) * 1.7).to(dev)
            w = (1.0 + 0.1 * torch.randn(dim, generator=g)).to(dev)
            y, r = torch.empty_like(x), torch.empty(batch, device=dev)
            assert lib.g_rmsnorm(P(x), P(w), P(y), P(r), Z(batch), Z(dim), ctypes.c_float(eps)) == 0
            out.update({f"rms{n}_x": x, f"rms{n}_w": w, f"rms{n}_out": y, f"rms{n}_norm2": r, f"rms{n}_eps": torch.tensor(eps)})

        # rotation: in [bs, len, hnum, dims], the row of sequence b at index l has position pos[b] + l
        # (rotary_embed.cu:19-29); the table [positions, dims, (cos, sin)] is the one of fill_rotary_cache
        # (v1/tensortype/common.cpp:6-24), whose numbers tests/golden/rotary_table.npz holds
        table = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "rotary_table.npz"))["case1"]  # 24 x 32
        bs, length, hnum, dims = 2, 7, 3, 32
        cs = torch.from_numpy(table.copy()).to(dev)
        x = torch.randn(bs, length, hnum, dims, generator=g).to(dev)
        pos = torch.tensor([0, 11], dtype=torch.int32, device=dev)
        y = torch.empty_like(x)
        assert lib.g_rotary(P(x), P(cs), P(pos), P(y), Z(bs), Z(hnum), Z(length), Z(dims)) == 0
        out.update(rot_x=x, rot_table=cs, rot_pos=pos, rot_out=y)

        # silu(act) * in
        act = (torch.randn(1000, generator=g) * 4).to(dev)
        inp = torch.randn(1000, generator=g).to(dev)
        y = torch.empty_like(act)
        assert lib.g_silu_product(P(act), P(inp), P(y), Z(1000)) == 0
        out.update(silu_act=act, silu_in=inp, silu_out=y)

        # causal mask: 5 new tokens after 4 cached ones, two sequences, the second with a masked-out key
        batch, new, full = 2, 5, 9
        m = torch.ones(batch, full, dtype=torch.int32)
        m[1, 2] = 0
        m = m.to(dev)
        y = torch.empty(batch, new, full, device=dev)
        assert lib.g_causal_mask(P(m), P(y), Z(batch), Z(new), Z(full)) == 0
        out.update(mask_in=m, mask_out=y)

        # samplers
        logits = (torch.randn(6, 1537, generator=g) * 2).to(dev)
        ids = torch.empty(6, dtype=torch.int32, device=dev)
        assert lib.g_top1(P(logits), P(ids), Z(6), Z(1537)) == 0
        out.update(top_logits=logits, top1_ids=ids.clone())
        temp, draws = 2.5, [0.02, 0.2, 0.31, 0.5, 0.77, 0.999]
        picks = []
        for u in draws:
            assert lib.g_top3(P(logits), P(ids), Z(6), Z(1537), ctypes.c_float(temp), ctypes.c_float(u)) == 0
            picks.append(ids.clone())
        out.update(top3_temperature=torch.tensor(temp), top3_draws=torch.tensor(draws), top3_ids=torch.stack(picks))

    arrays = {k: v.detach().cpu().numpy() for k, v in out.items()}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")
    np.savez_compressed(path, **arrays)
    print("wrote", path, {k: v.shape for k, v in arrays.items()})
    if len(sys.argv) > 2:                                   # a second place for the file (a run on another machine)
        os.makedirs(sys.argv[2], exist_ok=True)
        np.savez_compressed(os.path.join(sys.argv[2], "reference_kernels.npz"), **arrays)


if __name__ == "__main__":
    main()
