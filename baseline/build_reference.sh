#!/bin/bash
# Builds the unmodified vt-transformer v1 engine for sm_100 and links baseline/ref_driver.cpp against it.
#
#   baseline/build_reference.sh [REFERENCE_CHECKOUT]      (default: $VT_REFERENCE_CHECKOUT, else where this build mounts it)
#
# The checkout's v1/ tree is copied to baseline/_ref/src (the checkout itself is read-only) and compiled with the
# flags of its own makefiles (v1/tensortype/Makefile.cuda, v1/tensortype/cuda_kernels/CMakeLists.txt and
# bitsandbytes/CMakeLists.txt), except: the target architecture is sm_100 instead of 60/70/80/90; `-include
# cstdint` is given on the command line because common.hpp:47 names std::uintptr_t without including it (gcc 13);
# the tokenizer library (Rust) is left out, since only chat.cpp's text handling needs it.  No source file of the
# reference is changed.  Output: baseline/_ref/ref_driver.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${VT_REFERENCE_CHECKOUT:-/root/reference}}"
OUT="$HERE/_ref"
CUDA="${CUDA_DIR:-/usr/local/cuda}"
CUDNN_INC="${CUDNN_INC:-/usr/include/x86_64-linux-gnu}"
CUDNN_LIB="${CUDNN_LIB:-/usr/lib/x86_64-linux-gnu}"
ARCH="-gencode arch=compute_100,code=sm_100"
mkdir -p "$OUT/obj"
rm -rf "$OUT/src"
cp -r "$REF/v1" "$OUT/src"
TT="$OUT/src/tensortype"
CK="$TT/cuda_kernels"
BNB="$CK/bitsandbytes"
pids=()
for f in lt_sgemm causal_mask convert layernorm rmsnorm rotary_embed transpose_0213 gelu silu_product easy_sampling; do
    "$CUDA/bin/nvcc" -std=c++17 -O3 $ARCH -I"$CUDNN_INC" -Xcompiler -fPIC -c "$CK/$f.cu" -o "$OUT/obj/ck_$f.o" & pids+=($!)
done
for f in ops kernels; do
    "$CUDA/bin/nvcc" -std=c++17 -O3 --use_fast_math -DBUILD_CUDA $ARCH -rdc=true -I"$BNB/csrc" -I"$BNB/include" \
        -Xcompiler -fPIC -c "$BNB/csrc/$f.cu" -o "$OUT/obj/bnb_$f.o" & pids+=($!)
done
for f in common cpu_ops bitsandbytes; do
    g++ -O3 -std=c++17 -DBUILD_CUDA -I"$BNB/csrc" -I"$BNB/include" -I"$CUDA/include" -fPIC -c "$BNB/csrc/$f.cpp" \
        -o "$OUT/obj/bnb_$f.o" & pids+=($!)
done
INC="-I$TT -I$OUT/src/install/include -I$OUT/src/models/qwen2-7b -I$CUDA/include -I$CUDNN_INC -I$CK -I$BNB/csrc"
FLAGS="-O3 -include cstdint -Wno-maybe-uninitialized -Wno-strict-aliasing -Wno-uninitialized -fopenmp -D_USING_DEVICE_CUDA_ -std=c++17"
for f in context common dag tensortype host_tensor cuda_tensor nn_operators nn_kvcache; do
    g++ $FLAGS $INC -c "$TT/$f.cpp" -o "$OUT/obj/tt_$f.o" & pids+=($!)
done
g++ $FLAGS $INC -c "$HERE/ref_driver.cpp" -o "$OUT/obj/ref_driver.o" & pids+=($!)
for p in "${pids[@]}"; do wait "$p"; done
"$CUDA/bin/nvcc" $ARCH -dlink "$OUT/obj/bnb_ops.o" "$OUT/obj/bnb_kernels.o" -o "$OUT/obj/bnb_dlink.o"
g++ -fopenmp -o "$OUT/ref_driver" "$OUT/obj/ref_driver.o" "$OUT"/obj/tt_*.o "$OUT"/obj/ck_*.o "$OUT"/obj/bnb_*.o \
    -L"$CUDA/lib64" -L"$CUDNN_LIB" -lcudnn -lcudart -lcublas -lcublasLt -lcusparse -lcudadevrt
echo "built: $OUT/ref_driver"
