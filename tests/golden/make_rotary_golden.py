"""Makes tests/golden/rotary_table.npz from vt-transformer's own ``fill_rotary_cache``
(v1/tensortype/common.cpp:6-24), the one piece of its model code that compiles and runs on a
CPU.  Usage: python tests/golden/make_rotary_golden.py <path to the vt-transformer checkout>

The function is compiled as it stands (g++ needs ``-include cstdint`` for that file) into a
small program that prints the table for a few (length, dims, base); the numbers are stored
as float32.  tests/test_plain.py compares the plain implementation's table with them.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

CASES = [(40, 16, 10000.0), (24, 32, 1000000.0), (16, 48, 500000.0), (300, 128, 1000000.0)]

MAIN = r"""
#include <cstdio>
#include <vector>
namespace vt { template<typename T> void fill_rotary_cache(std::vector<T>&, int, int, float); }
int main(int argc, char** argv) {
    int len = atoi(argv[1]), dims = atoi(argv[2]); float base = atof(argv[3]);
    std::vector<float> d; vt::fill_rotary_cache<float>(d, len, dims, base);
    for (float v : d) printf("%.9g\n", v);
    return 0;
}
"""


def main():
    ref = sys.argv[1]
    tt = os.path.join(ref, "v1", "tensortype")
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "main.cpp"), "w") as f:
            f.write(MAIN)
        exe = os.path.join(tmp, "rot")
        subprocess.check_call(["g++", "-O0", "-std=c++17", "-include", "cstdint", "-include", "cstdlib", "-I", tt,
                               "-I", os.path.join(ref, "v1", "install", "include"),
                               os.path.join(tt, "common.cpp"), os.path.join(tmp, "main.cpp"), "-o", exe])
        out = {}
        for n, (length, dims, base) in enumerate(CASES):
            txt = subprocess.check_output([exe, str(length), str(dims), repr(base)]).decode()
            vals = np.array([float(x) for x in txt.split()], dtype=np.float32).reshape(length, dims, 2)
            out[f"case{n}"] = vals
            out[f"case{n}_args"] = np.array([length, dims, base], dtype=np.float64)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "rotary_table.npz"), **out)
    print("wrote rotary_table.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
