"""TEST INFRASTRUCTURE.  Compiles tests/cpp/kernels_driver.cc (the check of the C++ free functions in
fastertransformer_b200/shim/decode_kernels.h) against libftb200.so and the CPU restatement it compares them
with (oracle/libft_oracle.so).  The binary lands in tests/cpp/_build/ (git-ignored).

usage: python tests/cpp/build_kernels_driver.py
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "kernels_driver")


def build_kernels_driver():
    pkg = os.path.join(ROOT, "fastertransformer_b200")
    lib_dir, oracle_dir = os.path.join(pkg, "lib"), os.path.join(ROOT, "oracle")
    src = os.path.join(HERE, "kernels_driver.cc")
    deps = [src, os.path.join(pkg, "shim", "decode_kernels.h"), os.path.join(lib_dir, "libftb200.so"),
            os.path.join(oracle_dir, "libft_oracle.so")]
    for d in deps:
        if not os.path.exists(d):
            raise RuntimeError("missing %s: build the library and the restatement first" % d)
    if os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-x", "cu", src,
           "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(pkg, "shim"), "-L" + lib_dir, "-lftb200",
           "-L" + oracle_dir, "-lft_oracle",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../fastertransformer_b200/lib",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../oracle", "-o", OUT]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the kernels driver failed")
    return OUT


if __name__ == "__main__":
    print(build_kernels_driver())
