"""Build the sm_100a shared library of the decode-sampling kernels, in-tree.

`python -m fastertransformer_b200.build` compiles every .cu under csrc/ with nvcc for
compute_100a/sm_100a and links fastertransformer_b200/lib/libftb200.so.  Objects are rebuilt only
when a source or header is newer.  The flags mirror the reference's release build
(--use_fast_math, CMakeLists.txt:77 and :200-201 of FasterTransformer) because the kernels promise the
same approximate exp / log / divide instructions.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INC = os.path.join(os.path.dirname(HERE), "include")
OUT = os.path.join(HERE, "lib")
OBJ = os.path.join(OUT, "obj")
LIB = os.path.join(OUT, "libftb200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "--use_fast_math", "-lineinfo",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC", "-I" + INC, "-I" + CSRC,
]


def _newest_header():
    t = 0.0
    for d in (CSRC, INC):
        for root, _, files in os.walk(d):
            for f in files:
                if f.endswith((".h", ".cuh")):
                    t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return out


def _compile(src, obj, verbose):
    cmd = [NVCC] + FLAGS + ["-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(verbose=False, force=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr_t = _newest_header()
    jobs, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_").rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            for src, rc, log in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                if verbose or rc != 0:
                    sys.stderr.write(log)
                if rc != 0:
                    raise RuntimeError("nvcc failed on " + src)
    if jobs or not os.path.exists(LIB):
        r = subprocess.run([NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


def build_shim_driver():
    """Compile the C++ decode layers (shim/) with their test driver (tests/cpp/shim_driver.cc) against the
    library; the binary lands next to libftb200.so (same folder, found through its rpath)."""
    root = os.path.dirname(HERE)
    out = os.path.join(OUT, "shim_driver")
    srcs = [os.path.join(root, "tests", "cpp", "shim_driver.cc"), os.path.join(HERE, "shim", "DynamicDecodeLayer.cc")]
    deps = srcs + [os.path.join(HERE, "shim", "DynamicDecodeLayer.h"), os.path.join(HERE, "shim", "ft_compat.h"), LIB]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-x", "cu"] + srcs + [
        "-I" + INC, "-I" + os.path.join(HERE, "shim"), "-L" + OUT, "-lftb200", "-Xlinker", "-rpath", "-Xlinker",
        "$ORIGIN", "-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the shim driver failed")
    return out


def build_th_op():
    """Compile the torch custom class FasterTransformer.DynamicDecodeOp (th_op/DynamicDecodeOp.cc over the C++
    decode layers) into lib/libth_ftb200.so, next to libftb200.so which it links."""
    import torch
    from torch.utils import cpp_extension
    out = os.path.join(OUT, "libth_ftb200.so")
    srcs = [os.path.join(HERE, "th_op", "DynamicDecodeOp.cc"), os.path.join(HERE, "shim", "DynamicDecodeLayer.cc")]
    deps = srcs + [os.path.join(HERE, "shim", "DynamicDecodeLayer.h"), os.path.join(HERE, "shim", "ft_compat.h"), LIB]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cuda_home = os.path.dirname(os.path.dirname(NVCC))
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + srcs
    for inc in cpp_extension.include_paths() + [os.path.join(cuda_home, "include"), INC, os.path.join(HERE, "shim")]:
        cmd += ["-I" + inc]
    cmd += ["-L" + tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-L" + OUT, "-lftb200", "-L" + os.path.join(cuda_home, "lib64"), "-lcudart",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib, "-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("building the torch custom class failed")
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    print(build_shim_driver())
    print(build_th_op())
