"""Compile-time checks of the C++ decode layers (fastertransformer_b200/shim), no GPU needed.

1. Inside a FasterTransformer checkout the classes are built against the project's own Tensor, TensorMap and
   IAllocator (-DFTB200_WITH_FT_HEADERS): the translation unit must compile with the checkout on the include path
   (skipped when $FT_REFERENCE_ROOT, or a sibling `reference` directory, holds no checkout).
2. BaseSamplingLayer<T> is abstract through its pure-virtual runSampling(), the two sampling layers derive from it
   and are concrete, and the constructors take the reference's argument lists
   (layers/sampling_layers/BaseSamplingLayer.h:62-77, TopKSamplingLayer.h:55-67, TopPSamplingLayer.h:64-77).
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "fastertransformer_b200", "shim")
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _reference_root():
    for cand in (os.environ.get("FT_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "src", "fastertransformer", "utils", "Tensor.h")):
            return cand
    return None


def _compile(src, out, extra):
    cmd = [NVCC, "-std=c++17", "-x", "cu", "-c", src, "-o", out, "-I" + os.path.join(ROOT, "include"), "-I" + SHIM,
           "-gencode", "arch=compute_100a,code=sm_100a"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]


@pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not found")
def test_shim_compiles_against_the_reference_headers(tmp_path):
    ref = _reference_root()
    if ref is None:
        pytest.skip("no FasterTransformer checkout: set FT_REFERENCE_ROOT")
    _compile(os.path.join(SHIM, "DynamicDecodeLayer.cc"), str(tmp_path / "shim_ft.o"),
             ["-DFTB200_WITH_FT_HEADERS", "-DENABLE_BF16", "-I" + ref])


TRAITS = r"""
#include <type_traits>
#include "DynamicDecodeLayer.h"
using namespace fastertransformer;
template<typename T>
struct Checks {
    using Base = BaseSamplingLayer<T>;
    static_assert(std::is_abstract<Base>::value, "runSampling() must be pure virtual");
    static_assert(std::has_virtual_destructor<Base>::value, "");
    static_assert(std::is_base_of<Base, TopKSamplingLayer<T>>::value, "");
    static_assert(std::is_base_of<Base, TopPSamplingLayer<T>>::value, "");
    static_assert(!std::is_abstract<TopKSamplingLayer<T>>::value && !std::is_abstract<TopPSamplingLayer<T>>::value, "");
    static_assert(std::is_constructible<TopKSamplingLayer<T>, size_t, size_t, size_t, int, size_t, unsigned long long, float,
                                        float, float, cudaStream_t, cublasMMWrapper*, IAllocator*, bool>::value, "");
    static_assert(std::is_constructible<TopPSamplingLayer<T>, size_t, size_t, size_t, int, float, unsigned long long, float,
                                        float, float, cudaStream_t, cublasMMWrapper*, IAllocator*, bool,
                                        cudaDeviceProp*>::value, "");
    static_assert(std::is_constructible<DynamicDecodeLayer<T>, size_t, size_t, int, cudaStream_t, cublasMMWrapper*,
                                        IAllocator*, bool, cudaDeviceProp*>::value, "");
    static_assert(std::is_copy_constructible<TopKSamplingLayer<T>>::value, "");
};
// a sampler of the caller's own: derives from the base with the reference's constructor list and supplies runSampling()
template<typename T>
struct OwnSampler: BaseSamplingLayer<T> {
    using BaseSamplingLayer<T>::BaseSamplingLayer;
    int calls = 0;
    void runSampling(TensorMap*, TensorMap*) override { ++calls; }
};
template struct Checks<float>;
template struct Checks<half>;
template struct Checks<__nv_bfloat16>;
template struct OwnSampler<float>;
"""


@pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not found")
def test_base_sampling_layer_is_abstract_and_derivable(tmp_path):
    src = tmp_path / "traits.cc"
    src.write_text(TRAITS)
    _compile(str(src), str(tmp_path / "traits.o"), [])
