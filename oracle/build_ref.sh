#!/usr/bin/env bash
# TEST INFRASTRUCTURE.  Compiles the reference's own decode-sampling sources,
# where they lie, into oracle/_ref/libft_decode_ref.so together with
# oracle/ref_harness.cu.  Only object files and the shared library land in
# oracle/_ref/ (git-ignored), plus one test file of the reference placed there
# unchanged (oracle/_ref/th_op/test_th_decode_op.py: the reference's own test
# of its torch op, which tests/test_th_decode_op_gpu.py runs as it stands
# against this package's torch class).  Nothing of the reference enters history.
#
# usage: oracle/build_ref.sh [REFERENCE_ROOT]      (default: $FT_REFERENCE_ROOT)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${FT_REFERENCE_ROOT:-}}"
if [ -z "$REF" ]; then
    echo "usage: oracle/build_ref.sh REFERENCE_ROOT   (or set FT_REFERENCE_ROOT to a FasterTransformer checkout)" >&2
    exit 2
fi
OUT="$HERE/_ref"
OBJ="$OUT/obj"
mkdir -p "$OBJ"

if [ ! -d "$REF/src/fastertransformer" ]; then
    echo "reference tree not found at $REF - keeping any prebuilt $OUT/libft_decode_ref.so" >&2
    exit 0
fi

NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
# The reference's release configuration: fast math on (CMakeLists.txt:77, :200-201), NDEBUG (CMAKE_BUILD_TYPE
# Release: asserts off, log level INFO, utils/logger.h:84-88), C++17, bf16 enabled.
FLAGS=(-gencode arch=compute_100a,code=sm_100a -std=c++17 -O3 --use_fast_math -DNDEBUG -DENABLE_BF16
       --expt-relaxed-constexpr --expt-extended-lambda -Xcompiler -fPIC -Xcompiler -w -w
       -I"$REF")

S="$REF/src/fastertransformer"
SRCS=(
    "$S/kernels/sampling_penalty_kernels.cu"
    "$S/kernels/sampling_topk_kernels.cu"
    "$S/kernels/sampling_topp_kernels.cu"
    "$S/kernels/ban_bad_words.cu"
    "$S/kernels/stop_criteria_kernels.cu"
    "$S/kernels/online_softmax_beamsearch_kernels.cu"
    "$S/kernels/beam_search_penalty_kernels.cu"
    "$S/kernels/beam_search_topk_kernels.cu"
    "$S/kernels/logprob_kernels.cu"
    "$S/kernels/decoding_kernels.cu"
    "$S/layers/DynamicDecodeLayer.cc"
    "$S/layers/sampling_layers/BaseSamplingLayer.cc"
    "$S/layers/sampling_layers/TopKSamplingLayer.cu"
    "$S/layers/sampling_layers/TopPSamplingLayer.cu"
    "$S/layers/beam_search_layers/BaseBeamSearchLayer.cu"
    "$S/layers/beam_search_layers/BeamSearchLayer.cu"
    "$S/layers/beam_search_layers/OnlineBeamSearchLayer.cu"
    "$S/utils/Tensor.cc"
    "$S/utils/cuda_utils.cc"
    "$S/utils/logger.cc"
    "$S/utils/memory_utils.cu"
    "$HERE/ref_harness.cu"
)

JOBS="${JOBS:-$(nproc)}"
pids=()
objs=()
for src in "${SRCS[@]}"; do
    base="$(basename "$src")"
    obj="$OBJ/${base%.*}.o"
    objs+=("$obj")
    if [ -f "$obj" ] && [ "$obj" -nt "$src" ]; then
        continue
    fi
    ( "$NVCC" "${FLAGS[@]}" -x cu -c "$src" -o "$obj" ) &
    pids+=($!)
    while [ "$(jobs -rp | wc -l)" -ge "$JOBS" ]; do sleep 0.5; done
done
for p in "${pids[@]:-}"; do
    [ -n "$p" ] && wait "$p"
done

"$NVCC" -shared -o "$OUT/libft_decode_ref.so" "${objs[@]}" -lcudart -lcurand -lcublas -lcublasLt
echo "built $OUT/libft_decode_ref.so"
mkdir -p "$OUT/th_op"
cp "$REF/tests/unittests/th_op/test_th_decode_op.py" "$OUT/th_op/test_th_decode_op.py"
echo "placed $OUT/th_op/test_th_decode_op.py"
