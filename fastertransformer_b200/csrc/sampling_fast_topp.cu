// Single-pass decode-sampling kernel for the rows of the top-p layer, half and bfloat16 logits (a translation unit
// of its own: the two kernels compile side by side).
#include "fast_sampling.cuh"

namespace ftb200 {
template int fast_sampling_occupancy<FTB200_F16, true>(size_t, int*);
template int fast_sampling_occupancy<FTB200_BF16, true>(size_t, int*);
template int fast_sampling_launch<FTB200_F16, true>(const KParams&, int, size_t, cudaStream_t);
template int fast_sampling_launch<FTB200_BF16, true>(const KParams&, int, size_t, cudaStream_t);
}  // namespace ftb200
