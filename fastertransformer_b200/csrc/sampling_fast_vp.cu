// Single-pass kernel of the vocabulary-parallel local pass (top-k rows hand their candidates to the exchange
// record instead of drawing), half and bfloat16 logits.
#include "fast_sampling.cuh"

namespace ftb200 {
template int fast_sampling_occupancy<FTB200_F16, false, 1>(size_t, int*);
template int fast_sampling_occupancy<FTB200_BF16, false, 1>(size_t, int*);
template int fast_sampling_launch<FTB200_F16, false, 1>(const KParams&, int, size_t, cudaStream_t);
template int fast_sampling_launch<FTB200_BF16, false, 1>(const KParams&, int, size_t, cudaStream_t);
}  // namespace ftb200
