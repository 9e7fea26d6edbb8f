// Fused decode-sampling kernel, f16 logits.
#include "sampling_kernels.cuh"

namespace ftb200 {
template int sampling_occupancy<FTB200_F16>(size_t, int*);
template int sampling_launch<FTB200_F16>(const KParams&, int, size_t, cudaStream_t);
}  // namespace ftb200
