// Fused decode-sampling kernel, f32 logits.
#include "sampling_kernels.cuh"

namespace ftb200 {
template int sampling_occupancy<FTB200_F32>(size_t, int*);
template int sampling_launch<FTB200_F32>(const KParams&, int, size_t, cudaStream_t);
template int vp_merge_launch<FTB200_F32>(const KParams&, const u64*, int, int*, int, cudaStream_t);
}  // namespace ftb200
