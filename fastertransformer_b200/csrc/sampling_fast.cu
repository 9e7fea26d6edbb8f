// Single-pass decode-sampling kernel, half and bfloat16 logits.
#include "fast_sampling.cuh"

namespace ftb200 {
size_t fast_smem_for(int hash_slots, int vocab_padded)
{
    return fast_smem_bytes(hash_slots, vocab_padded);
}
template int fast_sampling_occupancy<FTB200_F16>(size_t, int*);
template int fast_sampling_occupancy<FTB200_BF16>(size_t, int*);
template int fast_sampling_launch<FTB200_F16>(const KParams&, int, size_t, cudaStream_t);
template int fast_sampling_launch<FTB200_BF16>(const KParams&, int, size_t, cudaStream_t);
}  // namespace ftb200
