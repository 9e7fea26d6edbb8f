// Single-pass decode-sampling kernels (top-k rows, top-p rows), half and bfloat16 logits.
#include "fast_sampling.cuh"

namespace ftb200 {
size_t fast_smem_for(int hash_slots, int vocab_padded, bool topp)
{
    return fast_smem_bytes(hash_slots, vocab_padded, topp);
}
int fast_max_history()
{
    return kFMaxHistAll;
}
int fast_max_words()
{
    return kFMaxWords;
}
template int fast_sampling_occupancy<FTB200_F16, false>(size_t, int*);
template int fast_sampling_occupancy<FTB200_BF16, false>(size_t, int*);
template int fast_sampling_launch<FTB200_F16, false>(const KParams&, int, size_t, cudaStream_t);
template int fast_sampling_launch<FTB200_BF16, false>(const KParams&, int, size_t, cudaStream_t);
}  // namespace ftb200
