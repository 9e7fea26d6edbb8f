// Bad-word ban (stand-alone form), stop-word criterion, length criterion and finished count.
#include <chrono>
#include <thread>

#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

// A word list is [2, L]: row 0 the concatenated token ids, row 1 the exclusive end offset of each word,
// padded with -1.  Returns true when word `i` matches the tail of the sequence ending at position
// `last` (inclusive) of column `col`, following parent_ids for beams.
// kernels/ban_bad_words.cu:49-75 (n_match = size-1, last = step-1) and
// kernels/stop_criteria_kernels.cu:53-75 (n_match = size, last = step).
__device__ __forceinline__ bool tail_matches(const int* ids, const int* parents, const int* words, int item_start,
                                             int n_match, int first_pos, size_t row_stride, size_t col_base,
                                             int beam_idx, int beam_width)
{
    int parent = beam_idx;
    for (int t = n_match - 1; t >= 0; --t) {
        const size_t at = (size_t)(first_pos + t) * row_stride + col_base + parent;
        if (ids[at] != words[item_start + t]) {
            return false;
        }
        if (beam_width > 1) {
            parent = parents[at];
            if (parent < 0 || parent >= beam_width) {
                return false;
            }
        }
    }
    return true;
}

template<typename T>
__global__ void ban_bad_words_kernel(T* logits, const int* output_ids, const int* parent_ids, int batch_size,
                                     int beam_width, const int* bad_words, int L, int share_words, int id_offset,
                                     int vocab_padded, int step)
{
    const int id        = blockIdx.x * blockDim.x + threadIdx.x;
    const int batch_idx = blockIdx.y / beam_width;
    const int beam_idx  = blockIdx.y % beam_width;
    const int* base     = share_words ? bad_words : bad_words + (size_t)batch_idx * 2 * L;
    const int* offs     = base + L;
    if (id >= L || offs[id] < 0) {
        return;
    }
    const int item_end = offs[id], item_start = id > 0 ? offs[id - 1] : 0, item_size = item_end - item_start;
    bool      ban = item_size == 1;
    if (item_size > 1 && step >= item_size - 1) {
        ban = tail_matches(output_ids, parent_ids, base, item_start, item_size - 1, step - (item_size - 1),
                           (size_t)batch_size * beam_width, (size_t)id_offset + (size_t)batch_idx * beam_width,
                           beam_idx, beam_width);
    }
    if (ban) {
        const int tok = base[item_end - 1];
        if (0 < tok && tok < vocab_padded) {
            logits[((size_t)batch_idx * beam_width + beam_idx) * vocab_padded + tok] = static_cast<T>(-INFINITY);
        }
    }
}

// One CTA: stop words for the local rows, then the length limit and the finished count for the batch.
__global__ void stop_criteria_kernel(const int* output_ids, const int* parent_ids, const int* stop_words, int L,
                                     uint8_t* finished, const uint32_t* limit, int id_offset, int local_batch,
                                     int batch_size, int beam_width, int step, int* count_out, int* count_host)
{
    __shared__ int s_count;
    if (threadIdx.x == 0) {
        s_count = 0;
    }
    if (stop_words != nullptr) {
        const int total = local_batch * beam_width * L;
        for (int w = threadIdx.x; w < total; w += blockDim.x) {
            const int id = w % L, bb = w / L;
            const int batch_idx = bb / beam_width, beam_idx = bb % beam_width;
            const int* base = stop_words + (size_t)batch_idx * 2 * L;
            const int* offs = base + L;
            if (offs[id] < 0) {
                continue;
            }
            const int item_end = offs[id], item_start = id > 0 ? offs[id - 1] : 0, item_size = item_end - item_start;
            if (step + 1 >= item_size
                && tail_matches(output_ids, parent_ids, base, item_start, item_size, step - (item_size - 1),
                                (size_t)batch_size * beam_width, (size_t)id_offset + (size_t)batch_idx * beam_width,
                                beam_idx, beam_width)) {
                finished[(size_t)id_offset + bb] = 1;
            }
        }
    }
    __syncthreads();
    if (limit != nullptr) {
        int mine = 0;
        for (int i = threadIdx.x; i < batch_size * beam_width; i += blockDim.x) {
            uint8_t f = finished[i] | ((uint32_t)step >= limit[i / beam_width] ? 1 : 0);
            finished[i] = f;
            mine += f ? 1 : 0;
        }
        for (int m = 16; m > 0; m >>= 1) {
            mine += __shfl_xor_sync(0xffffffffu, mine, m);
        }
        if ((threadIdx.x & 31) == 0 && mine) {
            atomicAdd(&s_count, mine);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            *count_out = s_count;
            if (count_host != nullptr) {
                *count_host = s_count;  // pinned host memory, written from here: no copy has to follow the kernel
            }
        }
    }
}

}  // namespace ftb200

using namespace ftb200;

extern "C" int ftb200_ban_bad_words(void* logits, int dtype, const int* output_ids, const int* parent_ids,
                                    int batch_size, int local_batch_size, int beam_width, const int* bad_words,
                                    int share_words, int bad_words_len, int id_offset, int vocab_size_padded, int step,
                                    void* stream)
{
    if (logits == nullptr || output_ids == nullptr || bad_words == nullptr || bad_words_len <= 0
        || (beam_width > 1 && parent_ids == nullptr) || dtype < 0 || dtype > 2) {
        set_error("ftb200_ban_bad_words: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (local_batch_size * beam_width == 0) {
        return FTB200_OK;
    }
    dim3 block(((bad_words_len + 31) / 32) * 32 < 256 ? ((bad_words_len + 31) / 32) * 32 : 256);
    dim3 grid((bad_words_len + block.x - 1) / block.x, local_batch_size * beam_width);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FTB200_F32) {
        ban_bad_words_kernel<<<grid, block, 0, st>>>((float*)logits, output_ids, parent_ids, batch_size, beam_width,
                                                     bad_words, bad_words_len, share_words, id_offset,
                                                     vocab_size_padded, step);
    }
    else if (dtype == FTB200_F16) {
        ban_bad_words_kernel<<<grid, block, 0, st>>>((__half*)logits, output_ids, parent_ids, batch_size, beam_width,
                                                     bad_words, bad_words_len, share_words, id_offset,
                                                     vocab_size_padded, step);
    }
    else {
        ban_bad_words_kernel<<<grid, block, 0, st>>>((__nv_bfloat16*)logits, output_ids, parent_ids, batch_size,
                                                     beam_width, bad_words, bad_words_len, share_words, id_offset,
                                                     vocab_size_padded, step);
    }
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}

extern "C" int ftb200_stop_criteria(const int* output_ids, const int* parent_ids, const int* stop_words,
                                    int stop_words_len, uint8_t* finished, const uint32_t* sequence_limit_length,
                                    int id_offset, int local_batch_size, int batch_size, int beam_width, int step,
                                    int* finished_count_dev, int* finished_count_host, void* stream)
{
    if (finished == nullptr || output_ids == nullptr || batch_size <= 0 || beam_width <= 0
        || (stop_words != nullptr && beam_width > 1 && parent_ids == nullptr)
        || (sequence_limit_length != nullptr && (finished_count_dev == nullptr || finished_count_host == nullptr))) {
        set_error("ftb200_stop_criteria: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (stop_words == nullptr && sequence_limit_length == nullptr) {
        return FTB200_OK;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // Where the host word is page-locked memory the kernel can reach (cudaHostAlloc / cudaMallocHost / a registered
    // range), the kernel stores the count there itself; otherwise a copy follows it.  Asked on every call: the
    // same address may be pageable memory the next time.
    int* direct = nullptr;
    if (sequence_limit_length != nullptr) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, finished_count_host) == cudaSuccess && attr.type == cudaMemoryTypeHost
            && attr.devicePointer != nullptr) {
            direct = (int*)attr.devicePointer;
        }
        (void)cudaGetLastError();  // (an unregistered pointer is reported as an error by older drivers)
    }
    stop_criteria_kernel<<<1, 1024, 0, st>>>(output_ids, parent_ids, stop_words_len > 0 ? stop_words : nullptr,
                                             stop_words_len, finished, sequence_limit_length, id_offset,
                                             local_batch_size, batch_size, beam_width, step, finished_count_dev, direct);
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    if (sequence_limit_length != nullptr && direct == nullptr) {
        FTB_CUDA_CHECK(cudaMemcpyAsync(finished_count_host, finished_count_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
    }
    return FTB200_OK;
}

extern "C" int ftb200_wait_should_stop(const int* finished_count_host, int batch_size, int beam_width, void* stream,
                                       int timeout_ms, int* should_stop)
{
    if (finished_count_host == nullptr || should_stop == nullptr) {
        set_error("ftb200_wait_should_stop: invalid argument");
        return FTB200_INVALID_ARG;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const auto   t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaStreamQuery(st);
        if (e == cudaSuccess) {
            break;
        }
        if (e != cudaErrorNotReady) {
            set_error(std::string("ftb200_wait_should_stop: ") + cudaGetErrorString(e));
            return FTB200_CUDA_ERROR;
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0);
        if (timeout_ms >= 0 && ms.count() > timeout_ms) {
            set_error("ftb200_wait_should_stop: the stream did not drain within the deadline");
            return FTB200_TIMEOUT;
        }
    }
    *should_stop = ((volatile const int*)finished_count_host)[0] == batch_size * beam_width ? 1 : 0;
    return FTB200_OK;
}
