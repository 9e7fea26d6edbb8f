// Caller-side steps either side of the per-step decode path: start-of-decoding state, back-tracking of beam
// parents into final sequences, ranking of archived hypotheses, and archiving of unfinished beams.
// Replaces invokeDecodingInitialize (kernels/decoding_kernels.cu:26-64), invokeGatherTree (:452-646),
// invokeFinalize (:698-804) and invokeInsertUnfinishedPath (kernels/beam_search_topk_kernels.cu:788-843).
//
// The reference walks every parent chain with one thread and dependent global loads (one thread per batch
// entry for the archive).  Here one CTA serves a batch entry: the whole CTA stages a tile of time levels of the
// id / parent tables in shared memory with coalesced loads, one thread per beam follows its chain through the
// tile in shared memory, and the CTA writes results back with coalesced stores.
#include <limits.h>

#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

namespace {

constexpr int kDkThreads = 256;
constexpr int kStage     = 2048;  // table entries (levels x beams) staged per tile
constexpr int kMaxBeams  = 1024;  // the reference's launch shapes stop here as well (:636-645, :787-789)
constexpr int kMaxArchiveBeams = 512;  // 2 * beam_width slots per entry have to fit a block there (:787-789)

template<typename T>
__device__ __forceinline__ T start_score_floor();
template<>
__device__ __forceinline__ float start_score_floor<float>()
{
    return -1e20f;
}
template<>
__device__ __forceinline__ __half start_score_floor<__half>()
{
    return __float2half(-65504.0f);
}
template<>
__device__ __forceinline__ __nv_bfloat16 start_score_floor<__nv_bfloat16>()
{
    return __float2bfloat16(-1e20f);
}

template<typename T>
__global__ void decoding_initialize_kernel(uint8_t* finished, int* sequence_length, int* word_ids, T* cum_log_probs,
                                           const int* sentence_ids, int n, int beam_width, int max_input_length)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += blockDim.x * gridDim.x) {
        finished[i]        = 0;
        sequence_length[i] = max_input_length;
        if (word_ids != nullptr) {
            word_ids[i] = sentence_ids[i / beam_width];
        }
        cum_log_probs[i] = (i % beam_width == 0) ? T(0.0f) : start_score_floor<T>();
    }
}

// ---- gather tree ------------------------------------------------------------------------------------------
struct GatherTree {
    int*       beams;
    int*       max_sequence_lengths;
    int        final_step;
    const int* input_lengths;
    int*       response_input_lengths;
    int        max_time, batch_size, beam_width;
    const int* step_ids;
    const int* parent_ids;
    const int* end_tokens;
    int        max_input_length;
    const int* prefix_lengths;
    const int* virtual_lengths;
    int        max_input_without_prompt_length, max_prefix_length;
    int*       output_ids;
};

__global__ void __launch_bounds__(kDkThreads) gather_tree_kernel(GatherTree p)
{
    __shared__ int     s_ids[kStage], s_par[kStage];
    __shared__ int     s_parent[kMaxBeams];
    __shared__ uint8_t s_bad[kMaxBeams];
    __shared__ int     s_maxlen;

    const int    b = blockIdx.x, K = p.beam_width, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const size_t BK = (size_t)p.batch_size * K, col0 = (size_t)b * K;
    const int    max_input_length = p.input_lengths == nullptr ? 0 : p.max_input_length;
    const int    prompt_len = p.prefix_lengths == nullptr ? 0 : p.prefix_lengths[b];
    const int    virt = p.virtual_lengths == nullptr ? 0 : p.virtual_lengths[b];
    const int    trimmed = p.max_prefix_length + (p.max_input_length - p.max_input_without_prompt_length);
    const int    end = p.end_tokens[b];
    auto         at = [&](int time, int beam) { return BK * (size_t)time + col0 + beam; };
    auto         in_len = [&](int beam) { return (p.input_lengths == nullptr ? 0 : p.input_lengths[col0 + beam]) - virt; };

    if (tid == 0) {
        s_maxlen = -1;
    }
    __syncthreads();
    // Every reference thread of a batch entry rewrites all of its lengths from the values it read; in lockstep
    // that is one update per entry, which is what is done here.
    for (int j = tid; j < K; j += kDkThreads) {
        const int tmp_len               = p.max_sequence_lengths[col0 + j] + p.final_step;
        p.max_sequence_lengths[col0 + j] = tmp_len - trimmed;
        if (p.response_input_lengths != nullptr) {
            p.response_input_lengths[col0 + j] = in_len(j) - prompt_len;
        }
        atomicMax(&s_maxlen, tmp_len);
    }
    __syncthreads();
    const int max_len = s_maxlen, top = min(p.max_time, max_len);
    if (top <= 0) {
        return;
    }

    // level top-1: the beam's own last token
    for (int beam = tid; beam < K; beam += kDkThreads) {
        const int shift = max_input_length - in_len(beam) + prompt_len;
        const int tgt   = top - 1 - shift;
        if (tgt >= 0) {  // the reference writes without this check
            p.beams[at(tgt, beam)] = p.step_ids[at(top - 1, beam)];
        }
        s_parent[beam] = p.parent_ids == nullptr ? 0 : p.parent_ids[at(top - 1, beam)] % K;
        s_bad[beam]    = 0;
    }
    // levels top-2 .. 0 in tiles of `tl` levels
    const int tl = kStage / K;
    for (int hi = top - 1; hi > 0; hi -= tl) {
        const int lo = max(0, hi - tl), n = (hi - lo) * K;
        __syncthreads();
        for (int e = tid; e < n; e += kDkThreads) {
            const size_t g = BK * (size_t)(lo + e / K) + col0 + e % K;
            s_ids[e]       = p.step_ids[g];
            s_par[e]       = p.parent_ids == nullptr ? 0 : p.parent_ids[g];
        }
        __syncthreads();
        for (int beam = tid; beam < K; beam += kDkThreads) {
            const int input_len = in_len(beam), shift = max_input_length - input_len + prompt_len;
            int       parent = s_parent[beam];
            bool      bad    = s_bad[beam];
            for (int level = hi - 1; level >= lo; --level) {
                if (level < prompt_len || (level >= input_len && level < max_input_length)) {
                    continue;
                }
                const int tgt = level >= max_input_length ? level - shift : level - prompt_len;
                if (parent < 0 || parent > K) {
                    p.beams[at(tgt, beam)] = end;
                    parent                 = -1;
                    bad                    = true;
                }
                else {
                    const int e            = (level - lo) * K + parent;
                    p.beams[at(tgt, beam)] = s_ids[e];
                    const int v            = s_par[e];  // in [0, K) on a well-formed tree: skip the division
                    parent                 = (unsigned)v < (unsigned)K ? v : v % K;
                }
            }
            s_parent[beam] = parent;
            s_bad[beam]    = bad;
        }
    }
    __syncthreads();

    // One warp per beam: end tokens after the sequence, nothing but end tokens after the first one, transposition.
    const int out_len = p.max_time - trimmed;
    for (int beam = wid; beam < K; beam += kDkThreads / 32) {
        const int shift = max_input_length - in_len(beam) + prompt_len;
        for (int t = max(0, max_len - shift) + lane; t < p.max_time - p.max_prefix_length; t += 32) {
            p.beams[at(t, beam)] = end;
        }
        __syncwarp();
        if (!s_bad[beam]) {
            int first = INT_MAX;
            for (int t = (max_input_length == 0 ? 1 : max_input_length) + lane; t < top; t += 32) {
                if (p.beams[at(t, beam)] == end) {
                    first = t;
                    break;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
            }
            if (first != INT_MAX) {
                for (int t = first + 1 + lane; t < top; t += 32) {
                    p.beams[at(t, beam)] = end;
                }
            }
        }
        __syncwarp();
        if (p.output_ids != nullptr) {
            int* out = p.output_ids + (col0 + beam) * (size_t)out_len;
            for (int j = lane; j < out_len; j += 32) {
                out[j] = p.beams[at(j, beam)];
            }
        }
    }
}

// ---- finalize ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kDkThreads) finalize_kernel(int* output_ids, int* sequence_lengths,
                                                              float* cum_log_probs, float* output_log_probs,
                                                              const int* topk_output_ids,
                                                              const int* topk_sequence_lengths, const float* scores,
                                                              const float* topk_cum_log_probs,
                                                              const float* topk_log_probs, const int* num_beams,
                                                              int K, int max_seq_len)
{
    __shared__ float s_score[2 * kMaxBeams];
    __shared__ int   s_rank[kMaxBeams];
    const int        b = blockIdx.x, tid = threadIdx.x, n = max(0, min(num_beams[b], 2 * K));
    for (int j = tid; j < n; j += kDkThreads) {
        s_score[j] = scores[(size_t)b * 2 * K + j];
    }
    // The reference picks the largest remaining score K times, the first index winning ties; once the n
    // archived entries are used up it finds entry 0 again.
    for (int i = tid; i < K; i += kDkThreads) {
        s_rank[i] = 0;
    }
    __syncthreads();
    for (int j = tid; j < n; j += kDkThreads) {
        const float s = s_score[j];
        int         r = 0;
        for (int l = 0; l < n; ++l) {
            const float o = s_score[l];
            r += (o > s) || (o == s && l < j);
        }
        if (r < K) {
            s_rank[r] = j;
        }
    }
    __syncthreads();
    for (int beam = tid; beam < K; beam += kDkThreads) {
        const size_t src = (size_t)b * 2 * K + s_rank[beam];
        sequence_lengths[(size_t)b * K + beam] = topk_sequence_lengths[src];
        if (cum_log_probs != nullptr) {
            cum_log_probs[(size_t)b * K + beam] = topk_cum_log_probs[src];
        }
    }
    for (int beam = 0; beam < K; ++beam) {
        const size_t src = ((size_t)b * 2 * K + s_rank[beam]) * (size_t)(max_seq_len + 1);
        const size_t dst = ((size_t)b * K + beam) * (size_t)max_seq_len;
        const int    len = topk_sequence_lengths[(size_t)b * 2 * K + s_rank[beam]];
        for (int i = tid; i < len; i += kDkThreads) {  // position 0 of the archive is the start token
            output_ids[dst + i] = topk_output_ids[src + i + 1];
            if (output_log_probs != nullptr) {
                output_log_probs[dst + i] = topk_log_probs[src + i + 1];
            }
        }
    }
}

// ---- archive of unfinished beams ----------------------------------------------------------------------------
struct InsertPath {
    int*         output_ids_tgt;
    int*         sequence_lengths_tgt;
    float*       cum_log_probs_tgt;
    float*       normed_scores;
    float*       log_probs_tgt;
    int*         num_beams;
    const uint8_t* is_done;
    const int*   output_ids_src;
    const int*   parent_ids_src;
    const int*   sequence_lengths_src;
    const float* log_probs_src;
    int          max_seq_len;
    float        length_penalty;
    const uint8_t* finished;
    const float* cum_log_probs;
    int          batch_size, beam_width;
};

__global__ void __launch_bounds__(kDkThreads) insert_unfinished_path_kernel(InsertPath p)
{
    __shared__ int   s_ids[kStage], s_par[kStage], s_out[kStage];
    __shared__ float s_lp[kStage], s_lpout[kStage];
    __shared__ int   s_prev[kMaxArchiveBeams], s_len[kMaxArchiveBeams];
    __shared__ int   s_top;

    const int b = blockIdx.x, K = p.beam_width, tid = threadIdx.x;
    if (p.is_done[b]) {
        return;
    }
    const size_t BK = (size_t)p.batch_size * K, col0 = (size_t)b * K;
    const int    first_slot = p.num_beams[b];
    const size_t row = (size_t)p.max_seq_len + 1;
    const bool   with_lp = p.log_probs_tgt != nullptr && p.log_probs_src != nullptr;
    if (tid == 0) {
        s_top = -1;
    }
    __syncthreads();
    for (int beam = tid; beam < K; beam += kDkThreads) {
        const int    len = p.sequence_lengths_src[col0 + beam];
        const size_t tgt = (size_t)b * 2 * K + beam + first_slot;
        const size_t g   = (size_t)len * BK + col0 + beam;
        s_len[beam]      = len;
        p.output_ids_tgt[tgt * row + len] = p.output_ids_src[g];
        if (with_lp) {
            p.log_probs_tgt[tgt * row + len] = p.log_probs_src[g];
        }
        s_prev[beam]                = p.parent_ids_src[g];
        p.sequence_lengths_tgt[tgt] = len;
        const float cum   = p.cum_log_probs[col0 + beam];
        const int   n_tok = p.finished[col0 + beam] ? len + 1 : len;
        p.normed_scores[tgt] =
            (p.length_penalty == 0.0f || n_tok == 1) ? cum : cum / powf((float)n_tok, p.length_penalty);
        p.cum_log_probs_tgt[tgt] = cum;
        atomicMax(&s_top, len);
    }
    __syncthreads();
    const int top = s_top, tl = kStage / K;
    for (int hi = top; hi > 0; hi -= tl) {  // levels hi-1 .. lo
        const int lo = max(0, hi - tl), n = (hi - lo) * K;
        __syncthreads();
        for (int e = tid; e < n; e += kDkThreads) {
            const size_t g = BK * (size_t)(lo + e / K) + col0 + e % K;
            s_ids[e]       = p.output_ids_src[g];
            s_par[e]       = p.parent_ids_src[g];
            if (with_lp) {
                s_lp[e] = p.log_probs_src[g];
            }
        }
        __syncthreads();
        for (int beam = tid; beam < K; beam += kDkThreads) {
            int prev = s_prev[beam];
            for (int level = min(hi, s_len[beam]) - 1; level >= lo; --level) {
                prev        = min(max(prev, 0), K - 1);  // the reference follows an out-of-range parent unchecked
                const int e = (level - lo) * K + prev, o = (level - lo) * K + beam;
                s_out[o]    = s_ids[e];
                if (with_lp) {
                    s_lpout[o] = s_lp[e];
                }
                prev = s_par[e];
            }
            s_prev[beam] = prev;
        }
        __syncthreads();
        // rows of the archive are contiguous in the level: flush level-major per beam
        const int levels = hi - lo;
        for (int e = tid; e < levels * K; e += kDkThreads) {
            const int beam = e / levels, level = lo + e % levels;
            if (level < s_len[beam]) {
                const size_t tgt = (size_t)b * 2 * K + beam + first_slot;
                const int    o   = (level - lo) * K + beam;
                p.output_ids_tgt[tgt * row + level] = s_out[o];
                if (with_lp) {
                    p.log_probs_tgt[tgt * row + level] = s_lpout[o];
                }
            }
        }
    }
    if (tid == 0) {
        p.num_beams[b] = first_slot + K;
    }
}

}  // namespace
}  // namespace ftb200

using namespace ftb200;

extern "C" int ftb200_decoding_initialize(uint8_t* finished, int* sequence_length, int* word_ids,
                                          void* cum_log_probs, int dtype, const int* sentence_ids, int batch_size,
                                          int beam_width, int max_input_length, void* stream)
{
    if (finished == nullptr || sequence_length == nullptr || cum_log_probs == nullptr || batch_size <= 0
        || beam_width <= 0 || (word_ids != nullptr && sentence_ids == nullptr)) {
        set_error("ftb200_decoding_initialize: invalid argument");
        return FTB200_INVALID_ARG;
    }
    const int    n = batch_size * beam_width, grid = (n + 255) / 256;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case FTB200_F32:
            decoding_initialize_kernel<float><<<grid, 256, 0, st>>>(finished, sequence_length, word_ids,
                                                                    (float*)cum_log_probs, sentence_ids, n,
                                                                    beam_width, max_input_length);
            break;
        case FTB200_F16:
            decoding_initialize_kernel<__half><<<grid, 256, 0, st>>>(finished, sequence_length, word_ids,
                                                                     (__half*)cum_log_probs, sentence_ids, n,
                                                                     beam_width, max_input_length);
            break;
        case FTB200_BF16:
            decoding_initialize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
                finished, sequence_length, word_ids, (__nv_bfloat16*)cum_log_probs, sentence_ids, n, beam_width,
                max_input_length);
            break;
        default:
            set_error("ftb200_decoding_initialize: unknown dtype");
            return FTB200_INVALID_ARG;
    }
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}

extern "C" int ftb200_gather_tree(const ftb200_gather_tree_params* a)
{
    if (a == nullptr || a->beams == nullptr || a->max_sequence_lengths == nullptr || a->step_ids == nullptr
        || a->end_tokens == nullptr || a->batch_size <= 0 || a->beam_width <= 0 || a->max_time < 0) {
        set_error("ftb200_gather_tree: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (a->beam_width > kMaxBeams) {
        set_error("ftb200_gather_tree: beam_width above 1024");
        return FTB200_UNSUPPORTED;
    }
    GatherTree p;
    p.beams                           = a->beams;
    p.max_sequence_lengths            = a->max_sequence_lengths;
    p.final_step                      = a->max_sequence_length_final_step;
    p.input_lengths                   = a->input_lengths;
    p.response_input_lengths          = a->response_input_lengths;
    p.max_time                        = a->max_time;
    p.batch_size                      = a->batch_size;
    p.beam_width                      = a->beam_width;
    p.step_ids                        = a->step_ids;
    p.parent_ids                      = a->parent_ids;
    p.end_tokens                      = a->end_tokens;
    p.max_input_length                = a->max_input_length;
    p.prefix_lengths                  = a->prefix_soft_prompt_lengths;
    p.virtual_lengths                 = a->p_prompt_tuning_prompt_lengths;
    p.max_input_without_prompt_length = a->max_input_without_prompt_length;
    p.max_prefix_length               = a->max_prefix_soft_prompt_length;
    p.output_ids                      = a->output_ids;
    gather_tree_kernel<<<a->batch_size, kDkThreads, 0, (cudaStream_t)a->stream>>>(p);
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}

extern "C" int ftb200_finalize(int* output_ids, int* sequence_lengths, float* cum_log_probs, float* output_log_probs,
                               const int* topk_output_ids, const int* topk_sequence_lengths, const float* scores,
                               const float* topk_cum_log_probs, const float* topk_log_probs, const int* num_beams,
                               int beam_width, int max_seq_len, int batch_size, void* stream)
{
    if (output_ids == nullptr || sequence_lengths == nullptr || topk_output_ids == nullptr
        || topk_sequence_lengths == nullptr || scores == nullptr || num_beams == nullptr || beam_width <= 0
        || batch_size <= 0 || max_seq_len < 0 || (cum_log_probs != nullptr && topk_cum_log_probs == nullptr)
        || (output_log_probs != nullptr && topk_log_probs == nullptr)) {
        set_error("ftb200_finalize: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if ((beam_width * 2 + 31) / 32 * 32 >= 1024) {  // FT_CHECK(block.x < 1024), decoding_kernels.cu:789
        set_error("ftb200_finalize: 2 * beam_width rounded up to a warp must stay below 1024");
        return FTB200_UNSUPPORTED;
    }
    finalize_kernel<<<batch_size, kDkThreads, 0, (cudaStream_t)stream>>>(
        output_ids, sequence_lengths, cum_log_probs, output_log_probs, topk_output_ids, topk_sequence_lengths, scores,
        topk_cum_log_probs, topk_log_probs, num_beams, beam_width, max_seq_len);
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}

extern "C" int ftb200_insert_unfinished_path(const ftb200_beam_hyps* hyps, const int* output_ids_src,
                                             const int* parent_ids_src, const int* sequence_lengths_src,
                                             const float* log_probs_src, int max_seq_len, float length_penalty,
                                             const uint8_t* finished, const float* cum_log_probs, int batch_size,
                                             int beam_width, void* stream)
{
    if (hyps == nullptr || hyps->output_ids_tgt == nullptr || hyps->sequence_lengths_tgt == nullptr
        || hyps->cum_log_probs == nullptr || hyps->normed_scores == nullptr || hyps->num_beams == nullptr
        || hyps->is_done == nullptr || output_ids_src == nullptr || parent_ids_src == nullptr
        || sequence_lengths_src == nullptr || finished == nullptr || cum_log_probs == nullptr || batch_size <= 0
        || beam_width <= 0 || max_seq_len < 0) {
        set_error("ftb200_insert_unfinished_path: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (beam_width > kMaxArchiveBeams) {
        set_error("ftb200_insert_unfinished_path: beam_width above 512");
        return FTB200_UNSUPPORTED;
    }
    InsertPath p;
    p.output_ids_tgt       = hyps->output_ids_tgt;
    p.sequence_lengths_tgt = hyps->sequence_lengths_tgt;
    p.cum_log_probs_tgt    = hyps->cum_log_probs;
    p.normed_scores        = hyps->normed_scores;
    p.log_probs_tgt        = hyps->log_probs;
    p.num_beams            = hyps->num_beams;
    p.is_done              = hyps->is_done;
    p.output_ids_src       = output_ids_src;
    p.parent_ids_src       = parent_ids_src;
    p.sequence_lengths_src = sequence_lengths_src;
    p.log_probs_src        = log_probs_src;
    p.max_seq_len          = max_seq_len;
    p.length_penalty       = length_penalty;
    p.finished             = finished;
    p.cum_log_probs        = cum_log_probs;
    p.batch_size           = batch_size;
    p.beam_width           = beam_width;
    insert_unfinished_path_kernel<<<batch_size, kDkThreads, 0, (cudaStream_t)stream>>>(p);
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}
