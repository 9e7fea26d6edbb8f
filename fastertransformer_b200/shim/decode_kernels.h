// Free functions with FasterTransformer's names and signatures for the kernels either side of the decode
// step, implemented on the libftb200 C ABI (include/ftb200.h).  They replace, one for one:
//   invokeLogProbFromLogits<T>    kernels/logprob_kernels.h:23-35
//   invokeDecodingInitialize<T>   kernels/decoding_kernels.h:25-34
//   invokeGatherTree (3 forms)    kernels/decoding_kernels.h:102-147   (with struct gatherTreeParam)
//   invokeFinalize                kernels/decoding_kernels.h:155-168
//   invokeInsertUnfinishedPath    kernels/beam_search_topk_kernels.h:87-92 (with struct BeamHypotheses)
// A call the library refuses throws std::runtime_error with the "[FT][ERROR]" prefix.
//
// Inside a FasterTransformer checkout do not include the project's decoding_kernels.h, logprob_kernels.h or
// beam_search_topk_kernels.h next to this header: the structs below carry the same names and fields.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <type_traits>

#include "ftb200.h"

namespace fastertransformer {

namespace ftb200_detail {
inline void kernel_check(int status, const char* what)
{
    if (status != FTB200_OK) {
        throw std::runtime_error(std::string("[FT][ERROR] ") + what + ": " + ftb200_last_error_string());
    }
}
template<typename T>
constexpr int dtype_of()
{
    return std::is_same<T, float>::value ? FTB200_F32 : std::is_same<T, half>::value ? FTB200_F16 : FTB200_BF16;
}
}  // namespace ftb200_detail

template<typename T>
void invokeLogProbFromLogits(float* cum_log_probs, const T* logits, const int* input_ids, const int* input_lengths,
                             const size_t max_input_length, const size_t batch_size, const size_t vocab_size,
                             const size_t vocab_size_padded, void* workspace, const size_t workspace_size,
                             cudaStream_t stream, const bool batch_first = false)
{
    ftb200_detail::kernel_check(
        ftb200_log_prob_from_logits(cum_log_probs, logits, ftb200_detail::dtype_of<T>(), input_ids, input_lengths,
                                    max_input_length, batch_size, vocab_size, vocab_size_padded, workspace,
                                    workspace_size, stream, batch_first ? 1 : 0),
        "invokeLogProbFromLogits");
}

template<typename T>
void invokeDecodingInitialize(bool* finished, int* sequence_length, int* word_ids, T* cum_log_probs,
                              const int* sentence_ids, const int batch_size, const int beam_width,
                              const int max_input_length, cudaStream_t stream)
{
    ftb200_detail::kernel_check(
        ftb200_decoding_initialize(reinterpret_cast<uint8_t*>(finished), sequence_length, word_ids, cum_log_probs,
                                   ftb200_detail::dtype_of<T>(), sentence_ids, batch_size, beam_width,
                                   max_input_length, stream),
        "invokeDecodingInitialize");
}

struct gatherTreeParam {
    int*         beams                           = nullptr;
    int*         max_sequence_lengths            = nullptr;
    int          max_sequence_length_final_step  = 0;
    const int*   input_lengths                   = nullptr;
    int*         response_input_lengths          = nullptr;
    int          max_time                        = 0;
    int          batch_size                      = 0;
    int          beam_width                      = 0;
    const int*   step_ids                        = nullptr;
    const int*   parent_ids                      = nullptr;
    const int*   end_tokens                      = nullptr;
    int          max_input_length                = 0;
    const int*   prefix_soft_prompt_lengths      = nullptr;
    const int*   p_prompt_tuning_prompt_lengths  = nullptr;
    int          max_input_without_prompt_length = 0;
    int          max_prefix_soft_prompt_length   = 0;
    int*         output_ids                      = nullptr;
    cudaStream_t stream                          = nullptr;
};

inline void invokeGatherTree(gatherTreeParam param)
{
    ftb200_gather_tree_params p;
    p.beams                           = param.beams;
    p.max_sequence_lengths            = param.max_sequence_lengths;
    p.max_sequence_length_final_step  = param.max_sequence_length_final_step;
    p.input_lengths                   = param.input_lengths;
    p.response_input_lengths          = param.response_input_lengths;
    p.max_time                        = param.max_time;
    p.batch_size                      = param.batch_size;
    p.beam_width                      = param.beam_width;
    p.step_ids                        = param.step_ids;
    p.parent_ids                      = param.parent_ids;
    p.end_tokens                      = param.end_tokens;
    p.max_input_length                = param.max_input_length;
    p.prefix_soft_prompt_lengths      = param.prefix_soft_prompt_lengths;
    p.p_prompt_tuning_prompt_lengths  = param.p_prompt_tuning_prompt_lengths;
    p.max_input_without_prompt_length = param.max_input_without_prompt_length;
    p.max_prefix_soft_prompt_length   = param.max_prefix_soft_prompt_length;
    p.output_ids                      = param.output_ids;
    p.stream                          = param.stream;
    ftb200_detail::kernel_check(ftb200_gather_tree(&p), "invokeGatherTree");
}

inline void invokeGatherTree(int* beams, int* max_sequence_lengths, const int max_time, const int batch_size,
                             const int beam_width, const int* step_ids, const int* parent_ids, const int* end_tokens,
                             const int max_input_length, cudaStream_t stream)
{
    gatherTreeParam param;
    param.beams                = beams;
    param.max_sequence_lengths = max_sequence_lengths;
    param.max_time             = max_time;
    param.batch_size           = batch_size;
    param.beam_width           = beam_width;
    param.step_ids             = step_ids;
    param.parent_ids           = parent_ids;
    param.end_tokens           = end_tokens;
    param.max_input_length     = max_input_length;
    param.stream               = stream;
    invokeGatherTree(param);
}

inline void invokeGatherTree(int* beams, int* max_sequence_lengths, const int max_time, const int batch_size,
                             const int beam_width, const int* step_ids, const int* parent_ids, const int* end_tokens,
                             cudaStream_t stream)
{
    invokeGatherTree(beams, max_sequence_lengths, max_time, batch_size, beam_width, step_ids, parent_ids, end_tokens,
                     1, stream);
}

inline void invokeFinalize(int* output_ids, int* sequence_lengths, float* cum_log_probs, float* output_log_probs,
                           const int* topk_output_ids, const int* topk_sequence_lengths, const float* scores,
                           const float* topk_cum_log_probs, const float* topk_log_probs, const int* num_beams,
                           const int beam_width, const int max_seq_len, const int batch_size, cudaStream_t stream)
{
    ftb200_detail::kernel_check(ftb200_finalize(output_ids, sequence_lengths, cum_log_probs, output_log_probs,
                                                topk_output_ids, topk_sequence_lengths, scores, topk_cum_log_probs,
                                                topk_log_probs, num_beams, beam_width, max_seq_len, batch_size,
                                                stream),
                                "invokeFinalize");
}

struct BeamHypotheses {
    int*   output_ids_tgt       = nullptr;
    int*   sequence_lengths_tgt = nullptr;
    float* cum_log_probs        = nullptr;
    float* normed_scores        = nullptr;
    float* log_probs            = nullptr;
    float* min_normed_scores    = nullptr;
    int*   num_beams            = nullptr;
    bool*  is_done              = nullptr;

    const int*   output_ids_src       = nullptr;
    const int*   parent_ids_src       = nullptr;
    const int*   sequence_lengths_src = nullptr;
    const int*   end_ids              = nullptr;
    const float* log_probs_src        = nullptr;

    int   step             = 0;
    int   ite              = 0;
    int   batch_size       = 0;
    int   local_batch_size = 0;
    int   max_seq_len      = 0;
    float length_penalty   = 0.0f;

    bool early_stopping         = true;
    bool is_return_normed_score = true;
};

inline void invokeInsertUnfinishedPath(BeamHypotheses beam_hyps, const bool* finished, const float* cum_log_probs,
                                       const int batch_size, const int beam_width, cudaStream_t stream)
{
    ftb200_beam_hyps h;
    h.output_ids_tgt       = beam_hyps.output_ids_tgt;
    h.sequence_lengths_tgt = beam_hyps.sequence_lengths_tgt;
    h.cum_log_probs        = beam_hyps.cum_log_probs;
    h.normed_scores        = beam_hyps.normed_scores;
    h.log_probs            = beam_hyps.log_probs;
    h.min_normed_scores    = beam_hyps.min_normed_scores;
    h.num_beams            = beam_hyps.num_beams;
    h.is_done              = reinterpret_cast<uint8_t*>(beam_hyps.is_done);
    h.early_stopping       = beam_hyps.early_stopping ? 1 : 0;
    ftb200_detail::kernel_check(
        ftb200_insert_unfinished_path(&h, beam_hyps.output_ids_src, beam_hyps.parent_ids_src,
                                      beam_hyps.sequence_lengths_src, beam_hyps.log_probs_src, beam_hyps.max_seq_len,
                                      beam_hyps.length_penalty, reinterpret_cast<const uint8_t*>(finished),
                                      cum_log_probs, batch_size, beam_width, stream),
        "invokeInsertUnfinishedPath");
}

}  // namespace fastertransformer
