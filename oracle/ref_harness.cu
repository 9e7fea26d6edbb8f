/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * C-ABI harness around the UNMODIFIED reference implementation of the decode
 * sampling path (FasterTransformer's DynamicDecodeLayer<T> and the kernels it
 * launches).  The reference sources are compiled where they lie by
 * oracle/build_ref.sh and linked with this file into
 * oracle/_ref/libft_decode_ref.so.  Only tests, the smoke check and the
 * benchmark's reference arm load that library; the product never does.
 *
 * Everything here is glue: raw pointers in, the reference's own
 * TensorMap-keyed API called underneath (layers/DynamicDecodeLayer.h:58-75).
 */
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <string>

#include "src/fastertransformer/kernels/beam_search_topk_kernels.h"
#include "src/fastertransformer/kernels/decoding_kernels.h"
#include "src/fastertransformer/kernels/logprob_kernels.h"
#include "src/fastertransformer/kernels/sampling_topk_kernels.h"
#include "src/fastertransformer/layers/DynamicDecodeLayer.h"
#include "src/fastertransformer/utils/Tensor.h"
#include "src/fastertransformer/utils/allocator.h"

namespace ft = fastertransformer;

/* memory_utils.cu references the weight-only-quantisation pre-processor, whose
 * sources need the un-vendored CUTLASS submodule.  The decode sampling path
 * never calls it; give the linker an aborting stand-in. */
namespace fastertransformer {
enum class QuantType;
template<typename ComputeType, typename WeightType>
void symmetric_quantize(int8_t*, ComputeType*, const WeightType*, const std::vector<size_t>&, QuantType)
{
    fprintf(stderr, "[ref_harness] symmetric_quantize stub called\n");
    abort();
}
template void symmetric_quantize<half, float>(int8_t*, half*, const float*, const std::vector<size_t>&, QuantType);
template void symmetric_quantize<half, half>(int8_t*, half*, const half*, const std::vector<size_t>&, QuantType);
#ifdef ENABLE_BF16
template void
symmetric_quantize<__nv_bfloat16, float>(int8_t*, __nv_bfloat16*, const float*, const std::vector<size_t>&, QuantType);
template void symmetric_quantize<__nv_bfloat16, __nv_bfloat16>(
    int8_t*, __nv_bfloat16*, const __nv_bfloat16*, const std::vector<size_t>&, QuantType);
template void symmetric_quantize<__nv_bfloat16, half>(
    int8_t*, __nv_bfloat16*, const half*, const std::vector<size_t>&, QuantType);
template void symmetric_quantize<half, __nv_bfloat16>(
    int8_t*, half*, const __nv_bfloat16*, const std::vector<size_t>&, QuantType);
#endif
}  // namespace fastertransformer

extern "C" {

struct ftref_runtime_args {
    /* host arrays; n_* is 0 (absent), 1 or batch */
    int             n_top_k;
    const uint32_t* top_k;
    int             n_top_p;
    const float*    top_p;
    int             n_temperature;
    const float*    temperature;
    int             n_repetition_penalty;
    const float*    repetition_penalty;
    int             n_presence_penalty;
    const float*    presence_penalty;
    int             n_min_length;
    const int*      min_length;
    int             n_len_penalty;
    const float*    len_penalty;
    int             n_diversity;
    const float*    beam_search_diversity_rate;
    int             n_random_seed;
    const uint64_t* random_seed;
    /* device arrays [batch] or null */
    const float*    top_p_decay;
    const float*    top_p_min;
    const uint32_t* top_p_reset_ids;
};

struct ftref_step_args {
    void*           logits; /* device [batch, beam, vocab_padded] */
    int             batch;
    int             beam;
    const void*     embedding_bias; /* device [vocab_padded] or null */
    int             step;
    int             max_input_length;
    int             ite;
    int             local_batch_size;
    const int*      end_id;                /* device [batch] */
    const int*      input_lengths;         /* device [batch*beam] or null */
    const uint32_t* sequence_limit_length; /* device [batch] or null */
    const int*      stop_words_list;       /* device [batch,2,len] or null */
    int             stop_words_len;
    const int*      bad_words_list; /* device [2,len] or [batch,2,len] or null */
    int             bad_words_len;
    int             bad_words_shared;
    const int*      src_cache_indirection; /* device [local_batch,beam,max_seq_len] or null */
    int             max_seq_len;
    /* runtime args forwarded for the beam path (host, [1] or [batch]) */
    int          n_temperature;
    const float* temperature;
    int          n_len_penalty;
    const float* len_penalty;
    int          n_repetition_penalty;
    const float* repetition_penalty;
    int          n_presence_penalty;
    const float* presence_penalty;
    int          n_min_length;
    const int*   min_length;
    int          n_diversity;
    const float* beam_search_diversity_rate;
    /* outputs */
    int*   output_ids;            /* device [max_seq_len, batch*beam] */
    bool*  finished;              /* device [batch*beam] or null */
    float* cum_log_probs;         /* device [batch*beam] or null */
    int*   parent_ids;            /* device [max_seq_len, batch*beam] or null */
    int*   sequence_length;       /* device [batch*beam] or null */
    float* output_log_probs;      /* device [output_log_probs_len, batch*beam] or null */
    int    output_log_probs_len;
    int*   tgt_cache_indirection; /* device or null */
    void*  beam_hyps;             /* host BeamHypotheses* or null */
    bool*  should_stop;           /* host [1] */
};

struct FtRef {
    int                                      dtype;
    int                                      vocab;
    int                                      vocab_padded;
    ft::Allocator<ft::AllocatorType::CUDA>*  alloc;
    ft::DynamicDecodeLayer<float>*           f32;
    ft::DynamicDecodeLayer<half>*            f16;
    cudaStream_t                             stream;
    cudaDeviceProp                           prop;
    std::string                              err;
};

static thread_local std::string g_err;

const char* ftref_last_error()
{
    return g_err.c_str();
}

void* ftref_create(int dtype, int vocab, int vocab_padded, void* stream)
{
    try {
        FtRef* h  = new FtRef();
        h->dtype  = dtype;
        h->vocab  = vocab;
        h->vocab_padded = vocab_padded;
        h->stream = (cudaStream_t)stream;
        int dev   = 0;
        cudaGetDevice(&dev);
        cudaGetDeviceProperties(&h->prop, dev);
        h->alloc = new ft::Allocator<ft::AllocatorType::CUDA>(dev);
        h->alloc->setStream(h->stream);
        h->f32 = nullptr;
        h->f16 = nullptr;
        if (dtype == 0) {
            h->f32 = new ft::DynamicDecodeLayer<float>(
                vocab, vocab_padded, 0, h->stream, nullptr, h->alloc, false, &h->prop);
        }
        else {
            h->f16 = new ft::DynamicDecodeLayer<half>(
                vocab, vocab_padded, 0, h->stream, nullptr, h->alloc, false, &h->prop);
        }
        return h;
    }
    catch (std::exception& e) {
        g_err = e.what();
        return nullptr;
    }
}

void ftref_destroy(void* hv)
{
    FtRef* h = (FtRef*)hv;
    if (!h)
        return;
    delete h->f32;
    delete h->f16;
    delete h->alloc;
    delete h;
}

#define ADD_HOST(map, key, n, ptr, type)                                                                               \
    if ((n) > 0 && (ptr) != nullptr)                                                                                   \
    (map).insert(key, ft::Tensor(ft::MEMORY_CPU, type, {(size_t)(n)}, ptr))

int ftref_setup(void* hv, int batch, int beam, const ftref_runtime_args* a)
{
    FtRef* h = (FtRef*)hv;
    try {
        ft::TensorMap m;
        ADD_HOST(m, "runtime_top_k", a->n_top_k, a->top_k, ft::TYPE_UINT32);
        ADD_HOST(m, "runtime_top_p", a->n_top_p, a->top_p, ft::TYPE_FP32);
        ADD_HOST(m, "temperature", a->n_temperature, a->temperature, ft::TYPE_FP32);
        ADD_HOST(m, "repetition_penalty", a->n_repetition_penalty, a->repetition_penalty, ft::TYPE_FP32);
        ADD_HOST(m, "presence_penalty", a->n_presence_penalty, a->presence_penalty, ft::TYPE_FP32);
        ADD_HOST(m, "min_length", a->n_min_length, a->min_length, ft::TYPE_INT32);
        ADD_HOST(m, "len_penalty", a->n_len_penalty, a->len_penalty, ft::TYPE_FP32);
        ADD_HOST(m, "beam_search_diversity_rate", a->n_diversity, a->beam_search_diversity_rate, ft::TYPE_FP32);
        ADD_HOST(m, "random_seed", a->n_random_seed, a->random_seed, ft::TYPE_UINT64);
        if (a->top_p_decay)
            m.insert("top_p_decay", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_FP32, {(size_t)batch}, a->top_p_decay));
        if (a->top_p_min)
            m.insert("top_p_min", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_FP32, {(size_t)batch}, a->top_p_min));
        if (a->top_p_reset_ids)
            m.insert("top_p_reset_ids",
                     ft::Tensor(ft::MEMORY_GPU, ft::TYPE_UINT32, {(size_t)batch}, a->top_p_reset_ids));
        if (h->dtype == 0)
            h->f32->setup(batch, beam, &m);
        else
            h->f16->setup(batch, beam, &m);
        return 0;
    }
    catch (std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

int ftref_forward(void* hv, const ftref_step_args* s)
{
    FtRef* h = (FtRef*)hv;
    try {
        const size_t B  = s->batch;
        const size_t K  = s->beam;
        const size_t BK = B * K;
        const size_t L  = s->max_seq_len;
        ft::DataType lt = h->dtype == 0 ? ft::TYPE_FP32 : ft::TYPE_FP16;

        uint32_t ite = (uint32_t)s->ite;
        int      step = s->step, mil = s->max_input_length, lbs = s->local_batch_size;

        ft::TensorMap in;
        in.insert("logits", ft::Tensor(ft::MEMORY_GPU, lt, {B, K, (size_t)h->vocab_padded}, s->logits));
        if (s->embedding_bias)
            in.insert("embedding_bias", ft::Tensor(ft::MEMORY_GPU, lt, {(size_t)h->vocab_padded}, s->embedding_bias));
        in.insert("step", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &step));
        in.insert("max_input_length", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &mil));
        in.insert("ite", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_UINT32, {1}, &ite));
        in.insert("local_batch_size", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &lbs));
        in.insert("end_id", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {B}, s->end_id));
        if (s->input_lengths)
            in.insert("input_lengths", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {B, K}, s->input_lengths));
        if (s->sequence_limit_length)
            in.insert("sequence_limit_length",
                      ft::Tensor(ft::MEMORY_GPU, ft::TYPE_UINT32, {B}, s->sequence_limit_length));
        if (s->stop_words_list)
            in.insert("stop_words_list",
                      ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {B, 2, (size_t)s->stop_words_len}, s->stop_words_list));
        if (s->bad_words_list) {
            if (s->bad_words_shared)
                in.insert("bad_words_list",
                          ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {2, (size_t)s->bad_words_len}, s->bad_words_list));
            else
                in.insert(
                    "bad_words_list",
                    ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {B, 2, (size_t)s->bad_words_len}, s->bad_words_list));
        }
        if (s->src_cache_indirection)
            in.insert("src_cache_indirection",
                      ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {(size_t)lbs, K, L}, s->src_cache_indirection));
        ADD_HOST(in, "temperature", s->n_temperature, s->temperature, ft::TYPE_FP32);
        ADD_HOST(in, "len_penalty", s->n_len_penalty, s->len_penalty, ft::TYPE_FP32);
        ADD_HOST(in, "repetition_penalty", s->n_repetition_penalty, s->repetition_penalty, ft::TYPE_FP32);
        ADD_HOST(in, "presence_penalty", s->n_presence_penalty, s->presence_penalty, ft::TYPE_FP32);
        ADD_HOST(in, "min_length", s->n_min_length, s->min_length, ft::TYPE_INT32);
        ADD_HOST(in, "beam_search_diversity_rate", s->n_diversity, s->beam_search_diversity_rate, ft::TYPE_FP32);

        ft::TensorMap out;
        out.insert("output_ids", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {L, B, K}, s->output_ids));
        if (s->finished)
            out.insert("finished", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_BOOL, {BK}, s->finished));
        if (s->cum_log_probs)
            out.insert("cum_log_probs", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_FP32, {BK}, s->cum_log_probs));
        if (s->parent_ids)
            out.insert("parent_ids", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {L, B, K}, s->parent_ids));
        if (s->sequence_length)
            out.insert("sequence_length", ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {BK}, s->sequence_length));
        if (s->output_log_probs)
            out.insert("output_log_probs",
                       ft::Tensor(ft::MEMORY_GPU, ft::TYPE_FP32, {(size_t)s->output_log_probs_len, BK},
                                  s->output_log_probs));
        if (s->tgt_cache_indirection)
            out.insert("tgt_cache_indirection",
                       ft::Tensor(ft::MEMORY_GPU, ft::TYPE_INT32, {(size_t)lbs, K, L}, s->tgt_cache_indirection));
        if (s->beam_hyps)
            out.insert("beam_hyps", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_VOID, {1}, s->beam_hyps));
        bool dummy_stop = false;
        out.insert("should_stop",
                   ft::Tensor(ft::MEMORY_CPU, ft::TYPE_BOOL, {1}, s->should_stop ? s->should_stop : &dummy_stop));

        if (h->dtype == 0)
            h->f32->forward(&out, &in);
        else
            h->f16->forward(&out, &in);
        return 0;
    }
    catch (std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

/* Size and field offsets of the reference's BeamHypotheses, so a test can build one from Python. */
int ftref_sizeof_beam_hyps()
{
    return (int)sizeof(ft::BeamHypotheses);
}

/* Uniforms drawn exactly as the reference kernels draw them (curand_uniform on
 * the row's XORWOW state, sampling_topk_kernels.cu:283), without touching the
 * caller's states: states are copied, n_draws uniforms per row are produced. */
__global__ void ftref_uniform_kernel(const curandState_t* states, int n, int n_draws, float* out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        curandState_t st = states[i];
        for (int d = 0; d < n_draws; ++d) {
            out[(size_t)d * n + i] = curand_uniform(&st);
        }
    }
}

int ftref_curand_init(void* states, int n, unsigned long long seed, const unsigned long long* seeds_dev, void* stream)
{
    if (seeds_dev)
        ft::invokeCurandBatchInitialize((curandState_t*)states, n, seeds_dev, (cudaStream_t)stream);
    else
        ft::invokeCurandInitialize((curandState_t*)states, n, seed, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int ftref_curand_uniforms(const void* states, int n, int n_draws, float* out_dev, void* stream)
{
    ftref_uniform_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        (const curandState_t*)states, n, n_draws, out_dev);
    return (int)cudaGetLastError();
}

/* invokeLogProbFromLogits<T> (kernels/logprob_kernels.cu:142-183) on device pointers; dtype 0 = float, 1 = half. */
int ftref_log_prob_from_logits(float* cum_log_probs, const void* logits, int dtype, const int* input_ids,
                               const int* input_lengths, size_t max_input_length, size_t batch_size,
                               size_t vocab_size, size_t vocab_size_padded, void* workspace, size_t workspace_size,
                               void* stream, int batch_first)
{
    if (dtype == 0) {
        ft::invokeLogProbFromLogits(cum_log_probs, (const float*)logits, input_ids, input_lengths, max_input_length,
                                    batch_size, vocab_size, vocab_size_padded, workspace, workspace_size,
                                    (cudaStream_t)stream, batch_first != 0);
    }
    else {
        ft::invokeLogProbFromLogits(cum_log_probs, (const half*)logits, input_ids, input_lengths, max_input_length,
                                    batch_size, vocab_size, vocab_size_padded, workspace, workspace_size,
                                    (cudaStream_t)stream, batch_first != 0);
    }
    return (int)cudaGetLastError();
}

/* invokeDecodingInitialize<T> (kernels/decoding_kernels.cu:49-64); dtype 0 float, 1 half, 2 bf16. */
int ftref_decoding_initialize(bool* finished, int* sequence_length, int* word_ids, void* cum_log_probs, int dtype,
                              const int* sentence_ids, int batch_size, int beam_width, int max_input_length,
                              void* stream)
{
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0) {
        ft::invokeDecodingInitialize(finished, sequence_length, word_ids, (float*)cum_log_probs, sentence_ids,
                                     batch_size, beam_width, max_input_length, st);
    }
    else if (dtype == 1) {
        ft::invokeDecodingInitialize(finished, sequence_length, word_ids, (half*)cum_log_probs, sentence_ids,
                                     batch_size, beam_width, max_input_length, st);
    }
    else {
        ft::invokeDecodingInitialize(finished, sequence_length, word_ids, (__nv_bfloat16*)cum_log_probs, sentence_ids,
                                     batch_size, beam_width, max_input_length, st);
    }
    return (int)cudaGetLastError();
}

/* invokeGatherTree(gatherTreeParam) (kernels/decoding_kernels.cu:636-646); the arguments are gatherTreeParam's
 * fields in their order. */
int ftref_gather_tree(int* beams, int* max_sequence_lengths, int max_sequence_length_final_step,
                      const int* input_lengths, int* response_input_lengths, int max_time, int batch_size,
                      int beam_width, const int* step_ids, const int* parent_ids, const int* end_tokens,
                      int max_input_length, const int* prefix_soft_prompt_lengths,
                      const int* p_prompt_tuning_prompt_lengths, int max_input_without_prompt_length,
                      int max_prefix_soft_prompt_length, int* output_ids, void* stream)
{
    ft::gatherTreeParam param;
    param.beams                           = beams;
    param.max_sequence_lengths            = max_sequence_lengths;
    param.max_sequence_length_final_step  = max_sequence_length_final_step;
    param.input_lengths                   = input_lengths;
    param.response_input_lengths          = response_input_lengths;
    param.max_time                        = max_time;
    param.batch_size                      = batch_size;
    param.beam_width                      = beam_width;
    param.step_ids                        = step_ids;
    param.parent_ids                      = parent_ids;
    param.end_tokens                      = end_tokens;
    param.max_input_length                = max_input_length;
    param.prefix_soft_prompt_lengths      = prefix_soft_prompt_lengths;
    param.p_prompt_tuning_prompt_lengths  = p_prompt_tuning_prompt_lengths;
    param.max_input_without_prompt_length = max_input_without_prompt_length;
    param.max_prefix_soft_prompt_length   = max_prefix_soft_prompt_length;
    param.output_ids                      = output_ids;
    param.stream                          = (cudaStream_t)stream;
    ft::invokeGatherTree(param);
    return (int)cudaGetLastError();
}

/* invokeFinalize (kernels/decoding_kernels.cu:773-804). */
int ftref_finalize(int* output_ids, int* sequence_lengths, float* cum_log_probs, float* output_log_probs,
                   const int* topk_output_ids, const int* topk_sequence_lengths, const float* scores,
                   const float* topk_cum_log_probs, const float* topk_log_probs, const int* num_beams, int beam_width,
                   int max_seq_len, int batch_size, void* stream)
{
    ft::invokeFinalize(output_ids, sequence_lengths, cum_log_probs, output_log_probs, topk_output_ids,
                       topk_sequence_lengths, scores, topk_cum_log_probs, topk_log_probs, num_beams, beam_width,
                       max_seq_len, batch_size, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

/* invokeInsertUnfinishedPath (kernels/beam_search_topk_kernels.cu:834-843). */
int ftref_insert_unfinished_path(int* output_ids_tgt, int* sequence_lengths_tgt, float* cum_log_probs_tgt,
                                 float* normed_scores, float* log_probs_tgt, int* num_beams, bool* is_done,
                                 const int* output_ids_src, const int* parent_ids_src,
                                 const int* sequence_lengths_src, const float* log_probs_src, int max_seq_len,
                                 float length_penalty, const bool* finished, const float* cum_log_probs,
                                 int batch_size, int beam_width, void* stream)
{
    ft::BeamHypotheses h;
    h.output_ids_tgt       = output_ids_tgt;
    h.sequence_lengths_tgt = sequence_lengths_tgt;
    h.cum_log_probs        = cum_log_probs_tgt;
    h.normed_scores        = normed_scores;
    h.log_probs            = log_probs_tgt;
    h.num_beams            = num_beams;
    h.is_done              = is_done;
    h.output_ids_src       = output_ids_src;
    h.parent_ids_src       = parent_ids_src;
    h.sequence_lengths_src = sequence_lengths_src;
    h.log_probs_src        = log_probs_src;
    h.end_ids              = nullptr;
    h.step                 = 0;
    h.ite                  = 0;
    h.batch_size           = batch_size;
    h.local_batch_size     = batch_size;
    h.max_seq_len          = max_seq_len;
    h.length_penalty       = length_penalty;
    ft::invokeInsertUnfinishedPath(h, finished, cum_log_probs, batch_size, beam_width, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

}  // extern "C"
