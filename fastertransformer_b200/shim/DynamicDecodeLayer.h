// C++ classes with FasterTransformer's names and interface for the decode step, implemented on the
// libftb200 C ABI (include/ftb200.h).  They replace, one for one:
//   DynamicDecodeLayer<T>     layers/DynamicDecodeLayer.h:58-75
//   BaseSamplingLayer<T>      layers/sampling_layers/BaseSamplingLayer.h:26-81
//   TopKSamplingLayer<T>      layers/sampling_layers/TopKSamplingLayer.h:55-71
//   TopPSamplingLayer<T>      layers/sampling_layers/TopPSamplingLayer.h:64-81
//   OnlineBeamSearchLayer<T>  layers/beam_search_layers/OnlineBeamSearchLayer.h:44-62
// Same constructor arguments, same setup()/forward() signatures, same TensorMap keys, dtypes and
// placement, same exception types (std::runtime_error with the "[FT][ERROR]" prefix, std::domain_error
// for k outside [1, 1024]).  T is float, half or __nv_bfloat16.
//
// Inside a FasterTransformer checkout compile with -DFTB200_WITH_FT_HEADERS: the project's own Tensor,
// TensorMap and IAllocator are used.  Elsewhere the stand-ins of ft_compat.h are.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#ifdef FTB200_WITH_FT_HEADERS
#include "src/fastertransformer/utils/Tensor.h"
#include "src/fastertransformer/utils/allocator.h"
namespace fastertransformer {
class cublasMMWrapper;
}
#else
#include "ft_compat.h"
#endif

namespace fastertransformer {

namespace ftb200_detail {
class DecodeCore;  // dtype-erased state and logic shared by the four class templates
}

template<typename T>
class DynamicDecodeLayer {
public:
    DynamicDecodeLayer(size_t vocab_size, size_t vocab_size_padded, int end_id, cudaStream_t stream,
                       cublasMMWrapper* cublas_wrapper, IAllocator* allocator, bool is_free_buffer_after_forward,
                       cudaDeviceProp* cuda_device_prop);
    ~DynamicDecodeLayer();
    DynamicDecodeLayer(DynamicDecodeLayer const& other);

    void setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args);
    void forward(TensorMap* output_tensors, TensorMap* input_tensors);
    void forward(std::unordered_map<std::string, Tensor>* output_tensors,
                 const std::unordered_map<std::string, Tensor>* input_tensors);

    // BaseLayer's stream accessors (layers/BaseLayer.h:43-51): later calls run on the new stream.
    void         setStream(cudaStream_t stream);
    cudaStream_t getStream();

private:
    std::unique_ptr<ftb200_detail::DecodeCore> core_;
};

// The base of the sampling layers (layers/sampling_layers/BaseSamplingLayer.h:26-81): constructor arguments,
// setup() and forward() as there, and the pure-virtual runSampling() that forward() ends with.
//
// In the reference forward() rewrites the logits (temperature, repetition or presence penalty, minimum
// length) and runSampling() of the derived class selects the token.  Here all of that is one kernel, so
// forward() checks the step's tensors, fixes the slice of the batch (`ite`, `local_batch_size`) and calls
// runSampling(), and runSampling() of the two classes below launches the fused step, penalties included.
// A class derived from this base outside the library therefore receives the logits as the caller gave them:
// the penalties stored by setup() are applied by TopKSamplingLayer / TopPSamplingLayer only.
template<typename T>
class BaseSamplingLayer {
public:
    BaseSamplingLayer(size_t max_batch_size, size_t vocab_size, size_t vocab_size_padded, int end_id, size_t top_k,
                      float top_p, unsigned long long random_seed, float temperature, float len_penalty,
                      float repetition_penalty, cudaStream_t stream, cublasMMWrapper* cublas_wrapper,
                      IAllocator* allocator, bool is_free_buffer_after_forward, cudaDeviceProp* cuda_device_prop);
    BaseSamplingLayer(BaseSamplingLayer const& other);
    virtual ~BaseSamplingLayer();

    // runtime_args as in the reference: runtime_top_k / runtime_top_p [1] or [batch], temperature,
    // repetition_penalty or presence_penalty, min_length, random_seed, top_p_decay / top_p_min / top_p_reset_ids.
    virtual void setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args);
    virtual void forward(TensorMap* output_tensors, TensorMap* input_tensors);
    virtual void forward(std::unordered_map<std::string, Tensor>*       output_tensors,
                         const std::unordered_map<std::string, Tensor>* input_tensors);
    // The positional form is as unsupported here as in the reference (BaseSamplingLayer.cc:214-219 throws).
    virtual void forward(std::vector<Tensor>* output_tensors, const std::vector<Tensor>* input_tensors);

    void         setStream(cudaStream_t stream);
    cudaStream_t getStream();

protected:
    virtual void runSampling(TensorMap* output_tensors, TensorMap* input_tensors) = 0;

    size_t vocab_size_;
    size_t vocab_size_padded_;
    std::unique_ptr<ftb200_detail::DecodeCore> core_;
};

// The two sampling layers used on their own (without the dispatcher): each owns its curand states and
// samples the rows its runtime arguments select; the other half of the argument block stays empty.
template<typename T>
class TopKSamplingLayer: public BaseSamplingLayer<T> {
public:
    TopKSamplingLayer(size_t max_batch_size, size_t vocab_size, size_t vocab_size_padded, int end_id, size_t top_k,
                      unsigned long long random_seed, float temperature, float len_penalty, float repetition_penalty,
                      cudaStream_t stream, cublasMMWrapper* cublas_wrapper, IAllocator* allocator,
                      bool is_free_buffer_after_forward);
    TopKSamplingLayer(TopKSamplingLayer<T> const& other);
    ~TopKSamplingLayer();
    void setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args) override;

private:
    void runSampling(TensorMap* output_tensors, TensorMap* input_tensors) override;
    using BaseSamplingLayer<T>::core_;
};

template<typename T>
class TopPSamplingLayer: public BaseSamplingLayer<T> {
public:
    TopPSamplingLayer(size_t max_batch_size, size_t vocab_size, size_t vocab_size_padded, int end_id, float top_p,
                      unsigned long long random_seed, float temperature, float len_penalty, float repetition_penalty,
                      cudaStream_t stream, cublasMMWrapper* cublas_wrapper, IAllocator* allocator,
                      bool is_free_buffer_after_forward, cudaDeviceProp* cuda_device_prop);
    TopPSamplingLayer(TopPSamplingLayer<T> const& other);
    ~TopPSamplingLayer();
    void setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args) override;

private:
    void runSampling(TensorMap* output_tensors, TensorMap* input_tensors) override;
    using BaseSamplingLayer<T>::core_;
};

template<typename T>
class OnlineBeamSearchLayer {
public:
    OnlineBeamSearchLayer(size_t max_batch_size, size_t head_num, size_t size_per_head, size_t beam_width,
                          size_t vocab_size, size_t vocab_size_padded, int end_id, float diversity_rate,
                          float temperature, float len_penalty, float repetition_penalty, cudaStream_t stream,
                          cublasMMWrapper* cublas_wrapper, IAllocator* allocator, bool is_free_buffer_after_forward);
    ~OnlineBeamSearchLayer();
    void setup(const size_t batch_size, TensorMap* runtime_args);
    void forward(TensorMap* output_tensors, TensorMap* input_tensors);

private:
    std::unique_ptr<ftb200_detail::DecodeCore> core_;
};

}  // namespace fastertransformer
