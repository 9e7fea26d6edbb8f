// Torch custom class `FasterTransformer.DynamicDecodeOp` (torch.classes.FasterTransformer.DynamicDecodeOp) with the
// reference's constructor, setup(), forward() and broadcast_from_last_pipeline() argument lists
// (th_op/common/DynamicDecodeOp.h:155-226, registration th_op/common/DynamicDecodeOp.cc:445-454), on top of the
// C++ DynamicDecodeLayer<T> of ../shim.  torch owns the tensors and the stream; every computation is a call into
// libftb200.
//
// Differences: bfloat16 logits are accepted next to float and half; tensor_para_size / pipeline_para_size other
// than 1 are refused (the reference initialises NCCL from MPI there, which this library leaves to its caller:
// the vocabulary-parallel entry points take the communicator's result as plain buffers).
#include <ATen/cuda/CUDAContext.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "DynamicDecodeLayer.h"

namespace ft = fastertransformer;
namespace th = torch;

namespace torch_ext {

namespace {

void check_tensor(const th::Tensor& t, bool cuda, at::ScalarType type, const char* name)
{
    TORCH_CHECK(t.is_cuda() == cuda, name, cuda ? " must be a CUDA tensor" : " must be a CPU tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == type, name, ": inconsistent tensor type");
}
void check_optional(const th::optional<th::Tensor>& t, bool cuda, at::ScalarType type, const char* name)
{
    if (t.has_value()) {
        check_tensor(t.value(), cuda, type, name);
    }
}
// CHECK_OPTIONAL_INPUT in the reference wants CUDA tensors for these; CHECK_OPTIONAL_CPU_INPUT host tensors.
#define FTB_OPT_CPU(x, type) check_optional(x, false, type, #x)
#define FTB_OPT_GPU(x, type) check_optional(x, true, type, #x)

std::vector<size_t> shape_of(const th::Tensor& t)
{
    std::vector<size_t> s;
    for (int i = 0; i < t.dim(); ++i) {
        s.push_back((size_t)t.size(i));
    }
    return s;
}
ft::Tensor as_ft(const th::Tensor& t, ft::DataType type)
{
    return ft::Tensor(t.is_cuda() ? ft::MEMORY_GPU : ft::MEMORY_CPU, type, shape_of(t), t.data_ptr());
}
void put(ft::TensorMap& m, const char* key, const th::optional<th::Tensor>& t, ft::DataType type)
{
    if (t.has_value()) {
        m.insert(key, as_ft(t.value(), type));
    }
}

class IDecode {
public:
    virtual ~IDecode() {}
    virtual void setup(size_t batch, size_t beam, ft::TensorMap* args)   = 0;
    virtual void forward(ft::TensorMap* out, ft::TensorMap* in)          = 0;
};

template<typename T>
class Decode: public IDecode {
    ft::CudaAllocator                          allocator_;
    cudaDeviceProp                             prop_;
    std::unique_ptr<ft::DynamicDecodeLayer<T>> layer_;

public:
    Decode(size_t vocab, size_t vocab_padded)
    {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaGetDeviceProperties(&prop_, dev);
        auto stream = at::cuda::getCurrentCUDAStream().stream();
        allocator_.setStream(stream);
        layer_.reset(new ft::DynamicDecodeLayer<T>(vocab, vocab_padded, 0, stream, nullptr, &allocator_, false, &prop_));
    }
    void setup(size_t batch, size_t beam, ft::TensorMap* args) override
    {
        layer_->setStream(at::cuda::getCurrentCUDAStream().stream());
        layer_->setup(batch, beam, args);
    }
    void forward(ft::TensorMap* out, ft::TensorMap* in) override
    {
        layer_->setStream(at::cuda::getCurrentCUDAStream().stream());
        layer_->forward(out, in);
    }
};

}  // namespace

class DynamicDecodeOp: public th::jit::CustomClassHolder {
public:
    DynamicDecodeOp(const int64_t vocab_size, const int64_t vocab_size_padded, const int64_t tensor_para_size,
                    const int64_t pipeline_para_size, at::ScalarType scalar_type):
        vocab_size_((size_t)vocab_size), vocab_size_padded_((size_t)vocab_size_padded), scalar_type_(scalar_type)
    {
        if (tensor_para_size != 1 || pipeline_para_size != 1) {
            throw std::runtime_error("[FT][ERROR] DynamicDecodeOp: tensor_para_size and pipeline_para_size must be 1");
        }
        switch (scalar_type_) {
            case at::ScalarType::Float: decode_.reset(new Decode<float>(vocab_size_, vocab_size_padded_)); break;
            case at::ScalarType::Half: decode_.reset(new Decode<half>(vocab_size_, vocab_size_padded_)); break;
            case at::ScalarType::BFloat16:
                decode_.reset(new Decode<__nv_bfloat16>(vocab_size_, vocab_size_padded_));
                break;
            default: throw std::runtime_error("Wrong tensor type.");
        }
    }

    void setup(int64_t batch_size, int64_t beam_width, th::optional<th::Tensor> runtime_top_k_opt,
               th::optional<th::Tensor> runtime_top_p_opt, th::optional<th::Tensor> temperature_opt,
               th::optional<th::Tensor> repetition_penalty_opt, th::optional<th::Tensor> presence_penalty_opt,
               th::optional<th::Tensor> min_length_opt, th::optional<th::Tensor> length_penalty_opt,
               th::optional<th::Tensor> beam_search_diversity_rate_opt, th::optional<th::Tensor> random_seed_opt,
               th::optional<th::Tensor> top_p_decay_opt, th::optional<th::Tensor> top_p_min_opt,
               th::optional<th::Tensor> top_p_reset_ids_opt)
    {
        FTB_OPT_CPU(runtime_top_k_opt, torch::kInt32);
        FTB_OPT_CPU(runtime_top_p_opt, torch::kFloat);
        FTB_OPT_CPU(temperature_opt, torch::kFloat);
        FTB_OPT_CPU(repetition_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(presence_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(min_length_opt, torch::kInt32);
        FTB_OPT_CPU(length_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(beam_search_diversity_rate_opt, torch::kFloat);
        FTB_OPT_CPU(random_seed_opt, torch::kInt64);
        FTB_OPT_GPU(top_p_decay_opt, torch::kFloat);
        FTB_OPT_GPU(top_p_min_opt, torch::kFloat);
        FTB_OPT_GPU(top_p_reset_ids_opt, torch::kInt32);

        ft::TensorMap args;
        put(args, "runtime_top_k", runtime_top_k_opt, ft::TYPE_UINT32);
        put(args, "runtime_top_p", runtime_top_p_opt, ft::TYPE_FP32);
        put(args, "temperature", temperature_opt, ft::TYPE_FP32);
        put(args, "repetition_penalty", repetition_penalty_opt, ft::TYPE_FP32);
        put(args, "presence_penalty", presence_penalty_opt, ft::TYPE_FP32);
        put(args, "min_length", min_length_opt, ft::TYPE_INT32);
        put(args, "len_penalty", length_penalty_opt, ft::TYPE_FP32);
        put(args, "beam_search_diversity_rate", beam_search_diversity_rate_opt, ft::TYPE_FP32);
        put(args, "random_seed", random_seed_opt, ft::TYPE_UINT64);
        // the reference files the decay under "top_p_decay_opt" (th_op/common/DynamicDecodeOp.cc:102), a key its
        // layer never reads; the layer's own key is used here
        put(args, "top_p_decay", top_p_decay_opt, ft::TYPE_FP32);
        put(args, "top_p_min", top_p_min_opt, ft::TYPE_FP32);
        put(args, "top_p_reset_ids", top_p_reset_ids_opt, ft::TYPE_UINT32);
        decode_->setup((size_t)batch_size, (size_t)beam_width, &args);
    }

    th::Tensor forward(th::Tensor logits, int64_t step, int64_t max_input_length, int64_t ite,
                       int64_t local_batch_size, th::Tensor end_id, th::optional<th::Tensor> runtime_top_k_opt,
                       th::optional<th::Tensor> runtime_top_p_opt, th::optional<th::Tensor> temperature_opt,
                       th::optional<th::Tensor> repetition_penalty_opt, th::optional<th::Tensor> presence_penalty_opt,
                       th::optional<th::Tensor> min_length_opt, th::optional<th::Tensor> length_penalty_opt,
                       th::optional<th::Tensor> beam_search_diversity_rate_opt,
                       th::optional<th::Tensor> top_p_decay_opt, th::optional<th::Tensor> top_p_min_opt,
                       th::optional<th::Tensor> top_p_reset_ids_opt, th::optional<th::Tensor> embedding_bias_opt,
                       th::optional<th::Tensor> input_lengths_opt, th::optional<th::Tensor> sequence_limit_length_opt,
                       th::optional<th::Tensor> stop_words_list_opt, th::optional<th::Tensor> bad_words_list_opt,
                       th::optional<th::Tensor> src_cache_indirection_opt, th::Tensor output_token_ids,
                       th::optional<th::Tensor> finished_opt, th::optional<th::Tensor> sequence_lengths_opt,
                       th::optional<th::Tensor> cum_log_probs_opt, th::optional<th::Tensor> output_log_probs_opt,
                       th::optional<th::Tensor> parent_ids_opt, th::optional<th::Tensor> tgt_cache_indirection_opt)
    {
        check_tensor(logits, true, scalar_type_, "logits");
        TORCH_CHECK(logits.dim() == 3, "logits is of shape (batch_size, beam_width, vocab_size_padded), but got dim=",
                    logits.dim());
        TORCH_CHECK((size_t)logits.size(2) == vocab_size_padded_, "logits is of shape (batch_size, beam_width, vocab_size(",
                    vocab_size_padded_, ")), but got the last dim=", logits.size(2));
        check_tensor(end_id, true, torch::kInt32, "end_id");
        FTB_OPT_CPU(runtime_top_k_opt, torch::kInt32);
        FTB_OPT_CPU(runtime_top_p_opt, torch::kFloat);
        FTB_OPT_CPU(temperature_opt, torch::kFloat);
        FTB_OPT_CPU(repetition_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(presence_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(min_length_opt, torch::kInt32);
        FTB_OPT_CPU(length_penalty_opt, torch::kFloat);
        FTB_OPT_CPU(beam_search_diversity_rate_opt, torch::kFloat);
        FTB_OPT_GPU(top_p_decay_opt, torch::kFloat);
        FTB_OPT_GPU(top_p_min_opt, torch::kFloat);
        FTB_OPT_GPU(top_p_reset_ids_opt, torch::kInt32);
        FTB_OPT_GPU(embedding_bias_opt, scalar_type_);
        FTB_OPT_GPU(input_lengths_opt, torch::kInt32);
        FTB_OPT_GPU(sequence_limit_length_opt, torch::kInt32);
        FTB_OPT_GPU(stop_words_list_opt, torch::kInt32);
        FTB_OPT_GPU(bad_words_list_opt, torch::kInt32);
        FTB_OPT_GPU(src_cache_indirection_opt, torch::kInt32);
        check_tensor(output_token_ids, true, torch::kInt32, "output_token_ids");
        FTB_OPT_GPU(finished_opt, torch::kBool);
        FTB_OPT_GPU(sequence_lengths_opt, torch::kInt32);
        FTB_OPT_GPU(cum_log_probs_opt, torch::kFloat32);
        FTB_OPT_GPU(output_log_probs_opt, torch::kFloat32);
        FTB_OPT_GPU(parent_ids_opt, torch::kInt32);
        FTB_OPT_GPU(tgt_cache_indirection_opt, torch::kInt32);

        th::Tensor should_stop = torch::zeros({}, torch::dtype(torch::kBool).requires_grad(false));
        int        step_i = (int)step, mil_i = (int)max_input_length, lbs_i = (int)local_batch_size;
        unsigned   ite_u = (unsigned)ite;
        const ft::DataType T = scalar_type_ == at::ScalarType::Float ? ft::TYPE_FP32 :
                               scalar_type_ == at::ScalarType::Half  ? ft::TYPE_FP16 :
                                                                       ft::TYPE_BF16;
        ft::TensorMap in;
        in.insert("logits", as_ft(logits, T));
        in.insert("step", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &step_i));
        in.insert("max_input_length", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &mil_i));
        in.insert("ite", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_UINT32, {1}, &ite_u));
        in.insert("local_batch_size", ft::Tensor(ft::MEMORY_CPU, ft::TYPE_INT32, {1}, &lbs_i));
        in.insert("end_id", as_ft(end_id, ft::TYPE_INT32));
        put(in, "runtime_top_k", runtime_top_k_opt, ft::TYPE_UINT32);
        put(in, "runtime_top_p", runtime_top_p_opt, ft::TYPE_FP32);
        put(in, "temperature", temperature_opt, ft::TYPE_FP32);
        put(in, "repetition_penalty", repetition_penalty_opt, ft::TYPE_FP32);
        put(in, "presence_penalty", presence_penalty_opt, ft::TYPE_FP32);
        put(in, "min_length", min_length_opt, ft::TYPE_INT32);
        put(in, "len_penalty", length_penalty_opt, ft::TYPE_FP32);
        put(in, "beam_search_diversity_rate", beam_search_diversity_rate_opt, ft::TYPE_FP32);
        put(in, "top_p_decay", top_p_decay_opt, ft::TYPE_FP32);
        put(in, "top_p_min", top_p_min_opt, ft::TYPE_FP32);
        put(in, "top_p_reset_ids", top_p_reset_ids_opt, ft::TYPE_UINT32);
        put(in, "embedding_bias", embedding_bias_opt, T);
        put(in, "input_lengths", input_lengths_opt, ft::TYPE_INT32);
        put(in, "sequence_limit_length", sequence_limit_length_opt, ft::TYPE_INT32);
        put(in, "stop_words_list", stop_words_list_opt, ft::TYPE_INT32);
        put(in, "bad_words_list", bad_words_list_opt, ft::TYPE_INT32);
        put(in, "src_cache_indirection", src_cache_indirection_opt, ft::TYPE_INT32);

        ft::TensorMap out;
        out.insert("output_ids", as_ft(output_token_ids, ft::TYPE_INT32));
        out.insert("should_stop", as_ft(should_stop, ft::TYPE_BOOL));
        put(out, "finished", finished_opt, ft::TYPE_BOOL);
        put(out, "sequence_length", sequence_lengths_opt, ft::TYPE_INT32);
        put(out, "parent_ids", parent_ids_opt, ft::TYPE_INT32);
        put(out, "cum_log_probs", cum_log_probs_opt, ft::TYPE_FP32);
        put(out, "output_log_probs", output_log_probs_opt, ft::TYPE_FP32);
        put(out, "tgt_cache_indirection", tgt_cache_indirection_opt, ft::TYPE_INT32);
        decode_->forward(&out, &in);
        return should_stop;
    }

    // With one pipeline stage there is nothing to send (th_op/common/DynamicDecodeOp.cc:191-195).
    void broadcastFromLastPipeline(std::vector<th::Tensor> tensors)
    {
        for (const auto& t : tensors) {
            TORCH_CHECK(t.is_cuda(), "broadcast_from_last_pipeline wants CUDA tensors");
            TORCH_CHECK(t.is_contiguous(), "broadcast_from_last_pipeline wants contiguous tensors");
        }
    }

private:
    size_t                   vocab_size_, vocab_size_padded_;
    at::ScalarType           scalar_type_;
    std::unique_ptr<IDecode> decode_;
};

}  // namespace torch_ext

static auto ftb200DynamicDecodeOpTHS =
    torch::jit::class_<torch_ext::DynamicDecodeOp>("FasterTransformer", "DynamicDecodeOp")
        .def(torch::jit::init<int64_t, int64_t, int64_t, int64_t, at::ScalarType>())
        .def("setup", &torch_ext::DynamicDecodeOp::setup)
        .def("forward", &torch_ext::DynamicDecodeOp::forward)
        .def("broadcast_from_last_pipeline", &torch_ext::DynamicDecodeOp::broadcastFromLastPipeline);
