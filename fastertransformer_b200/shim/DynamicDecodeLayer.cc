// Host side of the decode layers on the libftb200 C ABI.  The logic follows
//   DynamicDecodeLayer<T>::setup / forward    layers/DynamicDecodeLayer.cc:153-178, :191-474, :477-514
//   BaseSamplingLayer<T>::setup / forward     layers/sampling_layers/BaseSamplingLayer.cc:112-206, :255-359
//   TopKSamplingLayer<T>::setup               layers/sampling_layers/TopKSamplingLayer.cu:134-186
//   TopPSamplingLayer<T>::setup               layers/sampling_layers/TopPSamplingLayer.cu:184-253
//   BaseBeamSearchLayer<T>::forward           layers/beam_search_layers/BaseBeamSearchLayer.cu:197-275
// of FasterTransformer: broadcast of the runtime arguments to per-row device arrays with host mirrors, the
// host-side gating of each penalty, slicing by ite * local_batch_size, the stop criteria and should_stop.
// Every computation is one call into the C ABI; a non-zero status comes back as the exception type the
// reference throws.
#include "DynamicDecodeLayer.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <numeric>
#include <stdexcept>

#include "ftb200.h"

namespace fastertransformer {
namespace ftb200_detail {

static void check(int rc)
{
    if (rc == FTB200_OK) {
        return;
    }
    const std::string msg = ftb200_last_error_string();
    if (rc == FTB200_DOMAIN_ERROR) {
        throw std::domain_error(msg);
    }
    throw std::runtime_error("[FT][ERROR] " + msg);
}

static void check_cuda(cudaError_t e)
{
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string("[FT][ERROR] CUDA runtime error: ") + cudaGetErrorString(e));
    }
}

template<typename T>
struct DtypeOf;
template<>
struct DtypeOf<float> {
    static constexpr int value = FTB200_F32;
};
template<>
struct DtypeOf<half> {
    static constexpr int value = FTB200_F16;
};
template<>
struct DtypeOf<__nv_bfloat16> {
    static constexpr int value = FTB200_BF16;
};

enum class Mode { Dispatcher, TopKOnly, TopPOnly, BeamOnly };

// One reference sampling layer's buffers (BaseSamplingLayer.cc:29-53 and the TopK / TopP allocateBuffer).
struct SamplingState {
    void*             curand  = nullptr;  // curandState_t[batch]
    uint32_t*         top_ks  = nullptr;
    float*            top_ps  = nullptr;
    uint8_t*          skip    = nullptr;
    float*            initial = nullptr;  // top-p layer only
    float*            decay   = nullptr;
    float*            pmin    = nullptr;
    int32_t*          reset   = nullptr;
    std::vector<char> skip_host;
    bool              active = false;
};

class DecodeCore {
public:
    DecodeCore(Mode mode, int dtype, size_t vocab, size_t vocab_padded, cudaStream_t stream, IAllocator* allocator,
               bool free_after_forward):
        mode_(mode), dtype_(dtype), vocab_(vocab), vocab_padded_(vocab_padded), stream_(stream), allocator_(allocator),
        free_after_forward_(free_after_forward)
    {
        if (allocator_ == nullptr) {
            throw std::runtime_error("[FT][ERROR] allocator must not be null");
        }
    }

    ~DecodeCore()
    {
        releaseAll();
    }

    void setup(size_t batch_size, size_t beam_width, TensorMap* args);
    void forward(TensorMap* out, TensorMap* in);
    void checkStep(TensorMap* out, TensorMap* in) const;
    void setStream(cudaStream_t stream)
    {
        stream_ = stream;
        if (allocator_ != nullptr) {
            allocator_->setStream(stream);
        }
    }
    cudaStream_t getStream() const
    {
        return stream_;
    }
    DecodeCore* cloneConfiguration() const
    {
        return new DecodeCore(mode_, dtype_, vocab_, vocab_padded_, stream_, allocator_, free_after_forward_);
    }

private:
    static constexpr size_t kCurandStateBytes = 48;  // sizeof(curandState_t)

    template<typename U>
    U* alloc(size_t n, bool host = false)
    {
        void* p = allocator_->malloc(sizeof(U) * n, true, host);
        owned_.push_back({p, host});
        return (U*)p;
    }
    void releaseAll()
    {
        for (auto& o : owned_) {
            void* p = o.first;
            allocator_->free(&p, o.second);
        }
        owned_.clear();
        topk_ = SamplingState();
        topp_ = SamplingState();
        workspace_ = nullptr, workspace_bytes_ = 0;
        beam_ws_ = nullptr, beam_ws_bytes_ = 0;
        count_dev_ = nullptr, count_host_ = nullptr;
        orders_.clear();
    }

    // runtime argument [1] or [batch] -> vector [batch]
    template<typename U>
    std::vector<U> broadcast(TensorMap* args, const char* key, size_t batch, U def)
    {
        std::vector<U> v(batch, def);
        if (args != nullptr && args->isExist(key)) {
            const Tensor& t = args->at(key);
            const size_t  n = t.size();
            if (n != 1 && n != batch) {
                throw std::runtime_error(std::string("[FT][ERROR] ") + key + " must be of shape [1] or [batch_size]");
            }
            for (size_t i = 0; i < batch; ++i) {
                v[i] = t.getVal<U>(n == 1 ? 0 : i);
            }
        }
        return v;
    }
    template<typename U>
    U* upload(const std::vector<U>& v)
    {
        U* d = alloc<U>(v.size());
        check_cuda(cudaMemcpyAsync(d, v.data(), sizeof(U) * v.size(), cudaMemcpyHostToDevice, stream_));
        return d;
    }
    template<typename U>
    static bool differs(TensorMap* args, const char* key)
    {
        if (args == nullptr || !args->isExist(key)) {
            return false;
        }
        const Tensor& t = args->at(key);
        for (size_t i = 1; i < t.size(); ++i) {
            if (t.getVal<U>(i) != t.getVal<U>(0)) {
                return true;
            }
        }
        return false;
    }

    void sample(TensorMap* out, TensorMap* in, size_t batch, int step, int ite, size_t lbs, int mil);
    void beam(TensorMap* out, TensorMap* in);
    void stopCriteria(TensorMap* out, TensorMap* in, size_t batch, int step, size_t lbs, size_t lo, size_t beam_width);

    Mode         mode_;
    int          dtype_;
    size_t       vocab_, vocab_padded_;
    cudaStream_t stream_;
    IAllocator*  allocator_;
    bool         free_after_forward_;

    std::vector<std::pair<void*, bool>> owned_;
    size_t                              batch_ = 0, beam_width_ = 1;
    bool                                has_diff_runtime_args_ = false;
    std::vector<float>                  temperature_h_, penalty_h_;
    std::vector<int>                    min_length_h_;
    float*                              temperature_d_ = nullptr;
    float*                              penalty_d_     = nullptr;
    int*                                min_length_d_  = nullptr;
    int                                 penalty_type_  = FTB200_PENALTY_NONE;
    float                               penalty_default_ = 0.0f;
    SamplingState                       topk_, topp_;
    int                                 max_top_k_ = 1;
    std::vector<double>                 row_cost_;
    struct OrderBuf {
        std::vector<int> host;
        int*             dev = nullptr;
    };
    std::map<std::pair<size_t, size_t>, OrderBuf> orders_;  // launch orders by (first row, rows) of a slice
    void*                               workspace_ = nullptr;
    size_t                              workspace_bytes_ = 0;
    void*                               beam_ws_ = nullptr;
    size_t                              beam_ws_bytes_ = 0;
    int*                                count_dev_ = nullptr;
    int*                                count_host_ = nullptr;
};

void DecodeCore::setup(size_t batch_size, size_t beam_width, TensorMap* args)
{
    releaseAll();
    batch_      = batch_size;
    beam_width_ = beam_width;
    // hasDiffRuntimeArgs (DynamicDecodeLayer.cc:477-514): beam search then runs one batch entry at a time
    has_diff_runtime_args_ = differs<float>(args, "beam_search_diversity_rate") || differs<float>(args, "temperature")
                             || differs<float>(args, "len_penalty") || differs<float>(args, "repetition_penalty")
                             || differs<float>(args, "presence_penalty") || differs<int>(args, "min_length");
    if (beam_width != 1 || mode_ == Mode::BeamOnly) {
        return;  // the beam layers have no set-up (BaseBeamSearchLayer.cu:123-127)
    }
    const size_t B = batch_size;
    if (args != nullptr && args->isExist("repetition_penalty") && args->isExist("presence_penalty")) {
        throw std::runtime_error("[FT][ERROR] Found ambiguous parameters repetition_penalty and presence_penalty "
                                 "which are mutually exclusive. Please provide one of repetition_penalty or "
                                 "presence_penalty.");
    }
    // BaseSamplingLayer::setup
    temperature_h_ = broadcast<float>(args, "temperature", B, 1.0f);
    if (args != nullptr && args->isExist("repetition_penalty")) {
        penalty_type_    = FTB200_PENALTY_MULTIPLICATIVE;
        penalty_default_ = 1.0f;
        penalty_h_       = broadcast<float>(args, "repetition_penalty", B, 1.0f);
    }
    else if (args != nullptr && args->isExist("presence_penalty")) {
        penalty_type_    = FTB200_PENALTY_ADDITIVE;
        penalty_default_ = 0.0f;
        penalty_h_       = broadcast<float>(args, "presence_penalty", B, 0.0f);
    }
    else {
        penalty_type_    = FTB200_PENALTY_NONE;
        penalty_default_ = 0.0f;
        penalty_h_.assign(B, 0.0f);
    }
    min_length_h_  = broadcast<int>(args, "min_length", B, 0);
    temperature_d_ = upload(temperature_h_);
    penalty_d_     = upload(penalty_h_);
    min_length_d_  = upload(min_length_h_);

    const Tensor* seeds = (args != nullptr && args->isExist("random_seed")) ? &args->at("random_seed") : nullptr;
    auto init_states = [&](SamplingState& s) {
        s.curand = alloc<char>(B * kCurandStateBytes);
        s.top_ks = alloc<uint32_t>(B);
        s.top_ps = alloc<float>(B);
        s.skip   = alloc<uint8_t>(B);
        s.skip_host.assign(B, 1);
        if (seeds == nullptr) {
            check(ftb200_curand_init(s.curand, (int)B, 0ull, nullptr, stream_));
        }
        else if (seeds->size() == 1) {
            check(ftb200_curand_init(s.curand, (int)B, seeds->getVal<unsigned long long>(0), nullptr, stream_));
        }
        else {
            if (seeds->size() != B) {
                throw std::runtime_error("[FT][ERROR] random_seeds must be of shape [1] or [batch_size]");
            }
            unsigned long long* d = alloc<unsigned long long>(B);
            check_cuda(cudaMemcpyAsync(d, seeds->data, 8 * B, cudaMemcpyHostToDevice, stream_));
            check(ftb200_curand_init(s.curand, (int)B, 0ull, d, stream_));
        }
    };
    const Tensor* top_k = (args != nullptr && args->isExist("runtime_top_k")) ? &args->at("runtime_top_k") : nullptr;
    const Tensor* top_p = (args != nullptr && args->isExist("runtime_top_p")) ? &args->at("runtime_top_p") : nullptr;
    const size_t  nk    = top_k != nullptr ? top_k->size() : 1;
    const size_t  np    = top_p != nullptr ? top_p->size() : 0;
    uint32_t      k_max = 0, k_first = 0;
    for (size_t i = 0; top_k != nullptr && i < nk; ++i) {
        k_max = std::max(k_max, top_k->getVal<uint32_t>(i));
    }
    if (top_k != nullptr) {
        k_first = top_k->getVal<uint32_t>(0);
    }
    const float p_scalar = top_p != nullptr ? top_p->getVal<float>(0) : 0.0f;
    auto fetch_skip = [&](SamplingState& s) {
        std::vector<uint8_t> h(B);
        check_cuda(cudaMemcpyAsync(h.data(), s.skip, B, cudaMemcpyDeviceToHost, stream_));
        check_cuda(cudaStreamSynchronize(stream_));
        s.skip_host.assign(h.begin(), h.end());
    };
    if (mode_ != Mode::TopPOnly) {
        // TopKSamplingLayer::setup
        init_states(topk_);
        if (nk > 1) {
            check_cuda(cudaMemcpyAsync(topk_.top_ks, top_k->data, 4 * B, cudaMemcpyHostToDevice, stream_));
        }
        if (np > 1) {
            check_cuda(cudaMemcpyAsync(topk_.top_ps, top_p->data, 4 * B, cudaMemcpyHostToDevice, stream_));
        }
        check(ftb200_setup_topk_runtime_args((int)B, k_max, topk_.top_ks, (int)nk, p_scalar, topk_.top_ps, (int)np,
                                             topk_.skip, stream_));
        fetch_skip(topk_);
        std::vector<uint32_t> ks(B);
        check_cuda(cudaMemcpyAsync(ks.data(), topk_.top_ks, 4 * B, cudaMemcpyDeviceToHost, stream_));
        check_cuda(cudaStreamSynchronize(stream_));
        max_top_k_    = (int)*std::max_element(ks.begin(), ks.end());
        topk_.active  = true;
        row_cost_.assign(B, 1.0);
        for (size_t i = 0; i < B; ++i) {
            row_cost_[i] = 1.0 + ks[i] / 128.0;
        }
    }
    if (mode_ != Mode::TopKOnly && top_p != nullptr) {
        // TopPSamplingLayer::setup
        init_states(topp_);
        topp_.initial = alloc<float>(B);
        topp_.decay   = alloc<float>(B);
        topp_.pmin    = alloc<float>(B);
        topp_.reset   = alloc<int32_t>(B);
        if (nk > 1) {
            check_cuda(cudaMemcpyAsync(topp_.top_ks, top_k->data, 4 * B, cudaMemcpyHostToDevice, stream_));
        }
        if (np > 1) {
            check_cuda(cudaMemcpyAsync(topp_.top_ps, top_p->data, 4 * B, cudaMemcpyHostToDevice, stream_));
        }
        check(ftb200_setup_topp_runtime_args(
            (int)B, k_first, topp_.top_ks, (int)nk, p_scalar, topp_.top_ps, (int)np, topp_.skip, topp_.initial,
            topp_.decay, args->getPtr<float>("top_p_decay"), topp_.pmin, args->getPtr<float>("top_p_min"), topp_.reset,
            args->getPtr<uint32_t>("top_p_reset_ids"), stream_));
        fetch_skip(topp_);
        topp_.active = true;
        // top-p rows cost most (several reads of the row), then top-k by k: start the expensive rows first
        std::vector<float> ps(B);
        check_cuda(cudaMemcpyAsync(ps.data(), topp_.top_ps, 4 * B, cudaMemcpyDeviceToHost, stream_));
        check_cuda(cudaStreamSynchronize(stream_));
        if (row_cost_.size() != B) {
            row_cost_.assign(B, 1.0);
        }
        for (size_t i = 0; i < B; ++i) {
            if (!topk_.active || topk_.skip_host[i]) {
                row_cost_[i] = 10.0 + 8.0 * ps[i];
            }
        }
    }
    // the launch orders follow the new arguments: their buffers go back to the allocator
    for (auto& kv : orders_) {
        void* p = kv.second.dev;
        for (auto it = owned_.begin(); it != owned_.end(); ++it) {
            if (it->first == p) {
                owned_.erase(it);
                break;
            }
        }
        allocator_->free(&p, false);
    }
    orders_.clear();
}

// What the reference's BaseSamplingLayer<T>::forward asserts before it touches the logits
// (BaseSamplingLayer.cc:253-290): the step's tensors are there and the slice lies inside the batch set up.
void DecodeCore::checkStep(TensorMap* out, TensorMap* in) const
{
    if (out == nullptr || in == nullptr) {
        throw std::runtime_error("[FT][ERROR] forward() needs both tensor maps");
    }
    for (const char* key : {"logits", "step", "max_input_length", "end_id"}) {
        if (!in->isExist(key)) {
            throw std::runtime_error(std::string("[FT][ERROR] Cannot find a tensor of name ") + key + " in the tensor map");
        }
    }
    if (!out->isExist("output_ids")) {
        throw std::runtime_error("[FT][ERROR] Cannot find a tensor of name output_ids in the tensor map");
    }
    const Tensor& logits = in->at("logits");
    const size_t  B      = logits.shape.empty() ? 0 : logits.shape[0];
    const size_t  lbs    = in->isExist("local_batch_size") ? (size_t)in->getVal<int>("local_batch_size") : B;
    const size_t  ite    = (size_t)in->getVal<uint32_t>("ite", 0u);
    if (batch_ == 0 || lbs == 0 || (ite + 1) * lbs > batch_) {
        throw std::runtime_error("[FT][ERROR] the slice [ite * local_batch_size, (ite + 1) * local_batch_size) lies "
                                 "outside the batch given to setup()");
    }
}

void DecodeCore::forward(TensorMap* out, TensorMap* in)
{
    const Tensor& logits = in->at("logits");
    if (mode_ == Mode::BeamOnly || (logits.shape.size() == 3 && logits.shape[1] > 1)) {
        beam(out, in);
        return;
    }
    const size_t B    = logits.shape[0];
    const int    step = in->getVal<int>("step");
    const int    ite  = (int)in->getVal<uint32_t>("ite", 0u);
    const size_t lbs  = in->isExist("local_batch_size") ? (size_t)in->getVal<int>("local_batch_size") : B;
    const int    mil  = in->getVal<int>("max_input_length");
    sample(out, in, B, step, ite, lbs, mil);
    if (mode_ == Mode::Dispatcher) {
        stopCriteria(out, in, B, step, lbs, (size_t)ite * lbs, 1);
    }
    if (free_after_forward_) {
        // the reference frees its workspaces here; the per-row argument buffers and curand states stay
        void* p = workspace_;
        if (p != nullptr) {
            for (auto it = owned_.begin(); it != owned_.end(); ++it) {
                if (it->first == p) {
                    owned_.erase(it);
                    break;
                }
            }
            allocator_->free(&p, false);
            workspace_ = nullptr, workspace_bytes_ = 0;
        }
    }
}

void DecodeCore::sample(TensorMap* out, TensorMap* in, size_t B, int step, int ite, size_t lbs, int mil)
{
    const size_t lo = (size_t)ite * lbs;
    auto all_skipped = [&](const SamplingState& s) {
        if (!s.active) {
            return true;
        }
        for (size_t i = lo; i < lo + lbs; ++i) {
            if (!s.skip_host[i]) {
                return false;
            }
        }
        return true;
    };
    const bool topk_on = !all_skipped(topk_), topp_on = !all_skipped(topp_);
    if (!topk_on && !topp_on) {
        return;
    }
    const Tensor& logits = in->at("logits");
    const size_t  es     = dtype_ == FTB200_F32 ? 4 : 2;

    ftb200_sampling_params p;
    std::memset(&p, 0, sizeof(p));
    p.dtype             = dtype_;
    p.batch_size        = (int)B;
    p.local_batch_size  = (int)lbs;
    p.ite               = ite;
    p.vocab_size        = (int)vocab_;
    p.vocab_size_padded = (int)vocab_padded_;
    p.step              = step;
    p.max_input_length  = mil;
    p.logits            = (const char*)logits.data + lo * vocab_padded_ * es;
    p.embedding_bias    = in->getPtr<void>("embedding_bias");
    p.end_ids           = in->at("end_id").getPtrWithOffset<int>(lo);
    p.input_lengths     = in->isExist("input_lengths") ? in->at("input_lengths").getPtrWithOffset<int>(lo) : nullptr;
    p.output_ids        = out->at("output_ids").getPtr<int>();
    if (in->isExist("bad_words_list")) {
        const Tensor& bw     = in->at("bad_words_list");
        const bool    shared = bw.shape.size() == 2 || bw.shape[0] == 1;
        const size_t  L      = bw.shape.back();
        p.bad_words          = shared ? bw.getPtr<int>() : bw.getPtrWithOffset<int>(lo * 2 * L);
        p.bad_words_len      = (int)L;
        p.bad_words_shared   = shared ? 1 : 0;
    }
    // host-side gating of the penalty kernels (BaseSamplingLayer.cc:302-349)
    bool temp = false, pen = false;
    int  minlen = 0;
    for (size_t i = lo; i < lo + lbs; ++i) {
        temp   = temp || temperature_h_[i] != 1.0f;
        pen    = pen || penalty_h_[i] != penalty_default_;
        minlen = std::max(minlen, min_length_h_[i]);
    }
    p.temperature        = temperature_d_ + lo;
    p.apply_temperature  = (p.embedding_bias != nullptr || temp) ? 1 : 0;
    p.repetition_penalty = penalty_d_ + lo;
    p.penalty_type       = penalty_type_;
    p.apply_repetition   = (step > 1 && penalty_type_ != FTB200_PENALTY_NONE && pen) ? 1 : 0;
    p.min_lengths        = min_length_d_ + lo;
    p.apply_min_length   = minlen > step - mil ? 1 : 0;
    if (topk_on) {
        p.topk_states = (char*)topk_.curand + lo * kCurandStateBytes;
        p.topk_ks     = topk_.top_ks + lo;
        p.topk_ps     = topk_.top_ps + lo;
        p.topk_skip   = topk_.skip + lo;
        p.max_top_k   = max_top_k_;
    }
    if (topp_on) {
        p.topp_states     = (char*)topp_.curand + lo * kCurandStateBytes;
        p.topp_ps         = topp_.top_ps + lo;
        p.topp_skip       = topp_.skip + lo;
        p.topp_initial_ps = topp_.initial + lo;
        p.topp_decay      = topp_.decay + lo;
        p.topp_min        = topp_.pmin + lo;
        p.topp_reset_ids  = topp_.reset + lo;
    }
    p.sequence_length = out->isExist("sequence_length") ? out->at("sequence_length").getPtrWithOffset<int>(lo) : nullptr;
    p.finished        = out->isExist("finished") ? out->at("finished").getPtrWithOffset<uint8_t>(lo) : nullptr;
    p.cum_log_probs   = out->isExist("cum_log_probs") ? out->at("cum_log_probs").getPtrWithOffset<float>(lo) : nullptr;
    if (out->isExist("output_log_probs")) {
        // [request_output_len, batch] sliced at (step - max_input_length) (DynamicDecodeLayer.cc:427-435)
        p.output_log_probs = out->at("output_log_probs").getPtrWithOffset<float>((size_t)(step - mil) * B + lo);
    }
    // Launch order of the slice (costliest rows first), one device buffer per (first row, rows) pair seen since
    // the last setup(): a caller that walks its micro-batches with `ite` gets every order built once, and
    // forward() neither allocates nor waits for the stream after that.
    auto ord_it = orders_.find({lo, lbs});
    if (ord_it == orders_.end()) {
        OrderBuf ob;
        ob.host.resize(lbs);
        std::iota(ob.host.begin(), ob.host.end(), 0);
        std::stable_sort(ob.host.begin(), ob.host.end(),
                         [&](int a, int b) { return row_cost_[lo + a] > row_cost_[lo + b]; });
        ob.dev = alloc<int>(lbs);
        ord_it = orders_.emplace(std::make_pair(lo, lbs), std::move(ob)).first;
        // (the host vector lives in the map, so the copy may complete after this call returns)
        check_cuda(cudaMemcpyAsync(ord_it->second.dev, ord_it->second.host.data(), 4 * lbs, cudaMemcpyHostToDevice,
                                   stream_));
    }
    p.row_order = ord_it->second.dev;
    size_t need = 0;
    check(ftb200_sampling_workspace_bytes(dtype_, (int)lbs, (int)vocab_padded_, &need));
    if (workspace_ == nullptr || workspace_bytes_ < need) {
        workspace_       = alloc<char>(need);
        workspace_bytes_ = need;
    }
    p.workspace       = workspace_;
    p.workspace_bytes = workspace_bytes_;
    p.stream          = stream_;
    check(ftb200_decode_step_sampling(&p));
}

void DecodeCore::beam(TensorMap* out, TensorMap* in)
{
    const Tensor& logits = in->at("logits");
    const size_t  B = logits.shape[0], K = logits.shape[1], Vp = logits.shape[2];
    const int     step = in->getVal<int>("step");
    const int     ite  = (int)in->getVal<uint32_t>("ite", 0u);
    const size_t  lbs  = in->isExist("local_batch_size") ? (size_t)in->getVal<int>("local_batch_size") : B;
    const int     mil  = in->getVal<int>("max_input_length");
    const size_t  es   = dtype_ == FTB200_F32 ? 4 : 2;
    const Tensor& ids  = out->at("output_ids");
    const size_t  L    = ids.shape[0];
    if (!out->isExist("cum_log_probs")) {
        throw std::runtime_error("[FT][ERROR] cum_log_probs should be provided in beam search.");
    }
    if (in->isExist("bad_words_list")) {
        const Tensor& bw     = in->at("bad_words_list");
        const bool    shared = bw.shape.size() == 2 || bw.shape[0] == 1;
        const size_t  Lw     = bw.shape.back();
        check(ftb200_ban_bad_words((char*)logits.data + (size_t)ite * lbs * K * Vp * es, dtype_, ids.getPtr<int>(),
                                   out->at("parent_ids").getPtr<int>(), (int)B, (int)lbs, (int)K,
                                   shared ? bw.getPtr<int>() : bw.getPtrWithOffset<int>((size_t)ite * lbs * 2 * Lw),
                                   shared ? 1 : 0, (int)Lw, (int)((size_t)ite * lbs), (int)Vp, step, stream_));
    }
    if (in->isExist("repetition_penalty") && in->isExist("presence_penalty")) {
        throw std::runtime_error("[FT][ERROR] Found ambiguous parameters repetition_penalty and presence_penalty "
                                 "which are mutually exclusive.");
    }
    const size_t sub   = has_diff_runtime_args_ ? 1 : lbs;
    const size_t n_sub = lbs / sub;
    size_t       need  = 0;
    check(ftb200_beam_workspace_bytes((int)sub, (int)K, &need));
    if (beam_ws_ == nullptr || beam_ws_bytes_ < need) {
        beam_ws_       = alloc<char>(need);
        beam_ws_bytes_ = need;
    }
    for (size_t d = (size_t)ite * n_sub; d < ((size_t)ite + 1) * n_sub; ++d) {
        const size_t row0 = d * sub * K;
        // per sub-batch scalars: entry d of a [batch] argument when the arguments differ, else entry 0
        auto scalar_f = [&](const char* key, float def) {
            if (!in->isExist(key)) {
                return def;
            }
            const Tensor& t = in->at(key);
            return t.getVal<float>(t.size() > 1 ? d * sub : 0);
        };
        ftb200_beam_params p;
        std::memset(&p, 0, sizeof(p));
        p.dtype = dtype_, p.batch_size = (int)B, p.local_batch_size = (int)sub, p.ite = (int)d, p.beam_width = (int)K;
        p.vocab_size = (int)vocab_, p.vocab_size_padded = (int)Vp, p.step = step, p.max_input_length = mil;
        p.max_seq_len    = (int)L;
        p.logits         = (const char*)logits.data + row0 * Vp * es;
        p.embedding_bias = in->getPtr<void>("embedding_bias");
        p.end_ids        = in->at("end_id").getPtrWithOffset<int>(d * sub);
        p.input_lengths  = in->isExist("input_lengths") ? in->at("input_lengths").getPtrWithOffset<int>(row0) : nullptr;
        p.temperature    = scalar_f("temperature", 1.0f);
        if (in->isExist("repetition_penalty")) {
            p.penalty_type = FTB200_PENALTY_MULTIPLICATIVE, p.repetition_penalty = scalar_f("repetition_penalty", 1.0f);
        }
        else if (in->isExist("presence_penalty")) {
            p.penalty_type = FTB200_PENALTY_ADDITIVE, p.repetition_penalty = scalar_f("presence_penalty", 0.0f);
        }
        else {
            p.penalty_type = FTB200_PENALTY_NONE, p.repetition_penalty = 1.0f;
        }
        if (in->isExist("min_length")) {
            const Tensor& t = in->at("min_length");
            p.min_length    = t.getVal<int>(t.size() > 1 ? d * sub : 0);
        }
        p.diversity_rate   = scalar_f("beam_search_diversity_rate", 0.0f);
        p.length_penalty   = scalar_f("len_penalty", 0.0f);
        p.output_ids       = ids.getPtr<int>();
        p.parent_ids       = out->at("parent_ids").getPtr<int>();
        p.finished         = out->at("finished").getPtrWithOffset<uint8_t>(row0);
        p.sequence_length  = out->at("sequence_length").getPtrWithOffset<int>(row0);
        p.cum_log_probs    = out->at("cum_log_probs").getPtrWithOffset<float>(row0);
        p.output_log_probs = out->isExist("output_log_probs") ? out->at("output_log_probs").getPtr<float>() : nullptr;
        p.src_cache_indirection = in->getPtr<int>("src_cache_indirection");
        p.tgt_cache_indirection = out->getPtr<int>("tgt_cache_indirection");
        // beam_hyps: a host pointer; outside a FasterTransformer checkout it points to an ftb200_beam_hyps
        p.beam_hyps       = out->isExist("beam_hyps") ? out->at("beam_hyps").getPtr<const ftb200_beam_hyps>() : nullptr;
        p.workspace       = beam_ws_;
        p.workspace_bytes = beam_ws_bytes_;
        p.stream          = stream_;
        check(ftb200_beam_search_step(&p));
    }
    stopCriteria(out, in, B, step, lbs, (size_t)ite * lbs, K);
}

void DecodeCore::stopCriteria(TensorMap* out, TensorMap* in, size_t B, int step, size_t lbs, size_t lo, size_t beam_width)
{
    // stop words, length limit and should_stop (DynamicDecodeLayer.cc:447-473)
    const bool has_sw = in->isExist("stop_words_list"), has_lim = in->isExist("sequence_limit_length");
    if (!has_sw && !has_lim) {
        return;
    }
    if (count_dev_ == nullptr) {
        count_dev_  = alloc<int>(1);
        count_host_ = alloc<int>(1, true);
    }
    size_t     L  = 0;
    const int* sw = nullptr;
    if (has_sw) {
        const Tensor& t = in->at("stop_words_list");
        L               = t.shape.back();
        sw              = t.getPtrWithOffset<int>(lo * 2 * L);
    }
    check(ftb200_stop_criteria(out->at("output_ids").getPtr<int>(), out->getPtr<int>("parent_ids"), sw, (int)L,
                               out->at("finished").getPtr<uint8_t>(),
                               has_lim ? in->at("sequence_limit_length").getPtr<uint32_t>() : nullptr,
                               (int)(lo * beam_width), (int)lbs, (int)B, (int)beam_width, step, count_dev_, count_host_,
                               stream_));
    if (has_lim && out->isExist("should_stop")) {
        int stop = 0;
        check(ftb200_wait_should_stop(count_host_, (int)B, (int)beam_width, stream_, 10000, &stop));
        *out->at("should_stop").getPtr<bool>() = stop != 0;
    }
}

}  // namespace ftb200_detail

using ftb200_detail::DecodeCore;
using ftb200_detail::DtypeOf;
using ftb200_detail::Mode;

// ---- DynamicDecodeLayer ---------------------------------------------------------------------------
template<typename T>
DynamicDecodeLayer<T>::DynamicDecodeLayer(size_t vocab_size, size_t vocab_size_padded, int, cudaStream_t stream,
                                          cublasMMWrapper*, IAllocator* allocator, bool is_free_buffer_after_forward,
                                          cudaDeviceProp*):
    core_(new DecodeCore(Mode::Dispatcher, DtypeOf<T>::value, vocab_size, vocab_size_padded, stream, allocator,
                         is_free_buffer_after_forward))
{
}
template<typename T>
DynamicDecodeLayer<T>::~DynamicDecodeLayer() = default;
template<typename T>
DynamicDecodeLayer<T>::DynamicDecodeLayer(DynamicDecodeLayer const& other): core_(other.core_->cloneConfiguration())
{
    // like the reference's copy constructor: fresh sub-layers with the same configuration; what setup()
    // stored is not carried over, a copy has to be set up before use
}
template<typename T>
void DynamicDecodeLayer<T>::setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args)
{
    core_->setup(batch_size, beam_width, runtime_args);
}
template<typename T>
void DynamicDecodeLayer<T>::setStream(cudaStream_t stream)
{
    core_->setStream(stream);
}

template<typename T>
cudaStream_t DynamicDecodeLayer<T>::getStream()
{
    return core_->getStream();
}

template<typename T>
void DynamicDecodeLayer<T>::forward(TensorMap* output_tensors, TensorMap* input_tensors)
{
    core_->forward(output_tensors, input_tensors);
}
template<typename T>
void DynamicDecodeLayer<T>::forward(std::unordered_map<std::string, Tensor>*       output_tensors,
                                    const std::unordered_map<std::string, Tensor>* input_tensors)
{
    TensorMap in(*input_tensors), out(*output_tensors);
    core_->forward(&out, &in);
}

// ---- the sampling layers on their own ---------------------------------------------------------------
template<typename T>
BaseSamplingLayer<T>::BaseSamplingLayer(size_t, size_t vocab_size, size_t vocab_size_padded, int, size_t top_k, float,
                                        unsigned long long, float, float, float, cudaStream_t stream, cublasMMWrapper*,
                                        IAllocator* allocator, bool is_free_buffer_after_forward, cudaDeviceProp*):
    vocab_size_(vocab_size),
    vocab_size_padded_(vocab_size_padded),
    core_(new DecodeCore(top_k > 0 ? Mode::TopKOnly : Mode::TopPOnly, DtypeOf<T>::value, vocab_size, vocab_size_padded,
                         stream, allocator, is_free_buffer_after_forward))
{
    // the per-layer defaults (top_k, top_p, temperature, penalties, seed) are dead arguments in the reference
    // too: setup() reads everything from runtime_args (BaseSamplingLayer.cc:120-206)
}
template<typename T>
BaseSamplingLayer<T>::BaseSamplingLayer(BaseSamplingLayer const& other):
    vocab_size_(other.vocab_size_), vocab_size_padded_(other.vocab_size_padded_), core_(other.core_->cloneConfiguration())
{
}
template<typename T>
BaseSamplingLayer<T>::~BaseSamplingLayer() = default;
template<typename T>
void BaseSamplingLayer<T>::setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args)
{
    core_->setup(batch_size, beam_width, runtime_args);
}
template<typename T>
void BaseSamplingLayer<T>::forward(TensorMap* output_tensors, TensorMap* input_tensors)
{
    core_->checkStep(output_tensors, input_tensors);
    runSampling(output_tensors, input_tensors);
}
template<typename T>
void BaseSamplingLayer<T>::forward(std::unordered_map<std::string, Tensor>*       output_tensors,
                                   const std::unordered_map<std::string, Tensor>* input_tensors)
{
    TensorMap in(*input_tensors), out(*output_tensors);
    forward(&out, &in);
}
template<typename T>
void BaseSamplingLayer<T>::forward(std::vector<Tensor>*, const std::vector<Tensor>*)
{
    throw std::runtime_error("[FT][ERROR] the positional forward() of a sampling layer is not supported");
}
template<typename T>
void BaseSamplingLayer<T>::setStream(cudaStream_t stream)
{
    core_->setStream(stream);
}
template<typename T>
cudaStream_t BaseSamplingLayer<T>::getStream()
{
    return core_->getStream();
}

template<typename T>
TopKSamplingLayer<T>::TopKSamplingLayer(size_t max_batch_size, size_t vocab_size, size_t vocab_size_padded, int end_id,
                                        size_t top_k, unsigned long long random_seed, float temperature,
                                        float len_penalty, float repetition_penalty, cudaStream_t stream,
                                        cublasMMWrapper* cublas_wrapper, IAllocator* allocator,
                                        bool is_free_buffer_after_forward):
    BaseSamplingLayer<T>(max_batch_size, vocab_size, vocab_size_padded, end_id, top_k > 0 ? top_k : 1, 0.0f, random_seed,
                         temperature, len_penalty, repetition_penalty, stream, cublas_wrapper, allocator,
                         is_free_buffer_after_forward, nullptr)
{
}
template<typename T>
TopKSamplingLayer<T>::TopKSamplingLayer(TopKSamplingLayer<T> const& other): BaseSamplingLayer<T>(other)
{
}
template<typename T>
TopKSamplingLayer<T>::~TopKSamplingLayer() = default;
template<typename T>
void TopKSamplingLayer<T>::setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args)
{
    BaseSamplingLayer<T>::setup(batch_size, beam_width, runtime_args);
}
template<typename T>
void TopKSamplingLayer<T>::runSampling(TensorMap* output_tensors, TensorMap* input_tensors)
{
    core_->forward(output_tensors, input_tensors);
}

template<typename T>
TopPSamplingLayer<T>::TopPSamplingLayer(size_t max_batch_size, size_t vocab_size, size_t vocab_size_padded, int end_id,
                                        float top_p, unsigned long long random_seed, float temperature,
                                        float len_penalty, float repetition_penalty, cudaStream_t stream,
                                        cublasMMWrapper* cublas_wrapper, IAllocator* allocator,
                                        bool is_free_buffer_after_forward, cudaDeviceProp* cuda_device_prop):
    BaseSamplingLayer<T>(max_batch_size, vocab_size, vocab_size_padded, end_id, 0, top_p, random_seed, temperature,
                         len_penalty, repetition_penalty, stream, cublas_wrapper, allocator,
                         is_free_buffer_after_forward, cuda_device_prop)
{
}
template<typename T>
TopPSamplingLayer<T>::TopPSamplingLayer(TopPSamplingLayer<T> const& other): BaseSamplingLayer<T>(other)
{
}
template<typename T>
TopPSamplingLayer<T>::~TopPSamplingLayer() = default;
template<typename T>
void TopPSamplingLayer<T>::setup(const size_t batch_size, const size_t beam_width, TensorMap* runtime_args)
{
    BaseSamplingLayer<T>::setup(batch_size, beam_width, runtime_args);
}
template<typename T>
void TopPSamplingLayer<T>::runSampling(TensorMap* output_tensors, TensorMap* input_tensors)
{
    core_->forward(output_tensors, input_tensors);
}

// ---- online beam search -----------------------------------------------------------------------------
template<typename T>
OnlineBeamSearchLayer<T>::OnlineBeamSearchLayer(size_t, size_t, size_t, size_t, size_t vocab_size,
                                                size_t vocab_size_padded, int, float, float, float, float,
                                                cudaStream_t stream, cublasMMWrapper*, IAllocator* allocator,
                                                bool is_free_buffer_after_forward):
    core_(new DecodeCore(Mode::BeamOnly, DtypeOf<T>::value, vocab_size, vocab_size_padded, stream, allocator,
                         is_free_buffer_after_forward))
{
}
template<typename T>
OnlineBeamSearchLayer<T>::~OnlineBeamSearchLayer() = default;
template<typename T>
void OnlineBeamSearchLayer<T>::setup(const size_t batch_size, TensorMap* runtime_args)
{
    core_->setup(batch_size, 0, runtime_args);
}
template<typename T>
void OnlineBeamSearchLayer<T>::forward(TensorMap* output_tensors, TensorMap* input_tensors)
{
    core_->forward(output_tensors, input_tensors);
}

#define FTB200_INSTANTIATE(T)                                                                                          \
    template class DynamicDecodeLayer<T>;                                                                              \
    template class BaseSamplingLayer<T>;                                                                               \
    template class TopKSamplingLayer<T>;                                                                               \
    template class TopPSamplingLayer<T>;                                                                               \
    template class OnlineBeamSearchLayer<T>;
FTB200_INSTANTIATE(float)
FTB200_INSTANTIATE(half)
FTB200_INSTANTIATE(__nv_bfloat16)

}  // namespace fastertransformer
