// Test driver for the C++ decode layers (fastertransformer_b200/shim): runs a few decode steps through
// fastertransformer::DynamicDecodeLayer<T> on seeded inputs and prints the ids of every step, one line per
// step.  tests/test_shim_gpu.py feeds the same inputs to the Python host mirror and compares the lines.
//
//   shim_driver <dtype: f32|f16|bf16> <batch> <vocab> <steps> <case>
//     topk | topp | mixed | beam   through DynamicDecodeLayer<T>
//     topk_layer | topp_layer      through TopKSamplingLayer<T> / TopPSamplingLayer<T>, held and called as
//                                  BaseSamplingLayer<T>* (setup, forward -> runSampling)
//     slices                       the mixed case with the batch sent in two slices per step (ite 0 and 1); the
//                                  allocator counts live allocations and the run fails if that count moves after
//                                  the first step
//     e2e                          the mixed case timed end to end: every step copies the logits from pinned host
//                                  memory, runs forward() and reads the step's ids back; prints one line
//                                  "e2e tokens_per_s=... ms_per_step=... steps=... h2d_bytes=... d2h_bytes=..."
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "DynamicDecodeLayer.h"

using namespace fastertransformer;

static uint64_t mix(uint64_t x)  // splitmix64 finaliser: value i of the stream is mix(seed + i)
{
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}
static float unit(uint64_t seed, uint64_t i)  // in [-4, 4), a multiple of 1/8192: exact in every logits type
{
    return (float)((int)(mix(seed + i) >> 48) - 32768) / 8192.0f;
}

template<typename T>
static T convert(float x);
template<>
float convert<float>(float x) { return x; }
template<>
half convert<half>(float x) { return __float2half(x); }
template<>
__nv_bfloat16 convert<__nv_bfloat16>(float x) { return __float2bfloat16(x); }

template<typename U>
static U* to_device(const std::vector<U>& v)
{
    U* d = nullptr;
    cudaMalloc(&d, sizeof(U) * v.size());
    cudaMemcpy(d, v.data(), sizeof(U) * v.size(), cudaMemcpyHostToDevice);
    return d;
}

// CudaAllocator that counts what is live.
class CountingAllocator: public CudaAllocator {
public:
    mutable long live = 0, total = 0;
    void*        malloc(size_t size, const bool is_set_zero = true, bool is_host = false) override
    {
        void* p = CudaAllocator::malloc(size, is_set_zero, is_host);
        if (p != nullptr) {
            ++live, ++total;
        }
        return p;
    }
    void free(void** ptr, bool is_host = false) const override
    {
        if (ptr != nullptr && *ptr != nullptr) {
            --live;
        }
        CudaAllocator::free(ptr, is_host);
    }
};

// End-to-end rate of DynamicDecodeLayer<T>::forward with host buffers: two pinned logits buffers alternate, the
// copy of the next step's logits runs on a second stream under this step's kernels, the ids of every step are
// read back before the next forward() is issued.  All copies lie inside the timed region.
template<typename T>
static int run_e2e(DataType dt, int B, int V, int steps)
{
    const int     mil = 4, warm = 3, L = mil + warm + steps;
    cudaStream_t  stream, copy_stream;
    cudaStreamCreate(&stream);
    cudaStreamCreate(&copy_stream);
    CudaAllocator alloc;
    alloc.setStream(stream);
    DynamicDecodeLayer<T> layer(V, V, V - 1, stream, nullptr, &alloc, false, nullptr);
    std::vector<uint32_t>           top_k(B);
    std::vector<float>              top_p(B), rep(1, 1.2f);
    std::vector<unsigned long long> seeds(B);
    for (int i = 0; i < B; ++i) {
        const uint32_t ks[4] = {0, 1, 8, 64};
        const float    ps[3] = {0.0f, 0.5f, 0.9f};
        top_k[i] = ks[i % 4], top_p[i] = ps[(i / 4) % 3], seeds[i] = 100 + 7 * i;
    }
    TensorMap args;
    args.insert("runtime_top_k", Tensor(MEMORY_CPU, TYPE_UINT32, {(size_t)B}, top_k.data()));
    args.insert("runtime_top_p", Tensor(MEMORY_CPU, TYPE_FP32, {(size_t)B}, top_p.data()));
    args.insert("repetition_penalty", Tensor(MEMORY_CPU, TYPE_FP32, {1}, rep.data()));
    args.insert("random_seed", Tensor(MEMORY_CPU, TYPE_UINT64, {(size_t)B}, seeds.data()));
    layer.setup(B, 1, &args);

    std::vector<int> ids_h((size_t)L * B, 0);
    for (int t = 0; t < mil; ++t) {
        for (int b = 0; b < B; ++b) {
            ids_h[(size_t)t * B + b] = (int)(mix(9000 + t * 131 + b) % (uint64_t)V);
        }
    }
    int*      output_ids = to_device(ids_h);
    uint8_t*  finished   = to_device(std::vector<uint8_t>((size_t)B, 0));
    int*      seq_len    = to_device(std::vector<int>((size_t)B, mil));
    int*      end_ids    = to_device(std::vector<int>(B, V - 1));
    int*      in_len     = to_device(std::vector<int>((size_t)B, mil));
    uint32_t* seq_lim    = to_device(std::vector<uint32_t>(B, (uint32_t)L + 1));
    const size_t n = (size_t)B * V;
    T *          host[2], *dev[2];
    int*         ids_back = nullptr;
    cudaMallocHost(&ids_back, sizeof(int) * B);
    for (int b = 0; b < 2; ++b) {
        cudaMallocHost(&host[b], sizeof(T) * n);
        cudaMalloc(&dev[b], sizeof(T) * n);
        for (size_t i = 0; i < n; ++i) {
            host[b][i] = convert<T>(unit(1000003ull * (b + 1), i));
        }
    }
    cudaEvent_t copied[2], consumed[2], t0, t1;
    for (int b = 0; b < 2; ++b) {
        cudaEventCreateWithFlags(&copied[b], cudaEventDisableTiming);
        cudaEventCreateWithFlags(&consumed[b], cudaEventDisableTiming);
    }
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    bool should_stop = false;
    auto copy_in     = [&](int i) {
        const int b = i % 2;
        cudaStreamWaitEvent(copy_stream, consumed[b], 0);
        cudaMemcpyAsync(dev[b], host[b], sizeof(T) * n, cudaMemcpyHostToDevice, copy_stream);
        cudaEventRecord(copied[b], copy_stream);
    };
    auto one_step = [&](int i, int step) {
        const int b      = i % 2;
        int       step_v = step, mil_v = mil, lbs_v = B;
        uint32_t  ite_v = 0;
        TensorMap in, out;
        in.insert("logits", Tensor(MEMORY_GPU, dt, {(size_t)B, (size_t)V}, dev[b]));
        in.insert("step", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &step_v));
        in.insert("max_input_length", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &mil_v));
        in.insert("ite", Tensor(MEMORY_CPU, TYPE_UINT32, {1}, &ite_v));
        in.insert("local_batch_size", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &lbs_v));
        in.insert("end_id", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B}, end_ids));
        in.insert("input_lengths", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B}, in_len));
        in.insert("sequence_limit_length", Tensor(MEMORY_GPU, TYPE_UINT32, {(size_t)B}, seq_lim));
        out.insert("output_ids", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)L, (size_t)B, 1}, output_ids));
        out.insert("finished", Tensor(MEMORY_GPU, TYPE_BOOL, {(size_t)B}, finished));
        out.insert("sequence_length", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B}, seq_len));
        out.insert("should_stop", Tensor(MEMORY_CPU, TYPE_BOOL, {1}, &should_stop));
        cudaStreamWaitEvent(stream, copied[b], 0);
        layer.forward(&out, &in);
        cudaEventRecord(consumed[b], stream);
        cudaMemcpyAsync(ids_back, output_ids + (size_t)step * B, sizeof(int) * B, cudaMemcpyDeviceToHost, stream);
        cudaStreamSynchronize(stream);
    };
    int i = 0;
    for (int b = 0; b < 2; ++b) {
        cudaEventRecord(consumed[b], stream);
    }
    copy_in(0);
    for (; i < warm; ++i) {
        copy_in(i + 1);
        one_step(i, mil + i);
    }
    cudaDeviceSynchronize();
    // the buffer of step `warm` was copied during the warm-up; copy it again inside the timed region
    cudaEventRecord(t0, stream);
    copy_in(i);
    for (; i < warm + steps; ++i) {
        if (i + 1 < warm + steps) {
            copy_in(i + 1);
        }
        one_step(i, mil + i);
    }
    cudaEventRecord(t1, stream);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        std::fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(e));
        return 2;
    }
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, t0, t1);
    std::printf("e2e tokens_per_s=%.1f ms_per_step=%.4f steps=%d h2d_bytes=%zu d2h_bytes=%zu\n",
                (double)B * steps / (ms * 1e-3), ms / steps, steps, sizeof(T) * n, sizeof(int) * (size_t)B);
    return 0;
}

template<typename T>
static int run(DataType dt, int B, int V, int steps, std::string which)
{
    if (which == "e2e") {
        return run_e2e<T>(dt, B, V, steps);
    }
    const int     K   = which == "beam" ? 4 : 1;
    const int     mil = 4, L = mil + steps;
    cudaStream_t  stream;
    cudaStreamCreate(&stream);
    CountingAllocator alloc;
    alloc.setStream(stream);
    const bool slices = which == "slices";
    std::unique_ptr<DynamicDecodeLayer<T>> dispatcher;
    std::unique_ptr<BaseSamplingLayer<T>>  sampler;  // the derived layers are used through the base's interface
    if (which == "topk_layer") {
        sampler.reset(new TopKSamplingLayer<T>(B, V, V, V - 1, 1, 0ull, 1.0f, 1.0f, 1.0f, stream, nullptr, &alloc, false));
        which = "topk";
    }
    else if (which == "topp_layer") {
        sampler.reset(new TopPSamplingLayer<T>(B, V, V, V - 1, 0.5f, 0ull, 1.0f, 1.0f, 1.0f, stream, nullptr, &alloc, false,
                                               nullptr));
        which = "topp";
    }
    else {
        dispatcher.reset(new DynamicDecodeLayer<T>(V, V, V - 1, stream, nullptr, &alloc, false, nullptr));
        if (slices) {
            which = "mixed";
        }
    }
    std::function<void(size_t, size_t, TensorMap*)> do_setup = [&](size_t b, size_t k, TensorMap* a) {
        sampler ? sampler->setup(b, k, a) : dispatcher->setup(b, k, a);
    };
    std::function<void(TensorMap*, TensorMap*)> do_forward = [&](TensorMap* o, TensorMap* i) {
        sampler ? sampler->forward(o, i) : dispatcher->forward(o, i);
    };

    // runtime arguments (host tensors)
    std::vector<uint32_t>           top_k(B);
    std::vector<float>              top_p(B), temperature(B), rep(1, 1.2f), len_pen(1, 1.0f);
    std::vector<unsigned long long> seeds(B);
    for (int i = 0; i < B; ++i) {
        seeds[i]       = 100 + 7 * i;
        temperature[i] = 0.5f + 0.25f * (i % 4);
        if (which == "topk") {
            top_k[i] = 1 + (i * 5) % 40, top_p[i] = 0.0f;
        }
        else if (which == "topp") {
            top_k[i] = 0, top_p[i] = 0.3f + 0.1f * (i % 6);
        }
        else {
            const uint32_t ks[4] = {0, 1, 8, 64};
            const float    ps[3] = {0.0f, 0.5f, 0.9f};
            top_k[i] = ks[i % 4], top_p[i] = ps[(i / 4) % 3];
        }
    }
    TensorMap args;
    if (K == 1) {
        args.insert("runtime_top_k", Tensor(MEMORY_CPU, TYPE_UINT32, {(size_t)B}, top_k.data()));
        args.insert("runtime_top_p", Tensor(MEMORY_CPU, TYPE_FP32, {(size_t)B}, top_p.data()));
        args.insert("temperature", Tensor(MEMORY_CPU, TYPE_FP32, {(size_t)B}, temperature.data()));
        args.insert("repetition_penalty", Tensor(MEMORY_CPU, TYPE_FP32, {1}, rep.data()));
        args.insert("random_seed", Tensor(MEMORY_CPU, TYPE_UINT64, {(size_t)B}, seeds.data()));
    }
    else {
        args.insert("len_penalty", Tensor(MEMORY_CPU, TYPE_FP32, {1}, len_pen.data()));
    }
    do_setup(B, K, &args);

    // state
    std::vector<int> ids_h((size_t)L * B * K, 0);
    for (int t = 0; t < mil; ++t) {
        for (int b = 0; b < B * K; ++b) {
            ids_h[(size_t)t * B * K + b] = (int)(mix(9000 + t * 131 + b) % (uint64_t)V);
        }
    }
    int*     output_ids = to_device(ids_h);
    int*     parent_ids = to_device(std::vector<int>((size_t)L * B * K, 0));
    uint8_t* finished   = to_device(std::vector<uint8_t>((size_t)B * K, 0));
    int*     seq_len    = to_device(std::vector<int>((size_t)B * K, mil));
    std::vector<float> cum_h((size_t)B * K, 0.0f);
    for (int b = 0; b < B * K; ++b) {
        cum_h[b] = K > 1 ? -(float)(b % K) : 0.0f;
    }
    float* cum     = to_device(cum_h);
    int*   end_ids = to_device(std::vector<int>(B, V - 1));
    int*   in_len  = to_device(std::vector<int>((size_t)B * K, mil));
    int*   src_ci  = to_device(std::vector<int>((size_t)B * K * L, 0));
    int*   tgt_ci  = to_device(std::vector<int>((size_t)B * K * L, 0));
    std::vector<uint32_t> lim_h(B, (uint32_t)L);
    uint32_t*             seq_lim = to_device(lim_h);
    T*                    logits  = nullptr;
    cudaMalloc(&logits, sizeof(T) * (size_t)B * K * V);
    std::vector<T>   logits_h((size_t)B * K * V);
    std::vector<int> step_ids((size_t)B * K);
    bool             should_stop = false;

    for (int s = 0; s < steps; ++s) {
        const int step = mil + s;
        for (size_t i = 0; i < logits_h.size(); ++i) {
            logits_h[i] = convert<T>(unit(1000003ull * (s + 1), i));
        }
        cudaMemcpy(logits, logits_h.data(), sizeof(T) * logits_h.size(), cudaMemcpyHostToDevice);
        const int n_slices = slices ? 2 : 1;
        long      live_before = alloc.live;
        for (int sl = 0; sl < n_slices; ++sl) {
        int      step_v = step, mil_v = mil, lbs_v = B / n_slices;
        uint32_t ite_v = (uint32_t)sl;
        TensorMap in, out;
        if (K == 1) {
            in.insert("logits", Tensor(MEMORY_GPU, dt, {(size_t)B, (size_t)V}, logits));
        }
        else {
            in.insert("logits", Tensor(MEMORY_GPU, dt, {(size_t)B, (size_t)K, (size_t)V}, logits));
            in.insert("len_penalty", Tensor(MEMORY_CPU, TYPE_FP32, {1}, len_pen.data()));
            in.insert("src_cache_indirection", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B, (size_t)K, (size_t)L}, src_ci));
            out.insert("tgt_cache_indirection", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B, (size_t)K, (size_t)L}, tgt_ci));
            out.insert("parent_ids", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)L, (size_t)B, (size_t)K}, parent_ids));
        }
        in.insert("step", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &step_v));
        in.insert("max_input_length", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &mil_v));
        in.insert("ite", Tensor(MEMORY_CPU, TYPE_UINT32, {1}, &ite_v));
        in.insert("local_batch_size", Tensor(MEMORY_CPU, TYPE_INT32, {1}, &lbs_v));
        in.insert("end_id", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B}, end_ids));
        in.insert("input_lengths", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B, (size_t)K}, in_len));
        in.insert("sequence_limit_length", Tensor(MEMORY_GPU, TYPE_UINT32, {(size_t)B}, seq_lim));
        out.insert("output_ids", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)L, (size_t)B, (size_t)K}, output_ids));
        out.insert("finished", Tensor(MEMORY_GPU, TYPE_BOOL, {(size_t)B * K}, finished));
        out.insert("sequence_length", Tensor(MEMORY_GPU, TYPE_INT32, {(size_t)B * K}, seq_len));
        out.insert("cum_log_probs", Tensor(MEMORY_GPU, TYPE_FP32, {(size_t)B * K}, cum));
        out.insert("should_stop", Tensor(MEMORY_CPU, TYPE_BOOL, {1}, &should_stop));
        do_forward(&out, &in);
        }
        if (slices && s > 0 && alloc.live != live_before) {
            std::fprintf(stderr, "live allocations moved from %ld to %ld at step %d\n", live_before, alloc.live, step);
            return 4;
        }
        if (K > 1) {
            std::swap(src_ci, tgt_ci);
        }
        cudaStreamSynchronize(stream);
        cudaMemcpy(step_ids.data(), output_ids + (size_t)step * B * K, 4 * step_ids.size(), cudaMemcpyDeviceToHost);
        std::printf("step %d stop %d ids", step, should_stop ? 1 : 0);
        for (int v : step_ids) {
            std::printf(" %d", v);
        }
        std::printf("\n");
    }
    if (slices) {
        std::printf("allocations %ld live %ld\n", alloc.total, alloc.live);
    }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        std::fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(e));
        return 2;
    }
    return 0;
}

int main(int argc, char** argv)
{
    if (argc < 6) {
        std::fprintf(stderr, "usage: shim_driver f32|f16|bf16 batch vocab steps topk|topp|mixed|beam|topk_layer|topp_layer|slices|e2e\n");
        return 1;
    }
    const std::string dt = argv[1], which = argv[5];
    const int         B = std::atoi(argv[2]), V = std::atoi(argv[3]), steps = std::atoi(argv[4]);
    try {
        if (dt == "f32") {
            return run<float>(TYPE_FP32, B, V, steps, which);
        }
        if (dt == "f16") {
            return run<half>(TYPE_FP16, B, V, steps, which);
        }
        return run<__nv_bfloat16>(TYPE_BF16, B, V, steps, which);
    }
    catch (const std::exception& ex) {
        std::fprintf(stderr, "exception: %s\n", ex.what());
        return 3;
    }
}
