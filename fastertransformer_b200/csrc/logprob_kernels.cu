// Log-probabilities of given token ids under the soft-max of context logits, summed per sequence.
// Replaces invokeLogProbFromLogits (kernels/logprob_kernels.cu:142-183): log_probs_kernel (:36-103) and
// accumulate_log_probs (:105-140).
//
// The reference reads every row twice (maximum, then sum of exponentials) with one 1024-thread block per
// (step, sequence).  Here a row is read once with 16-byte loads, each thread keeping a running
// (maximum, scaled sum) pair that is merged across the block at the end, and a fixed grid of 8 CTAs per SM
// walks the rows.  Both kernels are bound by HBM: vocab * sizeof(T) bytes per counted (step, sequence).
#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

namespace {

constexpr int   kLpThreads = 256;
constexpr float kLog2e     = 1.4426950408889634f;

template<typename T>
struct LpType;
template<>
struct LpType<float> {
    static constexpr int   kPerVec = 4;
    static constexpr float kLowest = -FLT_MAX;
    __device__ static float get(const float* p) { return *p; }
    __device__ static void  unpack(const uint4& v, float* x)
    {
        x[0] = __uint_as_float(v.x);
        x[1] = __uint_as_float(v.y);
        x[2] = __uint_as_float(v.z);
        x[3] = __uint_as_float(v.w);
    }
};
template<>
struct LpType<__half> {
    static constexpr int   kPerVec = 8;
    static constexpr float kLowest = -65504.0f;  // the reference starts the maximum at -HALF_FLT_MAX (:58-59)
    __device__ static float get(const __half* p) { return __half2float(*p); }
    __device__ static void  unpack(const uint4& v, float* x)
    {
        const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            x[2 * i]       = f.x;
            x[2 * i + 1]   = f.y;
        }
    }
};
template<>
struct LpType<__nv_bfloat16> {
    static constexpr int   kPerVec = 8;
    static constexpr float kLowest = -FLT_MAX;
    __device__ static float get(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static void  unpack(const uint4& v, float* x)
    {
        const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i]     = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// (m, s) stands for s * exp(m): the sum of exp(x) over the elements seen so far, with m their maximum
// (or the type's lowest value when nothing larger was seen, as in the reference).
struct MaxSum {
    float m, s;
};

__device__ __forceinline__ float fast_exp(float d)
{
    return exp2f(d * kLog2e);  // __expf under the reference's fast-math build
}

__device__ __forceinline__ void add_one(MaxSum& a, float x)
{
    if (x > a.m) {
        a.s = a.s * fast_exp(a.m - x) + 1.0f;
        a.m = x;
    }
    else {
        a.s += fast_exp(x - a.m);
    }
}

__device__ __forceinline__ MaxSum merge(const MaxSum& a, const MaxSum& b)
{
    const float m = fmaxf(a.m, b.m);
    return {m, a.s * fast_exp(a.m - m) + b.s * fast_exp(b.m - m)};
}

template<typename T>
__device__ __forceinline__ void add_vec(MaxSum& a, const uint4& v)
{
    constexpr int N = LpType<T>::kPerVec;
    float         x[N];
    LpType<T>::unpack(v, x);
    float vm = x[0];
#pragma unroll
    for (int i = 1; i < N; ++i) {
        vm = fmaxf(vm, x[i]);
    }
    if (vm > a.m) {
        a.s *= fast_exp(a.m - vm);
        a.m = vm;
    }
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        t += fast_exp(x[i] - a.m);
    }
    a.s += t;
}

// One CTA per (step, sequence) row at a time.  Rows past a sequence's length are skipped without a read.
template<typename T>
__global__ void __launch_bounds__(kLpThreads) context_log_probs_kernel(float* log_probs, const T* logits,
                                                                        const int* ids, const int* lengths,
                                                                        int max_len, int batch, int vocab,
                                                                        size_t vocab_padded, int batch_first,
                                                                        long long rows)
{
    constexpr int N = LpType<T>::kPerVec;
    __shared__ MaxSum s_part[kLpThreads / 32];
    const int         tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int         steps = max_len - 1;

    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        int step, b;
        if (batch_first) {
            b    = (int)(r / steps);
            step = (int)(r % steps);
        }
        else {
            step = (int)(r / batch);
            b    = (int)(r % batch);
        }
        if (step >= lengths[b] - 1) {
            continue;
        }
        const size_t row_idx = batch_first ? (size_t)b * max_len + step : (size_t)step * batch + b;
        const T*     row     = logits + row_idx * vocab_padded;

        MaxSum acc{LpType<T>::kLowest, 0.0f};
        // Scalars up to the first 16-byte boundary, 16-byte vectors, scalars after the last full vector.
        const int mis  = (int)((reinterpret_cast<uintptr_t>(row) & 15) / sizeof(T));
        const int head = min(vocab, mis ? N - mis : 0);
        const int nvec = (vocab - head) / N;
        if (tid < head) {
            add_one(acc, LpType<T>::get(row + tid));
        }
        const uint4* vp = reinterpret_cast<const uint4*>(row + head);
        int          i  = tid;
        for (; i + 3 * kLpThreads < nvec; i += 4 * kLpThreads) {
            const uint4 v0 = ld_nc_v4(vp + i);
            const uint4 v1 = ld_nc_v4(vp + i + kLpThreads);
            const uint4 v2 = ld_nc_v4(vp + i + 2 * kLpThreads);
            const uint4 v3 = ld_nc_v4(vp + i + 3 * kLpThreads);
            add_vec<T>(acc, v0);
            add_vec<T>(acc, v1);
            add_vec<T>(acc, v2);
            add_vec<T>(acc, v3);
        }
        for (; i < nvec; i += kLpThreads) {
            add_vec<T>(acc, ld_nc_v4(vp + i));
        }
        const int tail0 = head + nvec * N;
        if (tail0 + tid < vocab) {  // fewer than N <= 8 elements remain
            add_one(acc, LpType<T>::get(row + tail0 + tid));
        }

#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxSum other{__shfl_xor_sync(0xffffffffu, acc.m, o), __shfl_xor_sync(0xffffffffu, acc.s, o)};
            acc = merge(acc, other);
        }
        if (lane == 0) {
            s_part[wid] = acc;
        }
        __syncthreads();
        if (tid == 0) {
            MaxSum tot = s_part[0];
#pragma unroll
            for (int w = 1; w < kLpThreads / 32; ++w) {
                tot = merge(tot, s_part[w]);
            }
            const size_t out = batch_first ? (size_t)b * steps + step : (size_t)step * batch + b;
            const size_t tok = batch_first ? (size_t)b * max_len + step + 1 : (size_t)(step + 1) * batch + b;
            const int    id  = ids[tok];
            // The reference reads logits[id] unchecked; an id outside the padded row gives NaN here.
            const float x = (id >= 0 && (size_t)id < vocab_padded) ? LpType<T>::get(row + id) : NAN;
            log_probs[out] = x - tot.m - __logf(tot.s + 1e-9f);
        }
        __syncthreads();
    }
}

// cum_log_probs[b] = sum over step < lengths[b] - 1 of log_probs[step, b], in a fixed order.
__global__ void __launch_bounds__(kLpThreads) sum_log_probs_kernel(float* cum, const float* log_probs,
                                                                    const int* lengths, int max_len, int batch,
                                                                    int batch_first)
{
    __shared__ float s_part[kLpThreads / 32];
    const int        b = blockIdx.x, tid = threadIdx.x;
    const int        n = min(lengths[b], max_len) - 1;
    const float*     p = log_probs + (batch_first ? (size_t)b * (max_len - 1) : (size_t)b);
    const size_t     stride = batch_first ? 1 : (size_t)batch;
    float            acc = 0.0f;
    for (int step = tid; step < n; step += kLpThreads) {
        acc += p[(size_t)step * stride];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
    }
    if ((tid & 31) == 0) {
        s_part[tid >> 5] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < kLpThreads / 32; ++w) {
            t += s_part[w];
        }
        cum[b] = t;
    }
}

template<typename T>
int launch_log_probs(float* cum, const void* logits, const int* ids, const int* lengths, size_t max_len,
                     size_t batch, size_t vocab, size_t vocab_padded, float* log_probs, cudaStream_t st,
                     int batch_first)
{
    // (asked per call: the attribute query is a host-side table look-up, and a process may drive several devices)
    int n_sm = 0, dev = 0;
    FTB_CUDA_CHECK(cudaGetDevice(&dev));
    FTB_CUDA_CHECK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    const long long rows = (long long)(max_len - 1) * (long long)batch;
    if (rows > 0) {
        const int grid = (int)std::min<long long>(rows, (long long)n_sm * 8);
        context_log_probs_kernel<T><<<grid, kLpThreads, 0, st>>>(log_probs, (const T*)logits, ids, lengths,
                                                                 (int)max_len, (int)batch, (int)vocab,
                                                                 vocab_padded, batch_first, rows);
        FTB_CUDA_CHECK(cudaGetLastError());
        note_launch(1);
    }
    sum_log_probs_kernel<<<(int)batch, kLpThreads, 0, st>>>(cum, log_probs, lengths, (int)max_len, (int)batch,
                                                           batch_first);
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}

}  // namespace
}  // namespace ftb200

using namespace ftb200;

extern "C" int ftb200_log_prob_from_logits(float* cum_log_probs, const void* logits, int dtype,
                                           const int* input_ids, const int* input_lengths,
                                           size_t max_input_length, size_t batch_size, size_t vocab_size,
                                           size_t vocab_size_padded, void* workspace, size_t workspace_size,
                                           void* stream, int batch_first)
{
    if (cum_log_probs == nullptr || logits == nullptr || input_ids == nullptr || input_lengths == nullptr
        || max_input_length == 0 || batch_size == 0 || vocab_size == 0 || vocab_size > vocab_size_padded
        || max_input_length > 0x7fffffffu || batch_size > 0x7fffffffu || vocab_size_padded > 0x7fffffffu) {
        set_error("ftb200_log_prob_from_logits: invalid argument");
        return FTB200_INVALID_ARG;
    }
    // The reference asserts this bound (logprob_kernels.cu:169); it holds one float per (step, sequence).
    if (workspace == nullptr || workspace_size < sizeof(float) * max_input_length * batch_size) {
        set_error("ftb200_log_prob_from_logits: workspace below sizeof(float) * max_input_length * batch_size");
        return FTB200_WORKSPACE_SMALL;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float*       lp = (float*)workspace;
    switch (dtype) {
        case FTB200_F32:
            return launch_log_probs<float>(cum_log_probs, logits, input_ids, input_lengths, max_input_length,
                                           batch_size, vocab_size, vocab_size_padded, lp, st, batch_first);
        case FTB200_F16:
            return launch_log_probs<__half>(cum_log_probs, logits, input_ids, input_lengths, max_input_length,
                                            batch_size, vocab_size, vocab_size_padded, lp, st, batch_first);
        case FTB200_BF16:
            return launch_log_probs<__nv_bfloat16>(cum_log_probs, logits, input_ids, input_lengths,
                                                   max_input_length, batch_size, vocab_size, vocab_size_padded, lp,
                                                   st, batch_first);
        default:
            set_error("ftb200_log_prob_from_logits: unknown dtype");
            return FTB200_INVALID_ARG;
    }
}
