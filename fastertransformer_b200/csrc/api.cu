// Error / version plumbing of the C ABI, curand state set-up and the runtime-argument
// normalisation kernels of the two sampling layers.
#include <curand_kernel.h>

#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

static thread_local std::string g_error;
static thread_local int         g_launches = 0;

void set_error(const std::string& msg)
{
    g_error = msg;
}
const char* get_error()
{
    return g_error.c_str();
}
void note_launch(int n)
{
    g_launches += n;
}
void reset_launch_count()
{
    g_launches = 0;
}

// curand_init(seed, 0, 0, &state[i]) per row, as kernels/sampling_topk_kernels.cu:32-55.
__global__ void curand_init_kernel(curandState_t* states, int n, unsigned long long seed,
                                   const unsigned long long* seeds)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        curand_init(seeds != nullptr ? seeds[i] : seed, 0, 0, &states[i]);
    }
}

__global__ void curand_peek_kernel(const curandState_t* states, int n, int n_draws, float* out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        curandState_t st = states[i];
        for (int d = 0; d < n_draws; ++d) {
            out[(size_t)d * n + i] = curand_uniform(&st);
        }
    }
}

// layers/sampling_layers/TopKSamplingLayer.cu:28-77
__global__ void setup_topk_args_kernel(int batch, u32 top_k, u32* top_ks, int top_ks_size, float top_p, float* top_ps,
                                       int top_ps_size, uint8_t* skip_decode)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < batch; i += gridDim.x * blockDim.x) {
        u32   k = top_ks_size > 1 ? top_ks[i] : top_k;
        float p = top_ps_size > 1 ? top_ps[i] : top_p;
        if (k == 0 && p == 0.0f) {
            k = 1;
        }
        if (k > 0 && p == 0.0f) {
            p = 1.0f;
        }
        top_ks[i]      = k > 1024u ? 1024u : k;
        top_ps[i]      = p < 0.0f ? 0.0f : (p > 1.0f ? 1.0f : p);
        skip_decode[i] = k == 0 ? 1 : 0;
    }
}

// layers/sampling_layers/TopPSamplingLayer.cu:30-109
__global__ void setup_topp_args_kernel(int batch, u32 top_k, u32* top_ks, int top_ks_size, float top_p, float* top_ps,
                                       int top_ps_size, uint8_t* skip_decode, float* initial_top_p,
                                       float* top_p_decay_buf, const float* top_p_decay, float* top_p_min_buf,
                                       const float* top_p_min, int32_t* top_p_reset_ids_buf,
                                       const uint32_t* top_p_reset_ids)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < batch; i += gridDim.x * blockDim.x) {
        u32   k = top_ks_size > 1 ? top_ks[i] : top_k;
        float p = top_ps_size > 1 ? top_ps[i] : top_p;
        if (k == 0 && p == 0.0f) {
            k = 1;
        }
        top_ks[i]      = k;
        top_ps[i]      = p < 0.0f ? 0.0f : (p > 1.0f ? 1.0f : p);
        skip_decode[i] = k > 0 ? 1 : 0;

        initial_top_p[i] = top_ps[i];
        float d          = top_p_decay == nullptr ? 1.0f : top_p_decay[i];
        if (d > 1.0f || d <= 0.0f) {
            d = 1.0f;
        }
        top_p_decay_buf[i] = d;
        float m            = top_p_min == nullptr ? 1e-6f : top_p_min[i];
        if (m > 1.0f || m <= 0.0f) {
            m = 0.5f;
        }
        top_p_min_buf[i]       = m;
        top_p_reset_ids_buf[i] = (int32_t)(top_p_reset_ids == nullptr ? -1 : top_p_reset_ids[i]);
    }
}

}  // namespace ftb200

using namespace ftb200;

extern "C" const char* ftb200_version(void)
{
    return "ftb200 0.1 (sm_100a)";
}

extern "C" const char* ftb200_last_error_string(void)
{
    return get_error();
}

extern "C" int ftb200_last_launch_count(void)
{
    return g_launches;
}

extern "C" int ftb200_curand_init(void* states, int n, unsigned long long seed, const unsigned long long* seeds,
                                  void* stream)
{
    if (states == nullptr || n < 0) {
        set_error("ftb200_curand_init: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (n == 0) {
        return FTB200_OK;
    }
    curand_init_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((curandState_t*)states, n, seed, seeds);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

extern "C" int ftb200_curand_peek_uniforms(const void* states, int n, int n_draws, float* out, void* stream)
{
    if (states == nullptr || out == nullptr || n < 0 || n_draws < 0) {
        set_error("ftb200_curand_peek_uniforms: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (n == 0 || n_draws == 0) {
        return FTB200_OK;
    }
    curand_peek_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        (const curandState_t*)states, n, n_draws, out);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

extern "C" int ftb200_setup_topk_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size,
                                              float top_p, float* top_ps, int top_ps_size, uint8_t* skip_decode,
                                              void* stream)
{
    if (batch < 0 || top_ks == nullptr || top_ps == nullptr || skip_decode == nullptr) {
        set_error("ftb200_setup_topk_runtime_args: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (batch == 0) {
        return FTB200_OK;
    }
    int block = batch < 256 ? batch : 256;
    setup_topk_args_kernel<<<(batch + block - 1) / block, block, 0, (cudaStream_t)stream>>>(
        batch, top_k, top_ks, top_ks_size, top_p, top_ps, top_ps_size, skip_decode);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

extern "C" int ftb200_setup_topp_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size,
                                              float top_p, float* top_ps, int top_ps_size, uint8_t* skip_decode,
                                              float* initial_top_p, float* top_p_decay_buf, const float* top_p_decay,
                                              float* top_p_min_buf, const float* top_p_min,
                                              int32_t* top_p_reset_ids_buf, const uint32_t* top_p_reset_ids,
                                              void* stream)
{
    if (batch < 0 || top_ks == nullptr || top_ps == nullptr || skip_decode == nullptr || initial_top_p == nullptr
        || top_p_decay_buf == nullptr || top_p_min_buf == nullptr || top_p_reset_ids_buf == nullptr) {
        set_error("ftb200_setup_topp_runtime_args: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (batch == 0) {
        return FTB200_OK;
    }
    int block = batch < 256 ? batch : 256;
    setup_topp_args_kernel<<<(batch + block - 1) / block, block, 0, (cudaStream_t)stream>>>(
        batch, top_k, top_ks, top_ks_size, top_p, top_ps, top_ps_size, skip_decode, initial_top_p, top_p_decay_buf,
        top_p_decay, top_p_min_buf, top_p_min, top_p_reset_ids_buf, top_p_reset_ids);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}
