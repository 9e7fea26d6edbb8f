// ftb200_decode_step_sampling_static: the fused decode-sampling step for callers that must not allocate.
//
// Some hosts of this library have no way to hand the kernels a scratch buffer of their own making:
//   * an inference server that reserves the whole GPU for its own memory pool at start-up, so that a
//     later cudaMalloc from a plug-in fails or fragments the pool;
//   * a plug-in whose per-step callback is forbidden to allocate (TensorRT's enqueue(), a Triton
//     backend's execute path) because allocation synchronises the device and adds jitter to every token.
// For them the scratch of the fused step lives in a fixed array inside the library image.  Every GPU that
// loads the library carries the array (kStaticScratchBytes) until the process exits, used or not, so it is
// kept small; shapes that need more are refused and have to be sent in slices (the `ite` /
// `local_batch_size` fields of the argument block exist for exactly that).
// The entry point itself allocates nothing and creates nothing: no cudaMalloc / cudaFree, no stream, no event
// (the single-pass kernels of the step run one after the other on the caller's stream here).
#include <mutex>

#include "common.cuh"
#include "ftb200.h"

namespace {

constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB per GPU

// Lives in device memory of every GPU that loads this library.  On the host side the name below is
// only a handle for the runtime: it is NOT a device address and must never be given to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex    g_mutex;
void*         g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device, looked up once per device.
int static_scratch(void** out)
{
    int dev = 0;
    FTB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        ftb200::set_error("ftb200_decode_step_sampling_static: device ordinal out of range");
        return FTB200_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        FTB_CUDA_CHECK(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return FTB200_OK;
}

}  // namespace

namespace ftb200 {
int decode_step_sampling_impl(const ftb200_sampling_params* p, bool fork);
}

extern "C" size_t ftb200_static_scratch_bytes(void)
{
    return kStaticScratchBytes;
}

extern "C" int ftb200_decode_step_sampling_static(const ftb200_sampling_params* p)
{
    if (p == nullptr) {
        ftb200::set_error("ftb200_decode_step_sampling_static: null argument block");
        return FTB200_INVALID_ARG;
    }
    size_t need = 0;
    int    rc   = ftb200_sampling_workspace_bytes(p->dtype, p->local_batch_size, p->vocab_size_padded, &need);
    if (rc != FTB200_OK) {
        return rc;
    }
    if (need > kStaticScratchBytes) {
        ftb200::set_error("ftb200_decode_step_sampling_static: this shape needs " + std::to_string(need)
                          + " bytes of scratch but the built-in area holds " + std::to_string(kStaticScratchBytes)
                          + "; send fewer rows per call (ite / local_batch_size) or use "
                            "ftb200_decode_step_sampling with a workspace of your own");
        return FTB200_WORKSPACE_SMALL;
    }
    void* scratch = nullptr;
    rc            = static_scratch(&scratch);
    if (rc != FTB200_OK) {
        return rc;
    }
    // Same step as the allocating caller's entry point, pointed at the built-in area.  That entry point
    // zeroes the row-ticket header of the scratch on the stream before it launches, which is all that has
    // to start at zero; whatever else the previous call left behind is overwritten before it is read.
    ftb200_sampling_params q = *p;
    q.workspace              = scratch;
    q.workspace_bytes        = kStaticScratchBytes;
    return ftb200::decode_step_sampling_impl(&q, false);
}
