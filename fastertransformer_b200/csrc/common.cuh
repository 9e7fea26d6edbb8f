// Shared device helpers for the decode-sampling kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <string>

namespace ftb200 {

typedef unsigned long long u64;
typedef unsigned int       u32;

// ---- error plumbing shared by the extern "C" entry points --------------------------------------
void        set_error(const std::string& msg);
const char* get_error();
void        note_launch(int n);
void        reset_launch_count();

#define FTB_CUDA_CHECK(expr)                                                                                           \
    do {                                                                                                               \
        cudaError_t e__ = (expr);                                                                                      \
        if (e__ != cudaSuccess) {                                                                                      \
            ftb200::set_error(std::string(#expr) + ": " + cudaGetErrorString(e__));                                    \
            return FTB200_CUDA_ERROR;                                                                                  \
        }                                                                                                              \
    } while (0)

// ---- order-preserving integer image of a float ---------------------------------------------------
// key(a) < key(b)  <=>  a < b   for all non-NaN a, b (with -0 < +0).
__device__ __forceinline__ u32 fkey(float x)
{
    u32 b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(u32 k)
{
    u32 b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

// 16-byte read-only load that does not pollute L1.
__device__ __forceinline__ uint4 ld_nc_v4(const void* p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Add to a counter that is known to live in shared memory.  Through a plain pointer the compiler has to
// emit a generic-address atomic; this states the address space.
__device__ __forceinline__ void smem_add(u32* p, u32 v)
{
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"((u32)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}

// The same on a 32-bit shared-memory address.
__device__ __forceinline__ void reds_add(u32 addr, u32 v)
{
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ u32 lds_u32(u32 addr)
{
    u32 v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void smem_or(u32* p, u32 v)
{
    asm volatile("red.shared.or.b32 [%0], %1;" ::"r"((u32)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ u32 smem_cas(u32* p, u32 expect, u32 want)
{
    u32 old;
    asm volatile("atom.shared.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old)
                 : "r"((u32)__cvta_generic_to_shared(p)), "r"(expect), "r"(want)
                 : "memory");
    return old;
}

__device__ __forceinline__ uint2 ld_nc_v2(const void* p)
{
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// Tells the compiler that a pointer loaded from a structure points into shared memory, so that it emits
// ld.shared / st.shared instead of generic accesses (every pointer of the kernel's shared-memory map qualifies).
#define FTB_ASSUME_SHARED(p) __builtin_assume(__isShared(p))

// ---- in-place ascending sort of u64 keys by a cooperating thread group ---------------------------
// Bitonic network in its "all ascending" form (first sub-step of every merge compares mirrored
// positions), which tolerates any n: positions >= n behave as +infinity and are never touched.
// `sync` is __syncthreads for a whole CTA or __syncwarp for one warp.
template<class Sync, bool SMEM = false>
__device__ __forceinline__ void group_sort_u64(u64* a, int n, int tid, int nthr, Sync sync)
{
    if (SMEM) {
        FTB_ASSUME_SHARED(a);
    }
    if (n < 2) {
        return;
    }
    int np = 1;
    while (np < n) {
        np <<= 1;
    }
    const int half = np >> 1;
    for (int k = 2; k <= np; k <<= 1) {
        const int hk = k >> 1;
        for (int i = tid; i < half; i += nthr) {
            int l = (i / hk) * k + (i % hk);
            int h = l ^ (k - 1);
            if (h < n) {
                u64 x = a[l], y = a[h];
                if (x > y) {
                    a[l] = y;
                    a[h] = x;
                }
            }
        }
        sync();
        for (int j = k >> 2; j > 0; j >>= 1) {
            for (int i = tid; i < half; i += nthr) {
                int l = 2 * i - (i & (j - 1));
                int h = l + j;
                if (h < n) {
                    u64 x = a[l], y = a[h];
                    if (x > y) {
                        a[l] = y;
                        a[h] = x;
                    }
                }
            }
            sync();
        }
    }
}

struct CtaSync {
    __device__ __forceinline__ void operator()() const
    {
        __syncthreads();
    }
};
struct WarpSync {
    __device__ __forceinline__ void operator()() const
    {
        __syncwarp();
    }
};

}  // namespace ftb200
