// Fused decode-sampling step for sm_100a: bad-word ban, temperature + bias, repetition / presence
// penalty, min-length mask, pad / end masks, soft-max statistics, top-k or top-p selection and the
// draw - one persistent kernel, one CTA per row at a time, logits read from HBM once.
//
// Results are bit-identical to FasterTransformer's kernel chain for the same inputs and curand
// states.  That includes the parts of the reference whose outcome depends on its launch geometry:
//   * top-k tie order: which of several equal logits is kept / drawn follows from the reference's
//     8-CTA x {128,256}-thread arg-max passes (kernels/sampling_topk_kernels.cu:130-312) and from the
//     reduction order of cub::BlockReduce, restated in resolve_topk_class() below;
//   * soft-max denominator: summed in the order of the reference's min(V,1024)-thread strided loop
//     plus butterfly reduction (kernels/sampling_topp_kernels.cu:1294-1345, reduce_kernel_utils.cuh:73-103);
//   * top-p prefix sum: cub::BlockScan<float,256> raking order over the sorted probabilities
//     (kernels/sampling_topp_kernels.cu:877-1004).
// The file is compiled with --use_fast_math like the reference's release build, so /, __expf and logf
// lower to the same approximate instructions.
#pragma once
#include <curand_kernel.h>

#include "sampling_params.cuh"

namespace ftb200 {

// Per-row constants, kept in registers / shared memory.
struct RowCtx {
    const char* rowp;   // first byte of the row
    int         head;   // elements before the first 16-byte aligned vector
    int         nvec;   // aligned 16-byte vectors
    float       inv_t;  // 1 / (temperature + 1e-6), fp32
    __half      inv_t_h;
    float       theta;  // repetition / presence penalty
    float       neg_max;  // -MAX_T_VAL of the reference's logits type
};

struct Smem {
    u32*   hist;   // [kNB]
    u64*   cand;   // [kCap]
    float* val2;   // [1024] exp values of the sorted top-k / soft-max partial sums
    u32*   flags;  // one bit per aligned vector: holds a token with a hash entry
    u32*   hash;   // open addressing, (id << 2) | flags
};

__device__ __forceinline__ u32 hash_slot(int id, int shift)
{
    return (u32)(id * 2654435761u) >> shift;
}

static __device__ void hash_insert(const KParams& P, const Smem& S, const RowCtx& C, int id, u32 flag)
{
    if (id < 0 || id >= P.vocab_padded) {
        return;
    }
    u32 h    = hash_slot(id, P.hash_shift);
    u32 want = ((u32)id << 2) | flag;
    for (int probe = 0; probe < P.hash_slots; ++probe) {
        u32 old = atomicCAS(&S.hash[h], kHashEmpty, want);
        if (old == kHashEmpty) {
            break;
        }
        if ((old >> 2) == (u32)id) {
            atomicOr(&S.hash[h], flag);
            break;
        }
        h = (h + 1) & (P.hash_slots - 1);
    }
    const int epv = P.dtype == FTB200_F32 ? 4 : 8;
    int       rel = id - C.head;
    if (rel >= 0 && rel < C.nvec * epv) {
        int j = rel / epv;
        atomicOr(&S.flags[j >> 5], 1u << (j & 31));
    }
}

__device__ __forceinline__ u32 hash_lookup(const KParams& P, const Smem& S, int id)
{
    u32 h = hash_slot(id, P.hash_shift);
    for (int probe = 0; probe < P.hash_slots; ++probe) {
        u32 v = S.hash[h];
        if (v == kHashEmpty) {
            return 0;
        }
        if ((v >> 2) == (u32)id) {
            return v & 3u;
        }
        h = (h + 1) & (P.hash_slots - 1);
    }
    return 0;
}

// Temperature (+ bias) exactly as the reference's kernels compute it in the logits type
// (sampling_penalty_kernels.cu:117-179): fp32 arithmetic for float, half arithmetic with the inverse
// temperature rounded to half for half.  bf16 inputs take the fp32 route on the up-cast value.
template<int DT>
__device__ __forceinline__ float temp_value(const KParams& P, const RowCtx& C, u32 bits, int v)
{
    if (DT == FTB200_F16) {
        __half h = __ushort_as_half((unsigned short)bits);
        if (P.apply_temp) {
            if (P.bias != nullptr) {
                h = __hadd(h, ((const __half*)P.bias)[v]);
            }
            h = __hmul(h, C.inv_t_h);
        }
        return __half2float(h);
    }
    float x = (DT == FTB200_F32) ? __uint_as_float(bits) : __uint_as_float(bits << 16);
    if (P.apply_temp) {
        if (P.bias != nullptr) {
            float b = (DT == FTB200_F32) ? ((const float*)P.bias)[v] :
                                           __bfloat162float(((const __nv_bfloat16*)P.bias)[v]);
            x       = x + b;
        }
        x = x * C.inv_t;
    }
    return x;
}

// Penalty / mask for a token that has a hash entry.  Order of the reference: ban (-inf), temperature,
// repetition penalty from the pre-penalty value, min-length mask (sampling_penalty_kernels.cu:367-424,
// :485-500; ban_bad_words.cu:77-85).  A dead token is reported as -inf.
template<int DT>
__device__ __forceinline__ float special_value(const KParams& P, const RowCtx& C, float y, u32 fl)
{
    if (fl & kFlagDead) {
        return -INFINITY;
    }
    if ((fl & kFlagHist) && P.apply_rep) {
        if (P.penalty_type == FTB200_PENALTY_MULTIPLICATIVE) {
            y = y < 0.0f ? y * C.theta : y / C.theta;
        }
        else if (P.penalty_type == FTB200_PENALTY_ADDITIVE) {
            y = y - C.theta;
        }
        if (DT == FTB200_F16) {
            y = __half2float(__float2half_rn(y));
        }
    }
    return y;
}

// Final value of column v (scalar access; used for row edges and the ordered soft-max pass).
template<int DT>
__device__ __forceinline__ float elem_at(const KParams& P, const Smem& S, const RowCtx& C, int v)
{
    if (v >= P.vocab) {
        return -INFINITY;
    }
    u32 bits;
    if (DT == FTB200_F32) {
        bits = __ldg((const u32*)C.rowp + v);
    }
    else {
        bits = __ldg((const unsigned short*)C.rowp + v);
    }
    float     y   = temp_value<DT>(P, C, bits, v);
    const int epv = DT == FTB200_F32 ? 4 : 8;
    int       rel = v - C.head;
    bool      sp  = true;
    if (rel >= 0 && rel < C.nvec * epv) {
        int j = rel / epv;
        sp    = (S.flags[j >> 5] >> (j & 31)) & 1u;
    }
    if (sp) {
        u32 fl = hash_lookup(P, S, v);
        if (fl) {
            y = special_value<DT>(P, C, y, fl);
        }
    }
    return y;
}

// Visit vectors [j0, j1) of the row (and the unaligned head / tail when `edges`), calling f(v, y)
// for every column with its final value.  All loads of a thread's batch are issued before use.
template<int DT, class F>
__device__ __forceinline__ void
stream_range(const KParams& P, const Smem& S, const RowCtx& C, int j0, int j1, bool edges, F&& f)
{
    constexpr int EPV = DT == FTB200_F32 ? 4 : 8;
    const int     tid = threadIdx.x;
    if (edges) {
        for (int v = tid; v < C.head; v += kThreads) {
            f(v, elem_at<DT>(P, S, C, v));
        }
        for (int v = C.head + C.nvec * EPV + tid; v < P.vocab_padded; v += kThreads) {
            f(v, elem_at<DT>(P, S, C, v));
        }
    }
    const uint4* vp = (const uint4*)(C.rowp + (size_t)C.head * (DT == FTB200_F32 ? 4 : 2));
    for (int jb = j0; jb < j1; jb += kThreads * kUnroll) {
        uint4 q[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int j = jb + u * kThreads + tid;
            if (j < j1) {
                q[u] = ld_nc_v4(vp + j);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int j = jb + u * kThreads + tid;
            if (j < j1) {
                const bool sp = (S.flags[j >> 5] >> (j & 31)) & 1u;
                const u32  w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
                const int  vb   = C.head + j * EPV;
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    u32 bits = (DT == FTB200_F32) ? w[e] : ((w[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
                    int v    = vb + e;
                    float y;
                    if (v >= P.vocab) {
                        y = -INFINITY;
                    }
                    else {
                        y = temp_value<DT>(P, C, bits, v);
                        if (sp) {
                            u32 fl = hash_lookup(P, S, v);
                            if (fl) {
                                y = special_value<DT>(P, C, y, fl);
                            }
                        }
                    }
                    f(v, y);
                }
            }
        }
    }
}

// ---- CTA-wide helpers ----------------------------------------------------------------------------

// Walk an array of per-bucket weights from the top bucket down and return the largest bucket index
// b such that sum_{b' >= b} w(b') >= target, or -1 when the total stays below target.
template<class W>
__device__ __noinline__ int find_from_top(W w, double target, double* total_out)
{
    __shared__ double s_part[kWarps];
    __shared__ int    s_found;
    constexpr int PER = kNB / kThreads;
    const int     tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) {
        s_found = -1;
    }
    double local = 0.0;
    for (int i = 0; i < PER; ++i) {
        local += w(kNB - 1 - (tid * PER + i));
    }
    double incl = local;
    for (int off = 1; off < 32; off <<= 1) {
        double t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) {
            incl += t;
        }
    }
    if (lane == 31) {
        s_part[wid] = incl;
    }
    __syncthreads();
    double base = 0.0;
    for (int i = 0; i < wid; ++i) {
        base += s_part[i];
    }
    double excl = base + incl - local;
    if (excl < target && excl + local >= target) {
        double run = excl;
        for (int i = 0; i < PER; ++i) {
            int b = kNB - 1 - (tid * PER + i);
            run += w(b);
            if (run >= target || i == PER - 1) {
                s_found = b;
                break;
            }
        }
    }
    __syncthreads();
    if (total_out != nullptr) {
        double tot = 0.0;
        for (int i = 0; i < kWarps; ++i) {
            tot += s_part[i];
        }
        *total_out = tot;
    }
    int r = s_found;
    __syncthreads();
    return r;
}

static __device__ float draw_uniform(curandState_t* states, int row)
{
    curandState_t st = states[row];
    float         u  = curand_uniform(&st);
    states[row]      = st;
    return u;
}

// The reference's blockReduceSum over blockDim = nvt threads (reduce_kernel_utils.cuh:73-103), applied to
// the per-thread partial sums held in `partial[0..nvt)`.  Executed by warp 0.
static __device__ float butterfly_block_sum(const float* partial, int nvt)
{
    const int lane   = threadIdx.x & 31;
    const int nwarps = (nvt + 31) / 32;
    float     mine   = 0.0f;
    for (int w = 0; w < nwarps; ++w) {
        int   i = w * 32 + lane;
        float v = i < nvt ? partial[i] : 0.0f;
        for (int m = 16; m > 0; m >>= 1) {
            v = v + __shfl_xor_sync(0xffffffffu, v, m);
        }
        if (lane == w) {
            mine = v;
        }
    }
    // second stage: threads with threadIdx < blockDim/32.f read shared[lane], others 0
    float v = ((float)lane < (float)nvt / 32.f) ? mine : 0.0f;
    for (int m = 16; m > 0; m >>= 1) {
        v = v + __shfl_xor_sync(0xffffffffu, v, m);
    }
    return v;
}

template<int DT>
__device__ __forceinline__ float round_to_T(float x)
{
    return DT == FTB200_F16 ? __half2float(__float2half_rn(x)) : x;
}

// ---- tie order of the reference's two-stage top-k -------------------------------------------------
// `cls[0..m)` holds the (~key(value) << 32 | column) entries of ONE value class (all equal values).
// The reference extracts equal values in this order:
//   stage 1 (per CTA lane = (col / BS1) % 8): thread-id descending, then column ascending, where
//     thread-id = col % BS1 - cub::BlockReduce keeps the right-hand operand on ties and every thread
//     holds its first maximum (sampling_topk_kernels.cu:178-202, reduce_kernel_utils.cuh:345-348);
//     only the first k of a lane survive;
//   stage 2 over slot i = lane * k + rank: (i % BS2) descending, then i ascending (:255-280).
// lane_base[l] = number of larger-valued candidates in lane l.  Returns the column of the class member
// whose final rank inside the class is `want`.  Overwrites cls.
static __device__ __noinline__ int resolve_topk_class(u64* cls, int m, int want, int k, int bs1, int bs2, const u32* lane_base)
{
    __shared__ int s_ans;
    __shared__ u32 s_lane_cnt[8];
    __shared__ u32 s_lane_start[8];
    const int      tid = threadIdx.x;
    if (m == 1) {
        return (int)(cls[0] & 0xffffffffu);
    }
    if (tid < 8) {
        s_lane_cnt[tid] = 0;
    }
    __syncthreads();
    for (int a = tid; a < m; a += kThreads) {
        const u32 col  = (u32)(cls[a] & 0xffffffffu);
        const u32 lane = (col / bs1) & 7u;
        const u32 t1   = col % bs1;
        atomicAdd(&s_lane_cnt[lane], 1u);
        cls[a] = ((u64)lane << 56) | ((u64)(bs1 - 1 - t1) << 40) | col;
    }
    __syncthreads();
    if (tid == 0) {
        u32 run = 0;
        for (int l = 0; l < 8; ++l) {
            s_lane_start[l] = run;
            run += s_lane_cnt[l];
        }
        s_ans = -1;
    }
    group_sort_u64(cls, m, tid, kThreads, CtaSync());
    __syncthreads();
    for (int a = tid; a < m; a += kThreads) {
        const u64 e    = cls[a];
        const u32 col  = (u32)(e & 0xffffffffu);
        const u32 lane = (u32)(e >> 56);
        const u32 r    = lane_base[lane] + ((u32)a - s_lane_start[lane]);
        u64       key  = ~0ull;
        if (r < (u32)k) {
            const u32 i2 = lane * k + r;
            key          = ((u64)(bs2 - 1 - (i2 % bs2)) << 48) | ((u64)i2 << 32) | col;
        }
        cls[a] = key;
    }
    __syncthreads();
    group_sort_u64(cls, m, tid, kThreads, CtaSync());
    __syncthreads();
    if (tid == 0) {
        u64 e = cls[want < m ? want : m - 1];
        s_ans = (e == ~0ull) ? -1 : (int)(e & 0xffffffffu);
    }
    __syncthreads();
    int r = s_ans;
    __syncthreads();
    return r;
}

// ---- per-row set-up ------------------------------------------------------------------------------
template<int DT>
__device__ __noinline__ void build_row(const KParams& P, const Smem& S, RowCtx& C, int r)
{
    constexpr int ES  = DT == FTB200_F32 ? 4 : 2;
    constexpr int EPV = DT == FTB200_F32 ? 4 : 8;
    const int     tid = threadIdx.x;

    C.rowp          = (const char*)P.logits + (size_t)r * P.vocab_padded * ES;
    const size_t ad = (size_t)C.rowp;
    int          hd = (int)(((16 - (ad & 15)) & 15) / ES);
    C.head          = hd < P.vocab_padded ? hd : P.vocab_padded;
    C.nvec          = (P.vocab_padded - C.head) / EPV;
    C.inv_t         = 1.0f;
    if (P.apply_temp) {
        C.inv_t = 1.0f / (P.temperature[r] + 1e-6f);
    }
    C.inv_t_h = __float2half_rn(C.inv_t);
    C.theta   = P.apply_rep ? P.rep_penalty[r] : 1.0f;
    C.neg_max = DT == FTB200_F16 ? -65504.0f : -FLT_MAX;

    for (int i = tid; i < P.hash_slots; i += kThreads) {
        S.hash[i] = kHashEmpty;
    }
    for (int i = tid; i < P.flag_words; i += kThreads) {
        S.flags[i] = 0;
    }
    __syncthreads();

    const size_t col = (size_t)P.ite * P.local_batch + r;
    // token history -> repetition / presence penalty (sampling_penalty_kernels.cu:385-410)
    if (P.apply_rep) {
        const int input_len = P.input_lengths != nullptr ? P.input_lengths[r] : P.max_input_len;
        for (int t = tid; t < P.step; t += kThreads) {
            if (t >= input_len && t < P.max_input_len) {
                continue;
            }
            hash_insert(P, S, C, P.output_ids[(size_t)t * P.batch_size + col], kFlagHist);
        }
    }
    // bad words (ban_bad_words.cu:35-85): a word bans its last token when the preceding tokens match
    // the tail of the generated sequence; token 0 can never be banned.
    if (P.bad_words != nullptr) {
        const int  L    = P.bad_words_len;
        const int* base = P.bad_words_shared ? P.bad_words : P.bad_words + (size_t)r * 2 * L;
        const int* offs = base + L;
        for (int i = tid; i < L; i += kThreads) {
            const int item_end = offs[i];
            if (item_end < 0) {
                continue;
            }
            const int item_start = i > 0 ? offs[i - 1] : 0;
            const int item_size  = item_end - item_start;
            bool      ban        = item_size == 1;
            if (item_size > 1 && P.step >= item_size - 1) {
                ban = true;
                for (int j = item_size - 2; j >= 0; --j) {
                    const int prev = P.output_ids[(size_t)(P.step - (item_size - 1) + j) * P.batch_size + col];
                    if (prev != base[item_start + j]) {
                        ban = false;
                        break;
                    }
                }
            }
            if (ban) {
                const int tok = base[item_end - 1];
                if (0 < tok && tok < P.vocab_padded) {
                    hash_insert(P, S, C, tok, kFlagDead);
                }
            }
        }
    }
    // min-length mask on the end token (sampling_penalty_kernels.cu:493-499)
    if (P.apply_minlen && tid == 0) {
        if (P.seq_len[r] + 1 - P.max_input_len < P.min_lengths[r]) {
            hash_insert(P, S, C, P.end_ids[r], kFlagDead);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ u64 warp_max_u64(u64 v)
{
    for (int m = 16; m > 0; m >>= 1) {
        u64 o = __shfl_xor_sync(0xffffffffu, v, m);
        v     = o > v ? o : v;
    }
    return v;
}

static __device__ u64 block_max_u64(u64 v)
{
    __shared__ u64 s_m[kWarps];
    __shared__ u64 s_out;
    v = warp_max_u64(v);
    if ((threadIdx.x & 31) == 0) {
        s_m[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 b = 0;
        for (int i = 0; i < kWarps; ++i) {
            b = s_m[i] > b ? s_m[i] : b;
        }
        s_out = b;
    }
    __syncthreads();
    u64 r = s_out;
    __syncthreads();
    return r;
}

static __device__ u32 block_sum_u32(u32 v)
{
    __shared__ u32 s_m[kWarps];
    __shared__ u32 s_out;
    for (int m = 16; m > 0; m >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, m);
    }
    if ((threadIdx.x & 31) == 0) {
        s_m[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        u32 b = 0;
        for (int i = 0; i < kWarps; ++i) {
            b += s_m[i];
        }
        s_out = b;
    }
    __syncthreads();
    u32 r = s_out;
    __syncthreads();
    return r;
}

// Drop candidates below thr_key, keeping the rest in any order.  Returns the new count.
static __device__ __noinline__ int compact_candidates(u64* cand, int n, u32 thr_key)
{
    __shared__ u32 s_new;
    if (threadIdx.x == 0) {
        s_new = 0;
    }
    __syncthreads();
    for (int base = 0; base < n; base += kThreads) {
        const int i    = base + threadIdx.x;
        u64       e    = 0;
        bool      keep = false;
        if (i < n) {
            e    = cand[i];
            keep = (~(u32)(e >> 32)) >= thr_key;
        }
        __syncthreads();
        if (keep) {
            cand[atomicAdd(&s_new, 1u)] = e;
        }
        __syncthreads();
    }
    return (int)s_new;
}

struct RowOut {
    int*     id_out;
    int      r;
    int      end_id;
};

__device__ __forceinline__ void write_lengths(const KParams& P, const RowOut& O, int id)
{
    // rows that were already finished never get here (sampling_topk_kernels.cu:307-310)
    if (P.seq_len != nullptr && P.finished != nullptr) {
        P.seq_len[O.r]  = P.seq_len[O.r] + 1;
        P.finished[O.r] = id == O.end_id ? 1 : 0;
    }
}

// The draw of topk_stage2_sampling (sampling_topk_kernels.cu:255-311) over `sorted` (value descending),
// then the tie-order resolution.  use_exp: values are logits (exp taken here) or probabilities.
static __device__ __noinline__ void topk_finish(const KParams& P, const Smem& S, const RowOut& O, u64* sorted, int n, int k, float u,
                            float top_p, bool use_exp, bool want_lp)
{
    __shared__ int   s_pick, s_lo, s_hi;
    __shared__ float s_e, s_sum;
    __shared__ u32   s_lane_base[8];
    const int        tid   = threadIdx.x;
    const int        k_eff = k < n ? k : n;
    if (tid < 8) {
        s_lane_base[tid] = 0;
    }
    if (tid == 0) {
        s_pick = -1;
        if (k_eff > 0) {
            const float s_max = fkey_inv(~(u32)(sorted[0] >> 32));
            float       sum   = 0.0f;
            for (int i = 0; i < k_eff; ++i) {
                float y   = fkey_inv(~(u32)(sorted[i] >> 32));
                float e   = use_exp ? __expf(y - s_max) : y;
                S.val2[i] = e;
                sum += e;
            }
            float rand_num = u * top_p * sum;
            int   pick     = k_eff - 1;
            for (int i = 0; i < k_eff; ++i) {
                rand_num = rand_num - S.val2[i];
                if (rand_num <= 0.0f || i == k - 1) {
                    pick = i;
                    break;
                }
            }
            s_pick = pick;
            s_e    = S.val2[pick];
            s_sum  = sum;
            s_lo   = pick;
            s_hi   = pick + 1;
        }
    }
    __syncthreads();
    const int pick = s_pick;
    if (pick < 0) {
        // no selectable token in the row: the reference reads out of bounds here; emit token 0
        if (tid == 0) {
            *O.id_out = 0;
            write_lengths(P, O, 0);
        }
        __syncthreads();
        return;
    }
    // extent of the value class of the picked entry
    const u32 kv = (u32)(sorted[pick] >> 32);
    for (int i = tid; i < n; i += kThreads) {
        if ((u32)(sorted[i] >> 32) == kv) {
            atomicMin(&s_lo, i);
            atomicMax(&s_hi, i + 1);
        }
    }
    __syncthreads();
    const int lo = s_lo, hi = s_hi;
    int       col;
    if (hi - lo == 1) {
        col = (int)(sorted[pick] & 0xffffffffu);
    }
    else {
        const u32 bs1 = P.max_top_k <= 16 ? 128 : 256;
        const u32 bs2 = P.max_top_k <= 32 ? 128 : 256;
        for (int i = tid; i < lo; i += kThreads) {
            u32 c = (u32)(sorted[i] & 0xffffffffu);
            atomicAdd(&s_lane_base[(c / bs1) & 7u], 1u);
        }
        __syncthreads();
        col = resolve_topk_class(sorted + lo, hi - lo, pick - lo, k, (int)bs1, (int)bs2, s_lane_base);
    }
    if (tid == 0) {
        if (col < 0) {
            col = 0;
        }
        *O.id_out = col;
        if (want_lp) {
            float log_prob = logf(s_e);
            if (P.cum_log_probs != nullptr) {
                P.cum_log_probs[O.r] += log_prob;
            }
            if (P.out_log_probs != nullptr) {
                P.out_log_probs[O.r] = log_prob - logf(s_sum);
            }
        }
        write_lengths(P, O, col);
    }
    __syncthreads();
}

// ---- top-k, k == 1, no log-probs: a single arg-max with the reference's tie order ------------------
template<int DT>
__device__ __noinline__ void row_argmax(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O)
{
    const u32 bs1  = P.max_top_k <= 16 ? 128 : 256;
    u64       best = 0;
    stream_range<DT>(P, S, C, 0, C.nvec, true, [&](int v, float y) {
        if (y > C.neg_max) {
            // value, then CTA lane descending, thread descending, column ascending
            u32 tie = ((((u32)v / bs1) & 7u) << 29) | (((u32)v % bs1) << 21) | (0x1fffffu - (u32)v);
            u64 c   = ((u64)fkey(y) << 32) | tie;
            best    = c > best ? c : best;
        }
    });
    best = block_max_u64(best);
    if (threadIdx.x == 0) {
        int id    = best == 0 ? 0 : (int)(0x1fffffu - (u32)(best & 0x1fffffu));
        *O.id_out = id;
        write_lengths(P, O, id);
    }
    __syncthreads();
}

// ---- top-k, k > 1, no log-probs: one pass, running threshold, candidates in shared memory ----------
template<int DT>
__device__ __noinline__ void row_topk(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O, u64* gscratch, int k,
                         float u, float top_p)
{
    __shared__ u32 s_n, s_ovf;
    const int      tid = threadIdx.x;
    constexpr int  VB  = kThreads * kUnroll;

    auto count_w = [&](int b) { return (double)S.hist[b]; };
    auto thr_of  = [&](int b) { return b < 0 ? 0u : ((u32)b << 20); };

    for (int i = tid; i < kNB; i += kThreads) {
        S.hist[i] = 0;
    }
    if (tid == 0) {
        s_n   = 0;
        s_ovf = 0;
    }
    __syncthreads();

    u64* cand = S.cand;
    int  n    = 0;
    bool slow = false;
    {
        // warm-up: histogram the first batch, derive a threshold, then collect that batch
        const int j1 = C.nvec < VB ? C.nvec : VB;
        stream_range<DT>(P, S, C, 0, j1, true, [&](int v, float y) {
            if (y > C.neg_max) {
                atomicAdd(&S.hist[fkey(y) >> 20], 1u);
            }
        });
        __syncthreads();
        u32 thr = thr_of(find_from_top(count_w, (double)k, nullptr));
        stream_range<DT>(P, S, C, 0, j1, true, [&](int v, float y) {
            if (y > C.neg_max) {
                u32 key = fkey(y);
                if (key >= thr) {
                    u32 pos = atomicAdd(&s_n, 1u);
                    if (pos < (u32)kCap) {
                        cand[pos] = ((u64)(~key) << 32) | (u32)v;
                    }
                    else {
                        s_ovf = 1;
                    }
                }
            }
        });
        __syncthreads();
        slow = s_ovf != 0;
        // remaining batches: histogram and collect what passes the current threshold
        for (int j0 = j1; j0 < C.nvec && !slow; j0 += VB) {
            const int je = j0 + VB < C.nvec ? j0 + VB : C.nvec;
            const u32 n0 = s_n;
            __syncthreads();
            stream_range<DT>(P, S, C, j0, je, false, [&](int v, float y) {
                if (y > C.neg_max) {
                    u32 key = fkey(y);
                    if (key >= thr) {
                        atomicAdd(&S.hist[key >> 20], 1u);
                        u32 pos = atomicAdd(&s_n, 1u);
                        if (pos < (u32)kCap) {
                            cand[pos] = ((u64)(~key) << 32) | (u32)v;
                        }
                        else {
                            s_ovf = 1;
                        }
                    }
                }
            });
            __syncthreads();
            if (s_ovf) {
                // the batch did not fit: raise the threshold, shrink, and collect the batch again
                thr   = thr_of(find_from_top(count_w, (double)k, nullptr));
                int m = compact_candidates(cand, (int)n0, thr);
                __syncthreads();
                if (tid == 0) {
                    s_n   = m;
                    s_ovf = 0;
                }
                __syncthreads();
                stream_range<DT>(P, S, C, j0, je, false, [&](int v, float y) {
                    if (y > C.neg_max) {
                        u32 key = fkey(y);
                        if (key >= thr) {
                            u32 pos = atomicAdd(&s_n, 1u);
                            if (pos < (u32)kCap) {
                                cand[pos] = ((u64)(~key) << 32) | (u32)v;
                            }
                            else {
                                s_ovf = 1;
                            }
                        }
                    }
                });
                __syncthreads();
                slow = s_ovf != 0;
            }
            else if (s_n > (u32)(kCap / 2)) {
                thr   = thr_of(find_from_top(count_w, (double)k, nullptr));
                int m = compact_candidates(cand, (int)s_n, thr);
                __syncthreads();
                if (tid == 0) {
                    s_n = m;
                }
                __syncthreads();
            }
        }
        if (!slow) {
            thr = thr_of(find_from_top(count_w, (double)k, nullptr));
            n   = compact_candidates(cand, (int)s_n, thr);
            __syncthreads();
        }
    }
    if (slow) {
        // Degenerate rows (huge tie classes, adversarial orderings): full histogram, then collect into
        // this CTA's global scratch, which holds a whole row.
        for (int i = tid; i < kNB; i += kThreads) {
            S.hist[i] = 0;
        }
        if (tid == 0) {
            s_n = 0;
        }
        __syncthreads();
        stream_range<DT>(P, S, C, 0, C.nvec, true, [&](int v, float y) {
            if (y > C.neg_max) {
                atomicAdd(&S.hist[fkey(y) >> 20], 1u);
            }
        });
        __syncthreads();
        const u32 thr = thr_of(find_from_top(count_w, (double)k, nullptr));
        cand          = gscratch;
        stream_range<DT>(P, S, C, 0, C.nvec, true, [&](int v, float y) {
            if (y > C.neg_max) {
                u32 key = fkey(y);
                if (key >= thr) {
                    u32 pos   = atomicAdd(&s_n, 1u);
                    cand[pos] = ((u64)(~key) << 32) | (u32)v;
                }
            }
        });
        __syncthreads();
        n = (int)s_n;
    }
    group_sort_u64(cand, n, tid, kThreads, CtaSync());
    __syncthreads();
    topk_finish(P, S, O, cand, n, k, u, top_p, true, false);
}

// ---- rows that need soft-max probabilities: top-p, and top-k when log-probs are requested -----------
__device__ __forceinline__ int lin_bucket(float y, float maxv)
{
    int q = (int)((maxv - y) * (float)kLinScale);
    q     = q < 0 ? 0 : (q > kNB - 1 ? kNB - 1 : q);
    return kNB - 1 - q;
}

template<int DT>
__device__ __noinline__ void row_softmax(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O, u64* gscratch,
                            bool is_topp, int k, float u, float top_p, bool want_lp)
{
    constexpr int ES  = DT == FTB200_F32 ? 4 : 2;
    __shared__ float s_S;
    __shared__ int   s_sel;
    __shared__ u32   s_big[32];
    __shared__ u32   s_nbig;
    const int        tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;

    // pass 1 (HBM): row maximum and its first column
    u64 best = 0;
    stream_range<DT>(P, S, C, 0, C.nvec, true, [&](int v, float y) {
        if (y > C.neg_max) {
            u64 c = ((u64)fkey(y) << 32) | (0xffffffffu - (u32)v);
            best  = c > best ? c : best;
        }
    });
    best = block_max_u64(best);
    if (best == 0) {
        if (tid == 0) {
            *O.id_out = 0;
            write_lengths(P, O, 0);
        }
        __syncthreads();
        return;
    }
    const float maxv   = fkey_inv((u32)(best >> 32));
    const int   argmax = (int)(0xffffffffu - (u32)(best & 0xffffffffu));

    for (int attempt = 0; attempt < 2; ++attempt) {
        const bool force_complete = attempt == 1;
        // pass 2 (L2): exponentials, the denominator in the reference's summation order, bucket counts
        for (int i = tid; i < kNB; i += kThreads) {
            S.hist[i] = 0;
        }
        __syncthreads();
        const int nvt = P.vocab < 1024 ? P.vocab : 1024;  // blockDim of addBiasSoftMax (:1364)
        float     acc[4] = {0.f, 0.f, 0.f, 0.f};
        const bool grouped = nvt == 1024 && (((size_t)C.rowp) % (4 * ES) == 0) && (C.head % 4 == 0);
        if (grouped) {
            // thread t owns virtual threads 4t..4t+3: one 4-element load per 1024-column chunk
            constexpr int UN = 8;
            for (int m0 = 0; m0 * 1024 < P.vocab_padded; m0 += UN) {
                u32 raw[UN][4];
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    const int v0 = (m0 + uu) * 1024 + 4 * tid;
                    if (v0 + 3 < P.vocab_padded) {
                        if (DT == FTB200_F32) {
                            uint4 q    = *(const uint4*)(C.rowp + (size_t)v0 * 4);
                            raw[uu][0] = q.x, raw[uu][1] = q.y, raw[uu][2] = q.z, raw[uu][3] = q.w;
                        }
                        else {
                            uint2 q    = *(const uint2*)(C.rowp + (size_t)v0 * 2);
                            raw[uu][0] = q.x & 0xffffu, raw[uu][1] = q.x >> 16;
                            raw[uu][2] = q.y & 0xffffu, raw[uu][3] = q.y >> 16;
                        }
                    }
                }
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    const int v0 = (m0 + uu) * 1024 + 4 * tid;
                    if (v0 >= P.vocab_padded) {
                        continue;
                    }
                    if (v0 + 3 < P.vocab_padded) {
                        bool sp = true;
                        if (v0 >= C.head) {
                            const int j = (v0 - C.head) / (DT == FTB200_F32 ? 4 : 8);
                            sp          = j >= C.nvec || ((S.flags[j >> 5] >> (j & 31)) & 1u);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int v = v0 + e;
                            float     y = -INFINITY;
                            if (v < P.vocab) {
                                y = temp_value<DT>(P, C, raw[uu][e], v);
                                if (sp) {
                                    u32 fl = hash_lookup(P, S, v);
                                    if (fl) {
                                        y = special_value<DT>(P, C, y, fl);
                                    }
                                }
                            }
                            if (y > C.neg_max) {
                                float ex = round_to_T<DT>(__expf(y - maxv));
                                acc[e] += ex;
                                atomicAdd(&S.hist[lin_bucket(y, maxv)], 1u);
                            }
                        }
                    }
                    else {
                        for (int e = 0; e < 4 && v0 + e < P.vocab_padded; ++e) {
                            float y = elem_at<DT>(P, S, C, v0 + e);
                            if (y > C.neg_max) {
                                float ex = round_to_T<DT>(__expf(y - maxv));
                                acc[e] += ex;
                                atomicAdd(&S.hist[lin_bucket(y, maxv)], 1u);
                            }
                        }
                    }
                }
            }
            __syncthreads();
            for (int e = 0; e < 4; ++e) {
                S.val2[4 * tid + e] = acc[e];
            }
        }
        else {
            // thread t owns virtual threads t, t+256, t+512, t+768
            for (int v0 = 0; v0 < P.vocab_padded; v0 += nvt) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int vt = tid + q * kThreads;
                    const int v  = v0 + vt;
                    if (vt < nvt && v < P.vocab_padded) {
                        float y = elem_at<DT>(P, S, C, v);
                        if (y > C.neg_max) {
                            float ex = round_to_T<DT>(__expf(y - maxv));
                            acc[q] += ex;
                            atomicAdd(&S.hist[lin_bucket(y, maxv)], 1u);
                        }
                    }
                }
            }
            __syncthreads();
            for (int q = 0; q < 4; ++q) {
                S.val2[tid + q * kThreads] = acc[q];
            }
        }
        __syncthreads();
        if (wid == 0) {
            float s = butterfly_block_sum(S.val2, nvt);
            if (lane == 0) {
                s_S = s;
            }
        }
        __syncthreads();
        const float denom = s_S + 1e-6f;

        if (is_topp) {
            // arg-max shortcut of topp_beam_topk_kernel (sampling_topp_kernels.cu:801-860)
            const float p_max = round_to_T<DT>(round_to_T<DT>(1.0f) / denom);
            if (p_max >= top_p) {
                if (tid == 0) {
                    *O.id_out = argmax;
                    if (want_lp) {
                        float lprob = logf(p_max);
                        if (P.cum_log_probs != nullptr) {
                            P.cum_log_probs[O.r] += lprob;
                        }
                        if (P.out_log_probs != nullptr) {
                            P.out_log_probs[O.r] = lprob;
                        }
                    }
                    write_lengths(P, O, argmax);
                }
                __syncthreads();
                return;
            }
        }
        const float rand_num = u * top_p;

        // choose the lowest bucket to collect
        int b_star;
        if (is_topp) {
            // lower bound of the probability mass of each bucket; 0.995 covers rounding of p to T
            const float  scale = 0.995f / denom;
            auto         w     = [&](int b) {
                const int q = kNB - 1 - b;
                if (q >= kNB - 1) {
                    return 0.0;
                }
                return (double)S.hist[b] * (double)(__expf(-(float)(q + 1) / (float)kLinScale) * scale);
            };
            b_star = find_from_top(w, (double)rand_num, nullptr);
        }
        else {
            auto w = [&](int b) { return (double)S.hist[b]; };
            b_star = find_from_top(w, (double)k, nullptr);
        }
        int b_thr = b_star - 1;
        if (b_thr < 0 || force_complete) {
            b_thr = 0;
        }
        const bool complete = b_thr == 0;

        // exclusive offsets from the top bucket down; hist becomes the scatter cursor
        u32 n_g;
        {
            constexpr int PER   = kNB / kThreads;
            u32           local = 0;
            for (int i = 0; i < PER; ++i) {
                const int b = kNB - 1 - (tid * PER + i);
                if (b >= b_thr) {
                    local += S.hist[b];
                }
            }
            u32 incl = local;
            for (int off = 1; off < 32; off <<= 1) {
                u32 t = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) {
                    incl += t;
                }
            }
            __shared__ u32 s_wtot[kWarps];
            if (lane == 31) {
                s_wtot[wid] = incl;
            }
            __syncthreads();
            u32 base = 0, tot = 0;
            for (int i = 0; i < kWarps; ++i) {
                if (i < wid) {
                    base += s_wtot[i];
                }
                tot += s_wtot[i];
            }
            n_g     = tot;
            u32 run = base + incl - local;
            for (int i = 0; i < PER; ++i) {
                const int b = kNB - 1 - (tid * PER + i);
                if (b >= b_thr) {
                    u32 c     = S.hist[b];
                    S.hist[b] = run;
                    run += c;
                }
            }
            __syncthreads();
        }
        const bool in_smem = n_g <= (u32)kCap;
        u64*       dest    = in_smem ? S.cand : gscratch;

        // pass 3 (L2): probabilities of the collected columns, written bucket by bucket
        stream_range<DT>(P, S, C, 0, C.nvec, true, [&](int v, float y) {
            if (y > C.neg_max) {
                const int b = lin_bucket(y, maxv);
                if (b >= b_thr) {
                    float ex  = round_to_T<DT>(__expf(y - maxv));
                    float pr  = round_to_T<DT>(ex / denom);
                    u32   pos = atomicAdd(&S.hist[b], 1u);
                    dest[pos] = ((u64)(~fkey(pr)) << 32) | (u32)v;
                }
            }
        });
        if (tid == 0) {
            s_nbig = 0;
        }
        __syncthreads();
        // order inside each bucket: probability descending, column ascending (the stable radix sort
        // of the reference leaves equal probabilities in column order)
        for (int b = kNB - 1 - wid; b >= b_thr; b -= kWarps) {
            const u32 lo = b == kNB - 1 ? 0u : S.hist[b + 1];
            const u32 hi = S.hist[b];
            const int m  = (int)(hi - lo);
            if (m < 2) {
                continue;
            }
            if (in_smem) {
                group_sort_u64(dest + lo, m, lane, 32, WarpSync());
            }
            else if (m <= kWarpTile) {
                u64* tile = S.cand + wid * kWarpTile;
                for (int i = lane; i < m; i += 32) {
                    tile[i] = dest[lo + i];
                }
                __syncwarp();
                group_sort_u64(tile, m, lane, 32, WarpSync());
                for (int i = lane; i < m; i += 32) {
                    dest[lo + i] = tile[i];
                }
                __syncwarp();
            }
            else if (lane == 0) {
                u32 slot = atomicAdd(&s_nbig, 1u);
                if (slot < 32) {
                    s_big[slot] = (u32)b;
                }
            }
        }
        __syncthreads();
        if (s_nbig > 0) {
            if (s_nbig > 32) {
                // too many oversized buckets to list: sort the whole collection
                group_sort_u64(dest, (int)n_g, tid, kThreads, CtaSync());
            }
            else {
                for (u32 i = 0; i < s_nbig; ++i) {
                    const int b  = (int)s_big[i];
                    const u32 lo = b == kNB - 1 ? 0u : S.hist[b + 1];
                    const u32 hi = S.hist[b];
                    group_sort_u64(dest + lo, (int)(hi - lo), tid, kThreads, CtaSync());
                }
            }
            __syncthreads();
        }

        if (!is_topp) {
            // top-k over probabilities: the k-th entry must not sit in the lowest collected class
            const int k_eff = k < (int)n_g ? k : (int)n_g;
            bool      ok    = complete || k_eff == 0
                      || (u32)(dest[k_eff - 1] >> 32) != (u32)(dest[n_g - 1] >> 32);
            if (!ok) {
                __syncthreads();
                continue;
            }
            topk_finish(P, S, O, dest, (int)n_g, k, u, top_p, false, want_lp);
            return;
        }

        // top-p: the block-wide inclusive scan of topp_sampling, 256 sorted probabilities per chunk,
        // in cub::BlockScan's raking order (32 segments of 8, Kogge-Stone across segment totals).
        if (wid == 0) {
            float     R       = 0.0f;
            int       sel     = -1;  // -1: threshold never reached, -2: ran out of collected data
            const int nchunks = (P.vocab_padded + 255) / 256;
            for (int c = 0; c < nchunks; ++c) {
                if (c * 256 >= (int)n_g) {
                    sel = complete ? -1 : -2;
                    break;
                }
                const int bi = c * 256 + lane * 8;
                float     x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    x[i] = bi + i < (int)n_g ? fkey_inv(~(u32)(dest[bi + i] >> 32)) : 0.0f;
                }
                float up = x[0];
#pragma unroll
                for (int i = 1; i < 8; ++i) {
                    up = up + x[i];
                }
                float inc = up;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    float t = __shfl_up_sync(0xffffffffu, inc, off);
                    if (lane >= off) {
                        inc = inc + t;
                    }
                }
                const float agg = __shfl_sync(0xffffffffu, inc, 31);
                const float ex  = __shfl_up_sync(0xffffffffu, inc, 1);
                float       o   = lane == 0 ? R : R + ex;
                u32         cnt = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o = o + x[i];
                    cnt += rand_num <= o ? 1u : 0u;
                }
                // a warp of the reference covers 4 of these lanes (32 consecutive probabilities)
                u32 c4 = cnt;
                c4 += __shfl_xor_sync(0xffffffffu, c4, 1);
                c4 += __shfl_xor_sync(0xffffffffu, c4, 2);
                const u32 any = __ballot_sync(0xffffffffu, c4 > 0);
                if (any) {
                    const int g   = (__ffs(any) - 1) >> 2;
                    const u32 pc  = __shfl_sync(0xffffffffu, c4, g * 4);
                    const int pos = c * 256 + g * 32 + (32 - (int)pc);
                    if (!complete && c * 256 + g * 32 + 31 >= (int)n_g) {
                        sel = -2;
                    }
                    else {
                        sel = pos;
                    }
                    break;
                }
                R = R + agg;
            }
            if (sel >= 0 && !complete && (u32)(dest[sel] >> 32) == (u32)(dest[n_g - 1] >> 32)) {
                sel = -2;  // the lowest collected class may be incomplete
            }
            if (lane == 0) {
                s_sel = sel;
            }
        }
        __syncthreads();
        const int sel = s_sel;
        if (sel == -2) {
            __syncthreads();
            continue;  // collect the whole row and repeat
        }
        if (tid == 0) {
            if (sel >= 0 && sel < (int)n_g) {
                const u64 e  = dest[sel];
                const int id = (int)(e & 0xffffffffu);
                *O.id_out    = id;
                if (want_lp) {
                    float lprob = logf(fkey_inv(~(u32)(e >> 32)));
                    if (P.cum_log_probs != nullptr) {
                        P.cum_log_probs[O.r] += lprob;
                    }
                    if (P.out_log_probs != nullptr) {
                        P.out_log_probs[O.r] = lprob;
                    }
                }
                write_lengths(P, O, id);
            }
            else {
                // cumulative sum never reached the draw: the reference leaves the best token in place
                // and updates neither length nor finished (sampling_topp_kernels.cu:954, :973-995)
                *O.id_out = (int)(dest[0] & 0xffffffffu);
            }
        }
        __syncthreads();
        return;
    }
}

template<int DT>
__device__ void process_row(const KParams& P, const Smem& S, int r, u64* gscratch)
{
    __shared__ float s_u;
    const int        tid = threadIdx.x;
    int              mode = 0;
    if (P.topk_states != nullptr && !(P.topk_skip != nullptr && P.topk_skip[r])) {
        mode = 1;
    }
    else if (P.topp_states != nullptr && !(P.topp_skip != nullptr && P.topp_skip[r])) {
        mode = 2;
    }
    RowOut O;
    O.r      = r;
    O.end_id = P.end_ids[r];
    O.id_out = P.output_ids + (size_t)P.step * P.batch_size + (size_t)P.ite * P.local_batch + r;

    const bool fin     = P.finished != nullptr ? P.finished[r] != 0 : false;
    const bool want_lp = P.cum_log_probs != nullptr || P.out_log_probs != nullptr;
    __syncthreads();  // every thread has read finished[r] before thread 0 may rewrite it

    if (mode == 1 && fin) {
        // sampling_topk_kernels.cu:249-252: end id, no draw, length unchanged
        if (tid == 0) {
            *O.id_out = O.end_id;
        }
    }
    else if (mode != 0) {
        if (tid == 0) {
            s_u = draw_uniform(mode == 1 ? P.topk_states : P.topp_states, r);
        }
        __syncthreads();
        const float u = s_u;
        if (mode == 2 && fin) {
            // one-hot row: probability 1/(1+1e-6) on the end id (sampling_topp_kernels.cu:1309-1341)
            if (tid == 0) {
                const float top_p = P.topp_ps[r];
                const float p0    = DT == FTB200_F16 ? __half2float(__float2half_rn(1.0f / (1.0f + 1e-6f))) :
                                                       1.0f / (1.0f + 1e-6f);
                *O.id_out         = O.end_id;
                if (p0 >= top_p || u * top_p <= p0) {
                    if (want_lp) {
                        float lprob = logf(p0);
                        if (P.cum_log_probs != nullptr) {
                            P.cum_log_probs[r] += lprob;
                        }
                        if (P.out_log_probs != nullptr) {
                            P.out_log_probs[r] = lprob;
                        }
                    }
                    if (P.seq_len != nullptr && P.finished != nullptr) {
                        P.finished[r] = 1;
                    }
                }
            }
        }
        else {
            RowCtx C;
            build_row<DT>(P, S, C, r);
            if (mode == 1) {
                int k = (int)P.topk_ks[r];
                k     = k < 1 ? 1 : (k > kMaxTopK ? kMaxTopK : k);
                const float top_p = P.topk_ps[r];
                if (want_lp) {
                    row_softmax<DT>(P, S, C, O, gscratch, false, k, u, top_p, true);
                }
                else if (k == 1) {
                    row_argmax<DT>(P, S, C, O);
                }
                else {
                    row_topk<DT>(P, S, C, O, gscratch, k, u, top_p);
                }
            }
            else {
                row_softmax<DT>(P, S, C, O, gscratch, true, 0, u, P.topp_ps[r], want_lp);
            }
        }
    }
    __syncthreads();
    // top-p decay / reset (sampling_topp_kernels.cu:1381-1408), applied to every row of the call
    if (P.topp_states != nullptr && P.topp_decay != nullptr && tid == 0) {
        const int id = *O.id_out;
        float     p  = P.topp_ps[r];
        if (id == P.topp_reset[r]) {
            p = P.topp_initial[r];
        }
        else {
            p = fmaxf(p * P.topp_decay[r], P.topp_min[r]);
        }
        P.topp_ps[r] = p;
    }
}

template<int DT>
__global__ void __launch_bounds__(kThreads, 3) decode_sampling_kernel(const __grid_constant__ KParams P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int                                s_row;
    Smem                                          S;
    S.cand  = (u64*)smem_raw;
    S.hist  = (u32*)(S.cand + kCap);
    S.val2  = (float*)(S.hist + kNB);
    S.flags = (u32*)(S.val2 + 1024);
    S.hash  = S.flags + P.flag_words;
    u64* gscratch = P.scratch + (size_t)blockIdx.x * P.scratch_stride;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) {
            s_row = (int)atomicAdd(P.ticket, 1u);
        }
        __syncthreads();
        const int r = s_row;
        if (r >= P.local_batch) {
            break;
        }
        process_row<DT>(P, S, r, gscratch);
    }
}


// ---- per-dtype launch glue (instantiated once per logits type, each in its own translation unit) ----
template<int DT>
int sampling_occupancy(size_t smem, int* per_sm)
{
    // one query per distinct shared-memory size; the answer is cached for the life of the process
    static size_t cached_smem[8];
    static int    cached_val[8];
    static int    n_cached = 0;
    for (int i = 0; i < n_cached; ++i) {
        if (cached_smem[i] == smem) {
            *per_sm = cached_val[i];
            return FTB200_OK;
        }
    }
    FTB_CUDA_CHECK(
        cudaFuncSetAttribute(decode_sampling_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    FTB_CUDA_CHECK(
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, decode_sampling_kernel<DT>, kThreads, smem));
    if (n_cached < 8) {
        cached_smem[n_cached] = smem;
        cached_val[n_cached]  = *per_sm;
        ++n_cached;
    }
    return FTB200_OK;
}

template<int DT>
int sampling_launch(const KParams& K, int grid, size_t smem, cudaStream_t st)
{
    decode_sampling_kernel<DT><<<grid, kThreads, smem, st>>>(K);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

}  // namespace ftb200
