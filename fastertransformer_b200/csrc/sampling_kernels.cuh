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

#include <mutex>
#include <type_traits>

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
    float* spre;   // per hash slot: value of that column after temperature, before penalty / ban
    float* sfin;   // per hash slot: final value of that column (-inf when banned or outside the vocabulary)
    unsigned short* hitq;  // [kThreads * kUnroll] vectors of the current batch that passed the packed filter
    u32*   nhit;   // [2] queue lengths, alternating per batch
};

__device__ __forceinline__ u64 global_timer_ns()
{
    u64 t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Diagnostic timeline: trace_mark(rec, i) stores the time at which thread 0 passed mark i of the current row.
// Marks (per row ticket, after the four header words row / CTA / start / end):
//   every soft-max row (top-p, top-k with log-probs)      two-pass top-k rows
//     0  row set-up done                                    0  row set-up done
//     1  maximum pass and special-column fetch done         1  slot-maximum pass and special-column fetch done
//    15  special columns compared with the maximum          2  cut chosen
//    16  (largest column penalised) slot maxima cleaned      9  packed filter done (word 14: queued vectors)
//     2  row maximum known                                  3  filtered pass done (word 18: candidates)
//    12  per-thread patch lists built                       4  special columns visited
//    13  ordered soft-max pass done (whole chunks)          5  sort and draw done
//     3  soft-max pass done (row tail included)
//    17  denominator reduced
//    19  provisional cut searched
//     4  provisional cut chosen
//   value-class path (16-bit top-p rows): 20 class count done, 5 special columns listed, 22 their sort done,
//     6 runs built (word 24 holds N | dense << 32 | runs << 40), 25 chunk aggregates done, 7 crossing found,
//     27 class of the crossing known, 8 class members collected; 11 class path left for the general path
//     (word 25: which check sent the row away).
constexpr int kTraceWords = 32;  // per row ticket: row, CTA, start, end, 28 marks
static __device__ void trace_mark(u64* rec, int i)
{
    if (rec != nullptr && threadIdx.x == 0) {
        rec[4 + i] = global_timer_ns();
    }
}

__device__ __forceinline__ u32 hash_slot(int id, int shift)
{
    return (u32)(id * 2654435761u) >> shift;
}

static __device__ void hash_insert(const KParams& P, const Smem& S, const RowCtx& C, int id, u32 flag)
{
    id -= P.vocab_offset;  // token id -> column of this (shard of the) vocabulary
    if (id < 0 || id >= P.vocab_padded) {
        return;
    }
    u32* const hash  = S.hash;
    u32* const flags = S.flags;
    FTB_ASSUME_SHARED(hash);
    FTB_ASSUME_SHARED(flags);
    u32 h    = hash_slot(id, P.hash_shift);
    u32 want = ((u32)id << 2) | flag;
    for (int probe = 0; probe < P.hash_slots; ++probe) {
        u32 old = smem_cas(&hash[h], kHashEmpty, want);
        if (old == kHashEmpty) {
            break;
        }
        if ((old >> 2) == (u32)id) {
            smem_or(&hash[h], flag);
            break;
        }
        h = (h + 1) & (P.hash_slots - 1);
    }
    const int sh  = P.dtype == FTB200_F32 ? 2 : 3;  // log2 of the columns per 16-byte vector
    int       rel = id - C.head;
    if (rel >= 0 && rel < (C.nvec << sh)) {
        int j   = rel >> sh;
        u32 bit = 1u << (j & 31);
        smem_or(&flags[j >> 5], bit);
    }
}

struct Xf;
__device__ __forceinline__ u32 hash_lookup_raw(const u32* hash, int shift, int mask, int id)
{
    FTB_ASSUME_SHARED(hash);
    u32 h = hash_slot(id, shift);
    for (int probe = 0; probe <= mask; ++probe) {
        u32 v = hash[h];
        if (v == kHashEmpty) {
            return 0;
        }
        if ((v >> 2) == (u32)id) {
            return v & 3u;
        }
        h = (h + 1) & mask;
    }
    return 0;
}

// The per-column arithmetic needs a handful of row constants.  They are gathered into one small value
// type that every loop copies into registers once: reading them through the kernel-argument block or
// through a reference inside a loop would cost a memory round trip per column.
struct Xf {
    const void* bias;
    float       inv_t, theta, neg_max;
    __half      inv_t_h;
    int         apply_temp, apply_rep, penalty_type, vocab, hash_shift, hash_mask;
    const u32*  hash;
};

__device__ __forceinline__ Xf make_xf(const KParams& P, const Smem& S, const RowCtx& C)
{
    Xf X;
    X.bias         = P.bias;
    X.inv_t        = C.inv_t;
    X.theta        = C.theta;
    X.neg_max      = C.neg_max;
    X.inv_t_h      = C.inv_t_h;
    X.apply_temp   = P.apply_temp;
    X.apply_rep    = P.apply_rep;
    X.penalty_type = P.penalty_type;
    X.vocab        = P.vocab;
    X.hash_shift   = P.hash_shift;
    X.hash_mask    = P.hash_slots - 1;
    X.hash         = S.hash;
    return X;
}

// Temperature (+ bias) exactly as the reference's kernels compute it in the logits type
// (sampling_penalty_kernels.cu:117-179): fp32 arithmetic for float, half arithmetic with the inverse
// temperature rounded to half for half.  bf16 inputs take the fp32 route on the up-cast value.
template<int DT>
__device__ __forceinline__ float temp_value(const Xf& X, u32 bits, int v)
{
    if (DT == FTB200_F16) {
        __half h = __ushort_as_half((unsigned short)bits);
        if (X.apply_temp) {
            if (X.bias != nullptr) {
                h = __hadd(h, ((const __half*)X.bias)[v]);
            }
            h = __hmul(h, X.inv_t_h);
        }
        return __half2float(h);
    }
    float x = (DT == FTB200_F32) ? __uint_as_float(bits) : __uint_as_float(bits << 16);
    if (X.apply_temp) {
        if (X.bias != nullptr) {
            float b = (DT == FTB200_F32) ? ((const float*)X.bias)[v] :
                                           __bfloat162float(((const __nv_bfloat16*)X.bias)[v]);
            x       = x + b;
        }
        x = x * X.inv_t;
    }
    return x;
}

// Penalty / mask for a token that has a hash entry.  Order of the reference: ban (-inf), temperature,
// repetition penalty from the pre-penalty value, min-length mask (sampling_penalty_kernels.cu:367-424,
// :485-500; ban_bad_words.cu:77-85).  A dead token is reported as -inf.
template<int DT>
__device__ __forceinline__ float special_value(const Xf& X, float y, u32 fl)
{
    if (fl & kFlagDead) {
        return -INFINITY;
    }
    if ((fl & kFlagHist) && X.apply_rep) {
        if (X.penalty_type == FTB200_PENALTY_MULTIPLICATIVE) {
            y = y < 0.0f ? y * X.theta : y / X.theta;
        }
        else if (X.penalty_type == FTB200_PENALTY_ADDITIVE) {
            y = y - X.theta;
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
    const Xf X = make_xf(P, S, C);
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
    float     y   = temp_value<DT>(X, bits, v);
    const int epv = DT == FTB200_F32 ? 4 : 8;
    int       rel = v - C.head;
    bool      sp  = true;
    if (rel >= 0 && rel < C.nvec * epv) {
        int j = rel / epv;
        sp    = (S.flags[j >> 5] >> (j & 31)) & 1u;
    }
    if (sp) {
        u32 fl = hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v);
        if (fl) {
            y = special_value<DT>(X, y, fl);
        }
    }
    return y;
}

// ---- streaming primitives ---------------------------------------------------------------------
// A row is read as 16-byte vectors.  Vectors that hold a token with a hash entry (history, banned,
// min-length) are skipped by the three loops below and visited by visit_specials(), together with
// the unaligned head / tail columns, so the hot loops carry no per-column look-up and do not diverge.
//
// B200 moves ~0.2 bytes per issued lane-instruction at full HBM rate, i.e. a 16-bit logit may cost
// about nine instructions.  The 16-bit loops therefore test two logits per instruction on the raw
// bit patterns (packed compare / max) and only unpack the rare vector that passes.

template<int DT>
__device__ __forceinline__ bool packed_ok(const KParams& P, const RowCtx& C)
{
    return DT != FTB200_F32 && P.bias == nullptr && C.inv_t > 0.0f;
}

// Largest raw 16-bit value r such that every column with final value >= thr_y has raw value >= r.
// Temperature is monotone for inv_t > 0; the margin covers the rounding of the forward computation.
template<int DT>
__device__ __forceinline__ u32 raw_threshold_pair(const KParams& P, const RowCtx& C, float thr_y)
{
    float t = thr_y;
    if (P.apply_temp && t > -FLT_MAX && t < FLT_MAX) {
        t = t / C.inv_t;
        t = t - fabsf(t) * (1.0f / 256.0f);
    }
    u32 r;
    if (DT == FTB200_F16) {
        t = fmaxf(t, -65504.0f);
        r = (u32)__half_as_ushort(__float2half_rd(t));
        if (thr_y <= -65504.0f) {
            r = 0xfc00u;  // -inf
        }
    }
    else {
        r = (u32)__bfloat16_as_ushort(__float2bfloat16_rd(t));
        if (thr_y <= -FLT_MAX) {
            r = 0xff80u;  // -inf
        }
    }
    return r | (r << 16);
}

template<int DT>
__device__ __forceinline__ u32 ge2_mask(u32 pair, u32 thr2)
{
    if (DT == FTB200_F16) {
        return __hge2_mask(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&thr2));
    }
    return __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&pair),
                       *reinterpret_cast<const __nv_bfloat162*>(&thr2));
}

template<int DT>
__device__ __forceinline__ u32 le2_mask(u32 pair, u32 thr2)
{
    if (DT == FTB200_F16) {
        return __hle2_mask(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&thr2));
    }
    return __hle2_mask(*reinterpret_cast<const __nv_bfloat162*>(&pair),
                       *reinterpret_cast<const __nv_bfloat162*>(&thr2));
}

// Smallest raw 16-bit value r such that every column with final value <= thr_y has raw value <= r.
template<int DT>
__device__ __forceinline__ u32 raw_ceiling_pair(const KParams& P, const RowCtx& C, float thr_y)
{
    float t = thr_y;
    if (P.apply_temp && t > -FLT_MAX && t < FLT_MAX) {
        t = t / C.inv_t;
        t = t + fabsf(t) * (1.0f / 256.0f);
    }
    u32 r;
    if (DT == FTB200_F16) {
        r = t >= 65504.0f ? 0x7c00u : (u32)__half_as_ushort(__float2half_ru(t));
    }
    else {
        r = t >= 3.38e38f ? 0x7f80u : (u32)__bfloat16_as_ushort(__float2bfloat16_ru(t));
    }
    return r | (r << 16);
}

template<int DT>
__device__ __forceinline__ u32 max2(u32 a, u32 b)
{
    if (DT == FTB200_F16) {
        __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<u32*>(&r);
    }
    __nv_bfloat162 r =
        __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<u32*>(&r);
}

template<int DT>
__device__ __forceinline__ const uint4* vec_base(const RowCtx& C)
{
    return (const uint4*)(C.rowp + (size_t)C.head * (DT == FTB200_F32 ? 4 : 2));
}

__device__ __forceinline__ u32 pick_word(const uint4& r, int i)
{
    return i < 2 ? (i == 0 ? r.x : r.y) : (i == 2 ? r.z : r.w);
}

template<int DT>
__device__ __forceinline__ u32 raw_bits(const uint4& r, int e)
{
    return DT == FTB200_F32 ? pick_word(r, e) : ((pick_word(r, e >> 1) >> ((e & 1) * 16)) & 0xffffu);
}

// f(v, y) for every column of the unflagged vectors in [j0, j1): exact final value, no filter.
template<int DT, class F>
__device__ __noinline__ void stream_all(const KParams& P, const Smem& S, const RowCtx& C, int j0, int j1, F&& f)
{
    const Xf X = make_xf(P, S, C);
    constexpr int EPV = DT == FTB200_F32 ? 4 : 8;
    const int     tid = threadIdx.x;
    const uint4*  vp  = vec_base<DT>(C);
#pragma unroll 1
    for (int j = j0 + tid; j < j1; j += kThreads) {
        const bool  sp = (S.flags[j >> 5] >> (j & 31)) & 1u;
        const uint4 r  = ld_nc_v4(vp + j);
        const int   vb = C.head + j * EPV;
#pragma unroll 1
        for (int e = 0; e < EPV; ++e) {
            int v = vb + e;
            if (sp && hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v)) {
                continue;  // special columns are reported by visit_specials
            }
            f(v, v >= P.vocab ? -INFINITY : temp_value<DT>(X, raw_bits<DT>(r, e), v));
        }
    }
}

// Hot side of the filtered stream: kUnroll 16-byte loads per thread, then one packed compare per two
// logits (16-bit types) or one multiply + compare per logit (fp32).  A vector with a passing column
// only has its batch-relative index queued in shared memory.  Takes nothing but scalars so that the
// whole loop lives in registers.
constexpr int kHotUnroll = 8;   // 16-byte loads in flight per thread in the register-only loops

constexpr int kHitCap   = kThreads * 16;  // entries of the hit queue (16-bit offsets)
constexpr int kHotBatch = kThreads * kHotUnroll;

// Queues the offsets (relative to jb) of the vectors of [jb, je) that may hold a passing column.  The
// counter keeps counting past the capacity so that the caller can see an overflow.
template<int DT, bool BAND = false>
__device__ __noinline__ void hot_filter(const uint4* vp, int jb, int je, float thr_y, u32 thr2, float inv, bool temp,
                                        unsigned short* hitq, u32* qn, u32 hi2 = 0)
{
    FTB_ASSUME_SHARED(hitq);
    FTB_ASSUME_SHARED(qn);
    const int tid = threadIdx.x;
    for (int j0 = jb; j0 < je; j0 += kHotBatch) {
        uint4 q[kHotUnroll];
#pragma unroll
        for (int u = 0; u < kHotUnroll; ++u) {
            int j = j0 + u * kThreads + tid;
            if (j < je) {
                q[u] = ld_nc_v4(vp + j);
            }
        }
#pragma unroll
        for (int u = 0; u < kHotUnroll; ++u) {
            if (j0 + u * kThreads + tid < je) {
                bool pass;
                if (DT == FTB200_F32) {
                    float a = __uint_as_float(q[u].x), b = __uint_as_float(q[u].y);
                    float c = __uint_as_float(q[u].z), d = __uint_as_float(q[u].w);
                    if (temp) {
                        a *= inv, b *= inv, c *= inv, d *= inv;  // the same multiply the exact path uses
                    }
                    pass = fmaxf(fmaxf(a, b), fmaxf(c, d)) >= thr_y;
                }
                else if (BAND) {
                    // columns inside [thr2, hi2]: both compares have to hold for the same half
                    pass = (((ge2_mask<DT>(q[u].x, thr2) & le2_mask<DT>(q[u].x, hi2))
                             | (ge2_mask<DT>(q[u].y, thr2) & le2_mask<DT>(q[u].y, hi2)))
                            | ((ge2_mask<DT>(q[u].z, thr2) & le2_mask<DT>(q[u].z, hi2))
                               | (ge2_mask<DT>(q[u].w, thr2) & le2_mask<DT>(q[u].w, hi2))))
                           != 0;
                }
                else {
                    pass = ((ge2_mask<DT>(q[u].x, thr2) | ge2_mask<DT>(q[u].y, thr2))
                            | (ge2_mask<DT>(q[u].z, thr2) | ge2_mask<DT>(q[u].w, thr2)))
                           != 0;
                }
                if (pass) {
                    const u32 pos = atomicAdd(qn, 1u);
                    if (pos < (u32)kHitCap) {
                        hitq[pos] = (unsigned short)(j0 - jb + u * kThreads + tid);
                    }
                }
            }
        }
    }
}

// hit(v, y) - or hit(v, y, raw bits) - for the columns of the unflagged vectors in [j0, j1) whose final
// value is >= thr().
// CTA-collective: every thread of the CTA must call it (it synchronises).
// Per batch: hot_filter() queues the vectors that may hold a passing column; after a barrier the queued
// vectors are fetched again (they are still in L1/L2) and handled one per thread, so the rare exact work
// runs dense instead of divergent.  thr() is read once per batch; a caller may raise it between batches.
// `span` is the number of vectors filtered per round: the default is one load batch, so that a caller can
// move its threshold often; a caller with a fixed threshold passes kWholeRow and the row is filtered in one
// go (a round whose hits do not fit the queue is repeated in single batches).
constexpr int kWholeRow = 65536;

template<int DT, class Thr, class Hit>
__device__ __noinline__ void
stream_filtered(const KParams& P, const Smem& S, const RowCtx& C, int j0, int j1, Thr&& thr, Hit&& hit, int span = kHotBatch,
                float thr_hi = INFINITY, u64* dbg = nullptr)
{
    const Xf X = make_xf(P, S, C);
    constexpr int   EPV   = DT == FTB200_F32 ? 4 : 8;
    const int       tid   = threadIdx.x;
    const uint4*    vp    = vec_base<DT>(C);
    const bool      fast  = DT == FTB200_F32 ? (P.bias == nullptr) : packed_ok<DT>(P, C);
    const bool      temp  = P.apply_temp != 0;
    const float     inv   = C.inv_t;
    const int       head  = C.head;
    const int       vocab = P.vocab;
    const u32*      flags = S.flags;
    unsigned short* hitq  = S.hitq;
    u32*            nhit  = S.nhit;
    FTB_ASSUME_SHARED(flags);
    FTB_ASSUME_SHARED(hitq);
    FTB_ASSUME_SHARED(nhit);
    int             par   = 0;
    if (!fast) {
        span = kHotBatch;
    }
    if (tid == 0) {
        nhit[0] = 0;
        nhit[1] = 0;
    }
    __syncthreads();
    for (int jb = j0; jb < j1;) {
        const int   je    = j1 - jb < span ? j1 : jb + span;
        const float thr_y = thr();
        const u32   thr2  = (fast && DT != FTB200_F32) ? raw_threshold_pair<DT>(P, C, thr_y) : 0u;
        const bool  band  = DT != FTB200_F32 && thr_hi < INFINITY;
        const u32   hi2   = (fast && band) ? raw_ceiling_pair<DT>(P, C, thr_hi) : 0u;
        if (fast) {
            if (band) {
                // a band of values: the hits of the packed filter are the columns between the two bounds
                hot_filter<DT, true>(vp, jb, je, thr_y, thr2, inv, temp, hitq, nhit + par, hi2);
            }
            else {
                hot_filter<DT>(vp, jb, je, thr_y, thr2, inv, temp, hitq, nhit + par);
            }
        }
        __syncthreads();
        // embedding bias or a non-positive temperature: every vector takes the exact path
        const int n = fast ? (int)nhit[par] : je - jb;
        if (dbg != nullptr) {
            trace_mark(dbg, 9);
            if (threadIdx.x == 0) {
                dbg[4 + 14] = (u64)n;
            }
        }
        if (fast && n > kHitCap) {
            // more hits than the queue holds: this round again, one load batch at a time
            __syncthreads();
            if (tid == 0) {
                nhit[par] = 0;
            }
            span = kHotBatch;
            __syncthreads();
            continue;
        }
        if (tid == 0) {
            nhit[par ^ 1] = 0;
        }
        // one column of a queued (or, without the filter, of every) vector: exact value, exact test
        auto column = [&](int j, const uint4& r, int e, bool sp) {
            const int v = head + j * EPV + e;
            if (v < vocab) {
                const u32   rb = raw_bits<DT>(r, e);
                const float y  = temp_value<DT>(X, rb, v);
                if (y >= thr_y) {
                    // special columns are reported by visit_specials with their final value
                    if (!(sp && hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v))) {
                        if constexpr (std::is_invocable_v<Hit, int, float, u32>) {
                            hit(v, y, rb);  // callers that bin by bit pattern
                        }
                        else {
                            hit(v, y);
                        }
                    }
                }
            }
        };
        // the next queued vector is on its way while this one is looked at
        int   j_next = 0;
        uint4 r_next = make_uint4(0u, 0u, 0u, 0u);
        if (tid < n) {
            j_next = jb + (fast ? (int)hitq[tid] : tid);
            r_next = ld_nc_v4(vp + j_next);
        }
#pragma unroll 1
        for (int i = tid; i < n; i += kThreads) {
            const int   j  = j_next;
            const uint4 r  = r_next;
            if (i + kThreads < n) {
                j_next = jb + (fast ? (int)hitq[i + kThreads] : i + kThreads);
                r_next = ld_nc_v4(vp + j_next);
            }
            const bool  sp = (flags[j >> 5] >> (j & 31)) & 1u;
            u32         pm = (1u << EPV) - 1u;  // columns of the vector that can pass
            if (DT != FTB200_F32 && fast) {
                // the packed compare that queued the vector says which halves can pass
                pm = 0;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const u32 word = pick_word(r, w);
                    u32       m    = ge2_mask<DT>(word, thr2);
                    if (band) {
                        m &= le2_mask<DT>(word, hi2);
                    }
                    pm |= ((m & 1u) | ((m >> 15) & 2u)) << (2 * w);
                }
            }
#pragma unroll 1
            while (pm != 0) {
                const int e = __ffs(pm) - 1;
                pm &= pm - 1;
                column(j, r, e, sp);
            }
        }
        __syncthreads();
        jb = je;
        par ^= 1;
    }
}

// Hot side of the row maximum: packed (16-bit) or plain (fp32) running maximum over raw values.
template<int DT>
__device__ __noinline__ u32 hot_max(const uint4* vp, int jn)
{
    const int tid   = threadIdx.x;
    float     best  = -INFINITY;
    u32       best2 = DT == FTB200_F16 ? 0xfc00fc00u : 0xff80ff80u;
    for (int jb = 0; jb < jn; jb += kThreads * kHotUnroll) {
        uint4 q[kHotUnroll];
#pragma unroll
        for (int u = 0; u < kHotUnroll; ++u) {
            int j = jb + u * kThreads + tid;
            if (j < jn) {
                q[u] = ld_nc_v4(vp + j);
            }
        }
#pragma unroll
        for (int u = 0; u < kHotUnroll; ++u) {
            if (jb + u * kThreads + tid < jn) {
                if (DT == FTB200_F32) {
                    best = fmaxf(best, fmaxf(fmaxf(__uint_as_float(q[u].x), __uint_as_float(q[u].y)),
                                             fmaxf(__uint_as_float(q[u].z), __uint_as_float(q[u].w))));
                }
                else {
                    best2 = max2<DT>(max2<DT>(best2, q[u].x), max2<DT>(q[u].y, max2<DT>(q[u].z, q[u].w)));
                }
            }
        }
    }
    return DT == FTB200_F32 ? __float_as_uint(best) : best2;
}

// Largest temperature-scaled value of the row (thread-local; -inf when none).  With include_flagged the
// hot loop covers every column as if none were penalised or banned; without it the special columns
// (those with a hash entry) are left out, at the price of a per-column look-up in flagged vectors.
// Order-preserving 16-bit key of a half / bfloat16 bit pattern (sign-magnitude -> unsigned order).
__device__ __forceinline__ u32 key16(u32 h)
{
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}
__device__ __forceinline__ u32 key16_inv(u32 k)
{
    return (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
}

// Per-thread maxima of eight disjoint column subsets ("slots"), see the two-pass top-k below.
constexpr int kSlotsPerThread = 8;
constexpr int kSlots          = kSlotsPerThread * kThreads;

template<int DT>
__device__ __forceinline__ void hot_slotmax_body(const uint4* vp, int jn, u32* slots)
{
    FTB_ASSUME_SHARED(slots);
    const int tid = threadIdx.x;
    if (DT == FTB200_F32) {
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a[i] = -INFINITY;
        }
        for (int jb = 0; jb < jn; jb += kThreads * kHotUnroll) {
            uint4 q[kHotUnroll];
#pragma unroll
            for (int u = 0; u < kHotUnroll; ++u) {
                const int j = jb + u * kThreads + tid;
                if (j < jn) {
                    q[u] = ld_nc_v4(vp + j);
                }
            }
#pragma unroll
            for (int u = 0; u < kHotUnroll; ++u) {
                if (jb + u * kThreads + tid < jn) {
                    const int h = (u & 1) * 4;
                    a[h + 0]    = fmaxf(a[h + 0], __uint_as_float(q[u].x));
                    a[h + 1]    = fmaxf(a[h + 1], __uint_as_float(q[u].y));
                    a[h + 2]    = fmaxf(a[h + 2], __uint_as_float(q[u].z));
                    a[h + 3]    = fmaxf(a[h + 3], __uint_as_float(q[u].w));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            slots[i * kThreads + tid] = fkey(a[i]);
        }
    }
    else {
        const u32 ninf = DT == FTB200_F16 ? 0xfc00fc00u : 0xff80ff80u;
        u32       a0 = ninf, a1 = ninf, a2 = ninf, a3 = ninf;
        for (int jb = 0; jb < jn; jb += kThreads * kHotUnroll) {
            uint4 q[kHotUnroll];
#pragma unroll
            for (int u = 0; u < kHotUnroll; ++u) {
                const int j = jb + u * kThreads + tid;
                if (j < jn) {
                    q[u] = ld_nc_v4(vp + j);
                }
            }
#pragma unroll
            for (int u = 0; u < kHotUnroll; ++u) {
                if (jb + u * kThreads + tid < jn) {
                    a0 = max2<DT>(a0, q[u].x);
                    a1 = max2<DT>(a1, q[u].y);
                    a2 = max2<DT>(a2, q[u].z);
                    a3 = max2<DT>(a3, q[u].w);
                }
            }
        }
        slots[0 * kThreads + tid] = key16(a0 & 0xffffu) << 16;
        slots[1 * kThreads + tid] = key16(a0 >> 16) << 16;
        slots[2 * kThreads + tid] = key16(a1 & 0xffffu) << 16;
        slots[3 * kThreads + tid] = key16(a1 >> 16) << 16;
        slots[4 * kThreads + tid] = key16(a2 & 0xffffu) << 16;
        slots[5 * kThreads + tid] = key16(a2 >> 16) << 16;
        slots[6 * kThreads + tid] = key16(a3 & 0xffffu) << 16;
        slots[7 * kThreads + tid] = key16(a3 >> 16) << 16;
    }
}

template<int DT>
__device__ __noinline__ void hot_slotmax(const uint4* vp, int jn, u32* slots)
{
    hot_slotmax_body<DT>(vp, jn, slots);
}

// Slot maxima that a pass over every column at its raw value left behind, made safe for taking the maximum over
// the ordinary columns: a slot whose maximum may be a special column's value before its penalty, and that lies
// above the largest slot no special column can top, is read again (its ~vocab/2048 columns, two bytes each)
// with the special columns left out.  The other such slots keep their value: they cannot hold the maximum.
// Returns false when more slots are affected than the list holds; the caller then reads the row again.
constexpr int kMaxDirtySlots = 64;
static __device__ u64 block_max_u64(u64 v);
template<int DT>
__device__ __noinline__ bool clean_special_slots(const KParams& P, const Smem& S, const RowCtx& C, u32* slots)
{
    static_assert(DT != FTB200_F32, "16-bit logits only");
    __shared__ u32 s_dirty[kMaxDirtySlots];
    __shared__ u32 s_nd;
    const Xf       X     = make_xf(P, S, C);
    const int      tid   = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int      nfull = P.vocab >= P.vocab_padded ? C.nvec : (P.vocab - C.head > 0 ? (P.vocab - C.head) / 8 : 0);
    FTB_ASSUME_SHARED(slots);
    if (tid == 0) {
        s_nd = 0;
    }
    // bit 0 of a slot word (keys sit in the upper half) marks a slot that a special column may top
    for (int i = tid; i < P.hash_slots; i += kThreads) {
        const u32 w = X.hash[i];
        if (w == kHashEmpty) {
            continue;
        }
        const int v = (int)(w >> 2), o = v - C.head;
        if (o < 0 || (o >> 3) >= nfull) {
            continue;
        }
        const int slot = (o & 7) * kThreads + ((o >> 3) & (kThreads - 1));
        if (S.spre[i] >= temp_value<DT>(X, key16_inv(slots[slot] >> 16), 0)) {
            smem_or(&slots[slot], 1u);
        }
    }
    __syncthreads();
    u32 safe = 0;
    for (int i = 0; i < kSlotsPerThread; ++i) {
        const u32 k = slots[i * kThreads + tid];
        safe        = (k & 1u) == 0 && k > safe ? k : safe;
    }
    safe = (u32)block_max_u64((u64)safe);
    for (int i = 0; i < kSlotsPerThread; ++i) {
        const int slot = i * kThreads + tid;
        const u32 k    = slots[slot];
        if (k & 1u) {
            slots[slot] = k & ~1u;
            if (k > safe) {
                const u32 at = atomicAdd(&s_nd, 1u);
                if (at < (u32)kMaxDirtySlots) {
                    s_dirty[at] = (u32)slot;
                }
            }
        }
    }
    __syncthreads();
    const u32 nd = s_nd;
    if (nd > (u32)kMaxDirtySlots) {
        return false;
    }
    const unsigned short* row16 = (const unsigned short*)C.rowp;
    for (u32 d = wid; d < nd; d += kWarps) {
        const int slot = (int)s_dirty[d], e = slot / kThreads, ts = slot % kThreads;
        u32       key = 0;
#pragma unroll 1
        for (int j = ts + kThreads * lane; j < nfull; j += kThreads * 32) {
            const int v = C.head + j * 8 + e;
            if (((S.flags[j >> 5] >> (j & 31)) & 1u) && hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v)) {
                continue;
            }
            const u32 k = key16((u32)__ldg(row16 + v));
            key         = k > key ? k : key;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const u32 other = __shfl_xor_sync(0xffffffffu, key, o);
            key             = other > key ? other : key;
        }
        if (lane == 0) {
            slots[slot] = key << 16;
        }
    }
    __syncthreads();
    return true;
}

// With clean_slots (the slot maxima of the 16-byte-vector part of the row, already free of special columns) the
// vector part is not read again.
template<int DT>
__device__ __noinline__ float stream_max(const KParams& P, const Smem& S, const RowCtx& C, bool include_flagged,
                                         u32* raw_key_max = nullptr, u32* slots = nullptr,
                                         const u32* clean_slots = nullptr)
{
    const Xf X = make_xf(P, S, C);
    constexpr int EPV   = DT == FTB200_F32 ? 4 : 8;
    const int     tid   = threadIdx.x;
    const uint4*  vp    = vec_base<DT>(C);
    const bool    pk    = packed_ok<DT>(P, C);
    const bool    fast  = (DT == FTB200_F32 ? (P.bias == nullptr && C.inv_t > 0.0f) : pk)
                      && (include_flagged || (DT != FTB200_F32 && clean_slots != nullptr));
    const int     nfull = P.vocab >= P.vocab_padded ? C.nvec : (P.vocab - C.head > 0 ? (P.vocab - C.head) / EPV : 0);
    float         best  = -INFINITY;
    u32           kraw  = 0;
    const int     jfast = fast ? nfull : 0;
    if (jfast > 0) {
        // temperature is monotone for inv_t > 0: the largest raw value gives the largest final value
        if (DT != FTB200_F32 && clean_slots != nullptr) {
            u32 km = 0;
            for (int i = 0; i < kSlotsPerThread; ++i) {
                const u32 k = clean_slots[i * kThreads + tid] >> 16;
                km          = k > km ? k : km;
            }
            kraw = km;
            best = temp_value<DT>(X, key16_inv(km), 0);
        }
        else if (DT != FTB200_F32 && slots != nullptr) {
            // same pass, but the eight per-thread subset maxima are kept (ordered keys << 16)
            hot_slotmax<DT>(vp, jfast, slots);
            u32 km = 0;
            for (int i = 0; i < kSlotsPerThread; ++i) {
                const u32 k = slots[i * kThreads + tid] >> 16;
                km          = k > km ? k : km;
            }
            kraw = km;
            best = temp_value<DT>(X, key16_inv(km), 0);
        }
        else {
        const u32 m = hot_max<DT>(vp, jfast);
        if (DT == FTB200_F32) {
            const float raw = __uint_as_float(m);
            best            = raw > -INFINITY ? temp_value<DT>(X, m, 0) : raw;
        }
        else {
            best = fmaxf(temp_value<DT>(X, m & 0xffffu, 0), temp_value<DT>(X, m >> 16, 0));
            const u32 ka = key16(m & 0xffffu), kb = key16(m >> 16);
            kraw         = ka > kb ? ka : kb;
        }
        }
    }
#pragma unroll 1
    for (int j = jfast + tid; j < C.nvec; j += kThreads) {
        const bool  sp = !include_flagged && ((S.flags[j >> 5] >> (j & 31)) & 1u);
        const uint4 r  = ld_nc_v4(vp + j);
        const int   vb = C.head + j * EPV;
#pragma unroll 1
        for (int e = 0; e < EPV; ++e) {
            const int v = vb + e;
            if (v < P.vocab && !(sp && hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v))) {
                const u32 rb = raw_bits<DT>(r, e);
                best         = fmaxf(best, temp_value<DT>(X, rb, v));
                if (DT != FTB200_F32) {
                    const u32 k = key16(rb);
                    kraw        = k > kraw ? k : kraw;
                }
            }
        }
    }
    if (raw_key_max != nullptr) {
        *raw_key_max = kraw;
    }
    return best;
}

// f(v, y) for every special column (history token, banned word, min-length mask: the entries of the
// hash table) with its final value, and for the unaligned head / tail columns of the row.
// Columns whose final value is below thr_y are not reported (pass -inf to see every column).
template<int DT, class F>
__device__ __noinline__ void visit_specials(const KParams& P, const Smem& S, const RowCtx& C, float thr_y, F&& f)
{
    constexpr int EPV = DT == FTB200_F32 ? 4 : 8;
    const Xf      X   = make_xf(P, S, C);
    const int     tid = threadIdx.x;
    const char*   rowp = C.rowp;
    const int     nslots = P.hash_slots;
    const float*  sfin   = S.sfin;
    FTB_ASSUME_SHARED(sfin);
    FTB_ASSUME_SHARED(X.hash);
#pragma unroll 1
    for (int i = tid; i < nslots; i += kThreads) {
        const u32 w = X.hash[i];
        if (w == kHashEmpty) {
            continue;
        }
        const int   v = (int)(w >> 2);
        const float y = sfin[i];
        if (y >= thr_y) {
            f(v, y);
        }
    }
    // row edges that no 16-byte vector covers; special ones were reported above
    const int tail0 = C.head + C.nvec * EPV;
    const int nedge = C.head + (P.vocab_padded - tail0);
#pragma unroll 1
    for (int i = tid; i < nedge; i += kThreads) {
        const int v = i < C.head ? i : tail0 + (i - C.head);
        if (hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v)) {
            continue;
        }
        float y = -INFINITY;
        if (v < X.vocab) {
            const u32 bits = DT == FTB200_F32 ? __ldg((const u32*)rowp + v) : (u32)__ldg((const unsigned short*)rowp + v);
            y              = temp_value<DT>(X, bits, v);
        }
        if (y >= thr_y) {
            f(v, y);
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

// Integer form of find_from_top over plain counts: the largest bucket b whose suffix sum reaches `target`
// (-1 when the total stays below), and the count strictly above it.
static __device__ __noinline__ int find_count_from_top(const u32* hist, u32 target, u32* above_out)
{
    __shared__ u32 s_part[kWarps];
    __shared__ int s_found;
    __shared__ u32 s_above;
    constexpr int  PER = kNB / kThreads;
    const int      tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    FTB_ASSUME_SHARED(hist);
    if (tid == 0) {
        s_found = -1;
        s_above = 0;
    }
    u32 c[PER], local = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        c[i] = hist[kNB - 1 - (tid * PER + i)];
        local += c[i];
    }
    u32 incl = local;
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) {
            incl += t;
        }
    }
    if (lane == 31) {
        s_part[wid] = incl;
    }
    __syncthreads();
    u32 base = 0;
    for (int i = 0; i < wid; ++i) {
        base += s_part[i];
    }
    const u32 excl = base + incl - local;
    if (excl < target && excl + local >= target) {
        u32 run = excl;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (run < target && run + c[i] >= target) {
                s_found = kNB - 1 - (tid * PER + i);
                s_above = run;
            }
            run += c[i];
        }
    }
    __syncthreads();
    const int r = s_found;
    *above_out  = s_above;
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

    if (tid == 0) {  // C is shared by the CTA; the barrier below publishes it
        C.rowp          = (const char*)P.logits + (size_t)r * P.vocab_padded * ES;
        const size_t ad = (size_t)C.rowp;
        int          hd = (int)(((16 - (ad & 15)) & 15) / ES);
        C.head          = hd < P.vocab_padded ? hd : P.vocab_padded;
        C.nvec          = (P.vocab_padded - C.head) / EPV;
        float inv_t     = 1.0f;
        if (P.apply_temp) {
            inv_t = 1.0f / (P.temperature[r] + 1e-6f);
        }
        C.inv_t   = inv_t;
        C.inv_t_h = __float2half_rn(inv_t);
        C.theta   = P.apply_rep ? P.rep_penalty[r] : 1.0f;
        C.neg_max = DT == FTB200_F16 ? -65504.0f : -FLT_MAX;
    }

    const size_t col = (size_t)P.ite * P.local_batch + r;
    // The global loads of this set-up are issued level by level, all independent ones together, so that a
    // thread waits for memory two or three times instead of once per token.
    // level 1: word-list offsets of this thread's bad word, first batch of history ids
    const int  L        = P.bad_words != nullptr ? P.bad_words_len : 0;
    const int* wbase    = L > 0 ? (P.bad_words_shared ? P.bad_words : P.bad_words + (size_t)r * 2 * L) : nullptr;
    const bool has_word = tid < L;  // lists longer than the CTA take the loop at the end
    int        item_end = -1, item_start = 0;
    if (has_word) {
        item_end   = wbase[L + tid];
        item_start = tid > 0 ? wbase[L + tid - 1] : 0;
    }
    constexpr int HB        = 4;
    const int     input_len = P.apply_rep ? (P.input_lengths != nullptr ? P.input_lengths[r] : P.max_input_len) : 0;
    const int     nhist     = P.apply_rep ? P.step : 0;
    int           ids[HB];
    bool          okh[HB];
#pragma unroll
    for (int q = 0; q < HB; ++q) {
        const int t = q * kThreads + tid;
        okh[q]      = t < nhist && !(t >= input_len && t < P.max_input_len);
        ids[q]      = okh[q] ? P.output_ids[(size_t)t * P.batch_size + col] : 0;
    }
    // level 2: the tokens of the word and the generated tokens it has to match (ban_bad_words.cu:35-85):
    // a word bans its last token when the preceding tokens match the tail of the generated sequence;
    // token 0 can never be banned.
    int  ban_tok = 0;
    bool ban     = false;
    if (has_word && item_end >= 0) {
        const int item_size = item_end - item_start;
        ban                 = item_size == 1;
        ban_tok             = wbase[item_end - 1];
        if (item_size > 1 && P.step >= item_size - 1) {
            ban = true;
            if (item_size <= 4) {
                int want[3], have[3];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const bool in = j < item_size - 1;
                    want[j]       = in ? wbase[item_start + j] : 0;
                    have[j]       = in ? P.output_ids[(size_t)(P.step - (item_size - 1) + j) * P.batch_size + col] : 0;
                }
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    ban = ban && want[j] == have[j];
                }
            }
            else {
                for (int j = item_size - 2; j >= 0; --j) {
                    const int prev = P.output_ids[(size_t)(P.step - (item_size - 1) + j) * P.batch_size + col];
                    if (prev != wbase[item_start + j]) {
                        ban = false;
                        break;
                    }
                }
            }
        }
    }
    // (the table is cleared while those loads are in flight)
    for (int i = tid; i < P.hash_slots; i += kThreads) {
        S.hash[i] = kHashEmpty;
    }
    for (int i = tid; i < P.flag_words; i += kThreads) {
        S.flags[i] = 0;
    }
    __syncthreads();
    // token history -> repetition / presence penalty (sampling_penalty_kernels.cu:385-410)
#pragma unroll
    for (int q = 0; q < HB; ++q) {
        if (okh[q]) {
            hash_insert(P, S, C, ids[q], kFlagHist);
        }
    }
    for (int t = HB * kThreads + tid; t < nhist; t += kThreads) {
        if (t >= input_len && t < P.max_input_len) {
            continue;
        }
        hash_insert(P, S, C, P.output_ids[(size_t)t * P.batch_size + col], kFlagHist);
    }
    if (ban && 0 < ban_tok && (P.vp_out != nullptr || ban_tok < P.vocab_padded)) {
        hash_insert(P, S, C, ban_tok, kFlagDead);
    }
    // word lists with more entries than the CTA has threads
    for (int i = tid + kThreads; i < L; i += kThreads) {
        const int* offs = wbase + L;
        const int  e1   = offs[i];
        if (e1 < 0) {
            continue;
        }
        const int s1   = offs[i - 1];
        const int size = e1 - s1;
        bool      b    = size == 1;
        if (size > 1 && P.step >= size - 1) {
            b = true;
            for (int j = size - 2; j >= 0; --j) {
                const int prev = P.output_ids[(size_t)(P.step - (size - 1) + j) * P.batch_size + col];
                if (prev != wbase[s1 + j]) {
                    b = false;
                    break;
                }
            }
        }
        if (b) {
            const int tok = wbase[e1 - 1];
            if (0 < tok && (P.vp_out != nullptr || tok < P.vocab_padded)) {
                hash_insert(P, S, C, tok, kFlagDead);
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

// Values of the special columns (before and after penalty / ban), fetched with all loads of a thread in
// flight together; every later visit of the specials reads shared memory only.  Called after the row's
// first streaming pass, when the row sits in L2 and the scattered 2-byte reads no longer go to DRAM.
template<int DT>
__device__ __noinline__ void fetch_specials(const KParams& P, const Smem& S, const RowCtx& C)
{
    const int tid = threadIdx.x;
    {
        const Xf      X  = make_xf(P, S, C);
        constexpr int SB = 8;
        u32* const    hash = S.hash;
        float* const  spre = S.spre;
        float* const  sfin = S.sfin;
        FTB_ASSUME_SHARED(hash);
        FTB_ASSUME_SHARED(spre);
        FTB_ASSUME_SHARED(sfin);
        for (int i0 = tid; i0 < P.hash_slots; i0 += kThreads * SB) {
            u32 w[SB], bits[SB];
#pragma unroll
            for (int q = 0; q < SB; ++q) {
                const int i = i0 + q * kThreads;
                w[q]        = i < P.hash_slots ? hash[i] : kHashEmpty;
            }
#pragma unroll
            for (int q = 0; q < SB; ++q) {
                // unconditional loads (column 0 stands in for an empty slot): all eight are in flight together
                const bool use = w[q] != kHashEmpty && (int)(w[q] >> 2) < P.vocab;
                const int  v   = use ? (int)(w[q] >> 2) : 0;
                bits[q] = DT == FTB200_F32 ? __ldg((const u32*)C.rowp + v) : (u32)__ldg((const unsigned short*)C.rowp + v);
            }
#pragma unroll
            for (int q = 0; q < SB; ++q) {
                const int i = i0 + q * kThreads;
                if (i < P.hash_slots) {
                    float pre = -INFINITY, fin = -INFINITY;
                    if (w[q] != kHashEmpty && (int)(w[q] >> 2) < P.vocab) {
                        pre = temp_value<DT>(X, bits[q], (int)(w[q] >> 2));
                        fin = special_value<DT>(X, pre, w[q] & 3u);
                    }
                    spre[i] = pre;
                    sfin[i] = fin;
                }
            }
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
    u64*     trace;  // this row's record of the diagnostic timeline, or null
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
    // e_i in parallel; the sum and the walk keep the reference's sequential order (:276-287)
    {
        const float s_max = k_eff > 0 ? fkey_inv(~(u32)(sorted[0] >> 32)) : 0.0f;
        for (int i = tid; i < k_eff; i += kThreads) {
            float y   = fkey_inv(~(u32)(sorted[i] >> 32));
            S.val2[i] = use_exp ? __expf(y - s_max) : y;
        }
    }
    __syncthreads();
    // The sum and the walk are chains of dependent adds in the reference's order (one thread).  The walk stores
    // every running value instead of testing it; the first one that ends the reference's loop is then found by
    // all threads.  Operands are fetched eight at a time so that the chains do not wait for shared memory.
    float* run = (float*)S.hist;  // [k_eff] running values; the bucket counts are not needed any more
    FTB_ASSUME_SHARED(run);
    __shared__ int s_walked;
    if (tid == 0) {
        s_pick   = k_eff > 0 ? k_eff - 1 : -1;
        s_walked = 0;
        if (k_eff > 0) {
            const float* val = S.val2;
            FTB_ASSUME_SHARED(val);
            const int k8  = k_eff & ~7;
            float     sum = 0.0f;
            float     v[8], w[8];
            if (k8 > 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = val[j];
                }
            }
            for (int i = 0; i < k8; i += 8) {
                if (i + 8 < k8) {  // the next eight are on their way while these are added
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        w[j] = val[i + 8 + j];
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    sum += v[j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = w[j];
                }
            }
            for (int i = k8; i < k_eff; ++i) {
                sum += val[i];
            }
            float rand_num = u * top_p * sum;
            int   walked   = 0;
            if (k8 > 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = val[j];
                }
            }
            // the terms are not negative, so the running value only falls: once a group of eight ends at or
            // below zero the reference's loop has stopped inside it
            for (int i = 0; i < k8 && !(rand_num <= 0.0f); i += 8) {
                if (i + 8 < k8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        w[j] = val[i + 8 + j];
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    rand_num   = rand_num - v[j];
                    run[i + j] = rand_num;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = w[j];
                }
                walked = i + 8;
            }
            if (walked == k8) {
                for (int i = k8; i < k_eff && !(rand_num <= 0.0f); ++i) {
                    rand_num = rand_num - val[i];
                    run[i]   = rand_num;
                    walked   = i + 1;
                }
            }
            s_walked = walked;
            s_sum    = sum;
        }
    }
    __syncthreads();
    for (int i = tid, nw = s_walked; i < nw; i += kThreads) {
        if (run[i] <= 0.0f || i == k - 1) {
            atomicMin(&s_pick, i);
            break;  // later entries of this thread are larger
        }
    }
    __syncthreads();
    if (tid == 0 && s_pick >= 0) {
        s_e  = S.val2[s_pick];
        s_lo = s_pick;
        s_hi = s_pick + 1;
    }
    __syncthreads();
    trace_mark(O.trace, 21);
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
    trace_mark(O.trace, 23);
    const int lo = s_lo, hi = s_hi;
    int       col;
    if (hi - lo == 1) {
        col = (int)(sorted[pick] & 0xffffffffu);
    }
    else {
        const u32 bs1 = P.max_top_k <= 16 ? 128 : 256;
        const u32 bs2 = P.max_top_k <= 32 ? 128 : 256;
        {
            // per-thread counts packed 8 x 8 bits (a thread sees at most kCap / kThreads entries), one atomic
            // per lane value and warp
            const int sh1   = bs1 == 128 ? 7 : 8;
            u64       packd = 0;
            for (int i = tid; i < lo; i += kThreads) {
                const u32 c = (u32)(sorted[i] & 0xffffffffu);
                packd += 1ull << (8 * ((c >> sh1) & 7u));
            }
            for (int l = 0; l < 8; ++l) {
                u32 cnt = (u32)(packd >> (8 * l)) & 0xffu;
                for (int m = 16; m > 0; m >>= 1) {
                    cnt += __shfl_xor_sync(0xffffffffu, cnt, m);
                }
                if ((tid & 31) == 0 && cnt != 0) {
                    atomicAdd(&s_lane_base[l], cnt);
                }
            }
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
    __shared__ u64 s_best;
    const u32      bs1 = P.max_top_k <= 16 ? 128 : 256;
    if (threadIdx.x == 0) {
        s_best = 0;
    }
    __syncthreads();
    const int sh1 = bs1 == 128 ? 7 : 8;
    auto consider = [&](int v, float y) {
        if (y > C.neg_max) {
            // value, then CTA lane descending, thread descending, column ascending
            u32 tie = ((((u32)v >> sh1) & 7u) << 29) | (((u32)v & (bs1 - 1)) << 21) | (0x1fffffu - (u32)v);
            const u64 c = ((u64)fkey(y) << 32) | tie;
            if (c > *(volatile u64*)&s_best) {
                atomicMax(&s_best, c);
            }
        }
    };
    // the filter threshold is the CTA's running maximum: only a handful of columns per row reach
    // the exact compare, so a warp almost never leaves the packed loop
    auto running = [&]() {
        const u64 b = *(volatile u64*)&s_best;
        return b == 0 ? -INFINITY : fkey_inv((u32)(b >> 32));
    };
    // one vector per thread seeds the maximum, one load batch sharpens it; the rest of the row is then filtered
    // in one round against that bound (a column above the maximum of the first 16 k is a rare event)
    const int jseed  = C.nvec < kThreads ? C.nvec : kThreads;
    const int jbatch = C.nvec < kHotBatch ? C.nvec : kHotBatch;
    stream_filtered<DT>(P, S, C, 0, jseed, running, consider);
    stream_filtered<DT>(P, S, C, jseed, jbatch, running, consider);
    stream_filtered<DT>(P, S, C, jbatch, C.nvec, running, consider, kWholeRow);
    fetch_specials<DT>(P, S, C);
    visit_specials<DT>(P, S, C, running(), consider);
    __syncthreads();
    if (threadIdx.x == 0) {
        const u64 best = s_best;
        int       id   = best == 0 ? 0 : (int)(0x1fffffu - (u32)(best & 0x1fffffu));
        *O.id_out      = id;
        write_lengths(P, O, id);
    }
    __syncthreads();
}

// Candidates (~key(value) << 32 | column) into value-descending order.  Up to half the candidate area a
// counting sort on the leading key bits does it in two sweeps (the other half receives the result); buckets
// that hold more than one distinct key - possible when the keys span more than 4096 values - are finished by
// a small sort each.  Larger sets take the bitonic network in place.  Returns where the sorted entries are.
static __device__ __noinline__ u64* sort_candidates(const Smem& S, u64* cand, int n)
{
    __shared__ u32 s_w[kWarps];
    __shared__ u32 s_bits[kNB / 32];
    const int      tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (n > kCap / 2 || cand != S.cand || n < 64) {
        group_sort_u64(cand, n, tid, kThreads, CtaSync());
        __syncthreads();
        return cand;
    }
    u64* dst = cand + kCap / 2;
    u32  kmin = 0xffffffffu, kmax = 0;
    for (int i = tid; i < n; i += kThreads) {
        const u32 k = (u32)(cand[i] >> 32);
        kmin        = k < kmin ? k : kmin;
        kmax        = k > kmax ? k : kmax;
    }
    kmin = ~(u32)block_max_u64((u64)(~kmin));
    kmax = (u32)block_max_u64((u64)kmax);
    int shift = 0;
    while (((kmax - kmin) >> shift) >= (u32)kNB) {
        ++shift;
    }
    u32* hist = S.hist;
    for (int i = tid; i < kNB; i += kThreads) {
        hist[i] = 0;
    }
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
        smem_add(&hist[((u32)(cand[i] >> 32) - kmin) >> shift], 1u);
    }
    __syncthreads();
    {
        // exclusive scan, ascending buckets: hist becomes the scatter cursor
        constexpr int PER = kNB / kThreads;
        u32           c[PER], mine = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            c[i] = hist[tid * PER + i];
            mine += c[i];
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) {
                incl += t;
            }
        }
        if (lane == 31) {
            s_w[wid] = incl;
        }
        __syncthreads();
        u32 base = 0;
        for (int i = 0; i < wid; ++i) {
            base += s_w[i];
        }
        u32 at = base + incl - mine;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            hist[tid * PER + i] = at;
            at += c[i];
        }
    }
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
        const u64 e = cand[i];
        dst[atomicAdd(&hist[((u32)(e >> 32) - kmin) >> shift], 1u)] = e;
    }
    __syncthreads();
    if (shift > 0) {
        // a bucket with two different keys next to each other has to be ordered
        for (int i = tid; i < kNB / 32; i += kThreads) {
            s_bits[i] = 0;
        }
        __syncthreads();
        for (int i = tid + 1; i < n; i += kThreads) {
            const u32 ka = (u32)(dst[i - 1] >> 32), kb = (u32)(dst[i] >> 32);
            const u32 ba = (ka - kmin) >> shift, bb = (kb - kmin) >> shift;
            if (ba == bb && ka != kb) {
                atomicOr(&s_bits[bb >> 5], 1u << (bb & 31));
            }
        }
        __syncthreads();
        for (int j = wid; j < kNB / 32; j += kWarps) {
            u32 word = s_bits[j];  // the same for every lane of the warp
            while (word != 0) {
                const u32 b  = (u32)j * 32u + (u32)(__ffs(word) - 1);
                const u32 hi = hist[b];  // cursor after the scatter = end of the bucket
                const u32 lo = b == 0 ? 0u : hist[b - 1];
                group_sort_u64(dst + lo, (int)(hi - lo), lane, 32, WarpSync());
                word &= word - 1;
            }
        }
        __syncthreads();
    }
    return dst;
}

// Common end of the top-k rows: sort the candidates (value descending), then either hand them to the
// vocabulary-parallel exchange or draw.
static __device__ __noinline__ void topk_tail(const KParams& P, const Smem& S, const RowOut& O, u64* cand, int n, int k, float u,
                                              float top_p)
{
    const int tid = threadIdx.x;
    cand          = sort_candidates(S, cand, n);
    trace_mark(O.trace, 10);
    if (P.vp_out != nullptr) {
        // Vocabulary-parallel local pass: hand over every column whose value reaches this shard's k-th
        // value, whole tie class included.  The global k-th value cannot be smaller than a shard's, so
        // the union over the shards holds every column the global selection and its tie order can touch.
        __shared__ int s_m;
        const int      k_eff = k < n ? k : n;
        if (tid == 0) {
            s_m = k_eff;
        }
        __syncthreads();
        if (k_eff > 0) {
            const u32 kv = (u32)(cand[k_eff - 1] >> 32);
            for (int i = k_eff + tid; i < n; i += kThreads) {
                if ((u32)(cand[i] >> 32) == kv) {
                    atomicMax(&s_m, i + 1);
                }
            }
        }
        __syncthreads();
        const int m   = s_m;
        u64*      out = P.vp_out + (size_t)O.r * (P.vp_cap + 2);
        if (tid == 0) {
            out[0] = m > P.vp_cap ? ~0ull : (u64)m;  // ~0: more ties than the exchange record holds
        }
        for (int i = tid; i < m && i < P.vp_cap; i += kThreads) {
            const u64 e = cand[i];
            out[1 + i]  = (e & 0xffffffff00000000ull) | (u64)((u32)(e & 0xffffffffu) + (u32)P.vocab_offset);
        }
        __syncthreads();
        return;
    }
    topk_finish(P, S, O, cand, n, k, u, top_p, true, false);
}

// ---- top-k in two passes -------------------------------------------------------------------------------
// Pass 1 (HBM) keeps, per thread, the running maximum of eight disjoint column subsets ("slots", 2048 per
// row).  The K-th largest slot maximum is a lower bound of the K-th largest column, usually a tight one:
// the largest columns of a row almost always sit in different slots.  Pass 2 (L2) collects the columns at
// or above that bound, which are then sorted and drawn from.  Special columns are counted separately
// (their final value is not the raw one), and the collected set is checked to hold at least k columns.
// Returns false when the row has to take the general one-pass path (too many specials, a candidate set
// that does not fit, a bound that the special columns invalidate).
template<int DT>
__device__ __noinline__ bool row_topk2(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O, int k, float u,
                                       float top_p)
{
    __shared__ u32 s_n, s_ovf;
    constexpr int  EPV = DT == FTB200_F32 ? 4 : 8;
    {
        // nothing but the arguments is live across the streaming call
        const int nfull0 = P.vocab >= P.vocab_padded ? C.nvec : (P.vocab - C.head > 0 ? (P.vocab - C.head) / EPV : 0);
        if (nfull0 * EPV < 8 * k || nfull0 < kThreads) {
            return false;  // short rows: the one-pass path is as good
        }
        trace_mark(O.trace, 0);
        hot_slotmax<DT>(vec_base<DT>(C), nfull0, (u32*)S.hitq);
        fetch_specials<DT>(P, S, C);
        trace_mark(O.trace, 1);
    }
    const Xf  X     = make_xf(P, S, C);
    const int tid   = threadIdx.x;
    u32*      slots = (u32*)S.hitq;  // [kSlots], free again before the filtered pass needs its queue
    u32*      hist  = S.hist;
    FTB_ASSUME_SHARED(slots);
    FTB_ASSUME_SHARED(hist);

    auto value_of_key = [&](u32 key) {
        if (DT == FTB200_F32) {
            return temp_value<DT>(X, __float_as_uint(fkey_inv(key)), 0);
        }
        return temp_value<DT>(X, key16_inv(key >> 16), 0);
    };
    // K-th largest slot key, 12 + 12 bits at a time.  The special columns may occupy slots without being
    // selectable at their raw value: those whose value before the penalty reaches the (coarse) bound are
    // added to K before the final selection.
    for (int i = tid; i < kNB; i += kThreads) {
        hist[i] = 0;
    }
    __syncthreads();
    for (int i = 0; i < kSlotsPerThread; ++i) {
        smem_add(&hist[slots[i * kThreads + tid] >> 20], 1u);
    }
    __syncthreads();
    u32 above = 0;
    int b1    = find_count_from_top(hist, (u32)k, &above);
    if (b1 < 0) {
        return false;
    }
    int K = k;
    {
        const float coarse = value_of_key((u32)b1 << 20);  // lower edge of the bucket: a bound below the K-th key
        u32         c      = 0;
        for (int i = tid; i < P.hash_slots; i += kThreads) {
            c += (X.hash[i] != kHashEmpty && S.spre[i] >= coarse) ? 1u : 0u;
        }
        const int s1 = (int)block_sum_u32(c);
        if (s1 > 0) {
            K = k + s1;
            if (K > 1600) {
                return false;
            }
            b1 = find_count_from_top(hist, (u32)K, &above);
            if (b1 < 0) {
                return false;
            }
        }
    }
    u32 key;
    if (DT != FTB200_F32) {
        // 16-bit keys have four bits left below the first level: sixteen counters, searched by every thread
        __shared__ u32 s_sub[16];
        if (tid < 16) {
            s_sub[tid] = 0;
        }
        __syncthreads();
        for (int i = 0; i < kSlotsPerThread; ++i) {
            const u32 kk = slots[i * kThreads + tid];
            if ((kk >> 20) == (u32)b1) {
                smem_add(&s_sub[(kk >> 16) & 0xfu], 1u);
            }
        }
        __syncthreads();
        const u32 need = (u32)K - above;
        u32       acc  = 0;
        int       b2   = 0;
        for (int b = 15; b >= 0; --b) {
            acc += s_sub[b];
            if (acc >= need) {
                b2 = b;
                break;
            }
        }
        key = ((u32)b1 << 20) | ((u32)b2 << 16);
    }
    else {
        for (int i = tid; i < kNB; i += kThreads) {
            hist[i] = 0;
        }
        __syncthreads();
        for (int i = 0; i < kSlotsPerThread; ++i) {
            const u32 kk = slots[i * kThreads + tid];
            if ((kk >> 20) == (u32)b1) {
                smem_add(&hist[(kk >> 8) & 0xfffu], 1u);
            }
        }
        __syncthreads();
        u32       above2 = 0;
        const int b2     = find_count_from_top(hist, (u32)K - above, &above2);
        key              = ((u32)b1 << 20) | ((u32)(b2 < 0 ? 0 : b2) << 8);
    }
    if (key == 0u) {
        return false;
    }
    const float thr_y = value_of_key(key);
    trace_mark(O.trace, 2);
    if (!(thr_y > C.neg_max)) {
        return false;
    }

    // pass 2: collect
    if (tid == 0) {
        s_n   = 0;
        s_ovf = 0;
    }
    __syncthreads();
    u64* cand = S.cand;
    FTB_ASSUME_SHARED(cand);
    auto push = [&](int v, float y) {
        if (y > C.neg_max) {
            // one atomic per warp: the lanes that arrive here together take consecutive positions
            const u32 act  = __activemask();
            const int lead = __ffs(act) - 1;
            const int lane = threadIdx.x & 31;
            u32       base = 0;
            if (lane == lead) {
                base = atomicAdd(&s_n, (u32)__popc(act));
            }
            base          = __shfl_sync(act, base, lead);
            const u32 pos = base + (u32)__popc(act & ((1u << lane) - 1u));
            if (pos < (u32)kCap) {
                cand[pos] = ((u64)(~fkey(y)) << 32) | (u32)v;
            }
            else {
                s_ovf = 1;
            }
        }
    };
    stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return thr_y; }, push, kWholeRow, INFINITY, O.trace);
    trace_mark(O.trace, 3);
    visit_specials<DT>(P, S, C, thr_y, push);
    __syncthreads();
    const int n = (int)s_n;
    if (O.trace != nullptr && threadIdx.x == 0) {
        O.trace[4 + 18] = (u64)n;
    }
    if (s_ovf || n < k) {
        __syncthreads();
        return false;
    }
    trace_mark(O.trace, 4);
    topk_tail(P, S, O, cand, n, k, u, top_p);
    trace_mark(O.trace, 5);
    return true;
}

// ---- top-k, k > 1, no log-probs: one pass, running threshold, candidates in shared memory ----------
template<int DT>
__device__ __noinline__ void row_topk(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O,
                                      u64* gscratch, int k, float u, float top_p)
{
    __shared__ u32 s_n, s_ovf;
    constexpr int  EPV = DT == FTB200_F32 ? 4 : 8;
    const int      tid = threadIdx.x;
    constexpr int  VB  = kHotBatch;

    fetch_specials<DT>(P, S, C);  // (a second fetch after the two-pass path gave up costs little: the row is in L2)
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
    u32  thr  = 0;  // order-preserving key of the current cut; columns below it cannot be in the top k
    auto histo = [&](int v, float y) {
        if (y > C.neg_max) {
            smem_add(&S.hist[fkey(y) >> 20], 1u);
        }
    };
    auto push = [&](int v, float y) {
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
    };
    auto histo_push = [&](int v, float y) {
        if (y > C.neg_max) {
            u32 key = fkey(y);
            if (key >= thr) {
                smem_add(&S.hist[key >> 20], 1u);
                u32 pos = atomicAdd(&s_n, 1u);
                if (pos < (u32)kCap) {
                    cand[pos] = ((u64)(~key) << 32) | (u32)v;
                }
                else {
                    s_ovf = 1;
                }
            }
        }
    };
    auto thr_f = [&]() { return thr == 0 ? -INFINITY : fkey_inv(thr); };
    {
        // warm-up: histogram the first columns, derive a cut from them (a valid lower bound of the k-th
        // value whatever the rest of the row holds), then collect those columns and the special ones
        int warm = (k * 8 > 2048 ? k * 8 : 2048) / EPV;
        warm     = (warm + kThreads - 1) / kThreads * kThreads;
        const int j1 = C.nvec < warm ? C.nvec : warm;
        stream_all<DT>(P, S, C, 0, j1, histo);
        __syncthreads();
        thr = thr_of(find_from_top(count_w, (double)k, nullptr));
        stream_filtered<DT>(P, S, C, 0, j1, thr_f, push);
        visit_specials<DT>(P, S, C, thr_f(), histo_push);
        __syncthreads();
        slow = s_ovf != 0;
        // the rest of the row: only columns at or above the cut are histogrammed and collected
        // batches double in size (up to VB vectors), so each one sends about k columns down the
        // exact path whatever k is, and the candidate buffer never sees a burst it cannot hold
        for (int j0 = j1, je = 0; j0 < C.nvec && !slow; j0 = je) {
            const int step = j0 < VB ? j0 : VB;
            je             = j0 + step < C.nvec ? j0 + step : C.nvec;
            const u32 n0 = s_n;
            __syncthreads();
            stream_filtered<DT>(P, S, C, j0, je, thr_f, histo_push);
            __syncthreads();
            if (s_ovf) {
                // the batch did not fit: raise the cut, shrink, and collect the batch again
                thr   = thr_of(find_from_top(count_w, (double)k, nullptr));
                int m = compact_candidates(cand, (int)n0, thr);
                __syncthreads();
                if (tid == 0) {
                    s_n   = m;
                    s_ovf = 0;
                }
                __syncthreads();
                stream_filtered<DT>(P, S, C, j0, je, thr_f, push);
                __syncthreads();
                slow = s_ovf != 0;
            }
            else if (s_n > (u32)(kCap / 2) || s_n - n0 > 96u) {
                // raise the cut while a batch still sends a noticeable number of columns down the
                // exact path
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
        stream_all<DT>(P, S, C, 0, C.nvec, histo);
        visit_specials<DT>(P, S, C, -INFINITY, histo);
        __syncthreads();
        thr  = thr_of(find_from_top(count_w, (double)k, nullptr));
        cand = gscratch;
        auto push_all = [&](int v, float y) {
            if (y > C.neg_max) {
                u32 key = fkey(y);
                if (key >= thr) {
                    cand[atomicAdd(&s_n, 1u)] = ((u64)(~key) << 32) | (u32)v;
                }
            }
        };
        stream_filtered<DT>(P, S, C, 0, C.nvec, thr_f, push_all);
        visit_specials<DT>(P, S, C, thr_f(), push_all);
        __syncthreads();
        n = (int)s_n;
    }
    topk_tail(P, S, O, cand, n, k, u, top_p);
}

// ---- rows that need soft-max probabilities: top-p, and top-k when log-probs are requested -----------
// The provisional histogram of a soft-max row counts every column within kTopSpan logit units of the row
// maximum (buckets above kTopBucket) and one column in sixteen of the rest: the few largest columns carry
// most of the probability mass, and a sample that hits or misses one of them would misplace the cut.
constexpr int   kTopBucket = kNB - 1 - 4 * kLinScale;
constexpr float kTopSpan   = 4.0f;

__device__ __forceinline__ int lin_bucket(float y, float maxv)
{
    int q = (int)((maxv - y) * (float)kLinScale);
    q     = q < 0 ? 0 : (q > kNB - 1 ? kNB - 1 : q);
    return kNB - 1 - q;
}

// One column into the provisional histogram: always when it lies in the exact region, else when sampled.
__device__ __forceinline__ void note_column(u32* hist, float y, float maxv, bool sampled, bool exact_top)
{
    const int b = lin_bucket(y, maxv);
    if (b > kTopBucket ? exact_top : sampled) {
        smem_add(&hist[b], 1u);
    }
}

// ---- ordered soft-max pass, lean form ----------------------------------------------------------------
// Thread t owns the reference's "virtual threads" 4t..4t+3; per 1024-column chunk it loads its four
// columns, takes the exponentials and adds them to four running sums, strictly in chunk order.  The
// special columns (history tokens, banned words, min-length mask) never enter the loop as a look-up:
// before the loop each one is filed, with its final value, in a short per-thread list ordered by chunk,
// and the loop only compares the chunk number with the head of its list.
constexpr int kPatchSlots = 16;  // special columns one thread may own; more -> general loop

template<int DT>
__device__ __noinline__ bool build_patches(const KParams& P, const Smem& S, const RowCtx& C, int nfull, u32* pkey,
                                           float* pval, u32* pcnt)
{
    __shared__ int s_over;
    const Xf       X   = make_xf(P, S, C);
    const int      tid = threadIdx.x;
    const float*   sfin = S.sfin;
    FTB_ASSUME_SHARED(sfin);
    FTB_ASSUME_SHARED(pkey);
    FTB_ASSUME_SHARED(pval);
    FTB_ASSUME_SHARED(pcnt);
    FTB_ASSUME_SHARED(X.hash);
    pcnt[tid]          = 0;
    if (tid == 0) {
        s_over = 0;
    }
    __syncthreads();
    const int limit = nfull * 1024;
    for (int i = tid; i < P.hash_slots; i += kThreads) {
        const u32 w = X.hash[i];
        if (w == kHashEmpty) {
            continue;
        }
        const int v = (int)(w >> 2);
        if (v >= limit) {
            continue;
        }
        const float y  = sfin[i];
        const int   t  = (v & 1023) >> 2;
        const u32   at = atomicAdd(&pcnt[t], 1u);
        if (at < (u32)kPatchSlots) {
            pkey[at * kThreads + t] = (u32)(((v >> 10) << 2) | (v & 3));
            pval[at * kThreads + t] = y;
        }
        else {
            s_over = 1;
        }
    }
    __syncthreads();
    if (s_over) {
        return false;
    }
    // each thread orders its own list by chunk
    const int n = (int)pcnt[tid];
    for (int a = 1; a < n; ++a) {
        const u32   k = pkey[a * kThreads + tid];
        const float y = pval[a * kThreads + tid];
        int         b = a - 1;
        while (b >= 0 && pkey[b * kThreads + tid] > k) {
            pkey[(b + 1) * kThreads + tid] = pkey[b * kThreads + tid];
            pval[(b + 1) * kThreads + tid] = pval[b * kThreads + tid];
            --b;
        }
        pkey[(b + 1) * kThreads + tid] = k;
        pval[(b + 1) * kThreads + tid] = y;
    }
    return true;
}

template<int DT, bool TEMP, bool EXACT_TOP>
__device__ __noinline__ void pass2_lean(const char* rowp, int nfull, float maxv, float inv_t, __half inv_t_h,
                                        u32 pkey, u32 pval, int pn, u32 hist, float* acc_out)
{
    // pkey, pval, hist: 32-bit shared-memory addresses (one register each, ld.shared / red.shared without a
    // generic-to-shared conversion per access)
    constexpr int ES  = DT == FTB200_F32 ? 4 : 2;
    constexpr int UN  = 8;
    const int     tid = threadIdx.x, wid = tid >> 5;
    float         a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    const float   ytop = maxv - kTopSpan - 0.02f;  // anything that can land above kTopBucket is at least this
    // head of this thread's patch list, held in registers one entry ahead of its use
    int           pi = 0;
    u32           nk = pn > 0 ? lds_u32(pkey + 4u * tid) : 0xffffffffu;
    float         nv = pn > 0 ? __uint_as_float(lds_u32(pval + 4u * tid)) : 0.0f;
    const char*   base = rowp + (size_t)tid * 4 * ES;
    auto value = [&](u32 bits) {
        if (DT == FTB200_F16) {
            __half h = __ushort_as_half((unsigned short)bits);
            if (TEMP) {
                h = __hmul(h, inv_t_h);
            }
            return __half2float(h);
        }
        float x = DT == FTB200_F32 ? __uint_as_float(bits) : __uint_as_float(bits << 16);
        if (TEMP) {
            x = x * inv_t;
        }
        return x;
    };
    for (int m0 = 0; m0 < nfull; m0 += UN) {
        uint4 raw[UN];  // 16-bit types use .x / .y only
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            if (m0 + uu < nfull) {
                const char* q = base + (size_t)(m0 + uu) * 1024 * ES;
                if (DT == FTB200_F32) {
                    raw[uu] = ld_nc_v4(q);
                }
                else {
                    const uint2 r = ld_nc_v2(q);
                    raw[uu].x = r.x, raw[uu].y = r.y;
                }
            }
        }
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            const int m = m0 + uu;
            if (m < nfull) {
                float y0, y1, y2, y3;
                if (DT == FTB200_F32) {
                    y0 = value(raw[uu].x), y1 = value(raw[uu].y), y2 = value(raw[uu].z), y3 = value(raw[uu].w);
                }
                else {
                    y0 = value(raw[uu].x & 0xffffu), y1 = value(raw[uu].x >> 16);
                    y2 = value(raw[uu].y & 0xffffu), y3 = value(raw[uu].y >> 16);
                }
                if ((int)(nk >> 2) == m) {
                    do {
                        const float yy = nv;
                        const u32   e  = nk & 3u;
                        y0             = e == 0 ? yy : y0;
                        y1             = e == 1 ? yy : y1;
                        y2             = e == 2 ? yy : y2;
                        y3             = e == 3 ? yy : y3;
                        ++pi;
                        nk = pi < pn ? lds_u32(pkey + 4u * (u32)(pi * kThreads + tid)) : 0xffffffffu;
                        nv = pi < pn ? __uint_as_float(lds_u32(pval + 4u * (u32)(pi * kThreads + tid))) : 0.0f;
                    } while ((int)(nk >> 2) == m);
                }
                // a column at or below -MAX adds exactly zero, as in the reference's loop
                a0 += round_to_T<DT>(__expf(y0 - maxv));
                a1 += round_to_T<DT>(__expf(y1 - maxv));
                a2 += round_to_T<DT>(__expf(y2 - maxv));
                a3 += round_to_T<DT>(__expf(y3 - maxv));
                if (((m + 2 * wid) & 15) == 0) {  // warp-uniform 1-in-16 sample for the provisional cut
                    const int b0 = lin_bucket(y0, maxv), b1 = lin_bucket(y1, maxv);
                    const int b2 = lin_bucket(y2, maxv), b3 = lin_bucket(y3, maxv);
                    reds_add(hist + 4u * (u32)b0, (y0 > -FLT_MAX && b0 <= kTopBucket) ? 1u : 0u);
                    reds_add(hist + 4u * (u32)b1, (y1 > -FLT_MAX && b1 <= kTopBucket) ? 1u : 0u);
                    reds_add(hist + 4u * (u32)b2, (y2 > -FLT_MAX && b2 <= kTopBucket) ? 1u : 0u);
                    reds_add(hist + 4u * (u32)b3, (y3 > -FLT_MAX && b3 <= kTopBucket) ? 1u : 0u);
                }
                if (EXACT_TOP && fmaxf(fmaxf(y0, y1), fmaxf(y2, y3)) >= ytop) {  // rare: a column of the exact region
                    const int b0 = lin_bucket(y0, maxv), b1 = lin_bucket(y1, maxv);
                    const int b2 = lin_bucket(y2, maxv), b3 = lin_bucket(y3, maxv);
                    if (b0 > kTopBucket) {
                        reds_add(hist + 4u * (u32)b0, 1u);
                    }
                    if (b1 > kTopBucket) {
                        reds_add(hist + 4u * (u32)b1, 1u);
                    }
                    if (b2 > kTopBucket) {
                        reds_add(hist + 4u * (u32)b2, 1u);
                    }
                    if (b3 > kTopBucket) {
                        reds_add(hist + 4u * (u32)b3, 1u);
                    }
                }
            }
        }
    }
    acc_out[0] = a0, acc_out[1] = a1, acc_out[2] = a2, acc_out[3] = a3;
}

// Pass 2 of a soft-max row (reads the row again, from L2): e = T(__expf(y - max)) for every column,
// summed per "virtual thread" exactly as addBiasSoftMax's min(V,1024)-thread strided loop does
// (kernels/sampling_topp_kernels.cu:1331-1334), plus the bucket counts.  The per-virtual-thread partial
// sums land in S.val2[0..nvt).
template<int DT>
__device__ __noinline__ void softmax_pass2(const KParams& P, const Smem& S, const RowCtx& C, float maxv, int nvt, u64* dbg,
                                           bool exact_top)
{
    const Xf X = make_xf(P, S, C);
    constexpr int ES  = DT == FTB200_F32 ? 4 : 2;
    const int     tid = threadIdx.x;
    u32*          hist = S.hist;
    const u32*    flags = S.flags;
    float*        val2 = S.val2;
    const char*   rowp = C.rowp;
    const int     vpad = P.vocab_padded, vocab = P.vocab, head = C.head, nvec = C.nvec;
    const float   neg_max = C.neg_max;
        float     acc[4] = {0.f, 0.f, 0.f, 0.f};
        const bool grouped = nvt == 1024 && (((size_t)rowp) % (4 * ES) == 0) && (head % 4 == 0);
        int        mstart  = 0;
        if (grouped && P.bias == nullptr) {
            // chunks that lie entirely inside the vocabulary take the lean loop
            const int nfull = (vocab < vpad ? vocab : vpad) / 1024;
            u32*      pkey  = (u32*)S.cand;
            float*    pval  = (float*)(pkey + kPatchSlots * kThreads);
            u32*      pcnt  = (u32*)S.hitq;
            if (nfull > 0 && build_patches<DT>(P, S, C, nfull, pkey, pval, pcnt)) {
                trace_mark(dbg, 12);
                const int pn = (int)pcnt[tid];
                if (P.apply_temp) {
                    if (exact_top) {
                        pass2_lean<DT, true, true>(rowp, nfull, maxv, C.inv_t, C.inv_t_h, (u32)__cvta_generic_to_shared(pkey), (u32)__cvta_generic_to_shared(pval), pn,
                                                    (u32)__cvta_generic_to_shared(hist), acc);
                    }
                    else {
                        pass2_lean<DT, true, false>(rowp, nfull, maxv, C.inv_t, C.inv_t_h, (u32)__cvta_generic_to_shared(pkey), (u32)__cvta_generic_to_shared(pval), pn,
                                                    (u32)__cvta_generic_to_shared(hist), acc);
                    }
                }
                else if (exact_top) {
                    pass2_lean<DT, false, true>(rowp, nfull, maxv, C.inv_t, C.inv_t_h, (u32)__cvta_generic_to_shared(pkey), (u32)__cvta_generic_to_shared(pval), pn,
                                                    (u32)__cvta_generic_to_shared(hist), acc);
                }
                else {
                    pass2_lean<DT, false, false>(rowp, nfull, maxv, C.inv_t, C.inv_t_h, (u32)__cvta_generic_to_shared(pkey), (u32)__cvta_generic_to_shared(pval), pn,
                                                    (u32)__cvta_generic_to_shared(hist), acc);
                }
                mstart = nfull;
                trace_mark(dbg, 13);
            }
        }
        if (grouped) {
            // thread t owns virtual threads 4t..4t+3: one 4-element load per 1024-column chunk
            constexpr int UN = 8;
            for (int m0 = mstart; m0 * 1024 < vpad; m0 += UN) {
                u32 raw[UN][4];
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    const int v0 = (m0 + uu) * 1024 + 4 * tid;
                    if (v0 + 3 < vpad) {
                        if (DT == FTB200_F32) {
                            uint4 q    = *(const uint4*)(rowp + (size_t)v0 * 4);
                            raw[uu][0] = q.x, raw[uu][1] = q.y, raw[uu][2] = q.z, raw[uu][3] = q.w;
                        }
                        else {
                            uint2 q    = *(const uint2*)(rowp + (size_t)v0 * 2);
                            raw[uu][0] = q.x & 0xffffu, raw[uu][1] = q.x >> 16;
                            raw[uu][2] = q.y & 0xffffu, raw[uu][3] = q.y >> 16;
                        }
                    }
                }
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    const int v0 = (m0 + uu) * 1024 + 4 * tid;
                    if (v0 >= vpad) {
                        continue;
                    }
                    const bool sampled = ((tid + m0 + uu) & 15) == 0;
                    if (v0 + 3 < vpad) {
                        bool sp = true;
                        if (v0 >= head) {
                            const int j = (v0 - head) / (DT == FTB200_F32 ? 4 : 8);
                            sp          = j >= nvec || ((flags[j >> 5] >> (j & 31)) & 1u);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int v = v0 + e;
                            float     y = -INFINITY;
                            if (v < vocab) {
                                y = temp_value<DT>(X, raw[uu][e], v);
                                if (sp) {
                                    u32 fl = hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v);
                                    if (fl) {
                                        y = special_value<DT>(X, y, fl);
                                    }
                                }
                            }
                            if (y > neg_max) {
                                float ex = round_to_T<DT>(__expf(y - maxv));
                                acc[e] += ex;
                                note_column(hist, y, maxv, sampled, exact_top);
                            }
                        }
                    }
                    else {
                        for (int e = 0; e < 4 && v0 + e < vpad; ++e) {
                            float y = elem_at<DT>(P, S, C, v0 + e);
                            if (y > neg_max) {
                                float ex = round_to_T<DT>(__expf(y - maxv));
                                acc[e] += ex;
                                note_column(hist, y, maxv, sampled, exact_top);
                            }
                        }
                    }
                }
            }
            __syncthreads();
            for (int e = 0; e < 4; ++e) {
                val2[4 * tid + e] = acc[e];
            }
        }
        else {
            // thread t owns virtual threads t, t+256, t+512, t+768
            for (int v0 = 0; v0 < vpad; v0 += nvt) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int vt = tid + q * kThreads;
                    const int v  = v0 + vt;
                    if (vt < nvt && v < vpad) {
                        float y = elem_at<DT>(P, S, C, v);
                        if (y > neg_max) {
                            float ex = round_to_T<DT>(__expf(y - maxv));
                            acc[q] += ex;
                            note_column(hist, y, maxv, ((vt + v0 / nvt) & 15) == 0, exact_top);
                        }
                    }
                }
            }
            __syncthreads();
            for (int q = 0; q < 4; ++q) {
                val2[tid + q * kThreads] = acc[q];
            }
        }
}

// ---- top-p over value classes (16-bit logits) --------------------------------------------------------
// A half / bfloat16 row holds few distinct values: every ordinary column with the same bit pattern has
// the same probability.  The sorted probability sequence the reference scans is therefore a short list
// of runs (probability, count): one per bit pattern above the cut, plus one per special column.  The
// scan is replayed over the runs in cub::BlockScan's order - no candidate list, no sort of the row -
// and only the value class that holds the crossing is collected, to find its J-th column (the
// reference's stable sort leaves equal probabilities in column order).
// Returns 1 when the row is finished, 0 when the caller has to take the general path.
// Dense form of the class count (16-bit logits): every column of the unflagged, fully valid vectors whose
// ordered key lies within `limit` patterns of the row's largest one is counted, straight from the bit
// pattern.  Used when a large part of the row lies above the cut, where queueing hits would queue everything.
template<int DT>
__device__ __noinline__ void hot_count_dense(const uint4* vp, int jn, const u32* flags, u32 kmax16, u32 limit, u32* hist,
                                             unsigned short* hitq, u32* qn)
{
    FTB_ASSUME_SHARED(flags);
    FTB_ASSUME_SHARED(hist);
    FTB_ASSUME_SHARED(hitq);
    FTB_ASSUME_SHARED(qn);
    constexpr int U   = 8;
    const int     tid = threadIdx.x;
    auto count2 = [&](u32 w) {
        const u32 m  = ((w >> 15) & 0x00010001u) * 0x7fffu;  // per half: 0x7fff when negative
        const u32 k2 = w ^ (m | 0x80008000u);                // ordered keys of both halves
        const u32 i0 = kmax16 - (k2 & 0xffffu), i1 = kmax16 - (k2 >> 16);
        if (i0 < limit) {
            smem_add(&hist[i0], 1u);
        }
        if (i1 < limit) {
            smem_add(&hist[i1], 1u);
        }
    };
    for (int jb = 0; jb < jn; jb += kThreads * U) {
        uint4 q[U];
        bool  ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = jb + u * kThreads + tid;
            ok[u]       = false;
            if (j < jn) {
                if ((flags[j >> 5] >> (j & 31)) & 1u) {
                    // a vector with a special column: queued, handled column by column afterwards
                    const u32 pos = atomicAdd(qn, 1u);
                    if (pos < (u32)kHitCap) {
                        hitq[pos] = (unsigned short)j;
                    }
                }
                else {
                    ok[u] = true;
                    q[u]  = ld_nc_v4(vp + j);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (ok[u]) {
                count2(q[u].x);
                count2(q[u].y);
                count2(q[u].z);
                count2(q[u].w);
            }
        }
    }
}

constexpr int kMaxRuns  = 4096;  // runs held in shared memory
constexpr int kMaxSpecs = 1024;  // special / edge columns above the cut
constexpr int kMaxAbove = 256;   // ordinary columns above a class window that does not reach the row maximum

template<int DT>
__device__ __noinline__ int row_topp_classes(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O,
                                             float maxv, float denom, float rand_num, float cut0, u32 kmax16,
                                             bool want_lp, bool dense, u32 k_cut_given = 0xffffffffu)
{
    __shared__ u32   s_ns, s_fail, s_wsum[kWarps], s_ncls, s_nabove;
    __shared__ int   s_c1, s_sel, s_imin, s_imax;
    __shared__ float s_R;
    __shared__ u64   s_above[kMaxAbove];  // columns above the class window: (~key(prob) << 32) | column
    const Xf         X   = make_xf(P, S, C);
    const int        tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const bool       complete = !(cut0 > -INFINITY);
    u64*             spec     = (u64*)S.hitq;            // [kMaxSpecs] (~key(prob) << 32) | column
    u32*             run_pr   = (u32*)S.cand;            // [kMaxRuns] runs, probability (float bits) descending;
                                                         // one element type for everything that shares this area
    u32*             run_st   = (u32*)S.cand + kMaxRuns; // [kMaxRuns] length, then first position of each run
    u32*             cls      = (u32*)S.cand;            // columns of the crossing class (after the replay)
    u32*             rank     = S.hist;                  // per pattern: count, then number of non-empty patterns before it
    float*           agg      = S.val2;                  // [1024] per-chunk aggregates
    FTB_ASSUME_SHARED(spec);
    FTB_ASSUME_SHARED(run_st);
    FTB_ASSUME_SHARED(rank);
    FTB_ASSUME_SHARED(agg);

    auto prob_of = [&](float y) {
        const float ex = round_to_T<DT>(__expf(y - maxv));
        return round_to_T<DT>(ex / denom);
    };
    auto prob_of_bin = [&](int idx) { return prob_of(temp_value<DT>(X, key16_inv(kmax16 - (u32)idx), 0)); };
    __syncthreads();  // a previous call's flags have been read by every thread
    for (int i = tid; i < kNB; i += kThreads) {
        S.hist[i] = 0;
    }
    if (tid == 0) {
        s_ns     = 0;
        s_fail   = 0;
        s_nabove = 0;
    }
    __syncthreads();
    // The cut in the pattern domain: the smallest ordered key whose value reaches cut0.  Everything at or
    // above that pattern is counted, so the collected classes are complete down to the value y_c.
    u32 k_cut = 0;
    if (k_cut_given != 0xffffffffu) {
        // the caller names the lowest pattern itself (the bottom of the class window): a search by value could
        // land on a lower pattern that rounds to the same value
        k_cut = k_cut_given;
    }
    else if (!complete) {
        u32 lo = 0, hi = kmax16;  // value(key) is monotone in the key
        while (lo < hi) {
            const u32 mid = (lo + hi) >> 1;
            if (temp_value<DT>(X, key16_inv(mid), 0) >= cut0) {
                hi = mid;
            }
            else {
                lo = mid + 1;
            }
        }
        k_cut = lo;
    }
    if (kmax16 - k_cut >= (u32)kNB) {
        // The patterns between the cut and the row maximum do not fit the window.  A peaked row has only a few
        // columns up there: the window is anchored at the cut instead, and the columns above it are listed one
        // by one (they join the runs like special columns do).  From here on kmax16 is the top of the window.
        if (complete || k_cut_given != 0xffffffffu) {
            { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 1; } return 0; }
        }
        kmax16 = k_cut + (u32)kNB - 1u;
        const float y_above = temp_value<DT>(X, key16_inv(kmax16 + 1u), 0);
        auto        above   = [&](int v, float y, u32 raw) {
            if (key16(raw) > kmax16 && y > C.neg_max) {
                const u32 pos = atomicAdd(&s_nabove, 1u);
                if (pos < (u32)kMaxAbove) {
                    s_above[pos] = ((u64)(~fkey(prob_of(y))) << 32) | (u32)v;
                }
            }
        };
        stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return y_above; }, above, kWholeRow);
        __syncthreads();
        if (s_nabove > (u32)kMaxAbove) {
            { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 1; } return 0; }
        }
    }
    const u32   limit = kmax16 - k_cut + 1u;
    const float y_c   = (complete && k_cut_given == 0xffffffffu) ? -INFINITY : temp_value<DT>(X, key16_inv(k_cut), 0);
    // pass 3 (L2): exact count of every bit pattern at or above the cut
    {
        constexpr int EPV = DT == FTB200_F32 ? 4 : 8;
        u32*          hist = S.hist;
        auto count = [&](int v, float y, u32 raw) {
            if (y > C.neg_max) {
                const u32 idx = kmax16 - key16(raw);
                if (idx < limit) {
                    smem_add(&hist[idx], 1u);
                }
            }
        };
        if (dense && DT != FTB200_F32) {
            const int nfull = P.vocab >= P.vocab_padded ? C.nvec : (P.vocab - C.head > 0 ? (P.vocab - C.head) / EPV : 0);
            if (tid == 0) {
                S.nhit[0] = 0;
            }
            __syncthreads();
            hot_count_dense<DT>(vec_base<DT>(C), nfull, S.flags, kmax16, limit, hist, S.hitq, S.nhit);
            // the vectors that reach past the vocabulary join the queue
            for (int j = nfull + tid; j < C.nvec; j += kThreads) {
                const u32 pos = atomicAdd(S.nhit, 1u);
                if (pos < (u32)kHitCap) {
                    S.hitq[pos] = (unsigned short)j;
                }
            }
            __syncthreads();
            const int nq = (int)S.nhit[0];
            if (nq > kHitCap || C.nvec > 65535) {
                { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 2; } return 0; }
            }
            const uint4* vp = vec_base<DT>(C);
            for (int i = tid; i < nq; i += kThreads) {
                const int   j  = (int)S.hitq[i];
                const bool  sp = (S.flags[j >> 5] >> (j & 31)) & 1u;
                const uint4 r  = ld_nc_v4(vp + j);
                for (int e = 0; e < EPV; ++e) {
                    const int v = C.head + j * EPV + e;
                    if (v < P.vocab && !(sp && hash_lookup_raw(X.hash, X.hash_shift, X.hash_mask, v))) {
                        const u32 raw = raw_bits<DT>(r, e);
                        count(v, temp_value<DT>(X, raw, v), raw);
                    }
                }
            }
            __syncthreads();
        }
        else {
            stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return y_c; }, count, kWholeRow);
        }
        trace_mark(O.trace, 20);
        // (the filtered stream is done with its hit queue: the list of specials may live there)
        visit_specials<DT>(P, S, C, y_c, [&](int v, float y) {
            if (y > C.neg_max) {
                const u32 pos = atomicAdd(&s_ns, 1u);
                if (pos < (u32)kMaxSpecs) {
                    spec[pos] = ((u64)(~fkey(prob_of(y))) << 32) | (u32)v;
                }
                else {
                    s_fail = 1;
                }
            }
        });
    }
    __syncthreads();
    {
        const u32 na = s_nabove, base = s_ns;
        if (base + na > (u32)kMaxSpecs) {
            s_fail = 1;  // (every thread writes the same value)
        }
        else {
            for (u32 i = tid; i < na; i += kThreads) {
                spec[base + i] = s_above[i];
            }
        }
        __syncthreads();
        if (tid == 0 && !s_fail) {
            s_ns = base + na;
        }
        __syncthreads();
    }
    trace_mark(O.trace, 5);
    if (s_fail) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 3; } return 0; }
    }
    const int ns = (int)s_ns;
    group_sort_u64<CtaSync, true>(spec, ns, tid, kThreads, CtaSync());
    __syncthreads();
    trace_mark(O.trace, 22);

    // Runs: the non-empty patterns in descending value with the specials merged in by probability (equal
    // probabilities: patterns first - the order inside a class of equal values changes no partial sum).
    constexpr int PER = kNB / kThreads;
    int           nA;
    for (int i = tid; i < kMaxRuns; i += kThreads) {
        run_st[i] = 0u;  // a position no pattern takes keeps length 0 and goes to a special column
    }
    __syncthreads();
    {
        u32 cnt[PER], mine = 0;
        for (int i = 0; i < PER; ++i) {
            cnt[i] = S.hist[tid * PER + i];
            mine += cnt[i] != 0 ? 1u : 0u;
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            u32 t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) {
                incl += t;
            }
        }
        if (lane == 31) {
            s_wsum[wid] = incl;
        }
        __syncthreads();
        u32 base = 0, tot = 0;
        for (int i = 0; i < kWarps; ++i) {
            if (i < wid) {
                base += s_wsum[i];
            }
            tot += s_wsum[i];
        }
        nA = (int)tot;
        if (nA + ns > kMaxRuns) {
            { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 4; } return 0; }
        }
        u32 at = base + incl - mine;
        for (int i = 0; i < PER; ++i) {
            const int idx = tid * PER + i;
            rank[idx]     = at;
            if (cnt[i] != 0) {
                const float pr = prob_of_bin(idx);
                const u32   kp = ~fkey(pr);  // ascending in this key = descending probability
                int         lo = 0, hi = ns; // number of specials with a strictly larger probability
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if ((u32)(spec[mid] >> 32) < kp) {
                        lo = mid + 1;
                    }
                    else {
                        hi = mid;
                    }
                }
                run_pr[at + lo] = __float_as_uint(pr);
                run_st[at + lo] = cnt[i];
                ++at;
            }
        }
    }
    __syncthreads();
    // Both lists keep their order in the merged sequence, and a pattern sits at (its rank among the patterns)
    // + (specials before it): the specials therefore fill the positions the patterns left free, in order.
    {
        constexpr int RPT  = kMaxRuns / kThreads;
        const int     Mtot = nA + ns;
        u32           freem = 0, mine = 0;
        for (int i = 0; i < RPT; ++i) {
            const int r = tid * RPT + i;
            if (r < Mtot && run_st[r] == 0u) {
                freem |= 1u << i;
                ++mine;
            }
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            u32 t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) {
                incl += t;
            }
        }
        __syncthreads();
        if (lane == 31) {
            s_wsum[wid] = incl;
        }
        __syncthreads();
        u32 j = incl - mine;
        for (int i = 0; i < wid; ++i) {
            j += s_wsum[i];
        }
        for (int i = 0; i < RPT; ++i) {
            if ((freem >> i) & 1u) {
                const int r = tid * RPT + i;
                run_pr[r]   = __float_as_uint(fkey_inv(~(u32)(spec[j] >> 32)));
                run_st[r]   = 1u;
                ++j;
            }
        }
    }
    __syncthreads();
    const int M = nA + ns;
    // the exponential has to be monotone over the patterns for the order of the runs to be the sorted order
    for (int i = tid; i + 1 < M; i += kThreads) {
        if (__uint_as_float(run_pr[i]) < __uint_as_float(run_pr[i + 1])) {
            s_fail = 1;
        }
    }
    __syncthreads();
    if (s_fail) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 5; } return 0; }
    }
    // exclusive scan of the run lengths -> first position of each run
    u32 N;
    {
        constexpr int RPT = kMaxRuns / kThreads;
        u32           c[RPT], mine = 0;
        for (int i = 0; i < RPT; ++i) {
            const int r = tid * RPT + i;
            c[i]        = r < M ? run_st[r] : 0u;
            mine += c[i];
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            u32 t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) {
                incl += t;
            }
        }
        __syncthreads();
        if (lane == 31) {
            s_wsum[wid] = incl;
        }
        __syncthreads();
        u32 base = 0, tot = 0;
        for (int i = 0; i < kWarps; ++i) {
            if (i < wid) {
                base += s_wsum[i];
            }
            tot += s_wsum[i];
        }
        N      = tot;
        u32 at = base + incl - mine;
        for (int i = 0; i < RPT; ++i) {
            const int r = tid * RPT + i;
            if (r < M) {
                run_st[r] = at;
                at += c[i];
            }
        }
    }
    __syncthreads();
    trace_mark(O.trace, 6);
    if (O.trace != nullptr && tid == 0) {
        O.trace[4 + 24] = (u64)N | ((u64)(dense ? 1 : 0) << 32) | ((u64)M << 40);
    }
    const int nch = (int)((N + 255u) / 256u);
    if (nch > 1024 || N == 0) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 6; } return 0; }
    }
    // run that holds position p
    auto run_of = [&](u32 p) {
        int lo = 0, hi = M - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (run_st[mid] <= p) {
                lo = mid;
            }
            else {
                hi = mid - 1;
            }
        }
        return lo;
    };
    // run at the first position of every chunk (the pattern counts are not needed any more): a lane then looks
    // for its own first run between two neighbouring entries, a handful of runs instead of all of them
    int* run_at = (int*)S.hist;
    FTB_ASSUME_SHARED(run_at);
    for (int c = tid; c <= nch; c += kThreads) {
        run_at[c] = c < nch ? run_of((u32)c * 256u) : M - 1;
    }
    __syncthreads();
    // the 8 consecutive values of this lane in chunk c
    auto load8 = [&](int c, float* x) {
        const u32 p0 = (u32)c * 256u + (u32)lane * 8u;
        int       i  = 0;
        if (p0 < N) {
            int lo = run_at[c], hi = run_at[c + 1];
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (run_st[mid] <= p0) {
                    lo = mid;
                }
                else {
                    hi = mid - 1;
                }
            }
            i = lo;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const u32 p = p0 + (u32)e;
            if (p < N) {
                if (i + 1 < M && run_st[i + 1] <= p) {
                    ++i;
                }
                x[e] = __uint_as_float(run_pr[i]);
            }
            else {
                x[e] = 0.0f;
            }
        }
    };
    // aggregate of every 256-value chunk in cub::BlockScan's raking order (32 segments of 8, Kogge-Stone
    // across the segment totals); the chunks are independent of the running prefix
    for (int c = wid; c < nch; c += kWarps) {
        float x[8];
        load8(c, x);
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
        if (lane == 31) {
            agg[c] = inc;
        }
    }
    __syncthreads();
    trace_mark(O.trace, 25);
    // running prefix chunk by chunk, as the reference's prefix functor accumulates it; stop a little early
    // (partial sums inside a chunk differ from prefix + aggregate only in the last bits)
    if (tid == 0) {
        float     R    = 0.0f;
        int       c1   = nch;
        const float stop = rand_num * (1.0f - 1e-4f);
        for (int c = 0; c < nch; ++c) {
            const float R2 = R + agg[c];
            if (R2 >= stop) {
                c1 = c;
                break;
            }
            R = R2;
        }
        s_c1 = c1;
        s_R  = R;
    }
    __syncthreads();
    if (s_c1 >= nch) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 7; } return 0; }
    }
    if (wid == 0) {
        float R   = s_R;
        int   sel = -2;
        for (int c = s_c1; c < nch; ++c) {
            float x[8];
            load8(c, x);
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
            const float ag  = __shfl_sync(0xffffffffu, inc, 31);
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
                const int g  = (__ffs(any) - 1) >> 2;
                const u32 pc = __shfl_sync(0xffffffffu, c4, g * 4);
                if (!complete && (u32)(c * 256 + g * 32 + 31) >= N) {
                    sel = -2;  // the 32 probabilities of that warp are not all known
                }
                else {
                    sel = c * 256 + g * 32 + (32 - (int)pc);
                }
                break;
            }
            R = R + ag;
        }
        if (lane == 0) {
            s_sel = sel;
        }
    }
    __syncthreads();
    const int sel = s_sel;
    trace_mark(O.trace, 7);
    if (sel < 0 || (u32)sel >= N) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 8; } return 0; }
    }
    // the class of the crossing: every column whose probability equals that of position sel
    const int   i_at  = run_of((u32)sel);
    const float p_sel = __uint_as_float(run_pr[i_at]);
    const u32   k_sel = fkey(p_sel);
    if (tid == 0) {
        s_ncls = 0;
        s_imin = 0x7fffffff;
        s_imax = -1;
    }
    __syncthreads();
    // first run of the class -> rank of the crossing inside the class
    {
        int lo = 0, hi = i_at;  // first run with probability == p_sel (runs are descending)
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (fkey(__uint_as_float(run_pr[mid])) > k_sel) {
                lo = mid + 1;
            }
            else {
                hi = mid;
            }
        }
        if (tid == 0) {
            s_c1 = sel - (int)run_st[lo];
        }
    }
    // bit patterns that map to this probability
    for (int i = 0; i < PER; ++i) {
        const int idx = tid * PER + i;
        if ((u32)idx <= kmax16) {
            const u32 raw = key16_inv(kmax16 - (u32)idx);
            if (fkey(prob_of(temp_value<DT>(X, raw, 0))) == k_sel) {
                atomicMin(&s_imin, idx);
                atomicMax(&s_imax, idx);
            }
        }
    }
    __syncthreads();  // the runs have been read for the last time: the class list takes their place
    if (s_imax >= kNB - 1) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 9; } return 0; }
    }
    // Special and edge columns of the class - all of them, also those below the cut: with probabilities
    // rounded to the logits type a class of equal probabilities can span several bit patterns and reach
    // below the counted range, and the rank of the crossing counts every column of the class.
    // Those at or above the cut are in the list (with the ordinary columns above the window); the rest come
    // from the table.
    for (int j = tid; j < ns; j += kThreads) {
        if ((u32)(spec[j] >> 32) == ~k_sel) {
            const u32 pos = atomicAdd(&s_ncls, 1u);
            if (pos < (u32)(2 * kMaxRuns)) {
                cls[pos] = (u32)(spec[j] & 0xffffffffu);
            }
        }
    }
    visit_specials<DT>(P, S, C, -INFINITY, [&](int v, float y) {
        if (y > C.neg_max && !(y >= y_c) && fkey(prob_of(y)) == k_sel) {
            const u32 pos = atomicAdd(&s_ncls, 1u);
            if (pos < (u32)(2 * kMaxRuns)) {
                cls[pos] = (u32)v;
            }
        }
    });
    __syncthreads();
    const int J = s_c1;
    trace_mark(O.trace, 27);
    if (s_imax >= 0) {
        const u32   k_hi  = kmax16 - (u32)s_imin, k_lo = kmax16 - (u32)s_imax;
        const float y_lo  = temp_value<DT>(X, key16_inv(k_lo), 0);
        const float y_hi  = temp_value<DT>(X, key16_inv(k_hi), 0);
        auto        member = [&](int v, float y, u32 raw) {
            const u32 k = key16(raw);
            if (k >= k_lo && k <= k_hi) {
                const u32 pos = atomicAdd(&s_ncls, 1u);
                if (pos < (u32)(2 * kMaxRuns)) {
                    cls[pos] = (u32)v;
                }
            }
        };
        stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return y_lo; }, member, kWholeRow, y_hi);
    }
    __syncthreads();
    const int ncls = (int)s_ncls;
    trace_mark(O.trace, 8);
    if (ncls > 2 * kMaxRuns || J >= ncls) {
        { if (O.trace != nullptr && threadIdx.x == 0) { O.trace[4 + 25] = 10; } return 0; }
    }
    // J-th smallest column of the class: members are counted per block of columns (reversed, so that the
    // walk from the top runs over ascending columns), the block holding rank J is found, and only the few
    // members of that block are ranked against each other.
    {
        __shared__ u32 s_blk[512];
        __shared__ u32 s_nblk;
        int            shift = 0;
        while (((P.vocab_padded - 1) >> shift) >= kNB) {
            ++shift;
        }
        for (int i = tid; i < kNB; i += kThreads) {
            S.hist[i] = 0;
        }
        if (tid == 0) {
            s_nblk = 0;
        }
        __syncthreads();
        for (int a = tid; a < ncls; a += kThreads) {
            smem_add(&S.hist[kNB - 1 - (int)(cls[a] >> shift)], 1u);
        }
        __syncthreads();
        u32       before = 0;
        const int bsel   = find_count_from_top(S.hist, (u32)(J + 1), &before);
        for (int a = tid; a < ncls; a += kThreads) {
            const int b = kNB - 1 - (int)(cls[a] >> shift);
            if (b == bsel) {
                s_blk[atomicAdd(&s_nblk, 1u)] = cls[a];
            }
        }
        __syncthreads();
        const int m  = (int)s_nblk;
        const int jj = J - (int)before;
        for (int a = tid; a < m; a += kThreads) {
            const u32 ca = s_blk[a];
            int       rk = 0;
            for (int b = 0; b < m; ++b) {
                rk += s_blk[b] < ca ? 1 : 0;
            }
            if (rk == jj) {
                s_sel = (int)ca;
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        const int id = s_sel;
        *O.id_out    = id;
        if (want_lp) {
            const float lprob = logf(p_sel);
            if (P.cum_log_probs != nullptr) {
                P.cum_log_probs[O.r] += lprob;
            }
            if (P.out_log_probs != nullptr) {
                P.out_log_probs[O.r] = lprob;
            }
        }
        write_lengths(P, O, id);
    }
    __syncthreads();
    return 1;
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

    // pass 1 (HBM): row maximum
    __shared__ int s_argmax;
    // The hot loop takes the maximum over every column as if no token were penalised or banned.  That
    // is the maximum of the ordinary columns unless a special column holds a pre-penalty value that
    // large; then the row is read again with the special columns left out.
    __shared__ int s_redo;
    if (tid == 0) {
        s_redo = 0;
    }
    trace_mark(O.trace, 0);
    u32        kraw       = 0;
    const bool have_slots = DT != FTB200_F32 && packed_ok<DT>(P, C);  // the max pass also leaves the slot maxima
    if (have_slots) {
        for (int i = 0; i < kSlotsPerThread; ++i) {
            ((u32*)S.hitq)[i * kThreads + tid] = 0;  // lowest key: a row too short for the vector pass leaves it
        }
    }
    float      tall       = stream_max<DT>(P, S, C, true, &kraw, have_slots ? (u32*)S.hitq : nullptr);
    fetch_specials<DT>(P, S, C);
    trace_mark(O.trace, 1);
    {
        // largest value and largest 16-bit pattern (as an ordered key) in one reduction
        const u64 m = block_max_u64(((u64)fkey(tall) << 32) | kraw);
        tall        = fkey_inv((u32)(m >> 32));
        kraw        = (u32)(m & 0xffffffffu);
    }
    float tmax = -INFINITY;
    {
        const Xf X = make_xf(P, S, C);
        bool     clash = false;
        for (int i = tid; i < P.hash_slots; i += kThreads) {
            const u32 w = X.hash[i];
            if (w != kHashEmpty) {
                clash |= S.spre[i] >= tall;
            }
        }
        if (clash) {
            s_redo = 1;
        }
    }
    trace_mark(O.trace, 15);
    __syncthreads();
    if (s_redo) {
        // the largest column is a penalised or banned one: take the maximum over the others from the slot
        // maxima where the pass left them, reading again only the slots a special column may top
        bool from_slots = false;
        if constexpr (DT != FTB200_F32) {
            if (have_slots) {
                from_slots = clean_special_slots<DT>(P, S, C, (u32*)S.hitq);
            }
        }
        trace_mark(O.trace, 16);
        tmax = from_slots ? stream_max<DT>(P, S, C, false, nullptr, nullptr, (const u32*)S.hitq) :
                            stream_max<DT>(P, S, C, false);
    }
    else {
        tmax = tall;
    }
    visit_specials<DT>(P, S, C, -INFINITY, [&](int v, float y) {
        if (y > C.neg_max) {
            tmax = fmaxf(tmax, y);
        }
    });
    const u64 best = block_max_u64(tmax > C.neg_max ? ((u64)fkey(tmax) << 32) | 1u : 0ull);
    if (best == 0) {
        if (tid == 0) {
            *O.id_out = 0;
            write_lengths(P, O, 0);
        }
        __syncthreads();
        return;
    }
    const float maxv = fkey_inv((u32)(best >> 32));
    trace_mark(O.trace, 2);

    // pass 2 (L2): exponentials, the denominator in the reference's summation order, and bucket counts
    // of every 16th group of columns.  Shared-memory atomics retire about one lane per clock, so a
    // full histogram would cost more than the rest of the row; the sample only has to place the cut.
    for (int i = tid; i < kNB; i += kThreads) {
        S.hist[i] = 0;
    }
    __syncthreads();
    if (have_slots) {
        // exact part of the provisional histogram: the slot maxima within kTopSpan of the row maximum.  A large
        // column that shares its slot with a larger one is missed, which only makes the cut more generous.
        const Xf   X     = make_xf(P, S, C);
        const u32* slots = (const u32*)S.hitq;
        for (int i = 0; i < kSlotsPerThread; ++i) {
            const float y = temp_value<DT>(X, key16_inv(slots[i * kThreads + tid] >> 16), 0);
            const int   b = lin_bucket(y, maxv);
            if (b > kTopBucket && y > C.neg_max) {
                smem_add(&S.hist[b], 1u);
            }
        }
        __syncthreads();
    }
    const int nvt = P.vocab < 1024 ? P.vocab : 1024;  // blockDim of addBiasSoftMax (:1364)
    softmax_pass2<DT>(P, S, C, maxv, nvt, O.trace, !have_slots);
    __syncthreads();
    trace_mark(O.trace, 3);
    {
        // the reference's blockReduceSum (reduce_kernel_utils.cuh:73-103) over nvt partial sums: every
        // 32-value butterfly is independent, so the warps of the CTA share them; warp 0 then runs the second
        // stage over the per-warp results (threads with threadIdx < blockDim / 32.f read their warp's result,
        // the others 0)
        __shared__ float s_vw[32];
        const int        nvw = (nvt + 31) / 32;
        for (int w = wid; w < nvw; w += kWarps) {
            const int i = w * 32 + lane;
            float     v = i < nvt ? S.val2[i] : 0.0f;
            for (int m = 16; m > 0; m >>= 1) {
                v = v + __shfl_xor_sync(0xffffffffu, v, m);
            }
            if (lane == 0) {
                s_vw[w] = v;
            }
        }
        __syncthreads();
        if (wid == 0) {
            float v = ((float)lane < (float)nvt / 32.f) ? s_vw[lane] : 0.0f;
            for (int m = 16; m > 0; m >>= 1) {
                v = v + __shfl_xor_sync(0xffffffffu, v, m);
            }
            if (lane == 0) {
                s_S = v;
            }
        }
    }
    __syncthreads();
    trace_mark(O.trace, 17);
    const float denom = s_S + 1e-6f;

    if (is_topp) {
        // arg-max shortcut of topp_beam_topk_kernel (sampling_topp_kernels.cu:801-860)
        const float p_max = round_to_T<DT>(round_to_T<DT>(1.0f) / denom);
        if (p_max >= top_p) {
            // first column holding the maximum (TopK<T,1>: larger value, then smaller column)
            if (tid == 0) {
                s_argmax = 0x7fffffff;
            }
            __syncthreads();
            auto first_max = [&](int v, float y) {
                if (y == maxv) {
                    atomicMin(&s_argmax, v);
                }
            };
            stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return maxv; }, first_max, kWholeRow);
            visit_specials<DT>(P, S, C, maxv, first_max);
            __syncthreads();
            const int argmax = s_argmax;
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
    __shared__ int s_bthr;

    // Provisional cut from the sample (x16), taken generously; the exact counts above it follow.
    int b_cut;
    {
        int b_est;
        auto weight = [&](int b) { return b > kTopBucket ? 1.0f : 16.0f; };
        if (is_topp) {
            const float scale = 1.0f / denom;
            auto        prob  = [&](int b) { return __expf(-((float)(kNB - 1 - b) + 0.5f) / (float)kLinScale) * scale; };
            // spread of the estimate: only the sampled buckets contribute, 240 n p^2 each
            float var = 0.0f;
            for (int b = tid; b <= kTopBucket; b += kThreads) {
                const float pb = prob(b);
                var += 240.0f * (float)S.hist[b] * pb * pb;
            }
            {
                __shared__ float s_var[kWarps];
                for (int m = 16; m > 0; m >>= 1) {
                    var += __shfl_xor_sync(0xffffffffu, var, m);
                }
                if (lane == 0) {
                    s_var[wid] = var;
                }
                __syncthreads();
                var = 0.0f;
                for (int i = 0; i < kWarps; ++i) {
                    var += s_var[i];
                }
                __syncthreads();
            }
            const float margin = 3.0f * sqrtf(var) + 0.01f;
            auto        w      = [&](int b) { return (double)S.hist[b] * (double)(prob(b) * weight(b)); };
            b_est = find_from_top(w, (double)(rand_num + margin), nullptr);
            trace_mark(O.trace, 19);
        }
        else {
            auto w = [&](int b) { return (double)weight(b) * (double)S.hist[b]; };
            b_est  = find_from_top(w, 1.25 * (double)k + 64.0, nullptr);
        }
        if (tid == 0) {
            int bt    = b_est < 0 ? 0 : b_est;
            u32 extra = 0;
            while (bt > 0 && extra < 8u) {
                --bt;
                extra += S.hist[bt];
            }
            s_bthr = bt;
        }
        __syncthreads();
        b_cut = s_bthr;
        __syncthreads();
    }

    trace_mark(O.trace, 4);
    if (is_topp && DT != FTB200_F32 && packed_ok<DT>(P, C)) {
        // value-class path: first with the provisional cut, then with every pattern the class window holds
        const u32   k_bot = kraw >= (u32)(kNB - 1) ? kraw - (u32)(kNB - 1) : 0u;
        const float cut_b = k_bot == 0u ? -INFINITY : temp_value<DT>(make_xf(P, S, C), key16_inv(k_bot), 0);
        const float cut_p = b_cut == 0 ? -INFINITY :
                                         maxv - (float)(kNB - b_cut) / (float)kLinScale - 1e-3f * fabsf(maxv) - 1e-3f;
        const float cut_a = fmaxf(cut_p, cut_b);
        // columns above the provisional cut, from the 1-in-16 sample: a dense row skips the hit queue
        // ... and above the top of a class window anchored at the provisional cut (when that one ends below the
        // row maximum)
        bool anchored = false;
        int  b_wtop   = kNB;
        if (cut_p > -INFINITY && cut_p < cut_b) {
            const Xf Xc = make_xf(P, S, C);
            u32      lo = 0, hi = kraw;  // lowest pattern whose value reaches the cut
            while (lo < hi) {
                const u32 mid = (lo + hi) >> 1;
                if (temp_value<DT>(Xc, key16_inv(mid), 0) >= cut_p) {
                    hi = mid;
                }
                else {
                    lo = mid + 1;
                }
            }
            if (lo + (u32)kNB <= kraw) {
                anchored = true;
                b_wtop   = lin_bucket(temp_value<DT>(Xc, key16_inv(lo + (u32)kNB), 0), maxv);
            }
        }
        u32 above = 0, above_w = 0;
        for (int i = tid; i < kNB; i += kThreads) {
            const u32 c = S.hist[i] * (i > kTopBucket ? 1u : 16u);
            above += i >= b_cut ? c : 0u;
            above_w += i >= b_wtop ? c : 0u;
        }
        above            = block_sum_u32(above);
        above_w          = block_sum_u32(above_w);
        // (the pass over bit patterns costs about as much as queueing 10 k columns one by one)
        const bool many  = above * 16u > (u32)P.vocab;
        const bool dense = cut_a <= cut_b || many;
        if (anchored && above_w <= (u32)(kMaxAbove / 2)) {
            // the nucleus reaches below the window of the maximum and the row is peaked: a window anchored at the
            // cut, the few columns above it listed one by one
            if (row_topp_classes<DT>(P, S, C, O, maxv, denom, rand_num, cut_p, kraw, want_lp, many)) {
                return;
            }
            if (O.trace != nullptr && tid == 0) {
                O.trace[4 + 26] = O.trace[4 + 25];  // why the anchored window gave up
            }
        }
        if (row_topp_classes<DT>(P, S, C, O, maxv, denom, rand_num, cut_a, kraw, want_lp, dense)) {
            return;
        }
        if (cut_b < cut_a && row_topp_classes<DT>(P, S, C, O, maxv, denom, rand_num, cut_b, kraw, want_lp, true, k_bot)) {
            return;
        }
        __syncthreads();
        trace_mark(O.trace, 11);
    }

    for (int attempt = 0; attempt < 2; ++attempt) {
        if (attempt == 1) {
            b_cut = 0;  // the provisional cut was too high: count and collect the whole row
        }
        // exact bucket counts of the columns above the provisional cut (filtered read from L2)
        for (int i = tid; i < kNB; i += kThreads) {
            S.hist[i] = 0;
        }
        __syncthreads();
        {
            const float cut0 = b_cut == 0 ? -INFINITY :
                                            maxv - (float)(kNB - b_cut) / (float)kLinScale - 1e-3f * fabsf(maxv) - 1e-3f;
            auto count = [&](int v, float y) {
                if (y > C.neg_max) {
                    const int b = lin_bucket(y, maxv);
                    if (b >= b_cut) {
                        smem_add(&S.hist[b], 1u);
                    }
                }
            };
            stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return cut0; }, count);
            visit_specials<DT>(P, S, C, cut0, count);
            __syncthreads();
        }

        // choose the lowest bucket to collect, now with a bound that holds
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
        // Collect below the deciding bucket until at least 64 more columns are in: the scan needs the
        // 32 entries after the crossing, and the crossing must not fall into the lowest collected
        // value class (which may continue below the cut).  16-bit logits leave many buckets empty.
        if (tid == 0) {
            int bt    = b_star < 0 ? b_cut : b_star;
            u32 extra = 0;
            while (bt > b_cut && extra < 64u) {
                --bt;
                extra += S.hist[bt];
            }
            // -1: the counted range does not reach far enough; the second attempt takes the whole row (a class
            // of equal probabilities - zeros after rounding to half, say - can be larger than any partial set)
            s_bthr = attempt == 1 ? 0 : ((b_cut > 0 && (b_star < 0 || extra < 64u)) ? -1 : bt);
        }
        __syncthreads();
        const int b_thr = s_bthr;
        __syncthreads();
        if (b_thr < 0) {
            continue;
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
        {
            const float cut = b_thr == 0 ? -INFINITY :
                                           maxv - (float)(kNB - b_thr) / (float)kLinScale - 1e-3f * fabsf(maxv) - 1e-3f;
            auto collect = [&](int v, float y) {
                if (y > C.neg_max) {
                    const int b = lin_bucket(y, maxv);
                    if (b >= b_thr) {
                        float ex  = round_to_T<DT>(__expf(y - maxv));
                        float pr  = round_to_T<DT>(ex / denom);
                        u32   pos = atomicAdd(&S.hist[b], 1u);
                        dest[pos] = ((u64)(~fkey(pr)) << 32) | (u32)v;
                    }
                }
            };
            stream_filtered<DT>(P, S, C, 0, C.nvec, [&]() { return cut; }, collect);
            visit_specials<DT>(P, S, C, cut, collect);
        }
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
        if (sel >= 0 && sel < (int)n_g) {
            // Equal probabilities stand in column order in the reference's stable sort.  The buckets above are
            // ordered by logit: probabilities rounded to the logits type can be equal across a bucket boundary,
            // so the whole run of entries equal to the selected one is put into column order before it is read.
            __shared__ int s_eq_lo, s_eq_hi;
            if (tid == 0) {
                s_eq_lo = sel;
                s_eq_hi = sel + 1;
            }
            __syncthreads();
            const u32 ksel = (u32)(dest[sel] >> 32);
            for (int i = tid; i < (int)n_g; i += kThreads) {
                if ((u32)(dest[i] >> 32) == ksel) {
                    atomicMin(&s_eq_lo, i);
                    atomicMax(&s_eq_hi, i + 1);
                }
            }
            __syncthreads();
            const int eq_lo = s_eq_lo, eq_hi = s_eq_hi;
            if (eq_hi - eq_lo > 1) {
                group_sort_u64(dest + eq_lo, eq_hi - eq_lo, tid, kThreads, CtaSync());
            }
            __syncthreads();
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

// Vocabulary-parallel local pass of a top-p row: largest final value of the shard's columns and the sum of
// exp(value - that maximum) over them, stored in the last word of the row's record as two floats.  The ranks
// combine the pairs as the reference's online soft-max does (reduce_md_op,
// kernels/online_softmax_beamsearch_kernels.cu:270-279), so the denominator is not summed in the single-GPU
// order: a draw that falls within rounding of a boundary may pick the neighbouring column.
template<int DT>
__device__ __noinline__ void row_vp_stats(const KParams& P, const Smem& S, const RowCtx& C, const RowOut& O)
{
    const int tid = threadIdx.x;
    float     m   = stream_max<DT>(P, S, C, false);  // ordinary columns (special ones are left out)
    fetch_specials<DT>(P, S, C);
    visit_specials<DT>(P, S, C, -INFINITY, [&](int v, float y) {
        if (y > C.neg_max) {
            m = fmaxf(m, y);
        }
    });
    const u64 best = block_max_u64(m > C.neg_max ? ((u64)fkey(m) << 32) | 1u : 0ull);
    float     maxv = -INFINITY, sum = 0.0f;
    if (best != 0) {
        maxv = fkey_inv((u32)(best >> 32));
        auto add = [&](int v, float y) {
            if (y > C.neg_max) {
                sum += __expf(y - maxv);
            }
        };
        stream_all<DT>(P, S, C, 0, C.nvec, add);
        visit_specials<DT>(P, S, C, -INFINITY, add);
    }
    // block-wide sum of the per-thread partial sums
    __shared__ float s_part[kWarps];
    for (int k = 16; k > 0; k >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, k);
    }
    if ((tid & 31) == 0) {
        s_part[tid >> 5] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
        for (int i = 0; i < kWarps; ++i) {
            t += s_part[i];
        }
        P.vp_out[(size_t)O.r * (P.vp_cap + 2) + P.vp_cap + 1] = ((u64)__float_as_uint(maxv) << 32) | __float_as_uint(t);
    }
    __syncthreads();
}

template<int DT>
__device__ void process_row(const KParams& P, const Smem& S, int r, u64* gscratch, u64* trace)
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
    // The per-row records live in shared memory: the row functions take them by reference, and a
    // reference to a stack object would turn every field access into a local-memory load.
    __shared__ RowOut s_O;
    __shared__ RowCtx s_C;
    RowOut&           O = s_O;
    if (tid == 0) {
        O.r      = r;
        O.end_id = P.end_ids[r];
        O.id_out = P.output_ids + (size_t)P.step * P.batch_size + (size_t)P.ite * P.local_batch + r;
        O.trace  = trace;
    }

    const bool fin     = P.finished != nullptr ? P.finished[r] != 0 : false;
    const bool want_lp = P.cum_log_probs != nullptr || P.out_log_probs != nullptr;
    __syncthreads();  // every thread has read finished[r] before thread 0 may rewrite it

    if (P.vp_out != nullptr) {
        // vocabulary-parallel local pass: candidates only; the merge draws
        if (mode == 1 && !fin) {
            RowCtx& C = s_C;
            build_row<DT>(P, S, C, r);
            int k = (int)P.topk_ks[r];
            k     = k < 1 ? 1 : (k > kMaxTopK ? kMaxTopK : k);
            if (!(P.bias == nullptr && C.inv_t > 0.0f && row_topk2<DT>(P, S, C, O, k, 0.0f, 1.0f))) {
                row_topk<DT>(P, S, C, O, gscratch, k, 0.0f, 1.0f);
            }
        }
        else if (mode == 2 && !fin) {
            // top-p row: the shard's (maximum, sum of exponentials) and its largest columns; the merge builds
            // the nucleus from the union
            RowCtx& C = s_C;
            build_row<DT>(P, S, C, r);
            row_vp_stats<DT>(P, S, C, O);
            int k = P.vp_cap > 128 ? P.vp_cap - 64 : P.vp_cap / 2;
            k     = k < 1 ? 1 : (k > kMaxTopK ? kMaxTopK : k);
            if (!(P.bias == nullptr && C.inv_t > 0.0f && row_topk2<DT>(P, S, C, O, k, 0.0f, 1.0f))) {
                row_topk<DT>(P, S, C, O, gscratch, k, 0.0f, 1.0f);
            }
        }
        else if (tid == 0) {
            P.vp_out[(size_t)r * (P.vp_cap + 2)] = 0;
        }
        __syncthreads();
        return;
    }
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
            RowCtx& C = s_C;
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
                else if (!(P.bias == nullptr && C.inv_t > 0.0f && row_topk2<DT>(P, S, C, O, k, u, top_p))) {
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
__global__ void __launch_bounds__(kThreads, 2) decode_sampling_kernel(const __grid_constant__ KParams P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int                                s_row;
    __shared__ Smem                               s_S;
    Smem&                                         S = s_S;
    if (threadIdx.x == 0) {
        S.cand  = (u64*)smem_raw;
        S.hist  = (u32*)(S.cand + kCap);
        S.val2  = (float*)(S.hist + kNB);
        S.flags = (u32*)(S.val2 + 1024);
        S.hash  = S.flags + P.flag_words;
        S.spre  = (float*)(S.hash + P.hash_slots);
        S.sfin  = S.spre + P.hash_slots;
        S.nhit  = (u32*)(S.sfin + P.hash_slots);
        S.hitq  = (unsigned short*)(S.nhit + 4);
    }
    u64* gscratch = P.scratch + (size_t)blockIdx.x * P.scratch_stride;
    // rows to serve: the whole local batch, or the list the single-pass kernel left behind
    const int n_rows = P.row_count_dev != nullptr ? (int)*P.row_count_dev : P.local_batch;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) {
            s_row = (int)atomicAdd(P.ticket, 1u);
        }
        __syncthreads();
        const int t = s_row;
        if (t >= n_rows) {
            break;
        }
        // rows are handed out costliest first when the caller supplied an order (longest-processing-
        // time-first keeps the last CTAs from finishing alone with an expensive row)
        const int r   = P.row_order != nullptr ? P.row_order[t] : t;
        u64*      rec = P.trace != nullptr ? P.trace + (size_t)t * kTraceWords : nullptr;
        if (rec != nullptr && threadIdx.x == 0) {
            rec[0] = (u64)r, rec[1] = (u64)blockIdx.x, rec[2] = global_timer_ns();
        }
        process_row<DT>(P, S, r, gscratch, rec);
        if (rec != nullptr && threadIdx.x == 0) {
            rec[3] = global_timer_ns();
        }
    }
}


// Merge of one top-p row: union of the shards' candidates, soft-max statistics combined, probabilities of the
// candidates, the reference's block-wide scan over them in sorted order (kernels/sampling_topp_kernels.cu:
// 877-1004) until the draw is crossed.  A row whose nucleus needs more columns than the shards sent is
// counted in `overflow` and gets id -1: the caller repeats it with a larger cap or on gathered logits.
template<int DT>
__device__ __noinline__ void vp_merge_topp_row(const KParams& P, const Smem& S, const u64* gathered, int nranks,
                                               int* overflow, int r)
{
    __shared__ float s_u, s_M, s_den;
    __shared__ u32   s_n, s_bad, s_all;
    __shared__ int   s_sel, s_lo, s_hi;
    const int        tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    int* const       id_out = P.output_ids + (size_t)P.step * P.batch_size + (size_t)P.ite * P.local_batch + r;
    const int        end_id = P.end_ids[r];
    const bool       fin    = P.finished != nullptr ? P.finished[r] != 0 : false;
    const float      top_p  = P.topp_ps[r];
    __syncthreads();
    __shared__ curandState_t s_before;  // the generator before this row's draw: an undecided row gets it back,
                                        // so that repeating the row draws the same number
    if (tid == 0) {
        s_before = P.topp_states[r];
        s_u   = draw_uniform(P.topp_states, r);  // every row of the top-p layer draws, finished or not
        s_n   = 0;
        s_bad = 0;
        s_all = 1;
        s_sel = -1;
    }
    __syncthreads();
    const float u = s_u;
    int         id = -1;
    bool        update_state = false;
    if (fin) {
        // one-hot row on the end id (sampling_topp_kernels.cu:1309-1341)
        const float p0 = DT == FTB200_F16 ? __half2float(__float2half_rn(1.0f / (1.0f + 1e-6f))) : 1.0f / (1.0f + 1e-6f);
        id             = end_id;
        if (tid == 0) {
            *id_out = id;
            if ((p0 >= top_p || u * top_p <= p0) && P.seq_len != nullptr && P.finished != nullptr) {
                P.finished[r] = 1;
            }
        }
    }
    else {
        // union of the candidates, statistics
        float M = -INFINITY;
        for (int q = 0; q < nranks; ++q) {
            const u64* rec = gathered + ((size_t)q * P.local_batch + r) * (P.vp_cap + 2);
            const u64  c   = rec[0];
            if (c == ~0ull) {
                if (tid == 0) {
                    s_bad = 1;
                }
                continue;
            }
            const u32 base = s_n;
            __syncthreads();
            if (base + (u32)c > (u32)kCap) {
                if (tid == 0) {
                    s_bad = 1;
                }
            }
            else {
                for (u32 i = tid; i < (u32)c; i += kThreads) {
                    S.cand[base + i] = rec[1 + i];
                }
                if (tid == 0) {
                    s_n = base + (u32)c;
                    const int k_local = P.vp_cap > 128 ? P.vp_cap - 64 : P.vp_cap / 2;
                    if ((int)c >= (k_local < kMaxTopK ? k_local : kMaxTopK)) {
                        s_all = 0;  // this shard may hold more columns than it sent
                    }
                }
            }
            M = fmaxf(M, __uint_as_float((u32)(rec[P.vp_cap + 1] >> 32)));
            __syncthreads();
        }
        if (tid == 0) {
            float den = 0.0f;
            for (int q = 0; q < nranks; ++q) {
                const u64 w = gathered[((size_t)q * P.local_batch + r) * (P.vp_cap + 2) + P.vp_cap + 1];
                const float m = __uint_as_float((u32)(w >> 32)), d = __uint_as_float((u32)w);
                if (m > -INFINITY) {
                    den += d * __expf(m - M);
                }
            }
            s_M   = M;
            s_den = den + 1e-6f;
        }
        __syncthreads();
        const int   n     = (int)s_n;
        const float denom = s_den;
        if (s_bad || n == 0 || !(M > -INFINITY)) {
            if (tid == 0) {
                atomicAdd(overflow, 1);
                *id_out            = -1;
                P.topp_states[r] = s_before;
            }
            __syncthreads();
            return;
        }
        group_sort_u64(S.cand, n, tid, kThreads, CtaSync());  // value descending, column ascending
        __syncthreads();
        // probabilities in place of the values (monotone: the order stays, equal probabilities are handled below)
        for (int i = tid; i < n; i += kThreads) {
            const u64   e  = S.cand[i];
            const float y  = fkey_inv(~(u32)(e >> 32));
            const float ex = round_to_T<DT>(__expf(y - M));
            const float pr = round_to_T<DT>(ex / denom);
            S.cand[i]      = ((u64)(~fkey(pr)) << 32) | (e & 0xffffffffu);
        }
        __syncthreads();
        const float p_max    = fkey_inv(~(u32)(S.cand[0] >> 32));
        const float rand_num = u * top_p;
        if (p_max >= top_p) {
            if (tid == 0) {
                s_sel = 0;  // arg-max shortcut of topp_beam_topk_kernel (sampling_topp_kernels.cu:801-860)
            }
        }
        else if (wid == 0) {
            float R   = 0.0f;
            int   sel = -1;
            for (int c = 0; c * 256 < n; ++c) {
                const int bi = c * 256 + lane * 8;
                float     x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    x[i] = bi + i < n ? fkey_inv(~(u32)(S.cand[bi + i] >> 32)) : 0.0f;
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
                u32 c4 = cnt;
                c4 += __shfl_xor_sync(0xffffffffu, c4, 1);
                c4 += __shfl_xor_sync(0xffffffffu, c4, 2);
                const u32 any = __ballot_sync(0xffffffffu, c4 > 0);
                if (any) {
                    const int g  = (__ffs(any) - 1) >> 2;
                    const u32 pc = __shfl_sync(0xffffffffu, c4, g * 4);
                    sel          = c * 256 + g * 32 + (32 - (int)pc);
                    if (!s_all && c * 256 + g * 32 + 31 >= n) {
                        sel = -2;  // the 32 probabilities of that warp are not all known
                    }
                    break;
                }
                R = R + agg;
            }
            if (sel >= n) {
                sel = -2;
            }
            if (sel == -1 && !s_all) {
                sel = -2;  // the draw lies beyond what the shards sent
            }
            if (lane == 0) {
                s_sel = sel;
            }
        }
        __syncthreads();
        int sel = s_sel;
        if (sel == -2) {
            if (tid == 0) {
                atomicAdd(overflow, 1);
                *id_out            = -1;
                P.topp_states[r] = s_before;
            }
            __syncthreads();
            return;
        }
        if (sel >= 0) {
            // equal probabilities stand in column order
            if (tid == 0) {
                s_lo = sel;
                s_hi = sel + 1;
            }
            __syncthreads();
            const u32 ksel = (u32)(S.cand[sel] >> 32);
            for (int i = tid; i < n; i += kThreads) {
                if ((u32)(S.cand[i] >> 32) == ksel) {
                    atomicMin(&s_lo, i);
                    atomicMax(&s_hi, i + 1);
                }
            }
            __syncthreads();
            const int lo = s_lo, hi = s_hi;
            if (!s_all && hi == n) {
                // the class of the crossing may continue in columns that were not sent
                if (tid == 0) {
                    atomicAdd(overflow, 1);
                    *id_out            = -1;
                    P.topp_states[r] = s_before;
                }
                __syncthreads();
                return;
            }
            if (hi - lo > 1) {
                group_sort_u64(S.cand + lo, hi - lo, tid, kThreads, CtaSync());
            }
            __syncthreads();
            id           = (int)(S.cand[sel] & 0xffffffffu);
            update_state = true;
        }
        else {
            // the cumulative sum never reached the draw: the best token, no length / finished update
            id = (int)(S.cand[0] & 0xffffffffu);
        }
        if (tid == 0) {
            *id_out = id;
            if (update_state && P.seq_len != nullptr && P.finished != nullptr) {
                P.seq_len[r]  = P.seq_len[r] + 1;
                P.finished[r] = id == end_id ? 1 : 0;
            }
        }
    }
    __syncthreads();
    // top-p decay / reset (sampling_topp_kernels.cu:1381-1408)
    if (P.topp_decay != nullptr && tid == 0) {
        float p = P.topp_ps[r];
        if (id == P.topp_reset[r]) {
            p = P.topp_initial[r];
        }
        else {
            p = fmaxf(p * P.topp_decay[r], P.topp_min[r]);
        }
        P.topp_ps[r] = p;
    }
    __syncthreads();
}

// Vocabulary-parallel merge: one CTA per row.  `gathered` holds, rank after rank, the records the local
// passes emitted ([rank][row][1 + cap]: count, then (~key(value) << 32 | global column) entries).  The
// union is sorted and handed to the same draw and tie-order code as the single-GPU path, so every rank
// arrives at the id the reference would sample from the full row.
template<int DT>
__global__ void __launch_bounds__(kThreads, 3)
vp_merge_kernel(const __grid_constant__ KParams P, const u64* gathered, int nranks, int* overflow)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float                              s_u;
    __shared__ u32                                s_n;
    __shared__ curandState_t                      s_before_k;  // generator of a top-k row before its draw
    constexpr int                                 kMergeRanks = 64;
    __shared__ u32                                s_off[kMergeRanks + 1];  // start of every rank's record in the union
    Smem                                          S;
    S.cand  = (u64*)smem_raw;
    S.hist  = (u32*)(S.cand + kCap);
    S.val2  = (float*)(S.hist + kNB);
    S.flags = nullptr, S.hash = nullptr, S.spre = nullptr, S.sfin = nullptr, S.hitq = nullptr, S.nhit = nullptr;
    const int tid = threadIdx.x;
    for (int r = blockIdx.x; r < P.local_batch; r += gridDim.x) {
        __syncthreads();
        const bool by_topk = P.topk_states != nullptr && !(P.topk_skip != nullptr && P.topk_skip[r]);
        const bool by_topp = !by_topk && P.topp_states != nullptr && !(P.topp_skip != nullptr && P.topp_skip[r]);
        if (by_topp) {
            vp_merge_topp_row<DT>(P, S, gathered, nranks, overflow, r);
            continue;
        }
        if (!by_topk) {
            continue;
        }
        RowOut O;
        O.r      = r;
        O.end_id = P.end_ids[r];
        O.id_out = P.output_ids + (size_t)P.step * P.batch_size + (size_t)P.ite * P.local_batch + r;
        O.trace  = nullptr;
        const bool fin = P.finished != nullptr ? P.finished[r] != 0 : false;
        __syncthreads();
        if (fin) {
            if (tid == 0) {
                *O.id_out = O.end_id;
            }
            continue;
        }
        if (tid == 0) {
            s_before_k = P.topk_states[r];
            s_u        = draw_uniform(P.topk_states, r);
            s_n        = 0;
        }
        __syncthreads();
        bool bad = false;
        for (int q = 0; q < nranks; ++q) {
            const u64* rec = gathered + ((size_t)q * P.local_batch + r) * (P.vp_cap + 2);
            const u64  c   = rec[0];
            if (c == ~0ull) {
                bad = true;
                continue;
            }
            const u32 base = s_n;
            __syncthreads();
            if (base + (u32)c > (u32)kCap) {
                bad = true;
            }
            else {
                for (u32 i = tid; i < (u32)c; i += kThreads) {
                    S.cand[base + i] = rec[1 + i];
                }
                if (tid == 0) {
                    if (q < kMergeRanks) {
                        s_off[q] = base, s_off[q + 1] = base + (u32)c;
                    }
                    s_n = base + (u32)c;
                }
            }
            __syncthreads();
        }
        if (bad) {
            if (tid == 0) {
                atomicAdd(overflow, 1);
                *O.id_out        = -1;
                P.topk_states[r] = s_before_k;  // repeating the row draws the same number
            }
            continue;
        }
        const int n      = (int)s_n;
        u64*      sorted = S.cand;
        if (nranks <= kMergeRanks && n <= kCap / 2) {
            // every rank's record is sorted already: the place of an entry in the union is its index in its own
            // record plus the number of smaller entries in each of the others (a binary search each; the entries are
            // distinct).  No sorting network, two barriers.
            u64* const dst = S.cand + kCap / 2;
            for (int a = tid; a < n; a += kThreads) {
                int q = 0;
                while (q + 1 < nranks && (u32)a >= s_off[q + 1]) {
                    ++q;
                }
                const u64 e    = S.cand[a];
                int       rank = a - (int)s_off[q];
                for (int o = 0; o < nranks; ++o) {
                    if (o == q) {
                        continue;
                    }
                    int lo = (int)s_off[o], hi = (int)s_off[o + 1];  // first entry of record o that is not below e
                    const int lo0 = lo;
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (S.cand[mid] < e) {
                            lo = mid + 1;
                        }
                        else {
                            hi = mid;
                        }
                    }
                    rank += lo - lo0;
                }
                dst[rank] = e;
            }
            __syncthreads();
            sorted = dst;
        }
        else {
            group_sort_u64(S.cand, n, tid, kThreads, CtaSync());
            __syncthreads();
        }
        int k = (int)P.topk_ks[r];
        k     = k < 1 ? 1 : (k > kMaxTopK ? kMaxTopK : k);
        topk_finish(P, S, O, sorted, n, k, s_u, P.topk_ps[r], true, false);
    }
}

template<int DT>
int vp_merge_launch(const KParams& K, const u64* gathered, int nranks, int* overflow, int grid, cudaStream_t st)
{
    const size_t smem = (size_t)kCap * 8 + (size_t)kNB * 4 + 1024 * 4;
    FTB_CUDA_CHECK(cudaFuncSetAttribute(vp_merge_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    vp_merge_kernel<DT><<<grid, kThreads, smem, st>>>(K, gathered, nranks, overflow);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

// ---- per-dtype launch glue (instantiated once per logits type, each in its own translation unit) ----
template<int DT>
int sampling_occupancy(size_t smem, int* per_sm)
{
    // One query per device and distinct shared-memory size; the answers are kept for the life of the process.  The
    // opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel: it is set on
    // every device before the first query there.
    constexpr int     kMaxDev = 64, kSizes = 8;
    static std::mutex mu;
    static bool       opted_in[kMaxDev];
    static size_t     cached_smem[kMaxDev][kSizes];
    static int        cached_val[kMaxDev][kSizes];
    static int        n_cached[kMaxDev];
    int               dev = 0;
    FTB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) {
        set_error("ftb200_decode_step_sampling: device ordinal out of range");
        return FTB200_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!opted_in[dev]) {
        FTB_CUDA_CHECK(
            cudaFuncSetAttribute(decode_sampling_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        opted_in[dev] = true;
    }
    for (int i = 0; i < n_cached[dev]; ++i) {
        if (cached_smem[dev][i] == smem) {
            *per_sm = cached_val[dev][i];
            return FTB200_OK;
        }
    }
    FTB_CUDA_CHECK(
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, decode_sampling_kernel<DT>, kThreads, smem));
    if (n_cached[dev] < kSizes) {
        cached_smem[dev][n_cached[dev]] = smem;
        cached_val[dev][n_cached[dev]]  = *per_sm;
        ++n_cached[dev];
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
