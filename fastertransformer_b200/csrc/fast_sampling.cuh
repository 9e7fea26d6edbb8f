// Single-pass form of the fused decode-sampling step for 16-bit logits (half / bfloat16) without an
// embedding bias: the kernel that serves the rows of a step first.  What it cannot decide from one pass
// (and every row kind it does not cover) is put on a list that decode_sampling_kernel works off afterwards,
// so the results are those of that kernel - and therefore the reference's - for every row.
//
// One CTA serves one row at a time; several CTAs share an SM, so that the fixed work of one row (set-up,
// threshold search, the draw) runs under the streaming of the others.  Per row:
//   1. a strided sample of 4096 columns gives, by bisection over the ordered 16-bit keys, a raw threshold
//      that about 2k (at least 128) columns of the row are expected to reach;
//   2. ONE pass over the row (16-byte loads, eight in flight per thread, one packed compare per two logits)
//      queues the vectors that hold a column at or above the threshold;
//   3. the queued vectors give the candidate columns and the count of every value class (bit pattern) above
//      the threshold; penalised / banned columns (token history, bad words, min-length) are taken out and
//      come back with their final values from a short list, as do the columns outside the aligned vectors;
//   4. the draw of topk_stage2_sampling (kernels/sampling_topk_kernels.cu:255-311) walks the classes from the
//      top - equal values add the same exponential, so the sorted sequence is (value, count) runs and no
//      sort of the candidates is needed - and the tie order inside the class the draw lands in follows
//      the reference's two-stage reduction (see resolve_topk_class).
// A row whose candidates turn out to be fewer than k, or that overflows one of the fixed-size tables, is
// left untouched (its generator state included) and goes to the list.
#pragma once
#include "sampling_kernels.cuh"

namespace ftb200 {

constexpr int kFCap      = 3840;  // candidate columns held in shared memory
constexpr int kFBins     = 2048;  // value classes (bit patterns) above the threshold
constexpr int kFSpecCap  = 128;   // listed columns (special or edge) at or above the threshold
constexpr int kFClsCap   = 768;   // members of the class the draw lands in
constexpr int kFRuns     = 1536;  // runs the draw may walk (classes + listed columns among the first k)
constexpr int kFRunBytes = kFRuns * 6 + kFBins * 2;  // top-k draw: value, count per run; class ranks
constexpr int kFPRuns    = 3584;  // top-p: runs of the replayed scan (probability, first position); a long history
                                  //        adds a run per listed column to the ~1500 patterns of a deep window
constexpr int kFPSpecCap = 2048;  // top-p: listed columns above the cut (a history of 2000 ids puts a thousand in a deep window)
constexpr int kFPClsCap  = 2048;  // top-p: members of the class the scan stops in
constexpr int kFSampleV  = 2;     // sampled vectors per thread (4096 columns per row)
constexpr int kFUnroll   = 8;     // 16-byte loads in flight per thread

// Shared-memory map of the single-pass kernel (dynamic shared memory, offsets fixed per launch).
struct FMap {
    u32*            cand;  // [kFCap]    (relative key << 20) | column
    u32*            emask; // [mask_words] per aligned vector one byte: which of its columns are special; after the
                           //              pass the same area holds the listed columns and the run arrays of the draw
    u32*            hash;  // [hash_slots] (id << 2) | flags, open addressing
    u32*            sval;  // [hash_slots] gathered raw word, then the final value of that column (float bits)
    u32*            hist;  // [kFBins]   columns per value class above the threshold
    u32*            stage; // [kFStageBytes / 4] token history, word list and last tokens of the row, as fetched
    uint4*          wbuf;  // [kWarps * kFRing] vectors parked during a pass (static shared memory of the kernel)
    unsigned short* wj;    // [kWarps * kFRing]
};

constexpr int kFMaxHist    = 1024;  // token-history entries the single-pass kernel stages at a time
constexpr int kFMaxHistAll = 4094;  // and in all (the table of special columns: step + words + 2 <= 4096)
constexpr int kFMaxWords   = 128;   // bad-word list length it stages
constexpr int kFStageBytes = 8192;  // >= (kFMaxHist + 2 * kFMaxWords + 4) * 4; later kFPSpecCap listed columns of a top-p row
// bytes of the per-vector mask area: one byte per aligned vector, and room for what follows the pass
__host__ __device__ inline size_t fast_mask_bytes(int vocab_padded, bool topp)
{
    const size_t need = ((size_t)vocab_padded / 8 + 16 + 15) / 16 * 16;
    size_t post = (size_t)kFSpecCap * 8 + (size_t)kFRunBytes;  // the top-k rows' kernel
    if (topp) {
        post = (size_t)kFPRuns * 8 > (size_t)kFPClsCap * 4 ? (size_t)kFPRuns * 8 : (size_t)kFPClsCap * 4;
    }
    return need > post ? need : post;
}
__host__ __device__ inline size_t fast_smem_bytes(int hash_slots, int vocab_padded, bool topp)
{
    const size_t sv = hash_slots > kFBins ? hash_slots : kFBins;  // the value area doubles as a class table
    return (size_t)kFCap * 4 + fast_mask_bytes(vocab_padded, topp) + (size_t)hash_slots * 4 + sv * 4 + (size_t)kFBins * 4
           + (topp ? (size_t)kFPSpecCap * 8 : (size_t)kFStageBytes);  // (the area is the last of the map)
}

__device__ __forceinline__ void cp_async4(u32 saddr, const void* g)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Row constants of the single-pass kernel (shared memory, written by thread 0).
struct FRow {
    const char* rowp;
    int         head, nfull, r, end_id, k;
    float       inv_t, theta, top_p, u;
    __half      inv_t_h;
    int*        id_out;
    u64*        trace;  // this row's record of the diagnostic timeline, or null
};

static __device__ void f_hash_insert(u32* hash, int slots, int shift, int id, u32 flag, int vocab_padded)
{
    if (id < 0 || id >= vocab_padded) {
        return;
    }
    FTB_ASSUME_SHARED(hash);
    u32       h    = hash_slot(id, shift);
    const u32 want = ((u32)id << 2) | flag;
    for (int probe = 0; probe < slots; ++probe) {
        const u32 old = smem_cas(&hash[h], kHashEmpty, want);
        if (old == kHashEmpty) {
            break;
        }
        if ((old >> 2) == (u32)id) {
            smem_or(&hash[h], flag);
            break;
        }
        h = (h + 1) & (slots - 1);
    }
}

// Value of a raw 16-bit pattern after temperature (no bias on this path).
template<int DT>
__device__ __forceinline__ float f_value(u32 raw, bool temp, float inv_t, __half inv_t_h)
{
    if (DT == FTB200_F16) {
        __half h = __ushort_as_half((unsigned short)raw);
        if (temp) {
            h = __hmul(h, inv_t_h);
        }
        return __half2float(h);
    }
    float x = __uint_as_float(raw << 16);
    if (temp) {
        x = x * inv_t;
    }
    return x;
}

// Slot of column `id` in the hash, -1 when it has none.
__device__ __forceinline__ int f_hash_find(const u32* hash, int shift, int mask, int id)
{
    FTB_ASSUME_SHARED(hash);
    u32 h = hash_slot(id, shift);
    for (int probe = 0; probe <= mask; ++probe) {
        const u32 v = hash[h];
        if (v == kHashEmpty) {
            return -1;
        }
        if ((v >> 2) == (u32)id) {
            return (int)h;
        }
        h = (h + 1) & mask;
    }
    return -1;
}

// What the pass over the row leaves behind, all in shared memory.
struct FSink {
    u32*                 cand;   // [kFCap] (relative key << 20) | column of every ordinary column at or above the threshold
    u32*                 hist;   // [kFBins] columns per relative key
    u32*                 sval;   // per hash slot: raw bits of that special column
    const u32*           hash;
    const unsigned char* emask;  // per aligned vector: bit e set = column e of the vector is special
    u32*                 ncand;
    u32*                 bad;    // set when a relative key does not fit the class table
    uint4*               wbuf;   // [kWarps][kFRing] vectors parked by the lanes of a warp
    unsigned short*      wj;     // [kWarps][kFRing] their vector indices
    int                  shift, mask, cap;
};

// One dense step of the side path: every live lane takes one parked vector of its warp, finds the columns at or
// above the threshold from the packed compares, leaves the raw values of special ones next to their hash slots
// and turns the others into candidates (one reservation in the candidate list per step and warp).
// BAND: the columns whose raw value lies in [thr_key, hi_key] are listed by column only (special ones left out).
template<int DT, bool BAND>
__device__ __forceinline__ void f_side_step(const uint4& v, int jj, bool live, int head, u32 thr_key, u32 thr2, u32 hi2,
                                            const FSink& K, u32& relmax)
{
    const int lane = threadIdx.x & 31;
    u32       pm   = 0;
    if (live) {
        u32 m0 = ge2_mask<DT>(v.x, thr2), m1 = ge2_mask<DT>(v.y, thr2);
        u32 m2 = ge2_mask<DT>(v.z, thr2), m3 = ge2_mask<DT>(v.w, thr2);
        if (BAND) {
            m0 &= le2_mask<DT>(v.x, hi2), m1 &= le2_mask<DT>(v.y, hi2);
            m2 &= le2_mask<DT>(v.z, hi2), m3 &= le2_mask<DT>(v.w, hi2);
        }
        pm = ((m0 & 1u) | ((m0 >> 15) & 2u)) | (((m1 & 1u) | ((m1 >> 15) & 2u)) << 2)
             | (((m2 & 1u) | ((m2 >> 15) & 2u)) << 4) | (((m3 & 1u) | ((m3 >> 15) & 2u)) << 6);
        if (BAND) {
            u32 t = pm;
            while (t != 0) {
                const int e = __ffs(t) - 1;
                t &= t - 1;
                if (hash_lookup_raw(K.hash, K.shift, K.mask, head + jj * 8 + e) != 0) {
                    pm &= ~(1u << e);
                }
            }
        }
        else {
            const u32 em = K.emask[jj];
            u32       sp = pm & em;
            pm &= ~em;
            while (sp != 0) {  // rare: a special column at or above the threshold
                const int e = __ffs(sp) - 1;
                sp &= sp - 1;
                const int slot = f_hash_find(K.hash, K.shift, K.mask, head + jj * 8 + e);
                if (slot >= 0) {
                    K.sval[slot] = raw_bits<DT>(v, e);
                }
            }
        }
    }
    const u32 n    = (u32)__popc(pm);
    u32       incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
        incl += lane >= o ? t : 0u;
    }
    const u32 total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) {
        return;
    }
    u32 base = 0;
    if (lane == 0) {
        base = atomicAdd(K.ncand, total);
    }
    base    = __shfl_sync(0xffffffffu, base, 0);
    u32 pos = base + incl - n;
    while (pm != 0) {
        const int e = __ffs(pm) - 1;
        pm &= pm - 1;
        if (BAND) {
            if (pos < (u32)K.cap) {
                K.cand[pos] = (u32)(head + jj * 8 + e);
            }
        }
        else {
            const u32 rel = key16(raw_bits<DT>(v, e)) - thr_key;
            if (rel >= (u32)kFBins) {
                *K.bad = 1;  // (the slot stays unwritten: the row is given up)
            }
            else {
                relmax = rel > relmax ? rel : relmax;
                if (pos < (u32)K.cap) {
                    K.cand[pos] = (rel << 20) | (u32)(head + jj * 8 + e);
                }
                smem_add(&K.hist[rel], 1u);
            }
        }
        ++pos;
    }
}

// The one pass over the row.  Eight 16-byte loads in flight per thread, one packed compare per two logits.
// A vector with a column at or above the threshold is a rare event for a lane but a common one for a warp, so
// a lane does not look at its own hit: it parks the vector in a small ring of its warp, and whenever 32
// vectors are parked the warp takes them one per lane (f_side_step).  Nothing of the row is read a second time.
constexpr int kFRing = 64;  // parked vectors per warp
template<int DT, bool BAND, int UNROLL>
__device__ __noinline__ void f_stream(const uint4* vp, int nfull, int head, u32 thr_key, u32 hi_key, const FSink& Ks,
                                      u32* relmax_out)
{
    const FSink K = Ks;  // (a copy in registers)
    FTB_ASSUME_SHARED(K.cand);
    FTB_ASSUME_SHARED(K.hist);
    FTB_ASSUME_SHARED(K.sval);
    FTB_ASSUME_SHARED(K.emask);
    FTB_ASSUME_SHARED(K.ncand);
    FTB_ASSUME_SHARED(K.bad);
    FTB_ASSUME_SHARED(K.wbuf);
    FTB_ASSUME_SHARED(K.wj);
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const u32 thr_raw = key16_inv(thr_key), hi_raw = key16_inv(hi_key);
    const u32 thr2 = thr_raw | (thr_raw << 16), hi2 = hi_raw | (hi_raw << 16);
    uint4* const          wbuf = K.wbuf + wid * kFRing;
    unsigned short* const wj   = K.wj + wid * kFRing;
    int  rd = 0, cnt = 0;  // ring read position and fill (the same in every lane)
    u32  relmax = 0;
    for (int jb = 0; jb < nfull; jb += kThreads * UNROLL) {
        uint4 q[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = jb + u * kThreads + tid;
            if (j < nfull) {
                q[u] = ld_nc_v4(vp + j);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j   = jb + u * kThreads + tid;
            bool      hit = false;
            if (j < nfull) {
                u32 m;
                if (BAND) {
                    m = ((ge2_mask<DT>(q[u].x, thr2) & le2_mask<DT>(q[u].x, hi2))
                         | (ge2_mask<DT>(q[u].y, thr2) & le2_mask<DT>(q[u].y, hi2)))
                        | ((ge2_mask<DT>(q[u].z, thr2) & le2_mask<DT>(q[u].z, hi2))
                           | (ge2_mask<DT>(q[u].w, thr2) & le2_mask<DT>(q[u].w, hi2)));
                }
                else {
                    m = (ge2_mask<DT>(q[u].x, thr2) | ge2_mask<DT>(q[u].y, thr2))
                        | (ge2_mask<DT>(q[u].z, thr2) | ge2_mask<DT>(q[u].w, thr2));
                }
                hit = m != 0;
            }
            const u32 hits = __ballot_sync(0xffffffffu, hit);
            if (hits == 0) {
                continue;
            }
            if (hit) {
                const int at = (rd + cnt + __popc(hits & ((1u << lane) - 1u))) & (kFRing - 1);
                wbuf[at]     = q[u];
                wj[at]       = (unsigned short)j;
            }
            cnt += __popc(hits);
            if (cnt >= 32) {
                __syncwarp();
                const int at = (rd + lane) & (kFRing - 1);
                f_side_step<DT, BAND>(wbuf[at], (int)wj[at], true, head, thr_key, thr2, hi2, K, relmax);
                rd = (rd + 32) & (kFRing - 1);
                cnt -= 32;
                __syncwarp();
            }
        }
    }
    __syncwarp();
    if (cnt > 0) {
        const int  at   = (rd + lane) & (kFRing - 1);
        const bool live = lane < cnt;
        uint4      v    = make_uint4(0u, 0u, 0u, 0u);
        int        jj   = 0;
        if (live) {
            v  = wbuf[at];
            jj = (int)wj[at];
        }
        f_side_step<DT, BAND>(v, jj, live, head, thr_key, thr2, hi2, K, relmax);
    }
    if (!BAND) {
        relmax = __reduce_max_sync(0xffffffffu, relmax);
        if (lane == 0 && relmax != 0) {
            atomicMax(relmax_out, relmax);
        }
    }
}

// The `want`-th largest of the CTA's per-thread sample maxima (ordered 16-bit keys in smax[kThreads]), by
// bisection inside one warp.  With `want` far below the number of threads it is, to within a few ranks, the
// `want`-th largest of all sampled columns - on the low side, which only lets a few more candidates through.
__device__ __forceinline__ u32 f_select_from_maxima(const unsigned short* smax, u32 want, u32* largest)
{
    FTB_ASSUME_SHARED(smax);
    const int lane = threadIdx.x & 31;
    u32       mine[kThreads / 32];
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) {
        mine[i] = smax[i * 32 + lane];
    }
    {
        u32 mx = 0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) {
            mx = mine[i] > mx ? mine[i] : mx;
        }
        *largest = __reduce_max_sync(0xffffffffu, mx);
    }
    u32 lo = 0, hi = 0xffffu;
#pragma unroll 1
    for (int it = 0; it < 16; ++it) {
        const u32 mid = (lo + hi + 1) >> 1;
        u32       c   = 0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) {
            c += mine[i] >= mid ? 1u : 0u;
        }
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= want) {
            lo = mid;
        }
        else {
            hi = mid - 1;
        }
    }
    return lo;
}

// Tie order inside one value class for m <= kThreads members (the rules of resolve_topk_class, by counting
// instead of sorting): member a of lane l = (col / bs1) % 8 has stage-1 rank
//   lane_base[l] + #{b in lane l : t1(b) > t1(a), or t1 equal and col(b) < col(a)},  t1 = col % bs1;
// members whose rank reaches k do not leave stage 1; the others are ordered by ((lane * k + rank) % bs2
// descending, lane * k + rank ascending).  Returns the column at position `want` of that order, -1 when
// there is none.  CTA-collective.
static __device__ int f_resolve_small(const u32* cols, int m, int want, int k, int bs1, int bs2, const u32* lane_base,
                                      u32* key2, int* s_ans)
{
    const int tid = threadIdx.x;
    FTB_ASSUME_SHARED(cols);
    FTB_ASSUME_SHARED(key2);
    if (tid == 0) {
        *s_ans = -1;
    }
    if (tid < m) {
        const u32 c = cols[tid], lane = (c / (u32)bs1) & 7u, t1 = c % (u32)bs1;
        u32       rk = 0;
        for (int b = 0; b < m; ++b) {
            const u32 cb = cols[b], lb = (cb / (u32)bs1) & 7u, tb = cb % (u32)bs1;
            rk += (lb == lane && (tb > t1 || (tb == t1 && cb < c))) ? 1u : 0u;
        }
        const u32 r = lane_base[lane] + rk;
        u32       key = 0xffffffffu;
        if (r < (u32)k) {
            const u32 i2 = lane * (u32)k + r;  // < 8 * 1024
            key          = (((u32)bs2 - 1u - (i2 % (u32)bs2)) << 16) | i2;
        }
        key2[tid] = key;
    }
    __syncthreads();
    if (tid < m) {
        const u32 mine = key2[tid];
        if (mine != 0xffffffffu) {
            int rk = 0;
            for (int b = 0; b < m; ++b) {
                rk += key2[b] < mine ? 1 : 0;
            }
            if (rk == (want < m ? want : m - 1)) {
                *s_ans = (int)cols[tid];
            }
        }
    }
    __syncthreads();
    const int ans = *s_ans;
    __syncthreads();
    return ans;
}

// Header of a row.  It is put together one row ahead by thread 0, in stages spread over the row in front, so
// that none of the dependent loads behind it (ticket -> row number -> per-row arguments and generator state) is
// waited for.
struct FHdr {
    int    t;  // ticket; >= the number of rows when none is left
    int    r, mode, fin, end_id, k;
    float  top_p, u, inv_t, theta;
    __half inv_t_h;
};
// landing zone of the next row's arguments (32-bit words; the two generator states sit on 16-byte boundaries)
constexpr int kFPreWords = 48;
enum { kPreStateK = 0, kPreStateP = 12, kPreSkipK = 24, kPreSkipP, kPreFin, kPreEnd, kPreK, kPrePk, kPrePp, kPreTemp,
       kPreRep };

__device__ __forceinline__ void cp_async16(u32 saddr, const void* g)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}

// Arguments of row nr on their way into pre[] (thread 0 only).
static __device__ void f_prefetch_header(const KParams& P, int nr, u32* pre)
{
    const u32 base = (u32)__cvta_generic_to_shared(pre);
    auto word = [&](int slot, const void* p) {
        cp_async4(base + 4u * (u32)slot, (const void*)((size_t)p & ~(size_t)3));
    };
    if (P.topk_states != nullptr) {
        const char* st = (const char*)(P.topk_states + nr);
        cp_async16(base + 4u * kPreStateK, st);
        cp_async16(base + 4u * kPreStateK + 16u, st + 16);
        cp_async16(base + 4u * kPreStateK + 32u, st + 32);
        word(kPreK, P.topk_ks + nr);
        word(kPrePk, P.topk_ps + nr);
        if (P.topk_skip != nullptr) {
            word(kPreSkipK, P.topk_skip + nr);
        }
    }
    if (P.topp_states != nullptr) {
        const char* st = (const char*)(P.topp_states + nr);
        cp_async16(base + 4u * kPreStateP, st);
        cp_async16(base + 4u * kPreStateP + 16u, st + 16);
        cp_async16(base + 4u * kPreStateP + 32u, st + 32);
        word(kPrePp, P.topp_ps + nr);
        if (P.topp_skip != nullptr) {
            word(kPreSkipP, P.topp_skip + nr);
        }
    }
    if (P.finished != nullptr) {
        word(kPreFin, P.finished + nr);
    }
    word(kPreEnd, P.end_ids + nr);
    if (P.apply_temp) {
        word(kPreTemp, P.temperature + nr);
    }
    if (P.apply_rep) {
        word(kPreRep, P.rep_penalty + nr);
    }
    cp_async_commit();
}

// Header of ticket nt / row nr from what f_prefetch_header brought in (thread 0 only, after its copies landed).
static __device__ void f_compose_header(const KParams& P, int nt, int nr, const u32* pre, FHdr& H)
{
    H.t = nt;
    if (nt >= P.local_batch) {
        return;
    }
    auto byte_at = [&](int slot, const void* p) { return (pre[slot] >> (8 * ((size_t)p & 3))) & 0xffu; };
    int  mode = 0;
    if (P.topk_states != nullptr && !(P.topk_skip != nullptr && byte_at(kPreSkipK, P.topk_skip + nr) != 0)) {
        mode = 1;
    }
    else if (P.topp_states != nullptr && !(P.topp_skip != nullptr && byte_at(kPreSkipP, P.topp_skip + nr) != 0)) {
        mode = 2;
    }
    H.r      = nr;
    H.mode   = mode;
    H.fin    = P.finished != nullptr ? (int)(byte_at(kPreFin, P.finished + nr) != 0) : 0;
    H.end_id = (int)pre[kPreEnd];
    int k    = (int)pre[kPreK];
    H.k      = k < 1 ? 1 : (k > kMaxTopK ? kMaxTopK : k);
    H.top_p  = __uint_as_float(mode == 1 ? pre[kPrePk] : pre[kPrePp]);
    float inv_t = 1.0f;
    if (P.apply_temp) {
        inv_t = 1.0f / (__uint_as_float(pre[kPreTemp]) + 1e-6f);
    }
    H.inv_t   = inv_t;
    H.inv_t_h = __float2half_rn(inv_t);
    H.theta   = P.apply_rep ? __uint_as_float(pre[kPreRep]) : 1.0f;
    H.u       = 0.0f;
    if (mode != 0) {
        // drawn from a copy: the state in memory moves on only when this kernel finishes the row
        curandState_t st = *(const curandState_t*)(pre + (mode == 1 ? kPreStateK : kPreStateP));
        H.u              = curand_uniform(&st);
    }
}

// Geometry of a row.
struct FGeo {
    const char* rowp;
    int         head, nfull;
};
__device__ __forceinline__ FGeo f_geometry(const KParams& P, int r)
{
    FGeo G;
    G.rowp          = (const char*)P.logits + (size_t)r * P.vocab_padded * 2;
    const size_t ad = (size_t)G.rowp;
    const int    hd = (int)(((16 - (ad & 15)) & 15) / 2);
    G.head          = hd < P.vocab_padded ? hd : P.vocab_padded;
    const int vend  = P.vocab < P.vocab_padded ? P.vocab : P.vocab_padded;
    G.nfull         = vend - G.head > 0 ? (vend - G.head) / 8 : 0;
    return G;
}


// ---- top-p rows ------------------------------------------------------------------------------------------
// After the pass a top-p row knows every column at or above the threshold (candidates, class counts, listed
// columns) and with them the row maximum.  What the reference does next, on probabilities
// (kernels/sampling_topp_kernels.cu:1294-1345 soft-max, :801-860 arg-max shortcut, :877-1004 sorted scan):
//   pass 2 (the row again, mostly from L2): the soft-max denominator in the reference's order - thread t owns
//     the "virtual threads" 4t..4t+3 (column mod 1024) and adds four exponentials per 1024-column chunk, strictly
//     in chunk order; special columns take their final value (the per-vector bytes say where they are).  The
//     same pass counts the bit patterns between a provisional cut and the threshold and lists the special
//     columns that fall there, so that the sorted probability sequence is known as (probability, count) runs
//     down to the cut;
//   the block scan of topp_sampling is replayed over the runs (cub::BlockScan<float,256> raking order: 32
//     segments of 8, Kogge-Stone over the segment totals, running prefix chunk by chunk);
//   the class (bit patterns of equal probability) that holds the crossing gives the id: its J-th column in
//     column order, from the candidate list or - below the threshold - from one filtered pass over the row.
// Whatever does not fit (crossing below the cut, tables too small) sends the row to the general kernel.

constexpr int kFMassBins = 128;  // sample mass per 16 bit patterns below the threshold

struct FTopp {
    u32   thr_key, relmax;
    int   n_ord, n_sp;
    float thr_y, neg_max, maxv;
};

template<int DT>
__device__ __forceinline__ float f_round_T(float x)
{
    return DT == FTB200_F16 ? __half2float(__float2half_rn(x)) : x;
}

static __device__ float f_block_sum(float v, float* s_w)
{
    for (int m = 16; m > 0; m >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, m);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
        s_w[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < kWarps; ++i) {
        t += s_w[i];
    }
    return t;
}

// ---- shared memory by 32-bit address (the hot loop of pass 2 keeps no generic pointer) ----
// (not volatile and without a memory clobber: the compiler may move and batch these reads - they are used on
//  tables that nobody writes while the loop around them runs)
__device__ __forceinline__ u32 lds_u8(u32 addr)
{
    u32 v;
    asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// The same under a predicate inside the instruction (no branch around it: a run of these stays one basic block).
__device__ __forceinline__ void reds_inc_if(u32 addr, u32 cond)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %1, 0;\n\t@p red.shared.add.u32 [%0], 1;\n\t}" ::"r"(addr), "r"(cond));
}
// Counter update whose result nobody in the surrounding loop reads: no memory clobber, so the arithmetic of
// neighbouring columns is free to move across it.
__device__ __forceinline__ void reds_add_free(u32 addr, u32 v)
{
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(addr), "r"(v));
}
__device__ __forceinline__ uint2 lds_v2(u32 addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cp_async8(u32 saddr, const void* g)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(saddr), "l"(g) : "memory");
}
template<int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ u32 atoms_add(u32 addr, u32 v)
{
    u32 old;
    asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void sts_u64(u32 addr, u64 v)
{
    asm volatile("st.shared.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ void sts_f32(u32 addr, float v)
{
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// flags of column `id` in the hash at shared address `hash` (0 when it has no entry)
__device__ __forceinline__ u32 f_lookup_saddr(u32 hash, int shift, int mask, int id)
{
    u32 h = hash_slot(id, shift);
    for (int probe = 0; probe <= mask; ++probe) {
        const u32 v = lds_u32(hash + 4u * h);
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

// Scalars of pass 2 (one argument block, by value: it travels in the parameter space of the call).
struct FPass2 {
    const char* rowp;
    int         nch, vocab, shift, mask, apply_rep, penalty_type;
    float       maxv, inv_t, theta, cut_y, thr_y, neg_max;
    u32         thr_key, lo_n;
    u32         emask, hash, hlo, spec, nspec, out;  // shared-memory addresses
    __half      inv_t_h;
};

// Pass 2 of a top-p row over the whole 1024-column chunks [0, nch) and the ragged rest up to `vocab`: thread t
// adds the exponentials of its four "virtual threads" chunk by chunk; with COUNTING the ordinary columns whose bit
// pattern lies in the lo_n patterns below the threshold are counted; special columns take their final value and
// are listed when it falls between the cut and the threshold.  The four sums go to out[4t .. 4t+3].
template<int DT, bool TEMP, bool COUNTING>
__device__ __noinline__ void f_pass2(const FPass2 A)
{
    const int    tid = threadIdx.x;
    const float  maxv = A.maxv, inv_t = A.inv_t;
    const __half inv_t_h = A.inv_t_h;
    const u32    thr_key = A.thr_key, lo_n = A.lo_n, hlo = A.hlo;
    float        a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    // final value of a special column (kernels/sampling_penalty_kernels.cu:367-424, :485-500; a dead one is -inf)
    auto special = [&](float y, u32 fl) {
        if (fl & kFlagDead) {
            return -INFINITY;
        }
        if ((fl & kFlagHist) && A.apply_rep) {
            if (A.penalty_type == FTB200_PENALTY_MULTIPLICATIVE) {
                y = y < 0.0f ? y * A.theta : y / A.theta;
            }
            else if (A.penalty_type == FTB200_PENALTY_ADDITIVE) {
                y = y - A.theta;
            }
            if (DT == FTB200_F16) {
                y = __half2float(__float2half_rn(y));
            }
        }
        return y;
    };
    auto patch = [&](float y, int v) {  // rare: column v is special
        const float yy = special(y, f_lookup_saddr(A.hash, A.shift, A.mask, v));
        if (yy >= A.cut_y && !(yy >= A.thr_y) && yy > A.neg_max) {  // (those at or above the threshold are listed already)
            const u32 pos = atoms_add(A.nspec, 1u);
            if (pos < (u32)kFPSpecCap) {
                sts_u64(A.spec + 8u * pos, ((u64)(~fkey(yy)) << 32) | (u32)v);
            }
        }
        return yy;
    };
    // A batch of UN chunks is worked on in stages, every stage over all 4 * UN columns of the thread: values,
    // final values of the special ones (rare), exponentials, the four running sums in chunk order, counts.  The
    // columns of a stage are independent of one another, so a warp has many instructions to issue between two
    // dependent ones.
    constexpr int UN     = 4;  // (larger batches run slower: the loop body then no longer sits in the instruction cache)
    const char*   base   = A.rowp + (size_t)tid * 8;
    const u32     embase = A.emask + (u32)(tid >> 1);
    const int     nch    = A.nch;
    const int     nib    = 4 * (tid & 1);
    // (threshold and cut both at or above +0: see the counting stage)
    const bool    pos_cut = thr_key - lo_n >= 0x8000u && thr_key > 0x8000u;
    const u32     thr_m1  = (thr_key & 0x7fffu) - 1u;
    for (int m0 = 0; m0 < nch; m0 += UN) {
        uint2 raw[UN];
        u32   em[UN];
        float y[UN][4];
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            const bool in = m0 + uu < nch;
            raw[uu]       = in ? ld_nc_v2(base + (size_t)(m0 + uu) * 2048) : make_uint2(0u, 0u);
            em[uu]        = in ? (lds_u8(embase + (u32)(m0 + uu) * 128u) >> nib) & 0xfu : 0u;
        }
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            y[uu][0] = f_value<DT>(raw[uu].x & 0xffffu, TEMP, inv_t, inv_t_h);
            y[uu][1] = f_value<DT>(raw[uu].x >> 16, TEMP, inv_t, inv_t_h);
            y[uu][2] = f_value<DT>(raw[uu].y & 0xffffu, TEMP, inv_t, inv_t_h);
            y[uu][3] = f_value<DT>(raw[uu].y >> 16, TEMP, inv_t, inv_t_h);
        }
        {
            // Special columns: rare for a thread, but some lane of a warp has one in nearly every batch.  One copy of
            // the code for the whole batch (the column is picked and put back with selects): a copy per column
            // made the loop body several times larger than the instruction cache likes.
            u32 todo = 0;
#pragma unroll
            for (int uu = 0; uu < UN; ++uu) {
                todo |= em[uu] << (4 * uu);
            }
            while (todo != 0) {
                const int j = __ffs(todo) - 1;
                todo &= todo - 1;
                float yv = 0.0f;
#pragma unroll
                for (int a = 0; a < 4 * UN; ++a) {
                    yv = j == a ? y[a >> 2][a & 3] : yv;
                }
                yv = patch(yv, (m0 + (j >> 2)) * 1024 + 4 * tid + (j & 3));
#pragma unroll
                for (int a = 0; a < 4 * UN; ++a) {
                    y[a >> 2][a & 3] = j == a ? yv : y[a >> 2][a & 3];
                }
            }
        }
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            // a column at or below -MAX adds exactly zero, as in the reference's loop; the chunks past the end of
            // the row are left out below
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                y[uu][e] = f_round_T<DT>(__expf(y[uu][e] - maxv));
            }
        }
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
            if (m0 + uu < nch) {
                a0 += y[uu][0], a1 += y[uu][1], a2 += y[uu][2], a3 += y[uu][3];
            }
        }
        if (COUNTING) {
            // Ordinary columns between the cut and the threshold, per bit pattern.  With the cut at or above +0 (the
            // usual case) the index below the threshold is a plain difference of the raw patterns: a negative
            // value, or one at or above the threshold, wraps to a huge index.
            if (pos_cut) {
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    if (m0 + uu < nch) {
                        const u32 i0 = thr_m1 - (raw[uu].x & 0xffffu), i1 = thr_m1 - (raw[uu].x >> 16);
                        const u32 i2 = thr_m1 - (raw[uu].y & 0xffffu), i3 = thr_m1 - (raw[uu].y >> 16);
                        const u32 ok = ~em[uu];
                        reds_inc_if(hlo + 4u * (i0 < lo_n ? i0 : 0u), (i0 < lo_n ? 1u : 0u) & ok);
                        reds_inc_if(hlo + 4u * (i1 < lo_n ? i1 : 0u), (i1 < lo_n ? 2u : 0u) & ok);
                        reds_inc_if(hlo + 4u * (i2 < lo_n ? i2 : 0u), (i2 < lo_n ? 4u : 0u) & ok);
                        reds_inc_if(hlo + 4u * (i3 < lo_n ? i3 : 0u), (i3 < lo_n ? 8u : 0u) & ok);
                    }
                }
            }
            else {
#pragma unroll
                for (int uu = 0; uu < UN; ++uu) {
                    if (m0 + uu < nch) {
                        const u32 i0 = thr_key - 1u - key16(raw[uu].x & 0xffffu), i1 = thr_key - 1u - key16(raw[uu].x >> 16);
                        const u32 i2 = thr_key - 1u - key16(raw[uu].y & 0xffffu), i3 = thr_key - 1u - key16(raw[uu].y >> 16);
                        if (i0 < lo_n && !(em[uu] & 1u)) {
                            reds_add_free(hlo + 4u * i0, 1u);
                        }
                        if (i1 < lo_n && !(em[uu] & 2u)) {
                            reds_add_free(hlo + 4u * i1, 1u);
                        }
                        if (i2 < lo_n && !(em[uu] & 4u)) {
                            reds_add_free(hlo + 4u * i2, 1u);
                        }
                        if (i3 < lo_n && !(em[uu] & 8u)) {
                            reds_add_free(hlo + 4u * i3, 1u);
                        }
                    }
                }
            }
        }
    }
    // the ragged rest of the row: columns nch * 1024 .. vocab - 1 (padding columns add nothing)
    {
        const int v0 = nch * 1024 + 4 * tid;
        if (v0 < A.vocab) {
            const unsigned short* row16 = (const unsigned short*)A.rowp;
            for (int e = 0; e < 4 && v0 + e < A.vocab; ++e) {
                const u32 r  = (u32)__ldg(row16 + v0 + e);
                const u32 fl = f_lookup_saddr(A.hash, A.shift, A.mask, v0 + e);
                float     yy = f_value<DT>(r, TEMP, inv_t, inv_t_h);
                if (fl != 0) {
                    yy = patch(yy, v0 + e);
                }
                const float ex = f_round_T<DT>(__expf(yy - maxv));
                a0 += e == 0 ? ex : 0.0f, a1 += e == 1 ? ex : 0.0f, a2 += e == 2 ? ex : 0.0f, a3 += e == 3 ? ex : 0.0f;
                if (COUNTING && fl == 0) {
                    const u32 i0 = thr_key - 1u - key16(r);
                    if (i0 < lo_n) {
                        reds_add_free(hlo + 4u * i0, 1u);
                    }
                }
            }
        }
    }
    sts_f32(A.out + 16u * (u32)tid, a0);
    sts_f32(A.out + 16u * (u32)tid + 4u, a1);
    sts_f32(A.out + 16u * (u32)tid + 8u, a2);
    sts_f32(A.out + 16u * (u32)tid + 12u, a3);
}

// Everything of a top-p row after the pass and the listed columns.  Returns true when the row is done.
template<int DT>
__device__ __forceinline__ bool fast_topp_tail(const KParams& P, const FMap& S, const FHdr& H, const FGeo& G, const FTopp T, u64* spec,
                               u32* s_nspec, const u32* s_mass, float mass_tail, u32 smax_key, u64* trace)
{
    __shared__ float s_w[kWarps], s_den, s_R;
    __shared__ u32   s_cut, s_wsum[kWarps], s_ncls, s_fail;
    __shared__ int   s_c1, s_sel, s_imin, s_imax, s_first;
    const int        tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const bool       temp = P.apply_temp != 0;
    u32* const       hist = S.hist;
    u32* const       hlo  = S.sval;
    u32* const       cand = S.cand;
    FTB_ASSUME_SHARED(hist);
    FTB_ASSUME_SHARED(hlo);
    FTB_ASSUME_SHARED(cand);
    FTB_ASSUME_SHARED(spec);
    const u32   thr_key = T.thr_key;
    const float maxv = T.maxv, neg_max = T.neg_max;
    const int   nfull = G.nfull;
    auto value_of = [&](u32 key) { return f_value<DT>(key16_inv(key), temp, H.inv_t, H.inv_t_h); };

    // ---- provisional cut: how far below the threshold the bit patterns have to be counted ----
    // Mass (sum of exp(value - maximum)) at or above the threshold is known exactly; below it the sampled columns
    // give an estimate per 16 bit patterns.  The cut is placed where the estimated cumulative share passes
    // 1.02 u p + 0.05: the part above the threshold is exact and the sampled part (3 % of the row, values under the
    // threshold only, so without the heavy tail of the exponentials) is within about 1.5 % of the total; a cut
    // that proves too high costs the row a trip through the general kernel, a low one more counting.
    float mhi = 0.0f;
    for (int b = tid; b <= (int)T.relmax; b += kThreads) {
        const u32 c = hist[b];
        if (c != 0) {
            mhi += (float)c * __expf(value_of(thr_key + (u32)b) - maxv);
        }
    }
    for (int i = tid; i < T.n_sp; i += kThreads) {
        mhi += __expf(fkey_inv(~(u32)(spec[i] >> 32)) - maxv);
    }
    mhi = f_block_sum(mhi, s_w);
    if (wid == 0) {
        // (warp 0: four mass bins per lane, a scan over the lanes; the sums are estimates, their order is free)
        static_assert(kFMassBins == 128, "four bins per lane");
        const float scale = __expf(value_of(smax_key) - maxv) * ((float)(nfull * 8) / (float)(kThreads * 8));
        float       mb[4], mine = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            mb[i] = (float)s_mass[lane * 4 + i] * (1.0f / 1048576.0f);
            mine += mb[i];
        }
        float incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            incl += lane >= o ? t : 0.0f;
        }
        const float lo_all = mass_tail + __shfl_sync(0xffffffffu, incl, 31);
        const float d_est  = mhi + scale * lo_all;
        const float share  = 1.02f * H.u * H.top_p + 0.05f;
        const float target = share * d_est;
        // first bin at which the running mass reaches the target (128: none)
        float acc   = mhi + scale * (incl - mine);
        int   first = kFMassBins;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc += scale * mb[i];
            if (acc >= target && first == kFMassBins) {
                first = lane * 4 + i;
            }
        }
        const u32 hit = __ballot_sync(0xffffffffu, first < kFMassBins);
        const int b   = hit != 0 ? __shfl_sync(0xffffffffu, first, __ffs(hit) - 1) : kFMassBins;
        if (lane == 0) {
            u32 cut = thr_key;
            if (mhi < target) {
                const u32 down = 16u * (u32)(b + 2);
                cut            = thr_key > down ? thr_key - down : 1u;
                if (thr_key - cut > (u32)kFBins) {
                    cut = thr_key - (u32)kFBins;
                }
            }
            s_cut  = cut;
            s_fail = 0;
        }
    }
    for (int i = tid; i < kFBins; i += kThreads) {
        hlo[i] = 0;  // (the raw values of the special columns are done with: the listed ones carry their final value)
    }
    __syncthreads();
    const u32   cut_key = s_cut;
    const float cut_y   = cut_key < thr_key ? value_of(cut_key) : T.thr_y;
    trace_mark(trace, 6);

    // ---- pass 2 ----
    float* const s_vt = (float*)S.wbuf;  // [1024] per-virtual-thread sums (the ring of the pass is idle)
    FTB_ASSUME_SHARED(s_vt);
    {
        FPass2 A;
        A.rowp = G.rowp, A.nch = P.vocab / 1024, A.vocab = P.vocab, A.shift = P.hash_shift, A.mask = P.hash_slots - 1;
        A.apply_rep = P.apply_rep, A.penalty_type = P.penalty_type;
        A.maxv = maxv, A.inv_t = H.inv_t, A.theta = H.theta, A.cut_y = cut_y, A.thr_y = T.thr_y, A.neg_max = neg_max;
        A.thr_key = thr_key, A.lo_n = thr_key - cut_key, A.inv_t_h = H.inv_t_h;
        A.emask = (u32)__cvta_generic_to_shared(S.emask), A.hash = (u32)__cvta_generic_to_shared(S.hash);
        A.hlo = (u32)__cvta_generic_to_shared(hlo), A.spec = (u32)__cvta_generic_to_shared(spec);
        A.nspec = (u32)__cvta_generic_to_shared(s_nspec), A.out = (u32)__cvta_generic_to_shared(s_vt);
        // (the common case without temperature comes in two forms: with and without the per-pattern count)
        if (temp) {
            f_pass2<DT, true, true>(A);
        }
        else if (cut_key < thr_key) {
            f_pass2<DT, false, true>(A);
        }
        else {
            f_pass2<DT, false, false>(A);
        }
    }
    __syncthreads();
    trace_mark(trace, 7);
    {
        // the reference's blockReduceSum (utils/reduce_kernel_utils.cuh:73-103) over the 1024 partial sums: a
        // butterfly inside every group of 32, then one over the 32 group results
        float* const s_vw = s_vt + 1024;  // [32] (the ring area holds 8 KB)
        for (int w = wid; w < 32; w += kWarps) {
            float v = s_vt[w * 32 + lane];
            for (int m = 16; m > 0; m >>= 1) {
                v = v + __shfl_xor_sync(0xffffffffu, v, m);
            }
            if (lane == 0) {
                s_vw[w] = v;
            }
        }
        __syncthreads();
        if (wid == 0) {
            float v = s_vw[lane];
            for (int m = 16; m > 0; m >>= 1) {
                v = v + __shfl_xor_sync(0xffffffffu, v, m);
            }
            if (lane == 0) {
                s_den = v;
            }
        }
    }
    __syncthreads();
    const float denom = s_den + 1e-6f;
    if (!(denom > 0.0f && denom < 3.0e38f)) {
        return false;  // (not a number, or out of range: nothing below may index with what would follow from it)
    }
    auto prob_of = [&](float y) { return f_round_T<DT>(f_round_T<DT>(__expf(y - maxv)) / denom); };
    const size_t col = (size_t)P.ite * P.local_batch + H.r;
    int* const   id_out = P.output_ids + (size_t)P.step * P.batch_size + col;
    const int    n_sp   = (int)*s_nspec;
    if (n_sp > kFPSpecCap) {
        return false;
    }

    // ---- arg-max shortcut of topp_beam_topk_kernel: the largest probability alone reaches p ----
    const float p_max = f_round_T<DT>(f_round_T<DT>(1.0f) / denom);
    if (p_max >= H.top_p) {
        // first column holding the maximum (larger value, then smaller column)
        if (tid == 0) {
            s_sel = 0x7fffffff;
        }
        __syncthreads();
        const u32 kmaxv = fkey(maxv);
        for (int i = tid; i < T.n_ord; i += kThreads) {
            const u32 e = cand[i];
            if ((e >> 20) == T.relmax && fkey(value_of(thr_key + (e >> 20))) == kmaxv) {
                atomicMin(&s_sel, (int)(e & 0xfffffu));
            }
        }
        for (int i = tid; i < n_sp; i += kThreads) {
            if (~(u32)(spec[i] >> 32) == kmaxv) {
                atomicMin(&s_sel, (int)(spec[i] & 0xffffffffu));
            }
        }
        __syncthreads();
        const int id = s_sel;
        if (id == 0x7fffffff) {
            return false;
        }
        if (tid == 0) {
            *id_out = id;
            if (P.seq_len != nullptr && P.finished != nullptr) {
                P.seq_len[H.r]  = P.seq_len[H.r] + 1;
                P.finished[H.r] = id == H.end_id ? 1 : 0;
            }
        }
        return true;
    }
    const float rand_num = H.u * H.top_p;

    // ---- runs: the counted bit patterns in descending value with the listed columns merged in by probability ----
    // pattern u of the window: key ktop - u, counted in hist (at or above the threshold) or hlo (below it)
    const u32 ktop = thr_key + T.relmax;
    const int npat = (int)(ktop - cut_key) + 1;
    if (npat > 16 * kThreads) {
        return false;
    }
    auto count_of = [&](int u) {
        const u32 key = ktop - (u32)u;
        return u >= npat ? 0u : (key >= thr_key ? hist[key - thr_key] : hlo[thr_key - 1u - key]);
    };
    // listed columns: value keys -> probability keys, sorted (probability descending, column ascending)
    for (int i = tid; i < n_sp; i += kThreads) {
        const u64 e = spec[i];
        spec[i]     = ((u64)(~fkey(prob_of(fkey_inv(~(u32)(e >> 32))))) << 32) | (e & 0xffffffffu);
    }
    __syncthreads();
    group_sort_u64<CtaSync, true>(spec, n_sp, tid, kThreads, CtaSync());
    __syncthreads();
    u32* const run_pr = S.emask;            // [kFPRuns] probability of the run (float bits), descending
    u32* const run_st = run_pr + kFPRuns;   // [kFPRuns] length, then first position of the run
    FTB_ASSUME_SHARED(run_pr);
    FTB_ASSUME_SHARED(run_st);
    constexpr int PER = 16;
    for (int i = tid; i < kFPRuns; i += kThreads) {
        run_st[i] = 0u;  // a position no pattern takes keeps length 0 and goes to a listed column
    }
    __syncthreads();
    int nA;
    {
        u32 cnt[PER], mine = 0;
        for (int i = 0; i < PER; ++i) {
            cnt[i] = count_of(tid * PER + i);
            mine += cnt[i] != 0 ? 1u : 0u;
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
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
        if (nA + n_sp > kFPRuns) {
            return false;
        }
        u32 at = base + incl - mine;
        for (int i = 0; i < PER; ++i) {
            if (cnt[i] != 0) {
                const float pr = prob_of(value_of(ktop - (u32)(tid * PER + i)));
                const u32   kp = ~fkey(pr);  // ascending in this key = descending probability
                int         lo = 0, hi = n_sp;  // listed columns with a strictly larger probability
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
    // both lists keep their order in the merged sequence: the listed columns fill the positions the patterns left
    // free, in order
    const int M = nA + n_sp;
    {
        constexpr int RPT = kFPRuns / kThreads;
        u32           freem = 0, mine = 0;
        for (int i = 0; i < RPT; ++i) {
            const int q = tid * RPT + i;
            if (q < M && run_st[q] == 0u) {
                freem |= 1u << i;
                ++mine;
            }
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
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
                const int q = tid * RPT + i;
                run_pr[q]   = __float_as_uint(fkey_inv(~(u32)(spec[j] >> 32)));
                run_st[q]   = 1u;
                ++j;
            }
        }
    }
    __syncthreads();
    // the exponential has to be monotone over the patterns for the order of the runs to be the sorted order
    for (int i = tid; i + 1 < M; i += kThreads) {
        if (__uint_as_float(run_pr[i]) < __uint_as_float(run_pr[i + 1])) {
            s_fail = 1;
        }
    }
    __syncthreads();
    if (s_fail) {
        return false;
    }
    // exclusive scan of the run lengths -> first position of each run
    u32 N;
    {
        constexpr int RPT = kFPRuns / kThreads;
        u32           c[RPT], mine = 0;
        for (int i = 0; i < RPT; ++i) {
            const int q = tid * RPT + i;
            c[i]        = q < M ? run_st[q] : 0u;
            mine += c[i];
        }
        u32 incl = mine;
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
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
            const int q = tid * RPT + i;
            if (q < M) {
                run_st[q] = at;
                at += c[i];
            }
        }
    }
    __syncthreads();
    trace_mark(trace, 8);
    if (trace != nullptr && tid == 0) {
        trace[4 + 20] = (u64)(thr_key - cut_key);
        trace[4 + 21] = (u64)N;
        trace[4 + 22] = (u64)T.n_ord;
    }
    const int nch = (int)((N + 255u) / 256u);
    if (nch > 1000 || N == 0) {
        return false;
    }
    auto run_of = [&](u32 p) {  // run that holds position p
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
    // run at the first position of every 256-entry chunk, and the chunk aggregates (the pattern counts below the
    // threshold are done with: both live where they were)
    int* const   run_at = (int*)hlo;              // [nch + 1]
    float* const agg    = (float*)(hlo + 1008);   // [nch]
    FTB_ASSUME_SHARED(run_at);
    FTB_ASSUME_SHARED(agg);
    for (int c = tid; c <= nch; c += kThreads) {
        run_at[c] = c < nch ? run_of((u32)c * 256u) : M - 1;
    }
    __syncthreads();
    auto load8 = [&](int c, float* x) {  // the 8 consecutive probabilities of this lane in chunk c
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
    // aggregate of every 256-value chunk in cub::BlockScan's raking order (32 segments of 8, Kogge-Stone across
    // the segment totals); the chunks are independent of the running prefix
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
            const float t = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) {
                inc = inc + t;
            }
        }
        if (lane == 31) {
            agg[c] = inc;
        }
    }
    __syncthreads();
    // running prefix chunk by chunk, as the reference's prefix functor accumulates it; stop a little early
    // (partial sums inside a chunk differ from prefix + aggregate only in the last bits)
    if (tid == 0) {
        float       R    = 0.0f;
        int         c1   = nch;
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
        return false;  // the draw lies beyond the counted range
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
                const float t = __shfl_up_sync(0xffffffffu, inc, off);
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
                if ((u32)(c * 256 + g * 32 + 31) >= N) {
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
    trace_mark(trace, 9);
    if (sel < 0 || (u32)sel >= N) {
        return false;
    }
    // ---- the class of the crossing: every column whose probability equals that of position sel ----
    const int   i_at  = run_of((u32)sel);
    const float p_sel = __uint_as_float(run_pr[i_at]);
    const u32   k_sel = fkey(p_sel);
    if (tid == 0) {
        s_ncls = 0;
        s_imin = 0x7fffffff;
        s_imax = -1;
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
        s_first = (int)run_st[lo];
    }
    __syncthreads();
    // bit patterns that map to this probability (one pattern past the counted range is looked at too: a class
    // that reaches down to the cut may go on below it)
    for (int i = 0; i < PER + 1; ++i) {
        const int u = tid * (PER + 1) + i;
        if (u <= npat && ktop >= (u32)u) {
            if (fkey(prob_of(value_of(ktop - (u32)u))) == k_sel) {
                atomicMin(&s_imin, u);
                atomicMax(&s_imax, u);
            }
        }
    }
    __syncthreads();
    const int J = sel - s_first;
    if (s_imax >= npat) {
        return false;
    }
    u32* const cls = S.emask;  // [kFPClsCap] columns of the class (the runs are done with)
    FTB_ASSUME_SHARED(cls);
    const int imin = s_imin, imax = s_imax;
    __syncthreads();
    // listed columns of the class
    for (int j = tid; j < n_sp; j += kThreads) {
        if ((u32)(spec[j] >> 32) == ~k_sel) {
            const u32 pos = atomicAdd(&s_ncls, 1u);
            if (pos < (u32)kFPClsCap) {
                cls[pos] = (u32)(spec[j] & 0xffffffffu);
            }
        }
    }
    if (imax >= 0) {
        const u32 k_hi = ktop - (u32)imin, k_lo = ktop - (u32)imax;
        if (k_lo >= thr_key) {
            // the class lies at or above the threshold: its ordinary columns are candidates
            for (int i = tid; i < T.n_ord; i += kThreads) {
                const u32 e = cand[i], key = thr_key + (e >> 20);
                if (key >= k_lo && key <= k_hi) {
                    const u32 pos = atomicAdd(&s_ncls, 1u);
                    if (pos < (u32)kFPClsCap) {
                        cls[pos] = e & 0xfffffu;
                    }
                }
            }
        }
        else {
            // below the threshold: one filtered pass over the row lists the ordinary columns of the band
            __syncthreads();
            __shared__ FSink s_band;
            if (tid == 0) {
                FSink& K = s_band;
                K.cand = cls, K.hist = S.hist, K.sval = S.sval, K.hash = S.hash, K.emask = (const unsigned char*)S.cand;
                K.ncand = &s_ncls, K.bad = &s_fail, K.shift = P.hash_shift, K.mask = P.hash_slots - 1, K.cap = kFPClsCap;
                K.wbuf = S.wbuf, K.wj = S.wj;
            }
            __syncthreads();
            f_stream<DT, true, kFUnroll>((const uint4*)(G.rowp + (size_t)G.head * 2), nfull, G.head, k_lo, k_hi, s_band, &s_fail);
            // row edges
            const int tail0 = G.head + nfull * 8;
            const int nedge = G.head + (P.vocab - tail0 > 0 ? P.vocab - tail0 : 0);
            for (int i = tid; i < nedge; i += kThreads) {
                const int v = i < G.head ? i : tail0 + (i - G.head);
                if (v < P.vocab && hash_lookup_raw(S.hash, P.hash_shift, P.hash_slots - 1, v) == 0) {
                    const u32 key = key16((u32)__ldg((const unsigned short*)G.rowp + v));
                    if (key >= k_lo && key <= k_hi) {
                        const u32 pos = atomicAdd(&s_ncls, 1u);
                        if (pos < (u32)kFPClsCap) {
                            cls[pos] = (u32)v;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    trace_mark(trace, 10);
    const int ncls = (int)s_ncls;
    if (ncls > kFPClsCap || J < 0 || J >= ncls) {
        return false;
    }
    // J-th smallest column of the class (the reference's stable sort leaves equal probabilities in column order)
    if (tid == 0) {
        s_sel = -1;
    }
    __syncthreads();
    for (int a = tid; a < ncls; a += kThreads) {
        const u32 ca = cls[a];
        int       rk = 0;
        for (int b = 0; b < ncls; ++b) {
            rk += cls[b] < ca ? 1 : 0;
        }
        if (rk == J) {
            s_sel = (int)ca;
        }
    }
    __syncthreads();
    const int id = s_sel;
    if (id < 0) {
        return false;
    }
    if (tid == 0) {
        *id_out = id;
        if (P.seq_len != nullptr && P.finished != nullptr) {
            P.seq_len[H.r]  = P.seq_len[H.r] + 1;
            P.finished[H.r] = id == H.end_id ? 1 : 0;
        }
    }
    return true;
}

// One row of the top-k layer (TOPP: of the top-p layer, up to the point where the two part).  Returns true when
// the row is done, false when it has to go to the list
// (nothing of the row's state has been touched then).  CTA-collective.  `stage1` / `stage2` are the hooks
// of the next row's header (run by thread 0 at points where the loads of the previous stage have had time
// to land).
// VP: the row of a vocabulary-parallel local pass (top-k rows only).  The logits are one column shard of the
// vocabulary: token ids become columns by subtracting P.vocab_offset, and instead of drawing the row hands every
// column whose value reaches the shard's k-th value (whole tie class) to the exchange record, as topk_tail does.
template<int DT, bool TOPP, int VP, class S1, class S2>
__device__ __forceinline__ bool fast_row(const KParams& P, const FMap& S, const FHdr& H, u64* trace, S1&& stage1, S2&& stage2)
{
    static_assert(!(TOPP && VP), "the record form serves top-k rows");
    const int id_shift = VP ? P.vocab_offset : 0;
    __shared__ u32   s_mass[kFMassBins];  // sample mass per bin, in units of 2^-20 (integer adds are native)
    __shared__ float s_mtail[kWarps];
    __shared__ u32   s_smaxkey, s_vmaxkey;
    __shared__ FSink s_sink;
    __shared__ u32            s_ncand, s_nspec, s_bad, s_ncls, s_lane_base[8], s_thr, s_relmax;
    __shared__ unsigned short s_smax[kThreads];
    __shared__ int            s_pick_idx, s_ans, s_nruns;
    __shared__ float          s_vsel;
    const int                 tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const bool                temp = P.apply_temp != 0;
    u32* const                hash = S.hash;
    u32* const                sval = S.sval;
    u32* const                hist = S.hist;
    u32* const                cand = S.cand;
    FTB_ASSUME_SHARED(hash);
    FTB_ASSUME_SHARED(sval);
    FTB_ASSUME_SHARED(hist);
    FTB_ASSUME_SHARED(cand);
    const int    r     = H.r;
    const FGeo   G     = f_geometry(P, r);
    const uint4* vp    = (const uint4*)(G.rowp + (size_t)G.head * 2);
    const int    nfull = G.nfull;
    const size_t col   = (size_t)P.ite * P.local_batch + r;

    // ---- everything the row's set-up needs is sent for at once: the sampled columns into registers, the
    //      token history, the word list and the last three tokens into shared memory (asynchronous copies) ----
    // sample: 16 blocks of 512 contiguous bytes spread over the row (one per warp and round), 4096 columns
    uint4 smp[kFSampleV];
#pragma unroll
    for (int v = 0; v < kFSampleV; ++v) {
        const int blk   = v * kWarps + wid;
        const int start = (int)(((long long)blk * (nfull - 32)) / (kFSampleV * kWarps - 1)) & ~31;
        smp[v]          = ld_nc_v4(vp + start + lane);
    }
    int* const stage_ids   = (int*)S.stage;                 // [kFMaxHist] history ids (-1: position not counted)
    int* const stage_words = stage_ids + kFMaxHist;         // [2 * kFMaxWords] the row's word list
    int* const stage_last  = stage_words + 2 * kFMaxWords;  // [3] tokens of steps step-3 .. step-1
    FTB_ASSUME_SHARED(stage_ids);
    FTB_ASSUME_SHARED(stage_words);
    FTB_ASSUME_SHARED(stage_last);
    const int  L     = P.bad_words != nullptr ? P.bad_words_len : 0;
    const int* wbase = L > 0 ? (P.bad_words_shared ? P.bad_words : P.bad_words + (size_t)r * 2 * L) : nullptr;
    const int  nhist = P.apply_rep ? P.step : 0;
    {
        // (input_lengths is read here, one dependent load: it is the same few cache lines for every row)
        const int input_len = P.apply_rep ? (P.input_lengths != nullptr ? P.input_lengths[r] : P.max_input_len) : 0;
        for (int t = tid; t < nhist && t < kFMaxHist; t += kThreads) {
            if (t >= input_len && t < P.max_input_len) {
                stage_ids[t] = -1;
            }
            else {
                cp_async4((u32)__cvta_generic_to_shared(&stage_ids[t]), P.output_ids + (size_t)t * P.batch_size + col);
            }
        }
        for (int i = tid; i < 2 * L; i += kThreads) {
            cp_async4((u32)__cvta_generic_to_shared(&stage_words[i]), wbase + i);
        }
        if (tid < 3 && P.step - 3 + tid >= 0) {
            cp_async4((u32)__cvta_generic_to_shared(&stage_last[tid]),
                      P.output_ids + (size_t)(P.step - 3 + tid) * P.batch_size + col);
        }
        cp_async_commit();
    }
    u32* const emask32 = S.emask;
    FTB_ASSUME_SHARED(emask32);
    for (int i = tid; i < P.hash_slots; i += kThreads) {
        hash[i] = kHashEmpty;
        sval[i] = 0xffffffffu;  // no raw value seen: the column lies below the threshold
    }
    for (int i = tid; i < kFBins; i += kThreads) {
        hist[i] = 0;
    }
    for (int i = tid; i < (nfull + 3) / 4; i += kThreads) {
        emask32[i] = 0;
    }
    if (tid < 8) {
        s_lane_base[tid] = 0;
    }
    if (tid == 0) {
        s_ncand = 0, s_nspec = 0, s_bad = 0, s_ncls = 0, s_relmax = 0, s_vmaxkey = 0;
        FSink& K = s_sink;
        K.cand = cand, K.hist = hist, K.sval = sval, K.hash = hash, K.emask = (const unsigned char*)S.emask;
        K.ncand = &s_ncand, K.bad = &s_bad, K.shift = P.hash_shift, K.mask = P.hash_slots - 1, K.cap = kFCap;
        K.wbuf = S.wbuf, K.wj = S.wj;
    }
    if (TOPP && tid < kFMassBins) {
        s_mass[tid] = 0u;
    }
    {
        // largest sampled column of this thread, as an ordered key
        u32 m2 = max2<DT>(max2<DT>(smp[0].x, smp[0].y), max2<DT>(smp[0].z, smp[0].w));
#pragma unroll
        for (int v = 1; v < kFSampleV; ++v) {
            m2 = max2<DT>(m2, max2<DT>(max2<DT>(smp[v].x, smp[v].y), max2<DT>(smp[v].z, smp[v].w)));
        }
        const u32 ka = key16(m2 & 0xffffu), kb = key16(m2 >> 16);
        s_smax[tid]  = (unsigned short)(ka > kb ? ka : kb);
    }
    cp_async_wait_all();  // history, word list and last tokens have landed
    __syncthreads();
    stage1();
    trace_mark(trace, 0);

    // ---- threshold from the sample (warp 0) while the other warps file the special columns: token history,
    //      banned words, min-length mask (the rules of build_row; kernels/sampling_penalty_kernels.cu:385-410,
    //      :493-499, kernels/ban_bad_words.cu:35-85) ----
    const int k      = H.k;
    const int ncols  = nfull * 8;
    // columns the threshold should let through: 2k, at least k + 256 (the estimate from a few sampled maxima
    // scatters widely); for k = 1 a handful is enough
    // (a top-p row of a smaller vocabulary aims lower: the estimate needs the wanted rank well inside the 256
    //  per-thread maxima of the sample, want_s <= 96 below)
    const int tp_cap = (int)(((long long)ncols * 96) / (kFSampleV * kThreads * 8));
    const int target = TOPP ? (tp_cap < 2048 ? tp_cap : 2048) : (k == 1 ? 64 : (2 * k > k + 256 ? 2 * k : k + 256));
    u32       want_s = (u32)(((long long)target * (kFSampleV * kThreads * 8) + ncols - 1) / ncols);
    want_s           = want_s < 3u ? 3u : want_s;
    bool words_ok    = true;
    if (wid == 0) {
        u32       kmx = 0;
        const u32 t   = f_select_from_maxima(s_smax, want_s, &kmx);
        if (lane == 0) {
            s_thr     = t;
            s_smaxkey = kmx;
        }
    }
    else {
        const int wt = tid - 32, wn = kThreads - 32;
        for (int t = wt; t < nhist && t < kFMaxHist; t += wn) {
            const int id = stage_ids[t];
            if (id >= 0) {
                f_hash_insert(hash, P.hash_slots, P.hash_shift, id - id_shift, kFlagHist, P.vocab_padded);
            }
        }
        for (int i = wt; i < L; i += wn) {
            const int e1 = stage_words[L + i];
            if (e1 < 0) {
                continue;
            }
            const int s1 = i > 0 ? stage_words[L + i - 1] : 0, size = e1 - s1;
            if (size > 4) {
                words_ok = false;  // longer words: the general kernel's loop
                continue;
            }
            bool b = size == 1;
            if (size > 1 && P.step >= size - 1) {
                b = true;
                for (int j = 0; j < size - 1; ++j) {
                    // generated token of step (step - (size - 1) + j)
                    b = b && stage_last[3 - (size - 1) + j] == stage_words[s1 + j];
                }
            }
            if (b) {
                const int tok = stage_words[e1 - 1];
                if (0 < tok && (VP || tok < P.vocab_padded)) {
                    f_hash_insert(hash, P.hash_slots, P.hash_shift, tok - id_shift, kFlagDead, P.vocab_padded);
                }
            }
        }
        if (P.apply_minlen && wt == 0) {
            if (P.seq_len[r] + 1 - P.max_input_len < P.min_lengths[r]) {
                f_hash_insert(hash, P.hash_slots, P.hash_shift, H.end_id - id_shift, kFlagDead, P.vocab_padded);
            }
        }
    }
    const bool long_words = __syncthreads_or(!words_ok);
    // a history of more than kFMaxHist ids comes through the staging area a tile at a time
    for (int base = kFMaxHist; base < nhist; base += kFMaxHist) {
        const int input_len = P.input_lengths != nullptr ? P.input_lengths[r] : P.max_input_len;
        for (int t = base + tid; t < nhist && t < base + kFMaxHist; t += kThreads) {
            if (t >= input_len && t < P.max_input_len) {
                stage_ids[t - base] = -1;
            }
            else {
                cp_async4((u32)__cvta_generic_to_shared(&stage_ids[t - base]), P.output_ids + (size_t)t * P.batch_size + col);
            }
        }
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();
        for (int t = base + tid; t < nhist && t < base + kFMaxHist; t += kThreads) {
            const int id = stage_ids[t - base];
            if (id >= 0) {
                f_hash_insert(hash, P.hash_slots, P.hash_shift, id - id_shift, kFlagHist, P.vocab_padded);
            }
        }
        __syncthreads();
    }
    stage2();
    // per-vector byte: which columns of the vector are special
    for (int i = tid; i < P.hash_slots; i += kThreads) {
        const u32 w = hash[i];
        if (w != kHashEmpty) {
            const int rel = (int)(w >> 2) - G.head;
            if (rel >= 0 && (rel >> 3) < nfull) {
                smem_or(&emask32[rel >> 5], (1u << (rel & 7)) << (8 * ((rel >> 3) & 3)));
            }
        }
    }
    const u32   thr_key = s_thr;
    const u32   thr_raw = key16_inv(thr_key);
    const float thr_y   = f_value<DT>(thr_raw, temp, H.inv_t, H.inv_t_h);
    const float neg_max = DT == FTB200_F16 ? -65504.0f : -FLT_MAX;
    if (TOPP) {
        // mass of the sampled columns below the threshold, per 16 bit patterns, relative to the largest sampled value
        // (the provisional cut of the second pass is placed with it)
        const float v_ref = f_value<DT>(key16_inv(s_smaxkey), temp, H.inv_t, H.inv_t_h);
        float       far   = 0.0f;
        {
            constexpr int v = 0;  // (half the sample is plenty here; the scale below accounts for it)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const u32 raw = raw_bits<DT>(smp[v], e);
                const u32 kk  = key16(raw);
                if (kk < thr_key && (raw & 0x7fffu) <= (DT == FTB200_F16 ? 0x7c00u : 0x7f80u)) {
                    const float w = __expf(f_value<DT>(raw, temp, H.inv_t, H.inv_t_h) - v_ref);
                    const u32   b = (thr_key - 1u - kk) >> 4;
                    if (b < (u32)kFMassBins) {
                        smem_add(&s_mass[b], (u32)(w * 1048576.0f));
                    }
                    else {
                        far += w;
                    }
                }
            }
        }
        for (int m = 16; m > 0; m >>= 1) {
            far += __shfl_xor_sync(0xffffffffu, far, m);
        }
        if (lane == 0) {
            s_mtail[wid] = far;
        }
    }
    __syncthreads();
    trace_mark(trace, 1);
    if (long_words || want_s > 96u || !(thr_y > neg_max) || thr_key == 0u) {
        return false;  // (uniform for the CTA)
    }

    // ---- the pass ----
    f_stream<DT, false, kFUnroll>(vp, nfull, G.head, thr_key, 0u, s_sink, &s_relmax);
    __syncthreads();
    trace_mark(trace, 2);
    trace_mark(trace, 3);
    trace_mark(trace, 4);
    // ---- listed columns: special ones with their final value, and the row's edges ----
    // (~key(value) << 32) | column.  Top-k rows: [kFSpecCap] where the per-vector bytes were (they are done with);
    // top-p rows: [kFPSpecCap] where the row's set-up data was (the bytes are needed once more)
    u64* const    spec     = TOPP ? (u64*)S.stage : (u64*)S.emask;
    constexpr int spec_cap = TOPP ? kFPSpecCap : kFSpecCap;
    FTB_ASSUME_SHARED(spec);
    {
        Xf X;
        X.bias = nullptr, X.inv_t = H.inv_t, X.theta = H.theta, X.neg_max = neg_max, X.inv_t_h = H.inv_t_h;
        X.apply_temp = P.apply_temp, X.apply_rep = P.apply_rep, X.penalty_type = P.penalty_type, X.vocab = P.vocab;
        X.hash_shift = P.hash_shift, X.hash_mask = P.hash_slots - 1, X.hash = hash;
        auto push = [&](int c, float y) {
            if (y >= thr_y && y > neg_max) {
                const u32 pos = atomicAdd(&s_nspec, 1u);
                if (pos < (u32)spec_cap) {
                    spec[pos] = ((u64)(~fkey(y)) << 32) | (u32)c;
                }
                if (TOPP) {
                    atomicMax(&s_vmaxkey, fkey(y));
                }
            }
        };
        for (int i = tid; i < P.hash_slots; i += kThreads) {
            const u32 w = hash[i];
            if (w == kHashEmpty) {
                continue;
            }
            const int id = (int)(w >> 2);
            if (id >= P.vocab) {
                continue;
            }
            const int rel = id - G.head;
            const u32 raw = (rel >= 0 && (rel >> 3) < nfull) ? sval[i] : (u32)__ldg((const unsigned short*)G.rowp + id);
            if (raw == 0xffffffffu) {
                continue;  // below the threshold before its penalty, and a penalty only lowers a value here
            }
            push(id, special_value<DT>(X, temp_value<DT>(X, raw, id), w & 3u));
        }
        const int tail0 = G.head + nfull * 8;
        const int nedge = G.head + (P.vocab - tail0 > 0 ? P.vocab - tail0 : 0);
        for (int i = tid; i < nedge; i += kThreads) {
            const int v = i < G.head ? i : tail0 + (i - G.head);
            if (v < P.vocab && hash_lookup_raw(hash, X.hash_shift, X.hash_mask, v) == 0) {
                push(v, temp_value<DT>(X, (u32)__ldg((const unsigned short*)G.rowp + v), v));
            }
        }
    }
    __syncthreads();
    trace_mark(trace, 5);
    const int n_ord = (int)s_ncand, n_sp = (int)s_nspec;
    if (s_bad || n_ord > kFCap || n_sp > spec_cap || n_ord + n_sp < (TOPP ? 1 : k)) {
        return false;
    }
    if constexpr (VP != 0) {
        // ---- vocabulary-parallel local pass: the record of this row (see topk_tail) ----
        const int n = n_ord + n_sp;
        if (n > kFCap / 2) {
            return false;  // (the entries are sorted as 64-bit words in the candidate area)
        }
        __shared__ int s_m;
        u64* const     big = (u64*)cand;
        FTB_ASSUME_SHARED(big);
        {
            constexpr int PER = (kFCap / 2 + kThreads - 1) / kThreads;
            u64           mine[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int a = tid + i * kThreads;
                mine[i]     = ~0ull;
                if (a < n_ord) {
                    const u32 e = cand[a];
                    const u32 kv = fkey(f_value<DT>(key16_inv(thr_key + (e >> 20)), temp, H.inv_t, H.inv_t_h));
                    mine[i]      = ((u64)(~kv) << 32) | (u64)(e & 0xfffffu);
                }
                else if (a < n) {
                    mine[i] = spec[a - n_ord];
                }
            }
            __syncthreads();  // every 32-bit entry has been read before the 64-bit ones take its place
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int a = tid + i * kThreads;
                if (a < n) {
                    big[a] = mine[i];
                }
            }
        }
        __syncthreads();
        group_sort_u64(big, n, tid, kThreads, CtaSync());
        __syncthreads();
        const int k_eff = k < n ? k : n;
        if (tid == 0) {
            s_m = k_eff;
        }
        __syncthreads();
        const u32 kv = (u32)(big[k_eff - 1] >> 32);
        if (DT == FTB200_F16 && temp && ~kv == fkey(thr_y)) {
            return false;  // half products round: patterns below the threshold may share the lowest class's value
        }
        for (int i = k_eff + tid; i < n; i += kThreads) {
            if ((u32)(big[i] >> 32) == kv) {
                atomicMax(&s_m, i + 1);
            }
        }
        __syncthreads();
        const int m   = s_m;
        u64*      out = P.vp_out + (size_t)r * (P.vp_cap + 2);
        if (tid == 0) {
            out[0] = m > P.vp_cap ? ~0ull : (u64)m;  // ~0: more ties than the exchange record holds
        }
        for (int i = tid; i < m && i < P.vp_cap; i += kThreads) {
            const u64 e = big[i];
            out[1 + i]  = (e & 0xffffffff00000000ull) | (u64)((u32)(e & 0xffffffffu) + (u32)P.vocab_offset);
        }
        return true;
    }
    if constexpr (TOPP) {
        if (n_ord < 1 || G.head != 0) {
            return false;  // (the second pass wants the row on a 16-byte boundary)
        }
        FTopp T;
        T.thr_key = thr_key, T.relmax = s_relmax, T.n_ord = n_ord, T.n_sp = n_sp;
        T.thr_y = thr_y, T.neg_max = neg_max;
        const float top_ord = f_value<DT>(key16_inv(thr_key + s_relmax), temp, H.inv_t, H.inv_t_h);
        const float top_sp  = s_vmaxkey != 0 ? fkey_inv(s_vmaxkey) : -INFINITY;
        T.maxv              = fmaxf(top_ord, top_sp);
        float mass_tail     = 0.0f;
        for (int i = 0; i < kWarps; ++i) {
            mass_tail += s_mtail[i];
        }
        return fast_topp_tail<DT>(P, S, H, G, T, spec, &s_nspec, s_mass, mass_tail, s_smaxkey, trace);
    }

    // ---- the draw (warp 0): runs of equal values from the top, then the reference's sequential sum and walk ----
    float* const          fe    = (float*)(spec + kFSpecCap);      // [kFRuns] value of the run
    unsigned short* const fc    = (unsigned short*)(fe + kFRuns);  // [kFRuns] columns of the run
    unsigned short* const crank = fc + kFRuns;                     // [kFBins] relative key of the a-th class from the top
    float* const          flat  = (float*)hist;                    // [k] exponentials of the first k entries (the counts are
                                                                   //     done with once the runs stand)
    FTB_ASSUME_SHARED(fe);
    FTB_ASSUME_SHARED(fc);
    FTB_ASSUME_SHARED(crank);
    FTB_ASSUME_SHARED(flat);
    if (wid == 0) {
        group_sort_u64<WarpSync, true>(spec, n_sp, lane, 32, WarpSync());
        __syncwarp();
        auto spec_above = [&](float v) {  // listed columns with a value strictly above v
            int       lo = 0, hi = n_sp;
            const u32 kc = ~fkey(v);
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if ((u32)(spec[mid] >> 32) < kc) {
                    lo = mid + 1;
                }
                else {
                    hi = mid;
                }
            }
            return lo;
        };
        // classes from the top bin down, 32 bins per trip, until they alone cover k columns (the listed columns
        // can only add to that); a class sits at (its rank among the classes) + (listed columns above it)
        int  nA = 0, covered = 0;
        bool over = false;
        for (int b0 = (int)s_relmax; b0 >= 0 && covered < k; b0 -= 32) {
            const int b   = b0 - lane;
            const u32 c   = b >= 0 ? hist[b] : 0u;
            const u32 any = __ballot_sync(0xffffffffu, c != 0);
            if (any == 0) {
                continue;
            }
            if (c != 0) {
                const float cv  = f_value<DT>(key16_inv(thr_key + (u32)b), temp, H.inv_t, H.inv_t_h);
                const int   a   = nA + __popc(any & ((1u << lane) - 1u));
                const int   pos = a + spec_above(cv);
                if (pos < kFRuns) {
                    fe[pos]  = cv;
                    fc[pos]  = (unsigned short)c;
                    crank[a] = (unsigned short)b;
                }
                else {
                    over = true;
                }
            }
            covered += (int)__reduce_add_sync(0xffffffffu, c);
            nA += __popc(any);
        }
        over = __any_sync(0xffffffffu, over);
        __syncwarp();
        // a listed column sits at (its rank among the listed columns) + (classes at or above its value); below
        // the last class taken the order no longer matters (k columns are covered before that)
        if (!over) {
            for (int i = lane; i < n_sp; i += 32) {
                const float sv = fkey_inv(~(u32)(spec[i] >> 32));
                int         lo = 0, hi = nA;  // classes (descending values) with value >= sv
                while (lo < hi) {
                    const int   mid = (lo + hi) >> 1;
                    const float cv  = f_value<DT>(key16_inv(thr_key + (u32)crank[mid]), temp, H.inv_t, H.inv_t_h);
                    if (cv >= sv) {
                        lo = mid + 1;
                    }
                    else {
                        hi = mid;
                    }
                }
                const int pos = i + lo;
                if (pos < kFRuns) {
                    fe[pos] = sv;
                    fc[pos] = 1;
                }
                else {
                    over = true;
                }
            }
            over = __any_sync(0xffffffffu, over);
        }
        const int nruns = nA + n_sp;
        __syncwarp();
        trace_mark(trace, 7);
        if (!over) {
            // the first k entries of the sorted sequence, as exponentials against the largest value: every run
            // writes its copies (the sequence the reference's thread 0 walks, sampling_topk_kernels.cu:276-287)
            const float vmax = fe[0];
            int         at   = 0;  // entries in front of the current batch of runs
            for (int p0 = 0; p0 < nruns && at < k; p0 += 32) {
                const int p    = p0 + lane;
                const int c    = p < nruns ? (int)fc[p] : 0;
                int       incl = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, o);
                    incl += lane >= o ? t : 0;
                }
                if (c != 0) {
                    const float e   = __expf(fe[p] - vmax);
                    const int   beg = at + incl - c;
                    const int   end = beg + c < k ? beg + c : k;
                    for (int i = beg; i < end; ++i) {
                        flat[i] = e;
                    }
                }
                at += __shfl_sync(0xffffffffu, incl, 31);
            }
            __syncwarp();
            trace_mark(trace, 8);
            if (lane == 0) {
                // dependent adds in the reference's order; operands come from shared memory eight at a time
                const int k8  = k & ~7;
                float     sum = 0.0f;
                for (int i = 0; i < k8; i += 8) {
                    const float4 a = *(const float4*)(flat + i), b = *(const float4*)(flat + i + 4);
                    sum += a.x, sum += a.y, sum += a.z, sum += a.w;
                    sum += b.x, sum += b.y, sum += b.z, sum += b.w;
                }
                for (int i = k8; i < k; ++i) {
                    sum += flat[i];
                }
                float rand_num = H.u * H.top_p * sum;
                int   pick     = k - 1;
                for (int i = 0; i < k; i += 8) {
                    float v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        v[j] = i + j < k ? flat[i + j] : 0.0f;
                    }
                    bool found = false;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (!found && i + j < k) {
                            rand_num -= v[j];
                            if (rand_num <= 0.0f || i + j == k - 1) {
                                pick  = i + j;
                                found = true;
                            }
                        }
                    }
                    if (found) {
                        break;
                    }
                }
                s_pick_idx = pick;
                // value of the picked entry: the run that holds position `pick`
                int acc = 0, prun = 0;
                for (int p = 0; p < nruns; ++p) {
                    acc += (int)fc[p];
                    if (acc > pick) {
                        prun = p;
                        break;
                    }
                }
                s_vsel = fe[prun];
            }
        }
        if (lane == 0) {
            s_nruns = over ? -1 : nruns;
        }
    }
    __syncthreads();
    trace_mark(trace, 9);
    if (s_nruns < 0) {
        return false;
    }
    // ---- the class the draw landed in: its members (all of them, also beyond the first k) and, per lane of
    //      the reference's first stage, the number of larger candidates ----
    const float vsel = s_vsel;
    const u32   ksel = fkey(vsel);
    if (DT == FTB200_F16 && temp && ksel == fkey(thr_y)) {
        return false;  // half products round: patterns below the threshold may share the lowest class's value
    }
    // (the run arrays are not needed any more: the class members take their place)
    u32* const cls  = (u32*)(spec + kFSpecCap);  // [kFClsCap]
    u32* const key2 = cls + kFClsCap;   // [kThreads] scratch of the small resolve
    FTB_ASSUME_SHARED(cls);
    const u32 bs1 = P.max_top_k <= 16 ? 128 : 256;
    const u32 bs2 = P.max_top_k <= 32 ? 128 : 256;
    const int sh1 = bs1 == 128 ? 7 : 8;
    {
        u32 packd_lo = 0, packd_hi = 0;  // 8 x 8-bit counters (a thread sees at most kFCap / kThreads entries)
        auto visit = [&](u32 kv, u32 c) {
            if (kv == ksel) {
                const u32 pos = atomicAdd(&s_ncls, 1u);
                if (pos < (u32)kFClsCap) {
                    cls[pos] = c;
                }
            }
            else if (kv > ksel) {
                const u32 l = (c >> sh1) & 7u;
                if (l < 4) {
                    packd_lo += 1u << (8 * l);
                }
                else {
                    packd_hi += 1u << (8 * (l - 4));
                }
            }
        };
        for (int i = tid; i < n_ord; i += kThreads) {
            const u32 e = cand[i];
            visit(fkey(f_value<DT>(key16_inv(thr_key + (e >> 20)), temp, H.inv_t, H.inv_t_h)), e & 0xfffffu);
        }
        for (int i = tid; i < n_sp; i += kThreads) {
            visit(~(u32)(spec[i] >> 32), (u32)(spec[i] & 0xffffffffu));
        }
        for (int l = 0; l < 8; ++l) {
            u32 cnt = ((l < 4 ? packd_lo : packd_hi) >> (8 * (l & 3))) & 0xffu;
            cnt     = __reduce_add_sync(0xffffffffu, cnt);
            if (lane == 0 && cnt != 0) {
                atomicAdd(&s_lane_base[l], cnt);
            }
        }
    }
    __syncthreads();
    trace_mark(trace, 10);
    const int m = (int)s_ncls;
    // number of candidates above the class = position of its first member in the sorted sequence
    int lo_cnt = 0;
    for (int l = 0; l < 8; ++l) {
        lo_cnt += (int)s_lane_base[l];
    }
    const int want = s_pick_idx - lo_cnt;
    if (m > kFClsCap || m < 1 || want < 0 || want >= m) {
        return false;  // (cannot happen for a consistent walk; the list takes the row if it does)
    }
    int idc;
    if (m == 1) {
        idc = (int)cls[0];
    }
    else if (m <= kThreads) {
        idc = f_resolve_small(cls, m, want, k, (int)bs1, (int)bs2, s_lane_base, key2, &s_ans);
    }
    else {
        // large classes: the sorting form, on 64-bit entries in the candidate area (its contents are done with)
        u64* big = (u64*)cand;
        for (int i = tid; i < m; i += kThreads) {
            big[i] = (u64)cls[i];
        }
        __syncthreads();
        idc = resolve_topk_class(big, m, want, k, (int)bs1, (int)bs2, s_lane_base);
    }
    if (tid == 0) {
        if (idc < 0) {
            idc = 0;
        }
        P.output_ids[(size_t)P.step * P.batch_size + col] = idc;
        if (P.seq_len != nullptr && P.finished != nullptr) {
            P.seq_len[r]  = P.seq_len[r] + 1;
            P.finished[r] = idc == H.end_id ? 1 : 0;
        }
    }
    return true;
}

template<int DT, bool TOPP, int VP = 0>
__global__ void __launch_bounds__(kThreads, TOPP ? 2 : 3) fast_sampling_kernel(const __grid_constant__ KParams P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ FHdr                               s_hdr[2];
    __shared__ __align__(16) u32                  s_pre[kFPreWords];
    __shared__ uint4                              s_wbuf[kWarps * 64];
    __shared__ unsigned short                     s_wj[kWarps * 64];
    FMap S;
    {
    S.wbuf = s_wbuf;
    S.wj   = s_wj;
    S.cand = (u32*)smem_raw;
    S.emask = S.cand + kFCap;
    S.hash  = S.emask + fast_mask_bytes(P.vocab_padded, TOPP) / 4;
    S.sval  = S.hash + P.hash_slots;
    S.hist  = S.sval + (P.hash_slots > kFBins ? P.hash_slots : kFBins);
    S.stage = S.hist + kFBins;
    }
    const int tid = threadIdx.x;
    // thread 0 keeps the next row's ticket and number between the stages
    int nt = 0, nr = 0;
    if (tid == 0) {
        nt = (int)atomicAdd(P.ticket + (TOPP ? 3 : 0), 1u);
        if (nt < P.local_batch) {
            nr = P.row_order != nullptr ? P.row_order[nt] : nt;
            f_prefetch_header(P, nr, s_pre);
            cp_async_wait_all();
        }
        f_compose_header(P, nt, nr, s_pre, s_hdr[0]);
    }
    for (int cur = 0;; cur ^= 1) {
        __syncthreads();
        const FHdr& H = s_hdr[cur];
        if (H.t >= P.local_batch) {
            break;
        }
        const int  r   = H.r;
        u64* const rec = P.trace != nullptr ? P.trace + ((size_t)H.t + (TOPP ? 2 * (size_t)P.local_batch : 0)) * kTraceWords : nullptr;
        if (tid == 0) {
            if (rec != nullptr) {
                rec[0] = (u64)r, rec[1] = (u64)blockIdx.x, rec[2] = global_timer_ns();
                rec[4 + 25] = (u64)clock64();
            }
            nt = (int)atomicAdd(P.ticket + (TOPP ? 3 : 0), 1u);  // stage 0 of the next row's header
        }
        auto stage1 = [&]() {
            if (tid == 0 && nt < P.local_batch) {
                nr = P.row_order != nullptr ? P.row_order[nt] : nt;
            }
        };
        auto stage2 = [&]() {
            if (tid == 0 && nt < P.local_batch) {
                f_prefetch_header(P, nr, s_pre);
            }
        };
        bool       done   = false;
        int* const id_out = P.output_ids + (size_t)P.step * P.batch_size + (size_t)P.ite * P.local_batch + r;
        const bool topp_row = H.mode == 2 && !H.fin;
        if (VP == 0 && topp_row != TOPP && !(TOPP && P.topk_states == nullptr)) {
            // the other kernel's row (a call without a top-k layer launches the top-p rows' kernel alone, and that one
            // then looks after every row)
            stage1();
            stage2();
            __syncthreads();
            if (tid == 0) {
                cp_async_wait_all();
                f_compose_header(P, nt, nr, s_pre, s_hdr[cur ^ 1]);
            }
            continue;
        }
        if (VP != 0 && !(H.mode == 1 && !H.fin)) {
            // vocabulary-parallel local pass: a top-p row is left to the general kernel (its statistics form), any
            // other row has nothing to send
            stage1();
            stage2();
            if (!topp_row) {
                if (tid == 0) {
                    P.vp_out[(size_t)r * (P.vp_cap + 2)] = 0;
                }
                done = true;
            }
        }
        else if (H.mode != 0 && !H.fin) {
            const FGeo G  = f_geometry(P, r);
            // (a penalty that can raise a value - repetition below 1, presence below 0 - would make columns
            //  under the threshold candidates: those rows go to the general kernel)
            const bool lowers = !P.apply_rep || (P.penalty_type == FTB200_PENALTY_MULTIPLICATIVE ? H.theta >= 1.0f :
                                                 P.penalty_type == FTB200_PENALTY_ADDITIVE ? H.theta >= 0.0f : true);
            const bool ok = lowers && G.nfull >= 2048 && G.nfull <= 65535 && H.inv_t > 0.0f && H.inv_t < 3.0e38f
                            && (P.apply_rep ? P.step : 0) <= kFMaxHistAll
                            && (P.bad_words != nullptr ? P.bad_words_len : 0) <= kFMaxWords;
            if (ok) {
                done = fast_row<DT, TOPP, VP>(P, S, H, rec, stage1, stage2);
                if (VP == 0 && done && tid == 0) {
                    curandState_t* states = H.mode == 1 ? P.topk_states : P.topp_states;
                    curandState_t  st     = states[r];
                    (void)curand_uniform(&st);
                    states[r] = st;
                }
            }
            else {
                stage1();
                stage2();
            }
        }
        else {
            stage1();
            stage2();
            if (H.mode == 0) {
                done = true;
            }
            else if (H.mode == 1) {
                // kernels/sampling_topk_kernels.cu:249-252: end id, no draw, length unchanged
                if (tid == 0) {
                    *id_out = H.end_id;
                }
                done = true;
            }
            else {
                // a finished row of the top-p layer: one-hot on the end id with probability 1 / (1 + 1e-6)
                // (kernels/sampling_topp_kernels.cu:1309-1341); the layer still draws
                if (tid == 0) {
                    const float p0 = DT == FTB200_F16 ? __half2float(__float2half_rn(1.0f / (1.0f + 1e-6f))) :
                                                        1.0f / (1.0f + 1e-6f);
                    *id_out        = H.end_id;
                    if ((p0 >= H.top_p || H.u * H.top_p <= p0) && P.seq_len != nullptr && P.finished != nullptr) {
                        P.finished[r] = 1;
                    }
                    curandState_t st = P.topp_states[r];
                    (void)curand_uniform(&st);
                    P.topp_states[r] = st;
                }
                done = true;
            }
        }
        __syncthreads();
        if (tid == 0) {
            if (rec != nullptr) {
                rec[3] = global_timer_ns();
                rec[4 + 26] = (u64)clock64();
                rec[4 + 27] = done ? 1 : 0;
            }
            if (!done) {
                P.redo_rows[atomicAdd(P.redo_count, 1u)] = r;
            }
            else if (VP == 0 && P.topp_states != nullptr && P.topp_decay != nullptr) {
                // top-p decay / reset (kernels/sampling_topp_kernels.cu:1381-1408), applied to every row of the call
                const int id = *id_out;
                float     p  = P.topp_ps[r];
                if (id == P.topp_reset[r]) {
                    p = P.topp_initial[r];
                }
                else {
                    p = fmaxf(p * P.topp_decay[r], P.topp_min[r]);
                }
                P.topp_ps[r] = p;
            }
            // the next row's header: its arguments were sent for before this row's pass
            cp_async_wait_all();
            f_compose_header(P, nt, nr, s_pre, s_hdr[cur ^ 1]);
        }
    }
}

template<int DT, bool TOPP, int VP = 0>
int fast_sampling_occupancy(size_t smem, int* per_sm)
{
    // per device: the opt-in to the shared-memory size (a per-device attribute of the kernel) and the answer
    constexpr int     kMaxDev = 64;
    static std::mutex mu;
    static size_t     set_smem[kMaxDev];
    static int        val[kMaxDev];
    int               dev = 0;
    FTB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) {
        set_error("ftb200_decode_step_sampling: device ordinal out of range");
        return FTB200_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (set_smem[dev] != smem) {
        FTB_CUDA_CHECK(cudaFuncSetAttribute(fast_sampling_kernel<DT, TOPP, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem));
        FTB_CUDA_CHECK(
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&val[dev], fast_sampling_kernel<DT, TOPP, VP>, kThreads, smem));
        set_smem[dev] = smem;
    }
    *per_sm = val[dev];
    return FTB200_OK;
}

template<int DT, bool TOPP, int VP = 0>
int fast_sampling_launch(const KParams& K, int grid, size_t smem, cudaStream_t st)
{
    fast_sampling_kernel<DT, TOPP, VP><<<grid, kThreads, smem, st>>>(K);
    FTB_CUDA_CHECK(cudaGetLastError());
    return FTB200_OK;
}

}  // namespace ftb200
