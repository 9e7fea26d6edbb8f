// Beam search, one step in one launch (sm_100a).
//
// One CTA per (batch entry, beam): penalties on the fly, one read of the row that yields the online
// soft-max statistics (max, sum of exponentials) and the row's best 2K columns.  The CTA that finishes
// last for a batch entry merges the K x 2K candidates, applies length penalty and diversity, archives
// finished hypotheses, picks the K live continuations, updates lengths / finished / parents and
// rewrites the KV-cache indirection - everything OnlineBeamSearchLayer<T>::forward launches
// (layers/beam_search_layers/BaseBeamSearchLayer.cu:181-289) in five kernels.
#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

constexpr int kBeamThreads = 256;
constexpr int kMaxBeam     = 64;

struct BeamK {
    int dtype, batch_size, local_batch, ite, K, vocab, vocab_padded, step, max_input_len, max_seq_len;
    const void* logits;
    const void* bias;
    const int*  end_ids;
    const int*  input_lengths;
    float       temperature, rep_penalty;
    int         penalty_type, min_length, apply_temp;
    float       diversity, length_penalty;
    int*        output_ids;
    int*        parent_ids;
    uint8_t*    finished;
    int*        seq_len;
    float*      cum_log_probs;
    float*      out_log_probs;
    const int*  src_indir;
    int*        tgt_indir;
    ftb200_beam_hyps hyps;
    int         has_hyps;
    // workspace
    u32*   arrivals;  // [local_batch]
    int*   cand_id;   // [local_batch, K, 2K]
    float* cand_val;  // [local_batch, K, 2K]  (already rounded to the logits type)
    const uint8_t* snap_finished;  // finished / sequence_length as they were before this step
    const int*     snap_seq_len;
};

template<int DT>
__device__ __forceinline__ float beam_round(float x)
{
    return DT == FTB200_F16 ? __half2float(__float2half_rn(x)) : x;
}

// logits value of column v with bias / temperature / pad mask applied in the logits type
// (kernels/beam_search_penalty_kernels.cu:24-87); bf16 goes the fp32 way on the up-cast value.
template<int DT>
__device__ __forceinline__ float beam_temp(const BeamK& P, u32 bits, int v)
{
    if (DT == FTB200_F16) {
        __half h = __ushort_as_half((unsigned short)bits);
        if (P.apply_temp) {
            if (v >= P.vocab) {
                return -65504.0f;
            }
            if (P.bias != nullptr) {
                h = __hadd(h, ((const __half*)P.bias)[v]);
            }
            h = __hmul(h, __float2half_rn(1.0f / (P.temperature + 1e-6f)));
        }
        return __half2float(h);
    }
    float x = DT == FTB200_F32 ? __uint_as_float(bits) : __uint_as_float(bits << 16);
    if (P.apply_temp) {
        if (v >= P.vocab) {
            return -FLT_MAX;
        }
        float b = 0.0f;
        if (P.bias != nullptr) {
            b = DT == FTB200_F32 ? ((const float*)P.bias)[v] : __bfloat162float(((const __nv_bfloat16*)P.bias)[v]);
        }
        x = (x + b) * (1.0f / (P.temperature + 1e-6f));
    }
    return x;
}

template<int DT>
__device__ __forceinline__ u32 beam_load(const void* row, int v)
{
    return DT == FTB200_F32 ? __ldg((const u32*)row + v) : (u32)__ldg((const unsigned short*)row + v);
}

struct MD {
    float m, d;
};
__device__ __forceinline__ MD md_merge(MD a, MD b)
{
    // kernels/online_softmax_beamsearch_kernels.cu:270-279
    const bool a_bigger = a.m > b.m;
    const MD   hi = a_bigger ? a : b, lo = a_bigger ? b : a;
    MD         r;
    r.d = hi.d + lo.d * __expf(lo.m - hi.m);
    r.m = hi.m;
    return r;
}

// (value desc, column asc) as one ascending u64
__device__ __forceinline__ u64 order_key(float val, u32 col)
{
    return ((u64)(~fkey(val)) << 32) | col;
}

template<int DT>
__global__ void __launch_bounds__(kBeamThreads) beam_step_kernel(const __grid_constant__ BeamK P)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // layout: u64 sortbuf[max(kBeamThreads * 8, K * 2K)] | int spec_id[step] | float spec_val[step]
    u64*             sortbuf = (u64*)smem_raw;
    __shared__ MD    s_md[kBeamThreads / 32];
    __shared__ int   s_nspec, s_last;
    __shared__ float s_old_cum[kMaxBeam];
    __shared__ int   s_newseq[kMaxBeam];

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int bb  = blockIdx.x;  // local batch-beam row
    const int b = bb / P.K, K = P.K, twoK = 2 * K;
    const int    V   = P.vocab_padded;
    const size_t ES  = DT == FTB200_F32 ? 4 : 2;
    const char*  row = (const char*)P.logits + (size_t)bb * V * ES;
    const float  MAXT = DT == FTB200_F16 ? 65504.0f : FLT_MAX;
    const int    sort_cap = kBeamThreads * 8 > K * twoK ? kBeamThreads * 8 : K * twoK;
    int*         spec_id  = (int*)(sortbuf + sort_cap);
    float*       spec_val = (float*)(spec_id + (P.step > 0 ? P.step : 1));

    const bool fin    = P.finished[bb] != 0;
    const int  end_id = P.end_ids[b];

    // ---- columns with a value of their own: repetition / presence penalty along the beam's ancestry
    //      (beam_search_penalty_kernels.cu:89-152: one thread walks parent_ids) and the min-length mask
    if (tid == 0) {
        int n = 0;
        if (!fin && P.penalty_type != FTB200_PENALTY_NONE && P.step > 0
            && P.rep_penalty != (P.penalty_type == FTB200_PENALTY_MULTIPLICATIVE ? 1.0f : 0.0f)) {
            const int    bbsize    = P.batch_size * K;
            const int    input_len = P.input_lengths != nullptr ? P.input_lengths[bb] : P.max_input_len;
            const int*   cur       = P.output_ids + (size_t)(P.step - 1) * bbsize + (size_t)P.ite * P.local_batch * K;
            const int*   parents   = P.parent_ids + (size_t)P.ite * K * P.local_batch;
            const float  pen       = beam_round<DT>(P.rep_penalty);
            auto         add       = [&](int id) {
                if (id < 0 || id >= V) {
                    return;
                }
                const float x = beam_temp<DT>(P, beam_load<DT>(row, id), id);
                float       y;
                if (P.penalty_type == FTB200_PENALTY_ADDITIVE) {
                    y = beam_round<DT>(x - pen);
                }
                else {
                    y = beam_round<DT>(x > 0.0f ? x / pen : x * pen);
                }
                spec_id[n]  = id;
                spec_val[n] = y;
                ++n;
            };
            add(cur[bb]);
            int parent_beam = bb % K;
            for (int i = P.step - 2; i >= 0; --i) {
                if (i >= input_len && i < P.max_input_len) {
                    continue;
                }
                parent_beam = parents[(size_t)i * bbsize + b * K + parent_beam];
                add(P.output_ids[(size_t)i * bbsize + b * K + parent_beam]);
            }
        }
        s_nspec = n;
    }
    __syncthreads();
    const int  nspec  = s_nspec;
    const bool minlen = !fin && (P.step - P.max_input_len < P.min_length)
                        && (P.seq_len[bb] + 1 - P.max_input_len < P.min_length);

    // value of column v as the reference's stage-1 kernel sees it (:410-432)
    auto value_of = [&](int v, u32 bits) -> float {
        if (fin) {
            return v == end_id ? MAXT : -MAXT;
        }
        if (minlen && v == end_id) {
            return -MAXT;
        }
        float y = beam_temp<DT>(P, bits, v);
        for (int i = 0; i < nspec; ++i) {  // later entries of the walk are older; the first match wins
            if (spec_id[i] == v) {
                y = spec_val[i];
                break;
            }
        }
        return y;
    };

    // ---- one pass: online soft-max statistics and this thread's best columns
    constexpr int LN = 8;  // per-thread list length; rows needing more than 8 winners take extra passes
    u64           best[LN];
#pragma unroll
    for (int i = 0; i < LN; ++i) {
        best[i] = ~0ull;
    }
    MD md{-MAXT, 0.0f};
    for (int v = tid; v < V; v += kBeamThreads) {
        const float y = value_of(v, fin ? 0u : beam_load<DT>(row, v));
        md            = md_merge(md, MD{y, 1.0f});
        const u64 kk  = order_key(y, (u32)v);
        if (kk < best[LN - 1]) {
            best[LN - 1] = kk;
#pragma unroll
            for (int i = LN - 1; i > 0; --i) {
                if (best[i] < best[i - 1]) {
                    u64 t       = best[i];
                    best[i]     = best[i - 1];
                    best[i - 1] = t;
                }
            }
        }
    }
    for (int off = 16; off > 0; off >>= 1) {
        MD o;
        o.m = __shfl_down_sync(0xffffffffu, md.m, off);
        o.d = __shfl_down_sync(0xffffffffu, md.d, off);
        md  = md_merge(md, o);
    }
    if (lane == 0) {
        s_md[wid] = md;
    }
    __syncthreads();
    md = s_md[0];
    for (int i = 1; i < kBeamThreads / 32; ++i) {
        md = md_merge(md, s_md[i]);
    }
    const float log_d = logf(md.d);
    const float cum   = P.cum_log_probs[bb];

    int*   my_id  = P.cand_id + (size_t)bb * twoK;
    float* my_val = P.cand_val + (size_t)bb * twoK;
    if (twoK <= LN) {
#pragma unroll
        for (int i = 0; i < LN; ++i) {
            sortbuf[tid * LN + i] = best[i];
        }
        __syncthreads();
        group_sort_u64(sortbuf, kBeamThreads * LN, tid, kBeamThreads, CtaSync());
        __syncthreads();
        if (tid < twoK) {
            const u64   e   = sortbuf[tid];
            const float u   = fkey_inv(~(u32)(e >> 32));
            const int   col = (int)(e & 0xffffffffu);
            my_id[tid]      = e == ~0ull ? -1 : bb * V + col;
            my_val[tid]     = beam_round<DT>(u - md.m - log_d + cum);
        }
    }
    else {
        // wide beams: extract the winners one by one, each pass over the row (it sits in L2 by now)
        __shared__ u64 s_prev;
        if (tid == 0) {
            s_prev = 0;
        }
        __syncthreads();
        for (int n = 0; n < twoK; ++n) {
            const u64 prev = s_prev;
            u64       mine = ~0ull;
            for (int v = tid; v < V; v += kBeamThreads) {
                const u64 kk = order_key(value_of(v, fin ? 0u : beam_load<DT>(row, v)), (u32)v);
                if ((n == 0 || kk > prev) && kk < mine) {
                    mine = kk;
                }
            }
            sortbuf[tid] = mine;
            __syncthreads();
            for (int s = kBeamThreads / 2; s > 0; s >>= 1) {
                if (tid < s && sortbuf[tid + s] < sortbuf[tid]) {
                    sortbuf[tid] = sortbuf[tid + s];
                }
                __syncthreads();
            }
            if (tid == 0) {
                const u64 e = sortbuf[0];
                s_prev      = e;
                my_id[n]    = e == ~0ull ? -1 : bb * V + (int)(e & 0xffffffffu);
                my_val[n]   = beam_round<DT>(fkey_inv(~(u32)(e >> 32)) - md.m - log_d + cum);
            }
            __syncthreads();
        }
    }

    // ---- the last CTA of this batch entry merges
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        s_last = atomicAdd(&P.arrivals[b], 1u) == (u32)(K - 1);
    }
    __syncthreads();
    if (!s_last) {
        return;
    }
    __threadfence();

    const int    ncand   = K * twoK;
    const int*   x       = P.cand_id + (size_t)b * ncand;
    const float* y       = P.cand_val + (size_t)b * ncand;
    const int    gbi     = P.ite * P.local_batch + b;
    int*         z       = P.output_ids + (size_t)P.step * P.batch_size * K + (size_t)P.ite * P.local_batch * K + b * K;
    int*         parents = P.parent_ids + (size_t)P.step * P.batch_size * K + (size_t)P.ite * P.local_batch * K + b * K;
    float*       v_cum   = P.cum_log_probs + b * K;
    float*       olp     = P.out_log_probs == nullptr ?
                               nullptr :
                               P.out_log_probs + (size_t)P.step * P.batch_size * K + (size_t)P.ite * P.local_batch * K;
    if (tid < K) {
        s_old_cum[tid] = v_cum[tid];
    }
    __syncthreads();
    bool skip_select = false;
    if (P.has_hyps) {
        // batch_topk_kernel, kernels/online_softmax_beamsearch_kernels.cu:129-138
        if (P.hyps.num_beams[gbi] == 0 && tid == 0) {
            P.hyps.min_normed_scores[gbi] = FLT_MAX;
        }
        else if (P.hyps.num_beams[gbi] == K) {
            skip_select = true;
        }
    }
    if (!skip_select) {
        // score of a candidate: length penalty with the length of the batch entry's FIRST indices, as the
        // reference indexes finished / sequence_lengths by the batch index (:148-156), plus diversity
        const int  len    = P.snap_finished[b] ? P.snap_seq_len[b] : P.snap_seq_len[b] + 1;
        const bool use_lp = !(P.length_penalty == 0.0f);
        for (int i = tid; i < ncand; i += kBeamThreads) {
            float e = y[i];
            if (use_lp && len != 1) {
                e = beam_round<DT>(e / beam_round<DT>(powf((float)len, P.length_penalty)));
            }
            if (DT == FTB200_F16) {
                // `elem += diversity_rate * (T)i` in half: the compiler contracts the half multiply and add of the
                // reference into one fused multiply-add, so the sum is rounded once (exact in double first)
                const double d = (double)beam_round<DT>(P.diversity) * (double)beam_round<DT>((float)(i % K)) + (double)e;
                e              = __half2float(__double2half(d));
            }
            else {
                e = e + P.diversity * (float)(i % K);
            }
            sortbuf[i] = x[i] < 0 ? ~0ull : order_key(e, (u32)i);
        }
        __syncthreads();
        group_sort_u64(sortbuf, ncand, tid, kBeamThreads, CtaSync());
        __syncthreads();
        if (tid == 0) {
            const int top_n = ncand < 2 * 4 ? ncand : (twoK <= 8 ? 8 : (twoK <= 16 ? 16 : (twoK <= 32 ? 32 : (twoK <= 64 ? 64 : 128))));
            int       selected = 0;
            for (int i = 0; i < top_n && i < ncand; ++i) {
                const u64 e = sortbuf[i];
                if (e == ~0ull) {
                    break;
                }
                const int   ci           = (int)(e & 0xffffffffu);
                const float normed_score = fkey_inv(~(u32)(e >> 32));
                const int   word         = x[ci];
                if (P.has_hyps && word % V == end_id) {
                    if (i < K) {
                        const int num_beam = P.hyps.num_beams[gbi];
                        int       beam_idx = num_beam;
                        bool      stop     = false;
                        if (num_beam == K) {
                            if (normed_score < P.hyps.min_normed_scores[gbi]) {
                                selected = K;
                                stop     = true;
                            }
                            else {
                                for (int j = 0; j < K; j++) {
                                    if (P.hyps.normed_scores[gbi * twoK + j] == P.hyps.min_normed_scores[gbi]) {
                                        beam_idx = j;
                                        P.hyps.num_beams[gbi]--;
                                        P.hyps.min_normed_scores[gbi]       = FLT_MAX;
                                        P.hyps.normed_scores[gbi * twoK + j] = normed_score;
                                        for (int l = 0; l < K; l++) {
                                            P.hyps.min_normed_scores[gbi] =
                                                fminf(P.hyps.min_normed_scores[gbi], P.hyps.normed_scores[gbi * twoK + l]);
                                        }
                                        break;
                                    }
                                }
                            }
                        }
                        if (stop) {
                            break;
                        }
                        const size_t tgt = ((size_t)gbi * twoK + beam_idx) * P.max_seq_len;
                        P.hyps.output_ids_tgt[tgt + P.step] = end_id;
                        if (P.hyps.log_probs != nullptr) {
                            P.hyps.log_probs[tgt + P.step] = y[ci] - s_old_cum[(word / V) % K];
                        }
                        int prev_id = (word / V) % K;
                        for (int j = P.step - 1; j >= 0; j--) {
                            const size_t src = (size_t)j * P.batch_size * K + (size_t)P.ite * P.local_batch * K + b * K + prev_id;
                            P.hyps.output_ids_tgt[tgt + j] = P.output_ids[src];
                            if (P.hyps.log_probs != nullptr && P.out_log_probs != nullptr) {
                                P.hyps.log_probs[tgt + j] = P.out_log_probs[src];
                            }
                            prev_id = P.parent_ids[src];
                        }
                        const int tb                      = gbi * twoK + beam_idx;
                        P.hyps.sequence_lengths_tgt[tb]   = P.step;
                        P.hyps.normed_scores[tb]          = normed_score;
                        P.hyps.min_normed_scores[gbi]     = fminf(P.hyps.min_normed_scores[gbi], normed_score);
                        P.hyps.num_beams[gbi]++;
                        P.hyps.cum_log_probs[tb]          = y[ci];
                    }
                }
                else if ((P.has_hyps && i < twoK) || (!P.has_hyps && i < K)) {
                    z[selected] = word;
                    if (olp != nullptr) {
                        olp[b * K + selected] = y[ci] - s_old_cum[(word / V) % K];
                    }
                    v_cum[selected] = y[ci];
                    selected++;
                }
                if (selected >= K) {
                    break;
                }
            }
            if (P.has_hyps) {
                // the reference indexes by the local batch index here (:254-261)
                if (P.hyps.num_beams[b] < K) {
                    P.hyps.is_done[b] = 0;
                }
                else if (P.hyps.early_stopping) {
                    P.hyps.is_done[b] = 1;
                }
            }
        }
        __syncthreads();
    }

    // ---- update_kernel (layers/beam_search_layers/OnlineBeamSearchLayer.cu:24-58): lengths follow the parent
    if (tid < K) {
        const int idx = b * K + tid;
        s_newseq[tid] = P.finished[idx] ? P.seq_len[idx] : P.seq_len[idx] + 1;
    }
    __syncthreads();
    if (tid < K) {
        const int idx     = b * K + tid;
        const int word    = z[tid];
        const int beam_id = (word / V) % K;
        const int word_id = word % V;
        P.seq_len[idx]    = s_newseq[beam_id];
        P.finished[idx]   = word_id == end_id ? 1 : 0;
        parents[tid]      = beam_id;
        z[tid]            = word_id;
    }
    __syncthreads();
    if (P.has_hyps && P.hyps.num_beams[gbi] == K && tid < K) {
        P.finished[b * K + tid] = 1;
    }
    __syncthreads();

    // ---- KV-cache indirection (layers/beam_search_layers/BaseBeamSearchLayer.cu:23-79)
    if (P.tgt_indir != nullptr && P.src_indir != nullptr) {
        const int L          = P.max_seq_len;
        const int start_step = P.step + 1 - L > 0 ? P.step + 1 - L : 0;
        const int num_steps  = P.step + 1 < L ? P.step + 1 : L;
        for (int i = tid; i < K * num_steps; i += kBeamThreads) {
            const int k = i / num_steps, t = i % num_steps + start_step;
            if (P.finished[b * K + k]) {
                continue;
            }
            const int    tc       = t % L;
            const int    src_beam = parents[k];
            const size_t base     = (size_t)b * K * L;
            P.tgt_indir[base + (size_t)k * L + tc] = t == P.step ? k : P.src_indir[base + (size_t)src_beam * L + tc];
        }
    }
}

}  // namespace ftb200

using namespace ftb200;

extern "C" int ftb200_beam_workspace_bytes(int local_batch_size, int beam_width, size_t* bytes)
{
    if (bytes == nullptr || local_batch_size < 0 || beam_width < 1 || beam_width > kMaxBeam) {
        set_error("ftb200_beam_workspace_bytes: invalid argument (beam_width must be 1..64)");
        return FTB200_INVALID_ARG;
    }
    const size_t rows = (size_t)local_batch_size * beam_width;
    *bytes            = 256 + (((size_t)local_batch_size * 4 + 255) / 256) * 256 + rows * 2 * beam_width * 8
             + ((rows + 255) / 256) * 256 + rows * 4;
    return FTB200_OK;
}

extern "C" int ftb200_beam_search_step(const ftb200_beam_params* p)
{
    reset_launch_count();
    if (p == nullptr || p->logits == nullptr || p->end_ids == nullptr || p->output_ids == nullptr
        || p->parent_ids == nullptr || p->finished == nullptr || p->sequence_length == nullptr
        || p->cum_log_probs == nullptr) {
        set_error("ftb200_beam_search_step: a required pointer is null (cum_log_probs is required in beam search)");
        return FTB200_INVALID_ARG;
    }
    if (p->beam_width < 2 || p->beam_width > kMaxBeam) {
        set_error("Topk kernel of beam search does not support beam_width=" + std::to_string(p->beam_width));
        return FTB200_DOMAIN_ERROR;
    }
    if (p->dtype < 0 || p->dtype > 2 || p->local_batch_size < 0 || p->vocab_size <= 0
        || p->vocab_size_padded < p->vocab_size || p->step < 0 || p->max_seq_len <= p->step) {
        set_error("ftb200_beam_search_step: bad shape or dtype");
        return FTB200_INVALID_ARG;
    }
    if (p->local_batch_size == 0) {
        return FTB200_OK;
    }
    size_t need = 0;
    ftb200_beam_workspace_bytes(p->local_batch_size, p->beam_width, &need);
    if (p->workspace == nullptr || p->workspace_bytes < need) {
        set_error("ftb200_beam_search_step: workspace too small, need " + std::to_string(need) + " bytes");
        return FTB200_WORKSPACE_SMALL;
    }
    BeamK K{};
    K.dtype = p->dtype, K.batch_size = p->batch_size, K.local_batch = p->local_batch_size, K.ite = p->ite;
    K.K = p->beam_width, K.vocab = p->vocab_size, K.vocab_padded = p->vocab_size_padded, K.step = p->step;
    K.max_input_len = p->max_input_length, K.max_seq_len = p->max_seq_len;
    K.logits = p->logits, K.bias = p->embedding_bias, K.end_ids = p->end_ids, K.input_lengths = p->input_lengths;
    K.temperature = p->temperature, K.rep_penalty = p->repetition_penalty, K.penalty_type = p->penalty_type;
    K.min_length = p->min_length, K.diversity = p->diversity_rate, K.length_penalty = p->length_penalty;
    // invokeAddBiasApplyPenalties gate, kernels/beam_search_penalty_kernels.cu:197
    K.apply_temp = (p->embedding_bias != nullptr || p->temperature != 1.0f || p->vocab_size != p->vocab_size_padded) ? 1 : 0;
    K.output_ids = p->output_ids, K.parent_ids = p->parent_ids, K.finished = p->finished;
    K.seq_len = p->sequence_length, K.cum_log_probs = p->cum_log_probs, K.out_log_probs = p->output_log_probs;
    K.src_indir = p->src_cache_indirection, K.tgt_indir = p->tgt_cache_indirection;
    K.has_hyps = (p->beam_hyps != nullptr && p->beam_hyps->num_beams != nullptr) ? 1 : 0;
    if (p->beam_hyps != nullptr) {
        K.hyps = *p->beam_hyps;
    }
    char* ws   = (char*)p->workspace;
    K.arrivals = (u32*)ws;
    const size_t rows = (size_t)p->local_batch_size * p->beam_width;
    K.cand_id  = (int*)(ws + (((size_t)p->local_batch_size * 4 + 255) / 256) * 256 + 256);
    K.cand_val = (float*)(K.cand_id + rows * 2 * p->beam_width);
    uint8_t* snap_fin = (uint8_t*)(K.cand_val + rows * 2 * p->beam_width);
    int*     snap_seq = (int*)(snap_fin + ((rows + 255) / 256) * 256);
    K.snap_finished   = snap_fin;
    K.snap_seq_len    = snap_seq;

    cudaStream_t st = (cudaStream_t)p->stream;
    FTB_CUDA_CHECK(cudaMemsetAsync(K.arrivals, 0, (size_t)p->local_batch_size * 4, st));
    // the merge of one batch entry reads finished / sequence_length of OTHER entries (the reference indexes
    // them by the batch index); give it the values from before any entry of this step was updated
    FTB_CUDA_CHECK(cudaMemcpyAsync(snap_fin, p->finished, rows, cudaMemcpyDeviceToDevice, st));
    FTB_CUDA_CHECK(cudaMemcpyAsync(snap_seq, p->sequence_length, rows * 4, cudaMemcpyDeviceToDevice, st));
    const int    twoK     = 2 * p->beam_width;
    const size_t sort_cap = (size_t)(kBeamThreads * 8 > p->beam_width * twoK ? kBeamThreads * 8 : p->beam_width * twoK);
    const size_t smem     = sort_cap * 8 + (size_t)(p->step > 0 ? p->step : 1) * 8 + 16;
    if (smem > 200 * 1024) {
        set_error("ftb200_beam_search_step: step too large for the shared-memory token list");
        return FTB200_UNSUPPORTED;
    }
    const int grid = p->local_batch_size * p->beam_width;
#define FTB_LAUNCH_BEAM(DT)                                                                                            \
    do {                                                                                                               \
        FTB_CUDA_CHECK(cudaFuncSetAttribute(beam_step_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                            200 * 1024));                                                              \
        beam_step_kernel<DT><<<grid, kBeamThreads, smem, st>>>(K);                                                     \
    } while (0)
    switch (p->dtype) {
        case FTB200_F32: FTB_LAUNCH_BEAM(FTB200_F32); break;
        case FTB200_F16: FTB_LAUNCH_BEAM(FTB200_F16); break;
        default: FTB_LAUNCH_BEAM(FTB200_BF16); break;
    }
#undef FTB_LAUNCH_BEAM
    FTB_CUDA_CHECK(cudaGetLastError());
    note_launch(1);
    return FTB200_OK;
}
