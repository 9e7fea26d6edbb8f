/*
 * TEST INFRASTRUCTURE - CPU restatement of FasterTransformer's decode sampling path.
 *
 * Plain C++ (no CUDA) that follows the reference's algorithm step by step so that the CUDA
 * kernels can be checked against it.  Only tests, the smoke check and the benchmark's cpu_baseline
 * leg may load this library; the product never does.
 *
 * Every function cites the reference code it restates (path:line inside the FasterTransformer tree,
 * paths relative to src/fastertransformer/).  Differences a CPU cannot avoid:
 *   - the reference is built with --use_fast_math, so its __expf / logf / division are the GPU's
 *     approximate instructions; here they are libm's expf / logf and IEEE division.  Values agree to a
 *     few ulp; a sampled id can differ only when a draw lands within that distance of a boundary.
 *   - uniforms are an input: the caller draws them with curand from the same states the kernels use.
 * Parity status: pinned against the reference's known-answer tests (tests/unittests/test_sampling_layer.cu,
 * tests/golden/) and against outputs of the compiled reference itself (oracle/_ref) on a B200.
 */
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../include/ftb200.h"

namespace {

typedef _Float16 half_t;

inline float bf16_to_float(uint16_t b)
{
    uint32_t u = (uint32_t)b << 16;
    float    f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline float half_bits_to_float(uint16_t b)
{
    half_t h;
    std::memcpy(&h, &b, 2);
    return (float)h;
}
inline float round_half(float x)
{
    return (float)(half_t)x;
}

struct RowView {
    int         dtype;
    const void* base;
    size_t      stride;
    float       get(size_t row, size_t v) const
    {
        switch (dtype) {
            case FTB200_F32: return ((const float*)base)[row * stride + v];
            case FTB200_F16: return half_bits_to_float(((const uint16_t*)base)[row * stride + v]);
            default: return bf16_to_float(((const uint16_t*)base)[row * stride + v]);
        }
    }
};

// Nearest half (ties to even) of a double, as a float: one rounding, for results the GPU forms with a fused
// half multiply-add.
static float round_half_from_double(double d)
{
    if (!(d == d) || d == 0.0 || std::isinf(d)) {
        return (float)d;
    }
    int    ex;
    double a = std::fabs(d);
    std::frexp(a, &ex);                        // a = m * 2^ex, m in [0.5, 1)
    int    e2      = ex - 1 < -14 ? -14 : ex - 1;  // exponent of the leading bit, clamped to the subnormal range
    double spacing = std::ldexp(1.0, e2 - 10);
    double r       = std::nearbyint(a / spacing) * spacing;
    if (r > 65504.0) {
        r = INFINITY;
    }
    return (float)(d < 0 ? -r : r);
}

// The logits type of the reference is float or half; bf16 inputs are handled as float on the up-cast.
struct TypeOps {
    bool  is_half;
    float max_t() const
    {
        return is_half ? 65504.0f : FLT_MAX;
    }
    float rnd(float x) const
    {
        return is_half ? round_half(x) : x;
    }
};

// kernels/ban_bad_words.cu:35-85 for beam_width == 1.
void ban_bad_words_row(std::vector<float>& x, const int* output_ids, int batch_size, size_t col, const int* words,
                       int L, int vocab_padded, int step)
{
    const int* offs = words + L;
    for (int i = 0; i < L; ++i) {
        if (offs[i] < 0) {
            continue;
        }
        const int item_end   = offs[i];
        const int item_start = i > 0 ? offs[i - 1] : 0;
        const int item_size  = item_end - item_start;
        bool      ban        = item_size == 1;
        if (item_size > 1 && step >= item_size - 1) {
            ban = true;
            for (int j = item_size - 2; j >= 0; --j) {
                int prev = output_ids[(size_t)(step - (item_size - 1) + j) * batch_size + col];
                if (prev != words[item_start + j]) {
                    ban = false;
                    break;
                }
            }
        }
        if (ban) {
            int tok = words[item_end - 1];
            if (0 < tok && tok < vocab_padded) {
                x[tok] = -INFINITY;
            }
        }
    }
}

// kernels/sampling_penalty_kernels.cu:117-179 (per-row temperature, bias, pad mask).
void temperature_row(std::vector<float>& x, const TypeOps& T, const RowView* bias, float temperature, int vocab,
                     int vocab_padded)
{
    const float inv = 1.0f / (temperature + 1e-6f);
    for (int v = 0; v < vocab_padded; ++v) {
        if (v < vocab) {
            if (T.is_half) {
                float h = x[v];
                if (bias) {
                    h = round_half(h + bias->get(0, v));
                }
                x[v] = round_half(h * round_half(inv));
            }
            else {
                float y = x[v];
                if (bias) {
                    y = y + bias->get(0, v);
                }
                x[v] = y * inv;
            }
        }
        else {
            // the half2 kernel leaves pad columns as they are (:171-177); the scalar one writes -MAX.
            // Both are overwritten by the end mask before selection.
            x[v] = -T.max_t();
        }
    }
}

// kernels/sampling_penalty_kernels.cu:367-424: every occurrence is computed from the pre-penalty value.
void repetition_row(std::vector<float>& x, const TypeOps& T, float theta, int type, const int* output_ids,
                    int batch_size, size_t col, int input_len, int max_input_len, int step, int vocab_padded)
{
    std::vector<std::pair<int, float>> upd;
    for (int t = 0; t < step; ++t) {
        if (t >= input_len && t < max_input_len) {
            continue;
        }
        int id = output_ids[(size_t)t * batch_size + col];
        if (id < 0 || id >= vocab_padded) {
            continue;
        }
        float logit = x[id], nv = logit;
        if (type == FTB200_PENALTY_ADDITIVE) {
            nv = logit - theta;
        }
        else if (type == FTB200_PENALTY_MULTIPLICATIVE) {
            nv = logit < 0.0f ? logit * theta : logit / theta;
        }
        upd.push_back({id, T.rnd(nv)});
    }
    for (auto& u : upd) {
        x[u.first] = u.second;
    }
}

// kernels/sampling_topk_kernels.cu:67-94.
void end_mask_row(std::vector<float>& x, const TypeOps& T, bool finished, int end_id, int vocab, int vocab_padded)
{
    for (int v = 0; v < vocab_padded; ++v) {
        if (v >= vocab) {
            x[v] = -T.max_t();
        }
        else if (finished) {
            x[v] = v == end_id ? T.max_t() : -T.max_t();
        }
    }
}

// warpReduceSum / blockReduceSum of kernels/reduce_kernel_utils.cuh:73-103 over `n` threads.
float butterfly_block_sum(const std::vector<float>& partial, int n)
{
    const int nwarps = (n + 31) / 32;
    float     shared[32];
    for (int i = 0; i < 32; ++i) {
        shared[i] = 0.0f;
    }
    for (int w = 0; w < nwarps; ++w) {
        float v[32], t[32];
        for (int l = 0; l < 32; ++l) {
            v[l] = w * 32 + l < n ? partial[w * 32 + l] : 0.0f;
        }
        for (int m = 16; m > 0; m >>= 1) {
            for (int l = 0; l < 32; ++l) {
                t[l] = v[l] + v[l ^ m];
            }
            std::memcpy(v, t, sizeof(v));
        }
        shared[w] = v[0];
    }
    float v[32], t[32];
    for (int l = 0; l < 32; ++l) {
        v[l] = ((float)l < (float)n / 32.f) ? shared[l] : 0.0f;
    }
    for (int m = 16; m > 0; m >>= 1) {
        for (int l = 0; l < 32; ++l) {
            t[l] = v[l] + v[l ^ m];
        }
        std::memcpy(v, t, sizeof(v));
    }
    return v[0];
}

// addBiasSoftMax, kernels/sampling_topp_kernels.cu:1294-1345 (bias is never passed by the layers).
void softmax_row(std::vector<float>& x, const TypeOps& T, bool finished, int end_id, int n, int n_padded)
{
    const int nthr    = n < 1024 ? n : 1024;
    float     max_val = -FLT_MAX;
    for (int v = 0; v < n_padded; ++v) {
        if (v < n) {
            if (finished) {
                x[v] = v == end_id ? T.max_t() : -T.max_t();
            }
        }
        else {
            x[v] = -T.max_t();
        }
        max_val = std::max(max_val, x[v]);
    }
    std::vector<float> partial(nthr, 0.0f);
    for (int v = 0; v < n_padded; ++v) {
        x[v] = T.rnd(expf(x[v] - max_val));
        partial[v % nthr] += x[v];
    }
    const float s = butterfly_block_sum(partial, nthr);
    for (int v = 0; v < n_padded; ++v) {
        x[v] = T.rnd(x[v] / (s + 1e-6f));
    }
}

struct Cand {
    float val;
    int   col;
};

// Two-stage top-k of kernels/sampling_topk_kernels.cu:130-312.  Stage 1: 8 CTAs per row, CTA `lane`
// owns columns with (col / BS1) % 8 == lane, thread col % BS1; k arg-max passes, each removing the
// winner.  Within a thread the first maximum wins (strict >, reduce_kernel_utils.cuh:329-336); across
// threads cub::BlockReduce keeps the right-hand operand on ties (reduce_topk_op_2, :345-348), i.e. the
// highest thread id.  Extracting k times with that rule equals taking the first k of the slice ordered
// by (value desc, thread desc, column asc).  Stage 2 repeats the scheme over the 8*k slots with BS2
// threads: (value desc, slot % BS2 desc, slot asc).  Values equal to -MAX are never selected.
std::vector<Cand> topk_two_stage(const std::vector<float>& x, const TypeOps& T, int vocab_padded, int k, int max_top_k)
{
    const int bs1 = max_top_k <= 16 ? 128 : 256;
    const int bs2 = max_top_k <= 32 ? 128 : 256;
    struct Slot {
        float val;
        int   col;
        int   slot;
    };
    std::vector<Slot> slots;
    for (int lane = 0; lane < 8; ++lane) {
        std::vector<Cand> mine;
        for (int base = lane * bs1; base < vocab_padded; base += bs1 * 8) {
            for (int t = 0; t < bs1 && base + t < vocab_padded; ++t) {
                if (x[base + t] > -T.max_t()) {
                    mine.push_back({x[base + t], base + t});
                }
            }
        }
        auto cmp = [&](const Cand& a, const Cand& b) {
            if (a.val != b.val) {
                return a.val > b.val;
            }
            int ta = a.col % bs1, tb = b.col % bs1;
            if (ta != tb) {
                return ta > tb;
            }
            return a.col < b.col;
        };
        size_t keep = std::min<size_t>(k, mine.size());
        std::partial_sort(mine.begin(), mine.begin() + keep, mine.end(), cmp);
        for (size_t j = 0; j < keep; ++j) {
            slots.push_back({mine[j].val, mine[j].col, lane * k + (int)j});
        }
    }
    auto cmp2 = [&](const Slot& a, const Slot& b) {
        if (a.val != b.val) {
            return a.val > b.val;
        }
        int ma = a.slot % bs2, mb = b.slot % bs2;
        if (ma != mb) {
            return ma > mb;
        }
        return a.slot < b.slot;
    };
    size_t keep = std::min<size_t>(k, slots.size());
    std::partial_sort(slots.begin(), slots.begin() + keep, slots.end(), cmp2);
    std::vector<Cand> out;
    for (size_t j = 0; j < keep; ++j) {
        out.push_back({slots[j].val, slots[j].col});
    }
    return out;
}

struct RowResult {
    int   id;
    bool  update_state;  // sequence_length / finished are rewritten
    bool  has_lp;
    float log_prob;      // added to cum_log_probs
    float out_log_prob;  // written to output_log_probs
};

// topk_stage2_sampling's draw, kernels/sampling_topk_kernels.cu:282-311.
RowResult topk_draw(const std::vector<Cand>& top, int k, float u, float top_p, bool probs)
{
    RowResult R{0, true, false, 0.f, 0.f};
    if (top.empty()) {
        return R;
    }
    std::vector<float> e(top.size());
    float              s_sum = 0.0f, s_max = top[0].val;
    for (size_t i = 0; i < top.size(); ++i) {
        e[i] = probs ? top[i].val : expf(top[i].val - s_max);
        s_sum += e[i];
    }
    float  rand_num = u * top_p * s_sum;
    size_t pick     = top.size() - 1;
    for (size_t i = 0; i < top.size(); ++i) {
        rand_num = rand_num - e[i];
        if (rand_num <= 0.0f || (int)i == k - 1) {
            pick = i;
            break;
        }
    }
    R.id           = top[pick].col;
    R.has_lp       = true;
    R.log_prob     = logf(e[pick]);
    R.out_log_prob = R.log_prob - logf(s_sum);
    return R;
}

// topp_beam_topk_kernel + segmented sort + topp_sampling, kernels/sampling_topp_kernels.cu:801-1004.
// The sort is a stable descending sort (equal probabilities stay in column order); the running sum is
// cub::BlockScan<float,256>::InclusiveSum with a running prefix: 32 raking threads each sum 8
// consecutive items left to right, a Kogge-Stone scan combines the 32 partials, and each item's result
// is prefix + partials-before + its segment's running sum.
RowResult topp_draw(const std::vector<float>& p, int vocab_padded, float u, float top_p)
{
    RowResult R{0, true, true, 0.f, 0.f};
    // arg-max shortcut: TopK<T,1> keeps the larger value, then the smaller column
    int best = 0;
    for (int v = 1; v < vocab_padded; ++v) {
        if (p[v] > p[best]) {
            best = v;
        }
    }
    if (p[best] >= top_p) {
        R.id       = best;
        R.log_prob = R.out_log_prob = logf(p[best]);
        return R;
    }
    std::vector<int> order(vocab_padded);
    for (int v = 0; v < vocab_padded; ++v) {
        order[v] = v;
    }
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return p[a] > p[b]; });
    const float rand_num = u * top_p;
    float       running  = 0.0f;
    const int   end      = (vocab_padded + 255) / 256 * 256;
    for (int c = 0; c < end; c += 256) {
        float x[256], out[256], up[32], inc[32];
        for (int t = 0; t < 256; ++t) {
            x[t] = c + t < vocab_padded ? p[order[c + t]] : 0.0f;
        }
        for (int j = 0; j < 32; ++j) {
            float s = x[8 * j];
            for (int i = 1; i < 8; ++i) {
                s = s + x[8 * j + i];
            }
            up[j] = inc[j] = s;
        }
        for (int off = 1; off < 32; off <<= 1) {
            float t[32];
            for (int j = 0; j < 32; ++j) {
                t[j] = j >= off ? inc[j] + inc[j - off] : inc[j];
            }
            std::memcpy(inc, t, sizeof(inc));
        }
        for (int j = 0; j < 32; ++j) {
            float o = j == 0 ? running : running + inc[j - 1];
            for (int i = 0; i < 8; ++i) {
                o              = o + x[8 * j + i];
                out[8 * j + i] = o;
            }
        }
        running = running + inc[31];
        // first warp with an active lane; lane = 32 - popcount of its mask (:963, :984)
        for (int w = 0; w < 8; ++w) {
            int cnt = 0;
            for (int l = 0; l < 32; ++l) {
                cnt += rand_num <= out[32 * w + l] ? 1 : 0;
            }
            if (cnt > 0) {
                int pos    = c + 32 * w + (32 - cnt);
                int col    = pos < vocab_padded ? order[pos] : order[0];
                R.id       = col;
                R.log_prob = R.out_log_prob = logf(p[col]);
                return R;
            }
        }
    }
    // never reached: the best token stays, nothing else is updated (:954)
    R.id           = order[0];
    R.update_state = false;
    R.has_lp       = false;
    return R;
}

}  // namespace

extern "C" {

/*
 * One decode step on the CPU.  Same argument block as ftb200_decode_step_sampling, with HOST pointers;
 * topk_states / topp_states point to float[local_batch_size] uniforms (the value curand_uniform
 * would return for each row this step).  Follows DynamicDecodeLayer::forward for beam_width == 1:
 * layers/DynamicDecodeLayer.cc:247-283, 389-445; BaseSamplingLayer::forward
 * (layers/sampling_layers/BaseSamplingLayer.cc:255-359); TopKSamplingLayer::runSampling
 * (TopKSamplingLayer.cu:189-267); TopPSamplingLayer::runSampling (TopPSamplingLayer.cu:256-342).
 */
int oracle_decode_step_sampling(const ftb200_sampling_params* p)
{
    const int     Vp = p->vocab_size_padded, V = p->vocab_size;
    const TypeOps T{p->dtype == FTB200_F16};
    const RowView L{p->dtype, p->logits, (size_t)Vp};
    RowView       biasv{p->dtype, p->embedding_bias, (size_t)Vp};
    const RowView* bias   = p->embedding_bias ? &biasv : nullptr;
    const float*  u_topk  = (const float*)p->topk_states;
    const float*  u_topp  = (const float*)p->topp_states;
    const bool    want_lp = p->cum_log_probs || p->output_log_probs;

    // rows are independent: one OpenMP thread per row, as many threads as OMP_NUM_THREADS allows
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < p->local_batch_size; ++r) {
        int mode = 0;
        if (u_topk && !(p->topk_skip && p->topk_skip[r])) {
            mode = 1;
        }
        else if (u_topp && !(p->topp_skip && p->topp_skip[r])) {
            mode = 2;
        }
        const size_t col    = (size_t)p->ite * p->local_batch_size + r;
        int*         id_out = p->output_ids + (size_t)p->step * p->batch_size + col;
        const bool   fin    = p->finished ? p->finished[r] != 0 : false;
        const int    end_id = p->end_ids[r];

        if (mode != 0) {
            std::vector<float> x(Vp);
            for (int v = 0; v < Vp; ++v) {
                x[v] = L.get(r, v);
            }
            if (p->bad_words && p->bad_words_len > 0) {
                const int* words =
                    p->bad_words_shared ? p->bad_words : p->bad_words + (size_t)r * 2 * p->bad_words_len;
                ban_bad_words_row(x, p->output_ids, p->batch_size, col, words, p->bad_words_len, Vp, p->step);
            }
            if (p->apply_temperature) {
                temperature_row(x, T, bias, p->temperature[r], V, Vp);
            }
            if (p->apply_repetition && p->penalty_type != FTB200_PENALTY_NONE) {
                const int input_len = p->input_lengths ? p->input_lengths[r] : p->max_input_length;
                repetition_row(x, T, p->repetition_penalty[r], p->penalty_type, p->output_ids, p->batch_size, col,
                               input_len, p->max_input_length, p->step, Vp);
            }
            if (p->apply_min_length) {
                // kernels/sampling_penalty_kernels.cu:493-499
                if (p->sequence_length[r] + 1 - p->max_input_length < p->min_lengths[r]) {
                    x[end_id] = -T.max_t();
                }
            }
            RowResult R{0, false, false, 0.f, 0.f};
            if (mode == 1) {
                end_mask_row(x, T, fin, end_id, V, Vp);
                if (want_lp) {
                    softmax_row(x, T, fin, end_id, V, Vp);
                }
                if (fin) {
                    // kernels/sampling_topk_kernels.cu:249-252
                    *id_out = end_id;
                }
                else {
                    int k = (int)p->topk_ks[r];
                    auto top = topk_two_stage(x, T, Vp, k, p->max_top_k);
                    R        = topk_draw(top, k, u_topk[r], p->topk_ps[r], want_lp);
                    R.has_lp = want_lp;
                    *id_out  = R.id;
                }
            }
            else {
                softmax_row(x, T, fin, end_id, V, Vp);
                R       = topp_draw(x, Vp, u_topp[r], p->topp_ps[r]);
                *id_out = R.id;
            }
            if (mode == 2 || !fin) {
                if (R.has_lp && want_lp) {
                    if (p->cum_log_probs) {
                        p->cum_log_probs[r] += R.log_prob;
                    }
                    if (p->output_log_probs) {
                        p->output_log_probs[r] = R.out_log_prob;
                    }
                }
                if (R.update_state && p->sequence_length && p->finished) {
                    p->sequence_length[r] = fin ? p->sequence_length[r] : p->sequence_length[r] + 1;
                    p->finished[r]        = *id_out == end_id ? 1 : 0;
                }
            }
        }
        // computeToppDecay, kernels/sampling_topp_kernels.cu:1381-1408
        if (u_topp && p->topp_decay && p->topp_min && p->topp_reset_ids && p->topp_initial_ps) {
            float tp = p->topp_ps[r];
            if (*id_out == p->topp_reset_ids[r]) {
                tp = p->topp_initial_ps[r];
            }
            else {
                tp = std::max(tp * p->topp_decay[r], p->topp_min[r]);
            }
            p->topp_ps[r] = tp;
        }
    }
    return 0;
}

/* setup_topk_runtime_args, layers/sampling_layers/TopKSamplingLayer.cu:28-77 (host arrays). */
void oracle_setup_topk_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size, float top_p,
                                    float* top_ps, int top_ps_size, uint8_t* skip_decode)
{
    for (int i = 0; i < batch; ++i) {
        uint32_t k = top_ks_size > 1 ? top_ks[i] : top_k;
        float    q = top_ps_size > 1 ? top_ps[i] : top_p;
        if (k == 0 && q == 0.0f) {
            k = 1;
        }
        if (k > 0 && q == 0.0f) {
            q = 1.0f;
        }
        top_ks[i]      = k > 1024u ? 1024u : k;
        top_ps[i]      = q < 0.0f ? 0.0f : (q > 1.0f ? 1.0f : q);
        skip_decode[i] = k == 0;
    }
}

/* set_topp_runtime_args, layers/sampling_layers/TopPSamplingLayer.cu:30-109 (host arrays). */
void oracle_setup_topp_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size, float top_p,
                                    float* top_ps, int top_ps_size, uint8_t* skip_decode, float* initial_top_p,
                                    float* decay_buf, const float* decay, float* min_buf, const float* top_p_min,
                                    int32_t* reset_buf, const uint32_t* reset_ids)
{
    for (int i = 0; i < batch; ++i) {
        uint32_t k = top_ks_size > 1 ? top_ks[i] : top_k;
        float    q = top_ps_size > 1 ? top_ps[i] : top_p;
        if (k == 0 && q == 0.0f) {
            k = 1;
        }
        top_ks[i]        = k;
        top_ps[i]        = q < 0.0f ? 0.0f : (q > 1.0f ? 1.0f : q);
        skip_decode[i]   = k > 0;
        initial_top_p[i] = top_ps[i];
        float d          = decay ? decay[i] : 1.0f;
        decay_buf[i]     = (d > 1.0f || d <= 0.0f) ? 1.0f : d;
        float m          = top_p_min ? top_p_min[i] : 1e-6f;
        min_buf[i]       = (m > 1.0f || m <= 0.0f) ? 0.5f : m;
        reset_buf[i]     = (int32_t)(reset_ids ? reset_ids[i] : (uint32_t)-1);
    }
}

/* stop_words_criterion, kernels/stop_criteria_kernels.cu:24-81, beam_width == 1. */
void oracle_stop_words(const int* output_ids, const int* stop_words, uint8_t* finished, int id_offset, int len,
                       int batch_size, int local_batch, int step)
{
    for (int b = 0; b < local_batch; ++b) {
        const int* words = stop_words + (size_t)b * 2 * len;
        const int* offs  = words + len;
        for (int i = 0; i < len; ++i) {
            if (offs[i] < 0) {
                continue;
            }
            const int item_end = offs[i], item_start = i > 0 ? offs[i - 1] : 0, item_size = item_end - item_start;
            bool      stop = false;
            if (step + 1 >= item_size) {
                stop = true;
                for (int j = item_size - 1; j >= 0; --j) {
                    int prev = output_ids[(size_t)(step - (item_size - 1) + j) * batch_size + id_offset + b];
                    if (prev != words[item_start + j]) {
                        stop = false;
                        break;
                    }
                }
            }
            if (stop) {
                finished[b] = 1;
            }
        }
    }
}

/* length_criterion, kernels/stop_criteria_kernels.cu:106-156: returns should_stop. */
int oracle_length_criterion(uint8_t* finished, const uint32_t* sequence_limit_length, int batch, int beam, int step)
{
    int sum = 0;
    for (int i = 0; i < batch * beam; ++i) {
        finished[i] |= (uint32_t)step >= sequence_limit_length[i / beam];
        sum += finished[i] ? 1 : 0;
    }
    return sum == batch * beam;
}

}  // extern "C"

// ================================================================================================
// Beam search step (beam_width > 1): OnlineBeamSearchLayer<T>::forward restated.
// ================================================================================================
namespace {

struct MDc {
    float m, d;
};
// reduce_md_op, kernels/online_softmax_beamsearch_kernels.cu:270-279
MDc md_op(MDc a, MDc b)
{
    bool a_bigger = a.m > b.m;
    MDc  hi = a_bigger ? a : b, lo = a_bigger ? b : a, r;
    r.d = hi.d + lo.d * expf(lo.m - hi.m);
    r.m = hi.m;
    return r;
}
// cub::BlockReduce (warp-shuffle reductions): inside a warp lane l takes op(own, lane l+off) for
// off = 1,2,4,8,16 while l+off stays inside the warp; warp results are folded left to right.
MDc block_reduce_md(std::vector<MDc> v)
{
    const int n = (int)v.size();
    std::vector<MDc> warp;
    for (int w0 = 0; w0 < n; w0 += 32) {
        MDc x[32];
        int cnt = std::min(32, n - w0);
        for (int l = 0; l < 32; ++l) {
            x[l] = l < cnt ? v[w0 + l] : MDc{0, 0};
        }
        for (int off = 1; off < 32; off <<= 1) {
            MDc t[32];
            for (int l = 0; l < 32; ++l) {
                t[l] = (l + off <= cnt - 1) ? md_op(x[l], x[l + off]) : x[l];
            }
            std::memcpy(x, t, sizeof(x));
        }
        warp.push_back(x[0]);
    }
    MDc r = warp[0];
    for (size_t w = 1; w < warp.size(); ++w) {
        r = md_op(r, warp[w]);
    }
    return r;
}

}  // namespace

extern "C" int oracle_beam_search_step(const ftb200_beam_params* p)
{
    const int     K = p->beam_width, V = p->vocab_size_padded, twoK = 2 * K, LB = p->local_batch_size;
    const TypeOps T{p->dtype == FTB200_F16};
    const RowView L{p->dtype, p->logits, (size_t)V};
    RowView       biasv{p->dtype, p->embedding_bias, (size_t)V};
    const bool    apply_temp = p->embedding_bias || p->temperature != 1.0f || p->vocab_size != V;
    const int     bbsize = p->batch_size * K;
    const int     rows = LB * K;
    const int     launcher_maxk = K <= 4 ? 4 : K <= 8 ? 8 : K <= 16 ? 16 : K <= 32 ? 32 : 64;
    const int     block_sz = launcher_maxk < 16 ? (launcher_maxk < 8 ? 256 : 128) : 64;
    int           voc_parts = 4;
    if (rows < 256) {
        voc_parts = std::min(128, (240 + rows - 1) / rows);
    }
    std::vector<int>   cand_id((size_t)rows * twoK);
    std::vector<float> cand_val((size_t)rows * twoK);
    const std::vector<uint8_t> fin0(p->finished, p->finished + rows);
    const std::vector<int>     seq0(p->sequence_length, p->sequence_length + rows);

    for (int bb = 0; bb < rows; ++bb) {
        const int b = bb / K, end_id = p->end_ids[b];
        std::vector<float> x(V);
        for (int v = 0; v < V; ++v) {
            x[v] = L.get(bb, v);
        }
        // invokeAddBiasApplyPenalties, kernels/beam_search_penalty_kernels.cu:175-267
        if (apply_temp) {
            const float inv = 1.0f / (p->temperature + 1e-6f);
            for (int v = 0; v < V; ++v) {
                if (v < p->vocab_size) {
                    float bv = p->embedding_bias ? biasv.get(0, v) : 0.0f;
                    x[v]     = T.is_half ? round_half(round_half(x[v] + bv) * round_half(inv)) : (x[v] + bv) * inv;
                }
                else {
                    x[v] = -T.max_t();
                }
            }
        }
        if (p->penalty_type != FTB200_PENALTY_NONE && p->step > 0
            && p->repetition_penalty != (p->penalty_type == FTB200_PENALTY_MULTIPLICATIVE ? 1.0f : 0.0f)) {
            const int   input_len = p->input_lengths ? p->input_lengths[bb] : p->max_input_length;
            const float pen       = T.rnd(p->repetition_penalty);
            std::vector<std::pair<int, float>> upd;
            auto add = [&](int id) {
                float lg = x[id];
                float nv = p->penalty_type == FTB200_PENALTY_ADDITIVE ? lg - pen : (lg > 0.0f ? lg / pen : lg * pen);
                upd.push_back({id, T.rnd(nv)});
            };
            const int* cur     = p->output_ids + (size_t)(p->step - 1) * bbsize + (size_t)p->ite * LB * K;
            const int* parents = p->parent_ids + (size_t)p->ite * K * LB;
            add(cur[bb]);
            int parent_beam = bb % K;
            for (int i = p->step - 2; i >= 0; --i) {
                if (i >= input_len && i < p->max_input_length) {
                    continue;
                }
                parent_beam = parents[(size_t)i * bbsize + b * K + parent_beam];
                add(p->output_ids[(size_t)i * bbsize + b * K + parent_beam]);
            }
            for (auto& u : upd) {
                x[u.first] = u.second;
            }
        }
        if (p->step - p->max_input_length < p->min_length
            && p->sequence_length[bb] + 1 - p->max_input_length < p->min_length) {
            x[end_id] = -T.max_t();
        }
        // stage 1 + stage 2, kernels/online_softmax_beamsearch_kernels.cu:366-514
        const bool fin = p->finished[bb];
        if (fin) {
            for (int v = 0; v < V; ++v) {
                x[v] = v == end_id ? T.max_t() : -T.max_t();
            }
        }
        const int        v_local = (V + voc_parts - 1) / voc_parts;
        std::vector<MDc> parts;
        for (int part = 0; part < voc_parts; ++part) {
            const int s0 = v_local * part, s1 = std::min(V, s0 + v_local);
            std::vector<MDc> thr(block_sz, MDc{-T.max_t(), 0.0f});
            for (int t = 0; t < block_sz; ++t) {
                for (int v = s0 + t; v < s1; v += block_sz) {
                    thr[t] = md_op(thr[t], MDc{x[v], 1.0f});
                }
            }
            parts.push_back(block_reduce_md(thr));
        }
        const int stage2_threads = voc_parts <= 32 ? 32 : voc_parts <= 64 ? 64 : 128;
        std::vector<MDc> st2(stage2_threads, MDc{-T.max_t(), 0.0f});
        for (int i = 0; i < voc_parts; ++i) {
            st2[i] = parts[i];
        }
        const MDc total = block_reduce_md(st2);
        std::vector<int> order(V);
        for (int v = 0; v < V; ++v) {
            order[v] = v;
        }
        std::partial_sort(order.begin(), order.begin() + std::min(twoK, V), order.end(), [&](int a, int c) {
            return x[a] != x[c] ? x[a] > x[c] : a < c;
        });
        const float d_total_log = logf(total.d);
        for (int i = 0; i < twoK; ++i) {
            const int v                      = i < V ? order[i] : -1;
            cand_id[(size_t)bb * twoK + i]  = v < 0 ? -1 : bb * V + v;
            cand_val[(size_t)bb * twoK + i] = v < 0 ? -INFINITY : T.rnd(x[v] - total.m - d_total_log + p->cum_log_probs[bb]);
        }
    }

    // batch_topk_kernel, :99-262
    const ftb200_beam_hyps* H = (p->beam_hyps && p->beam_hyps->num_beams) ? p->beam_hyps : nullptr;
    const int top_n = twoK <= 8 ? 8 : twoK <= 16 ? 16 : twoK <= 32 ? 32 : twoK <= 64 ? 64 : 128;
    for (int b = 0; b < LB; ++b) {
        const int    ncand = K * twoK, gbi = p->ite * LB + b, end_id = p->end_ids[b];
        const int*   x     = &cand_id[(size_t)b * ncand];
        const float* y     = &cand_val[(size_t)b * ncand];
        int*   z     = p->output_ids + (size_t)p->step * bbsize + (size_t)p->ite * LB * K + b * K;
        int*   par   = p->parent_ids + (size_t)p->step * bbsize + (size_t)p->ite * LB * K + b * K;
        float* v_cum = p->cum_log_probs + b * K;
        float* olp   = p->output_log_probs ? p->output_log_probs + (size_t)p->step * bbsize + (size_t)p->ite * LB * K : nullptr;
        std::vector<float> old_cum(v_cum, v_cum + K);
        bool skip = false;
        if (H) {
            if (H->num_beams[gbi] == 0) {
                H->min_normed_scores[gbi] = FLT_MAX;
            }
            else if (H->num_beams[gbi] == K) {
                skip = true;
            }
        }
        if (!skip) {
            const int len = fin0[b] ? seq0[b] : seq0[b] + 1;
            std::vector<float> e(ncand);
            std::vector<int>   ord;
            for (int i = 0; i < ncand; ++i) {
                float s = y[i];
                if (p->length_penalty != 0.0f && len != 1) {
                    s = T.rnd(s / T.rnd(powf((float)len, p->length_penalty)));
                }
                // `elem += diversity_rate * (T)i` (online_softmax_beamsearch_kernels.cu:157): in half the multiply
                // and the add are contracted into one fused multiply-add, so the sum is rounded once
                if (T.is_half) {
                    e[i] = round_half_from_double((double)T.rnd(p->diversity_rate) * (double)T.rnd((float)(i % K)) + (double)s);
                }
                else {
                    e[i] = std::fmaf(p->diversity_rate, (float)(i % K), s);
                }
                if (x[i] >= 0) {
                    ord.push_back(i);
                }
            }
            std::sort(ord.begin(), ord.end(), [&](int a, int c) { return e[a] != e[c] ? e[a] > e[c] : a < c; });
            int selected = 0;
            for (int i = 0; i < top_n && i < (int)ord.size(); ++i) {
                const int   ci = ord[i], word = x[ci];
                const float normed = e[ci];
                if (H && word % V == end_id) {
                    if (i < K) {
                        const int num_beam = H->num_beams[gbi];
                        int       beam_idx = num_beam;
                        if (num_beam == K) {
                            if (normed < H->min_normed_scores[gbi]) {
                                break;
                            }
                            for (int j = 0; j < K; ++j) {
                                if (H->normed_scores[gbi * twoK + j] == H->min_normed_scores[gbi]) {
                                    beam_idx = j;
                                    H->num_beams[gbi]--;
                                    H->min_normed_scores[gbi]        = FLT_MAX;
                                    H->normed_scores[gbi * twoK + j] = normed;
                                    for (int l = 0; l < K; ++l) {
                                        H->min_normed_scores[gbi] = std::min(H->min_normed_scores[gbi], H->normed_scores[gbi * twoK + l]);
                                    }
                                    break;
                                }
                            }
                        }
                        const size_t tgt = ((size_t)gbi * twoK + beam_idx) * p->max_seq_len;
                        H->output_ids_tgt[tgt + p->step] = end_id;
                        if (H->log_probs) {
                            H->log_probs[tgt + p->step] = y[ci] - old_cum[(word / V) % K];
                        }
                        int prev_id = (word / V) % K;
                        for (int j = p->step - 1; j >= 0; --j) {
                            const size_t src = (size_t)j * bbsize + (size_t)p->ite * LB * K + b * K + prev_id;
                            H->output_ids_tgt[tgt + j] = p->output_ids[src];
                            if (H->log_probs && p->output_log_probs) {
                                H->log_probs[tgt + j] = p->output_log_probs[src];
                            }
                            prev_id = p->parent_ids[src];
                        }
                        const int tb                = gbi * twoK + beam_idx;
                        H->sequence_lengths_tgt[tb] = p->step;
                        H->normed_scores[tb]        = normed;
                        H->min_normed_scores[gbi]   = std::min(H->min_normed_scores[gbi], normed);
                        H->num_beams[gbi]++;
                        H->cum_log_probs[tb] = y[ci];
                    }
                }
                else if ((H && i < twoK) || (!H && i < K)) {
                    z[selected] = word;
                    if (olp) {
                        olp[b * K + selected] = y[ci] - old_cum[(word / V) % K];
                    }
                    v_cum[selected] = y[ci];
                    ++selected;
                }
                if (selected >= K) {
                    break;
                }
            }
            if (H) {
                if (H->num_beams[b] < K) {
                    H->is_done[b] = 0;
                }
                else if (H->early_stopping) {
                    H->is_done[b] = 1;
                }
            }
        }
        // update_kernel, layers/beam_search_layers/OnlineBeamSearchLayer.cu:24-58
        std::vector<int> newseq(K);
        for (int k = 0; k < K; ++k) {
            const int idx = b * K + k;
            newseq[k]     = p->finished[idx] ? p->sequence_length[idx] : p->sequence_length[idx] + 1;
        }
        for (int k = 0; k < K; ++k) {
            const int idx = b * K + k, word = z[k], beam_id = (word / V) % K, word_id = word % V;
            p->sequence_length[idx] = newseq[beam_id];
            p->finished[idx]        = word_id == end_id;
            par[k]                  = beam_id;
            z[k]                    = word_id;
        }
        if (H && H->num_beams[gbi] == K) {
            for (int k = 0; k < K; ++k) {
                p->finished[b * K + k] = 1;
            }
        }
        // update_indir_cache_kernel, layers/beam_search_layers/BaseBeamSearchLayer.cu:23-50
        if (p->tgt_cache_indirection && p->src_cache_indirection) {
            const int Lq = p->max_seq_len, start = std::max(0, p->step + 1 - Lq), num = std::min(p->step + 1, Lq);
            for (int k = 0; k < K; ++k) {
                if (p->finished[b * K + k]) {
                    continue;
                }
                for (int t = start; t < start + num; ++t) {
                    const int    tc   = t % Lq;
                    const size_t base = (size_t)b * K * Lq;
                    p->tgt_cache_indirection[base + (size_t)k * Lq + tc] =
                        t == p->step ? k : p->src_cache_indirection[base + (size_t)par[k] * Lq + tc];
                }
            }
        }
    }
    return 0;
}

// invokeLogProbFromLogits, kernels/logprob_kernels.cu:142-183: log_probs_kernel (:36-103) per (step, sequence)
// with block_size threads (:165), then accumulate_log_probs (:105-140).  The partial maxima and sums follow the
// kernel's thread striding and its block reductions; expf/logf stand for the fast-math __expf/__logf.
// `log_probs` (may be null) receives the per-step values in the kernel's workspace layout.
extern "C" int oracle_log_prob_from_logits(float* cum_log_probs, float* log_probs, const void* logits, int dtype,
                                           const int* input_ids, const int* input_lengths, size_t max_input_length,
                                           size_t batch_size, size_t vocab_size, size_t vocab_size_padded,
                                           int batch_first)
{
    const int    nthr  = vocab_size < 1024 ? (int)((vocab_size + 31) / 32 * 32) : 1024;
    const float  lowest = dtype == FTB200_F16 ? -65504.0f : -FLT_MAX;
    const size_t steps = max_input_length - 1;
    const RowView L{dtype, logits, vocab_size_padded};
    std::vector<float> lp(steps * batch_size, 0.0f);
#pragma omp parallel for schedule(dynamic)
    for (long long r = 0; r < (long long)(steps * batch_size); ++r) {
        const size_t b = batch_first ? (size_t)r / steps : (size_t)r % batch_size;
        const size_t step = batch_first ? (size_t)r % steps : (size_t)r / batch_size;
        if ((int)step >= input_lengths[b] - 1) {
            continue;
        }
        const size_t row = batch_first ? b * max_input_length + step : step * batch_size + b;
        float        mx  = lowest;  // the maximum is exact whatever the order
        for (size_t v = 0; v < vocab_size; ++v) {
            mx = std::fmax(mx, L.get(row, v));
        }
        std::vector<float> partial(nthr, 0.0f);
        for (int t = 0; t < nthr; ++t) {
            float s = 0.0f;
            for (size_t v = t; v < vocab_size; v += nthr) {
                s += std::exp(L.get(row, v) - mx);
            }
            partial[t] = s;
        }
        const float  sum = butterfly_block_sum(partial, nthr);
        const size_t out = batch_first ? b * steps + step : step * batch_size + b;
        const size_t tok = batch_first ? b * max_input_length + step + 1 : (step + 1) * batch_size + b;
        lp[out]          = L.get(row, (size_t)input_ids[tok]) - mx - std::log(sum + 1e-9f);
    }
    for (size_t b = 0; b < batch_size; ++b) {
        std::vector<float> partial(nthr, 0.0f);
        const size_t       stride = batch_first ? 1 : batch_size;
        const float*       p = lp.data() + (batch_first ? b * steps : b);
        for (int t = 0; t < nthr; ++t) {
            float s = 0.0f;
            for (long long step = t; step < (long long)input_lengths[b] - 1 && step < (long long)steps; step += nthr) {
                s += p[(size_t)step * stride];
            }
            partial[t] = s;
        }
        cum_log_probs[b] = butterfly_block_sum(partial, nthr);
    }
    if (log_probs) {
        std::memcpy(log_probs, lp.data(), lp.size() * sizeof(float));
    }
    return 0;
}

// ---- caller-side steps ---------------------------------------------------------------------------------------

// decodingInitialize, kernels/decoding_kernels.cu:26-47.  cum_log_probs comes back as float whatever `dtype`
// (the value the typed store would hold).
extern "C" int oracle_decoding_initialize(uint8_t* finished, int* sequence_length, int* word_ids,
                                          float* cum_log_probs, int dtype, const int* sentence_ids, int batch_size,
                                          int beam_width, int max_input_length)
{
    float floor_v = -1e20f;
    if (dtype == FTB200_F16) {
        floor_v = -65504.0f;
    }
    else if (dtype == FTB200_BF16) {
        uint32_t u;
        std::memcpy(&u, &floor_v, 4);
        u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;  // round to nearest even on 16 bits
        std::memcpy(&floor_v, &u, 4);
    }
    for (int i = 0; i < batch_size * beam_width; ++i) {
        finished[i]        = 0;
        sequence_length[i] = max_input_length;
        if (word_ids != nullptr) {
            word_ids[i] = sentence_ids[i / beam_width];
        }
        cum_log_probs[i] = i % beam_width == 0 ? 0.0f : floor_v;
    }
    return 0;
}

// gatherTree, kernels/decoding_kernels.cu:452-583, one (entry, beam) at a time.  The length update that every
// thread of an entry repeats (:496-511) is done once per entry: the outcome when the entry's threads run in
// lockstep.
extern "C" int oracle_gather_tree(const ftb200_gather_tree_params* p)
{
    const int K = p->beam_width, B = p->batch_size;
    const int max_input_length = p->input_lengths == nullptr ? 0 : p->max_input_length;
    const int trimmed = p->max_prefix_soft_prompt_length + (p->max_input_length - p->max_input_without_prompt_length);
    for (int batch = 0; batch < B; ++batch) {
        const int prompt_len = p->prefix_soft_prompt_lengths ? p->prefix_soft_prompt_lengths[batch] : 0;
        const int virt = p->p_prompt_tuning_prompt_lengths ? p->p_prompt_tuning_prompt_lengths[batch] : 0;
        int       max_len = -1;
        for (int j = 0; j < K; ++j) {
            const int tmp_len = p->max_sequence_lengths[batch * K + j] + p->max_sequence_length_final_step;
            p->max_sequence_lengths[batch * K + j] = tmp_len - trimmed;
            if (p->response_input_lengths) {
                p->response_input_lengths[batch * K + j] =
                    (p->input_lengths ? p->input_lengths[batch * K + j] : 0) - virt - prompt_len;
            }
            max_len = std::max(max_len, tmp_len);
        }
        const int top = std::min(p->max_time, max_len);
        if (top <= 0) {
            continue;
        }
        const int end = p->end_tokens[batch];
        for (int beam = 0; beam < K; ++beam) {
            const int i = batch * K + beam;
            const int input_len = (p->input_lengths ? p->input_lengths[i] : 0) - virt;
            auto      ix = [&](int t, int bm) { return (size_t)B * K * t + (size_t)K * batch + bm; };
            const int shift = max_input_length - input_len + prompt_len;
            if (top - 1 - shift >= 0) {
                p->beams[ix(top - 1 - shift, beam)] = p->step_ids[ix(top - 1, beam)];
            }
            int  parent = p->parent_ids ? p->parent_ids[ix(top - 1, beam)] % K : 0;
            bool found_bad = false;
            for (int level = top - 2; level >= 0; --level) {
                if (level < prompt_len || (level >= input_len && level < max_input_length)) {
                    continue;
                }
                const int tgt = level >= max_input_length ? level - shift : level - prompt_len;
                if (parent < 0 || parent > K) {
                    p->beams[ix(tgt, beam)] = end;
                    parent                  = -1;
                    found_bad               = true;
                }
                else {
                    p->beams[ix(tgt, beam)] = p->step_ids[ix(level, parent)];
                    parent                  = p->parent_ids ? p->parent_ids[ix(level, parent)] % K : 0;
                }
            }
            for (int t = std::max(0, max_len - shift); t < p->max_time - p->max_prefix_soft_prompt_length; ++t) {
                p->beams[ix(t, beam)] = end;
            }
            if (!found_bad) {
                bool finished = false;
                for (int t = max_input_length == 0 ? 1 : max_input_length; t < top; ++t) {
                    if (finished) {
                        p->beams[ix(t, beam)] = end;
                    }
                    else if (p->beams[ix(t, beam)] == end) {
                        finished = true;
                    }
                }
            }
            const int out_len = p->max_time - trimmed;
            if (p->output_ids) {
                for (int j = 0; j < out_len; ++j) {
                    p->output_ids[(size_t)i * out_len + j] = p->beams[(size_t)j * B * K + i];
                }
            }
        }
    }
    return 0;
}

// finalize, kernels/decoding_kernels.cu:698-771: beam_width rounds of "largest remaining score, first index wins".
// Shared-memory slots past num_beams[b] are not initialised there; here they never match.
extern "C" int oracle_finalize(int* output_ids, int* sequence_lengths, float* cum_log_probs, float* output_log_probs,
                               const int* topk_output_ids, const int* topk_sequence_lengths, const float* scores,
                               const float* topk_cum_log_probs, const float* topk_log_probs, const int* num_beams,
                               int beam_width, int max_seq_len, int batch_size)
{
    const int K = beam_width;
    for (int b = 0; b < batch_size; ++b) {
        const int          n = std::max(0, std::min(num_beams[b], 2 * K));
        std::vector<float> s(scores + (size_t)b * 2 * K, scores + (size_t)b * 2 * K + n);
        std::vector<int>   rank(K, 0);
        for (int i = 0; i < K; ++i) {
            float mx = -FLT_MAX;
            for (int j = 0; j < n; ++j) {
                mx = std::max(mx, s[j]);
            }
            for (int j = 0; j < n; ++j) {
                if (s[j] == mx) {
                    rank[i] = j;
                    s[j]    = -FLT_MAX;
                    break;
                }
            }
        }
        for (int beam = 0; beam < K; ++beam) {
            const size_t src = (size_t)b * 2 * K + rank[beam];
            const int    len = topk_sequence_lengths[src];
            sequence_lengths[b * K + beam] = len;
            if (cum_log_probs) {
                cum_log_probs[b * K + beam] = topk_cum_log_probs[src];
            }
            for (int i = 0; i < len; ++i) {
                output_ids[((size_t)b * K + beam) * max_seq_len + i] = topk_output_ids[src * (max_seq_len + 1) + i + 1];
                if (output_log_probs) {
                    output_log_probs[((size_t)b * K + beam) * max_seq_len + i] =
                        topk_log_probs[src * (max_seq_len + 1) + i + 1];
                }
            }
        }
    }
    return 0;
}

// insertUnfinishedPath, kernels/beam_search_topk_kernels.cu:788-832.
extern "C" int oracle_insert_unfinished_path(const ftb200_beam_hyps* h, const int* output_ids_src,
                                             const int* parent_ids_src, const int* sequence_lengths_src,
                                             const float* log_probs_src, int max_seq_len, float length_penalty,
                                             const uint8_t* finished, const float* cum_log_probs, int batch_size,
                                             int beam_width)
{
    const int    K = beam_width;
    const size_t BK = (size_t)batch_size * K, row = (size_t)max_seq_len + 1;
    const bool   with_lp = h->log_probs != nullptr && log_probs_src != nullptr;
    for (int bid = 0; bid < batch_size; ++bid) {
        if (h->is_done[bid]) {
            continue;
        }
        const int tgt_start = h->num_beams[bid];
        for (int i = 0; i < K; ++i) {
            const size_t src = (size_t)bid * K + i, tgt = (size_t)bid * K * 2 + i + tgt_start;
            const int    length = sequence_lengths_src[src];
            h->output_ids_tgt[tgt * row + length] = output_ids_src[length * BK + src];
            if (with_lp) {
                h->log_probs[tgt * row + length] = log_probs_src[length * BK + src];
            }
            int prev = parent_ids_src[length * BK + src];
            for (int j = length - 1; j >= 0; --j) {
                prev = std::min(std::max(prev, 0), K - 1);
                const size_t g = j * BK + (size_t)bid * K + prev;
                h->output_ids_tgt[tgt * row + j] = output_ids_src[g];
                if (with_lp) {
                    h->log_probs[tgt * row + j] = log_probs_src[g];
                }
                prev = parent_ids_src[g];
            }
            h->sequence_lengths_tgt[tgt] = length;
            const int   n_tok = finished[src] ? length + 1 : length;
            const float cum = cum_log_probs[src];
            h->normed_scores[tgt] = (length_penalty == 0.0f || n_tok == 1) ? cum : cum / powf((float)n_tok, length_penalty);
            h->cum_log_probs[tgt] = cum;
            h->num_beams[bid]++;
        }
    }
    return 0;
}
