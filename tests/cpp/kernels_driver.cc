// TEST INFRASTRUCTURE.  Drives the C++ free functions of fastertransformer_b200/shim/decode_kernels.h
// (invokeLogProbFromLogits, invokeDecodingInitialize, invokeGatherTree, invokeFinalize,
// invokeInsertUnfinishedPath) on seeded inputs and compares them with the CPU restatement
// (oracle/libft_oracle.so, linked in).  Prints one "PASS <name>" or "FAIL <name> ..." line per check and
// exits non-zero on any failure.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "decode_kernels.h"

extern "C" {
int oracle_log_prob_from_logits(float*, float*, const void*, int, const int*, const int*, size_t, size_t, size_t,
                                size_t, int);
int oracle_decoding_initialize(uint8_t*, int*, int*, float*, int, const int*, int, int, int);
int oracle_gather_tree(const ftb200_gather_tree_params*);
int oracle_finalize(int*, int*, float*, float*, const int*, const int*, const float*, const float*, const float*,
                    const int*, int, int, int);
int oracle_insert_unfinished_path(const ftb200_beam_hyps*, const int*, const int*, const int*, const float*, int,
                                  float, const uint8_t*, const float*, int, int);
}

namespace ft = fastertransformer;

static uint64_t g_state = 12345;
static uint32_t rnd()
{
    g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)(g_state >> 33);
}
static int   rint_in(int lo, int hi) { return lo + (int)(rnd() % (uint32_t)(hi - lo)); }  // [lo, hi)
static float runit() { return (float)(rnd() & 0xffff) / 65536.0f; }

template<typename U>
static U* dev(const std::vector<U>& v)
{
    U* d = nullptr;
    cudaMalloc(&d, sizeof(U) * (v.size() ? v.size() : 1));
    cudaMemcpy(d, v.data(), sizeof(U) * v.size(), cudaMemcpyHostToDevice);
    return d;
}
template<typename U>
static std::vector<U> host(const U* d, size_t n)
{
    std::vector<U> v(n);
    cudaMemcpy(v.data(), d, sizeof(U) * n, cudaMemcpyDeviceToHost);
    return v;
}
static int g_fail = 0;
template<typename U>
static void expect_equal(const char* name, const std::vector<U>& a, const std::vector<U>& b, double tol = 0.0)
{
    size_t bad = a.size() != b.size();
    for (size_t i = 0; i < a.size() && i < b.size(); ++i) {
        const double d = std::fabs((double)a[i] - (double)b[i]);
        bad += d > tol * (1.0 + std::fabs((double)b[i]));
    }
    if (bad) {
        printf("FAIL %s: %zu of %zu differ\n", name, bad, a.size());
        ++g_fail;
    }
    else {
        printf("PASS %s\n", name);
    }
}

static void check_log_probs()
{
    const size_t       L = 9, B = 5, V = 777, VP = 784;
    std::vector<float> x(L * B * VP);
    std::vector<half>  xh(x.size());
    for (size_t i = 0; i < x.size(); ++i) {
        x[i]  = runit() * 6 - 3;
        xh[i] = __float2half(x[i]);
    }
    std::vector<int> ids(L * B), len(B);
    for (auto& v : ids) {
        v = rint_in(0, (int)V);
    }
    for (auto& v : len) {
        v = rint_in(1, (int)L + 1);
    }
    float *d_cum = dev(std::vector<float>(B)), *d_ws = dev(std::vector<float>(L * B));
    int *  d_ids = dev(ids), *d_len = dev(len);
    {
        float* d_x = dev(x);
        ft::invokeLogProbFromLogits(d_cum, d_x, d_ids, d_len, L, B, V, VP, d_ws, sizeof(float) * L * B, nullptr);
        std::vector<float> want(B);
        oracle_log_prob_from_logits(want.data(), nullptr, x.data(), FTB200_F32, ids.data(), len.data(), L, B, V, VP, 0);
        expect_equal("invokeLogProbFromLogits<float>", host(d_cum, B), want, 1e-5);
    }
    {
        half* d_x = dev(xh);
        ft::invokeLogProbFromLogits(d_cum, d_x, d_ids, d_len, L, B, V, VP, d_ws, sizeof(float) * L * B, nullptr);
        std::vector<float> want(B);
        oracle_log_prob_from_logits(want.data(), nullptr, xh.data(), FTB200_F16, ids.data(), len.data(), L, B, V, VP, 0);
        expect_equal("invokeLogProbFromLogits<half>", host(d_cum, B), want, 1e-5);
    }
    bool threw = false;
    try {
        ft::invokeLogProbFromLogits(d_cum, (const float*)d_ws, d_ids, d_len, L, B, V, VP, d_ws, 4, nullptr);
    }
    catch (const std::runtime_error&) {
        threw = true;
    }
    expect_equal("invokeLogProbFromLogits small workspace throws", std::vector<int>{threw}, std::vector<int>{1});
}

static void check_initialize()
{
    const int        B = 6, K = 4, n = B * K;
    std::vector<int> sid(B);
    for (auto& v : sid) {
        v = rint_in(0, 500);
    }
    bool*  d_fin;
    cudaMalloc(&d_fin, n);
    int *  d_seq = dev(std::vector<int>(n)), *d_word = dev(std::vector<int>(n)), *d_sid = dev(sid);
    float* d_cum = dev(std::vector<float>(n));
    ft::invokeDecodingInitialize(d_fin, d_seq, d_word, d_cum, d_sid, B, K, 33, nullptr);
    std::vector<uint8_t> fin(n);
    std::vector<int>     seq(n), word(n);
    std::vector<float>   cum(n);
    oracle_decoding_initialize(fin.data(), seq.data(), word.data(), cum.data(), FTB200_F32, sid.data(), B, K, 33);
    expect_equal("invokeDecodingInitialize finished", host((uint8_t*)d_fin, n), fin);
    expect_equal("invokeDecodingInitialize sequence_length", host(d_seq, n), seq);
    expect_equal("invokeDecodingInitialize word_ids", host(d_word, n), word);
    expect_equal("invokeDecodingInitialize cum_log_probs", host(d_cum, n), cum);
}

static void check_gather_tree()
{
    const int        B = 7, K = 4, T = 40, M = 6, n = B * K;
    std::vector<int> step(T * n), par(T * n), end(B), in_len(n), seq(n);
    for (auto& v : step) {
        v = rint_in(0, 9);
    }
    for (auto& v : par) {
        v = rint_in(0, K);
    }
    for (int b = 0; b < B; ++b) {
        end[b]       = rint_in(0, 9);
        const int il = rint_in(1, M + 1);
        for (int k = 0; k < K; ++k) {
            in_len[b * K + k] = il;
            seq[b * K + k]    = rint_in(M, T);
        }
    }
    // the full parameter block
    {
        ft::gatherTreeParam p;
        int *d_beams = dev(std::vector<int>(T * n, -7)), *d_seq = dev(seq), *d_out = dev(std::vector<int>(T * n, -7));
        p.beams = d_beams, p.max_sequence_lengths = d_seq, p.max_sequence_length_final_step = 1;
        p.input_lengths = dev(in_len), p.max_time = T, p.batch_size = B, p.beam_width = K;
        p.step_ids = dev(step), p.parent_ids = dev(par), p.end_tokens = dev(end), p.max_input_length = M;
        p.max_input_without_prompt_length = M, p.output_ids = d_out;
        ft::invokeGatherTree(p);
        std::vector<int>          beams(T * n, -7), seq2 = seq, out(T * n, -7);
        ftb200_gather_tree_params o{};
        o.beams = beams.data(), o.max_sequence_lengths = seq2.data(), o.max_sequence_length_final_step = 1;
        o.input_lengths = in_len.data(), o.max_time = T, o.batch_size = B, o.beam_width = K;
        o.step_ids = step.data(), o.parent_ids = par.data(), o.end_tokens = end.data(), o.max_input_length = M;
        o.max_input_without_prompt_length = M, o.output_ids = out.data();
        oracle_gather_tree(&o);
        expect_equal("invokeGatherTree(param) beams", host(d_beams, T * n), beams);
        expect_equal("invokeGatherTree(param) output_ids", host(d_out, T * n), out);
        expect_equal("invokeGatherTree(param) lengths", host(d_seq, n), seq2);
    }
    // the short form
    {
        int *d_beams = dev(std::vector<int>(T * n, -7)), *d_seq = dev(seq);
        ft::invokeGatherTree(d_beams, d_seq, T, B, K, dev(step), dev(par), dev(end), nullptr);
        std::vector<int>          beams(T * n, -7), seq2 = seq;
        ftb200_gather_tree_params o{};
        o.beams = beams.data(), o.max_sequence_lengths = seq2.data(), o.max_time = T, o.batch_size = B;
        o.beam_width = K, o.step_ids = step.data(), o.parent_ids = par.data(), o.end_tokens = end.data();
        o.max_input_length = 1;
        oracle_gather_tree(&o);
        expect_equal("invokeGatherTree(short) beams", host(d_beams, T * n), beams);
        expect_equal("invokeGatherTree(short) lengths", host(d_seq, n), seq2);
    }
}

static void check_archive_and_finalize()
{
    const int            B = 5, K = 4, L = 21, n = B * K;
    std::vector<int>     ids((L + 1) * n), par((L + 1) * n), len(n), nb(B, 0);
    std::vector<float>   lp((L + 1) * n), cum(n);
    std::vector<uint8_t> fin(n), done(B, 0);
    for (auto& v : ids) {
        v = rint_in(0, 1000);
    }
    for (auto& v : par) {
        v = rint_in(0, K);
    }
    for (auto& v : lp) {
        v = -runit();
    }
    for (int i = 0; i < n; ++i) {
        len[i] = rint_in(1, L + 1);
        cum[i] = -20 * runit();
        fin[i] = rnd() % 3 == 0;
    }
    done[2] = 1;
    const size_t         slots = (size_t)B * 2 * K;
    std::vector<int>     t_ids(slots * (L + 1), -7), t_len(slots, -7);
    std::vector<float>   t_cum(slots, -7), t_nrm(slots, -7), t_lp(slots * (L + 1), -7);
    ft::BeamHypotheses   h;
    h.output_ids_tgt = dev(t_ids), h.sequence_lengths_tgt = dev(t_len), h.cum_log_probs = dev(t_cum);
    h.normed_scores = dev(t_nrm), h.log_probs = dev(t_lp), h.num_beams = dev(nb);
    h.is_done = (bool*)dev(done);
    h.output_ids_src = dev(ids), h.parent_ids_src = dev(par), h.sequence_lengths_src = dev(len);
    h.log_probs_src = dev(lp), h.max_seq_len = L, h.length_penalty = 0.7f;
    ft::invokeInsertUnfinishedPath(h, (const bool*)dev(fin), dev(cum), B, K, nullptr);

    ftb200_beam_hyps o{};
    std::vector<int> nb2 = nb;
    o.output_ids_tgt = t_ids.data(), o.sequence_lengths_tgt = t_len.data(), o.cum_log_probs = t_cum.data();
    o.normed_scores = t_nrm.data(), o.log_probs = t_lp.data(), o.num_beams = nb2.data(), o.is_done = done.data();
    oracle_insert_unfinished_path(&o, ids.data(), par.data(), len.data(), lp.data(), L, 0.7f, fin.data(), cum.data(),
                                  B, K);
    expect_equal("invokeInsertUnfinishedPath output_ids_tgt", host(h.output_ids_tgt, t_ids.size()), t_ids);
    expect_equal("invokeInsertUnfinishedPath log_probs", host(h.log_probs, t_lp.size()), t_lp);
    expect_equal("invokeInsertUnfinishedPath normed_scores", host(h.normed_scores, slots), t_nrm, 2e-6);
    expect_equal("invokeInsertUnfinishedPath num_beams", host(h.num_beams, B), nb2);

    // rank what was archived (entry 2 holds nothing: num_beams 0)
    int *  d_out = dev(std::vector<int>(n * L, -7)), *d_len = dev(std::vector<int>(n, -7));
    float *d_cum = dev(std::vector<float>(n, -7)), *d_lp = dev(std::vector<float>(n * L, -7));
    ft::invokeFinalize(d_out, d_len, d_cum, d_lp, h.output_ids_tgt, h.sequence_lengths_tgt, h.normed_scores,
                       h.cum_log_probs, h.log_probs, h.num_beams, K, L, B, nullptr);
    std::vector<int>   out(n * L, -7), olen(n, -7);
    std::vector<float> ocum(n, -7), olp(n * L, -7);
    // slot 0 of the empty entry holds the fill value as its length: keep the copy loop away from it
    t_len[2 * 2 * K] = 0;
    cudaMemcpy(h.sequence_lengths_tgt, t_len.data(), sizeof(int) * slots, cudaMemcpyHostToDevice);
    ft::invokeFinalize(d_out, d_len, d_cum, d_lp, h.output_ids_tgt, h.sequence_lengths_tgt, h.normed_scores,
                       h.cum_log_probs, h.log_probs, h.num_beams, K, L, B, nullptr);
    oracle_finalize(out.data(), olen.data(), ocum.data(), olp.data(), t_ids.data(), t_len.data(), t_nrm.data(),
                    t_cum.data(), t_lp.data(), nb2.data(), K, L, B);
    expect_equal("invokeFinalize output_ids", host(d_out, n * L), out);
    expect_equal("invokeFinalize sequence_lengths", host(d_len, n), olen);
    expect_equal("invokeFinalize cum_log_probs", host(d_cum, n), ocum);
    expect_equal("invokeFinalize output_log_probs", host(d_lp, n * L), olp);
}

int main()
{
    check_log_probs();
    check_initialize();
    check_gather_tree();
    check_archive_and_finalize();
    cudaDeviceSynchronize();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        printf("FAIL cuda: %s\n", cudaGetErrorString(e));
        return 2;
    }
    return g_fail ? 1 : 0;
}
