// Constants and the kernel argument block of the fused decode-sampling step.
#pragma once
#include <curand_kernel.h>

#include "common.cuh"
#include "ftb200.h"

namespace ftb200 {

constexpr int kThreads   = 256;
constexpr int kWarps     = kThreads / 32;
constexpr int kNB        = 4096;  // histogram buckets
constexpr int kCap       = 4096;  // candidate slots held in shared memory
constexpr int kUnroll    = 8;     // 16-byte loads in flight per thread
constexpr int kMaxTopK   = 1024;
constexpr int kLinScale  = 64;    // linear buckets per logit unit below the row maximum
constexpr int kWarpTile  = kCap / kWarps;
constexpr u32 kHashEmpty = 0xffffffffu;
constexpr u32 kFlagHist  = 1u;  // id occurs in the row's token history -> repetition / presence penalty
constexpr u32 kFlagDead  = 2u;  // banned word or min-length mask -> can never be selected

struct KParams {
    int dtype, batch_size, local_batch, ite, vocab, vocab_padded, step, max_input_len;
    const void* logits;
    const void* bias;
    const int*  end_ids;
    const int*  input_lengths;
    int*        output_ids;
    const int*  bad_words;
    int         bad_words_len, bad_words_shared;
    const float* temperature;
    int          apply_temp;
    const float* rep_penalty;
    int          penalty_type, apply_rep;
    const int*   min_lengths;
    int          apply_minlen;
    curandState_t* topk_states;
    const u32*     topk_ks;
    const float*   topk_ps;
    const uint8_t* topk_skip;
    int            max_top_k;
    curandState_t* topp_states;
    float*         topp_ps;
    const uint8_t* topp_skip;
    const float*   topp_initial;
    const float*   topp_decay;
    const float*   topp_min;
    const int*     topp_reset;
    int*     seq_len;
    uint8_t* finished;
    float*   cum_log_probs;
    float*   out_log_probs;
    const int* row_order;
    u64*     vp_out;        // vocabulary-parallel local pass: [local_batch][1 + vp_cap] records, else null
    int      vp_cap;
    int      vocab_offset;  // first token id of this shard of the vocabulary (0 when not sharded)
    u32*     ticket;
    // Rows the single-pass kernel leaves to decode_sampling_kernel: it appends them to redo_rows and counts them
    // in redo_count; decode_sampling_kernel launched with row_count_dev != null serves row_order[0 .. *row_count_dev).
    u32*       redo_count;
    int*       redo_rows;
    const u32* row_count_dev;
    u64*     trace;           // optional per-row timeline: {row, CTA, start ns, end ns} per ticket, else null
    u64*     scratch;         // per-CTA candidate overflow area
    size_t   scratch_stride;  // u64 entries per CTA
    int      hash_slots, hash_shift, flag_words;
};

}  // namespace ftb200
