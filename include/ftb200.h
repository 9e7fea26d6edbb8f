/*
 * ftb200.h - C ABI of the B200 (sm_100a) decode-sampling kernels.
 *
 * This is the boundary a FasterTransformer build binds to in place of its own
 * kernels/ directory for the per-step token-selection path.  Every entry point
 * is `extern "C"`, takes plain pointers and sizes, returns an int status
 * (0 = OK, see ftb200_status) and never throws.  All device pointers belong to
 * the caller; all work is enqueued on the caller's stream.
 *
 * Each declaration names the reference interface it replaces, as
 * path:line inside the FasterTransformer source tree.
 */
#ifndef FTB200_H
#define FTB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    FTB200_OK              = 0,
    FTB200_INVALID_ARG     = 1, /* null pointer, bad shape, unsupported dtype ...                      */
    FTB200_DOMAIN_ERROR    = 2, /* top-k outside [1,1024]: the reference throws std::domain_error      */
    FTB200_CUDA_ERROR      = 3, /* a CUDA runtime call failed; see ftb200_last_error_string()          */
    FTB200_WORKSPACE_SMALL = 4, /* workspace_bytes below ftb200_sampling_workspace_bytes()             */
    FTB200_UNSUPPORTED     = 5, /* shape outside what the kernels handle (e.g. history too long)       */
    FTB200_TIMEOUT         = 6  /* a bounded wait ran out                                              */
} ftb200_status;

typedef enum {
    FTB200_F32  = 0,
    FTB200_F16  = 1,
    FTB200_BF16 = 2 /* not in the reference: computed as the fp32 path on the up-cast values */
} ftb200_dtype;

/* Mirrors RepetitionPenaltyType, kernels/penalty_types.h:24-28. */
typedef enum {
    FTB200_PENALTY_ADDITIVE       = 0, /* presence penalty:   x - theta                    */
    FTB200_PENALTY_MULTIPLICATIVE = 1, /* repetition penalty: x < 0 ? x * theta : x / theta */
    FTB200_PENALTY_NONE           = 2
} ftb200_penalty_type;

const char* ftb200_version(void);
/* Text of the last failure on the calling thread ("" if none). */
const char* ftb200_last_error_string(void);

/* ------------------------------------------------------------------------------------------
 * curand state set-up.  `states` is curandState_t[n] (XORWOW, 48 bytes each), the same layout
 * the reference keeps per layer (layers/sampling_layers/BaseSamplingLayer.h:38).
 * Replaces invokeCurandInitialize / invokeCurandBatchInitialize,
 * kernels/sampling_topk_kernels.cu:39-65.  `seeds` (device, n values) wins over `seed` when non-null.
 * ------------------------------------------------------------------------------------------ */
int ftb200_curand_init(void* states, int n, unsigned long long seed, const unsigned long long* seeds, void* stream);

/* Draw `n_draws` uniforms per row from COPIES of the states (the states are not advanced).
 * out is device float [n_draws, n].  Test/diagnostic helper; curand_uniform as the kernels call it. */
int ftb200_curand_peek_uniforms(const void* states, int n, int n_draws, float* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Runtime-argument normalisation.
 * top-k layer: setup_topk_runtime_args<1024>, layers/sampling_layers/TopKSamplingLayer.cu:28-77
 *   k==0&&p==0 -> k=1;  k>0&&p==0 -> p=1;  k clipped to 1024;  p clipped to [0,1];  skip = (k==0).
 * top-p layer: set_topp_runtime_args, layers/sampling_layers/TopPSamplingLayer.cu:30-109
 *   k==0&&p==0 -> k=1;  p clipped;  skip = (k>0);  initial_top_p/decay/min/reset-id buffers filled.
 * top_ks/top_ps are device arrays [batch] that already hold the per-row values when
 * top_ks_size/top_ps_size > 1 and are overwritten with the normalised values.
 * ------------------------------------------------------------------------------------------ */
int ftb200_setup_topk_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size, float top_p,
                                   float* top_ps, int top_ps_size, uint8_t* skip_decode, void* stream);
int ftb200_setup_topp_runtime_args(int batch, uint32_t top_k, uint32_t* top_ks, int top_ks_size, float top_p,
                                   float* top_ps, int top_ps_size, uint8_t* skip_decode, float* initial_top_p,
                                   float* top_p_decay_buf, const float* top_p_decay, float* top_p_min_buf,
                                   const float* top_p_min, int32_t* top_p_reset_ids_buf,
                                   const uint32_t* top_p_reset_ids, void* stream);

/* ------------------------------------------------------------------------------------------
 * One fused decode-sampling step.
 *
 * Replaces, for beam_width == 1, everything DynamicDecodeLayer::forward launches between the
 * logits GEMM and the stop criteria (layers/DynamicDecodeLayer.cc:247-283, 389-445):
 *   invokeBanBadWords                       kernels/ban_bad_words.cu:88-120
 *   invokeBatchApplyTemperaturePenalty      kernels/sampling_penalty_kernels.cu:181-206
 *   invokeBatchApplyRepetitionPenalty       kernels/sampling_penalty_kernels.cu:426-459
 *   invokeMinLengthPenalty                  kernels/sampling_penalty_kernels.cu:502-517
 *   invokeAddBiasEndMask                    kernels/sampling_topk_kernels.cu:96-110
 *   invokeAddBiasSoftMax                    kernels/sampling_topp_kernels.cu:1347-1356
 *   invokeBatchTopKSampling                 kernels/sampling_topk_kernels.cu:345-396
 *   invokeTopPInitialize / invokeBatchTopPSampling   kernels/sampling_topp_kernels.cu:790-799, 1006-1170
 *   invokeComputeToppDecay                  kernels/sampling_topp_kernels.cu:1410-1427
 * The logits are read, never written.  Results (ids, flags, lengths) equal the reference's.
 * ------------------------------------------------------------------------------------------ */
typedef struct ftb200_sampling_params {
    /* ---- geometry ---- */
    int dtype;             /* ftb200_dtype of logits and embedding_bias                              */
    int batch_size;        /* rows of the whole request batch = row stride of output_ids            */
    int local_batch_size;  /* rows handled by this call                                              */
    int ite;               /* micro-batch index; local row r is global row ite*local_batch_size + r  */
    int vocab_size;
    int vocab_size_padded; /* row stride of logits; columns >= vocab_size are masked                 */
    int step;              /* position being generated; ids land in output_ids[step, :]              */
    int max_input_length;

    /* ---- inputs (device) ---- */
    const void* logits;         /* [local_batch_size, vocab_size_padded], first local row            */
    const void* embedding_bias; /* [vocab_size_padded] or null                                       */
    const int*  end_ids;        /* [local_batch_size]                                                */
    const int*  input_lengths;  /* [local_batch_size] or null                                        */
    int*        output_ids;     /* [max_seq_len, batch_size], whole tensor: history in, new ids out  */
    const int*  bad_words;      /* [2, bad_words_len] (shared) or [local_batch_size, 2, len]; null ok */
    int         bad_words_len;
    int         bad_words_shared;

    /* ---- per-row runtime arguments (device, [local_batch_size]) and the host-side gating the
     *      reference applies before each penalty kernel (BaseSamplingLayer.cc:302-349) ---- */
    const float* temperature;
    int          apply_temperature; /* embedding_bias != null || any temperature != 1              */
    const float* repetition_penalty;
    int          penalty_type;      /* ftb200_penalty_type                                          */
    int          apply_repetition;  /* step > 1 && type != NONE && any row != default               */
    const int*   min_lengths;
    int          apply_min_length;  /* any min_length > step - max_input_length                     */

    /* ---- top-k layer state (null topk_states: layer absent) ---- */
    void*           topk_states; /* curandState_t[local_batch_size]                                  */
    const uint32_t* topk_ks;     /* normalised k per row                                             */
    const float*    topk_ps;     /* normalised p per row                                             */
    const uint8_t*  topk_skip;   /* 1 = row not handled by the top-k layer                           */
    int             max_top_k;   /* max k over the WHOLE batch (selects the reference's block sizes,
                                    sampling_topk_kernels.cu:388-392, which fix its tie order)      */

    /* ---- top-p layer state (null topp_states: layer absent) ---- */
    void*          topp_states;
    float*         topp_ps;      /* in/out: decayed after the step                                   */
    const uint8_t* topp_skip;
    const float*   topp_initial_ps;
    const float*   topp_decay;
    const float*   topp_min;
    const int32_t* topp_reset_ids;

    /* ---- outputs (device, first local row; null = not wanted) ---- */
    int*     sequence_length;
    uint8_t* finished; /* bool[local_batch_size], in/out */
    float*   cum_log_probs;
    float*   output_log_probs; /* [local_batch_size] slice for this step */

    /* ---- scheduling hint (device, [local_batch_size], a permutation of 0..local_batch_size-1; null = row
     *      order).  Rows are started in this order; listing the expensive rows first (top-p, large k)
     *      shortens the tail of the launch.  Results do not depend on it. ---- */
    const int* row_order;

    /* ---- scratch ---- */
    void*  workspace;
    size_t workspace_bytes;
    void*  stream;
} ftb200_sampling_params;

/* Bytes of scratch ftb200_decode_step_sampling needs for this shape (depends on dtype, vocab and the
 * SM count of the current device).  Replaces the nullptr-workspace size queries of
 * invokeTopKSampling / invokeTopPSampling (TopKSamplingLayer.cu:93-108, TopPSamplingLayer.cu:120-141). */
int ftb200_sampling_workspace_bytes(int dtype, int local_batch_size, int vocab_size_padded, size_t* bytes);

/* Limits (FTB200_UNSUPPORTED beyond them): vocab_size_padded <= 2^21; with a repetition or presence penalty
 * on, step + bad_words_len + 2 <= 4096 - the columns that need individual treatment (token history, banned
 * words, min-length mask) are kept in a shared-memory table, two slots per column, and 8192 slots is what fits
 * next to the other tables of the kernel.  Without a penalty the history does not enter the table and only
 * bad_words_len + 2 <= 4096 applies. */
int ftb200_decode_step_sampling(const ftb200_sampling_params* p);

/* Number of kernels the last ftb200_decode_step_sampling call on this thread launched. */
int ftb200_last_launch_count(void);

/* Diagnostic, no counterpart in the reference: when `device_buf` is not null every later
 * ftb200_decode_step_sampling call writes records of 32 uint64 each, {row, CTA, start, end, 28 phase marks}
 * with the times in nanoseconds of the GPU's global timer (a mark the row did not pass is left untouched).
 * With R = local_batch_size the record of the single-pass top-k kernel's ticket t lies at device_buf[32 t..],
 * the general kernel's at device_buf[32 (R + t)..] and the single-pass top-p kernel's at
 * device_buf[32 (2 R + t)..]: the buffer must hold 3 * 256 bytes per row of the call.  Pass null to switch the
 * trace off (the default). */
int ftb200_set_row_trace(uint64_t* device_buf);

/* Diagnostic, no counterpart in the reference.  ftb200_decode_step_sampling serves 16-bit logits of at least
 * 16400 columns (no embedding bias, no log-probabilities) in up to three launches: a single-pass kernel for the
 * top-p rows and one for the top-k rows side by side (one read of each row for a top-k row, several rows in
 * flight per SM), then the general kernel on the rows those two leave behind; ftb200_vocab_parallel_local does
 * the same with the top-k rows' kernel in its record form.  ftb200_set_single_pass(0) sends every row to the
 * general kernel (the results are the same either way; tests compare the two); 1 (the default) restores the
 * single-pass kernels.  Process-wide. */
int ftb200_set_single_pass(int on);

/* ------------------------------------------------------------------------------------------
 * Bad-word ban as a stand-alone call (the fused step above already applies it; this entry serves
 * callers that use the kernel by itself, e.g. the beam-search path).  Writes -inf into the logits.
 * Replaces invokeBanBadWords, kernels/ban_bad_words.cu:88-120 (same argument meaning).
 * ------------------------------------------------------------------------------------------ */
int ftb200_ban_bad_words(void* logits, int dtype, const int* output_ids, const int* parent_ids, int batch_size,
                         int local_batch_size, int beam_width, const int* bad_words, int share_words,
                         int bad_words_len, int id_offset, int vocab_size_padded, int step, void* stream);

/* ------------------------------------------------------------------------------------------
 * Stop criteria after the ids of `step` are written: stop-word match, sequence-length limit, and the
 * count of finished sequences.  One launch.
 * Replaces invokeStopWordsCriterion (kernels/stop_criteria_kernels.cu:83-104) and
 * invokeLengthCriterion (:129-157).  The reference spins on a pinned int without bound; here the count
 * is copied to `finished_count_host` (pinned, 1 int) on the stream and ftb200_wait_should_stop waits for
 * it with a deadline.
 *   stop_words            [local_batch_size, 2, stop_words_len] for the local rows, or null
 *   finished              bool[batch_size*beam_width], whole batch
 *   sequence_limit_length uint32[batch_size], or null (then only stop words run and nothing is counted)
 * ------------------------------------------------------------------------------------------ */
int ftb200_stop_criteria(const int* output_ids, const int* parent_ids, const int* stop_words, int stop_words_len,
                         uint8_t* finished, const uint32_t* sequence_limit_length, int id_offset,
                         int local_batch_size, int batch_size, int beam_width, int step, int* finished_count_dev,
                         int* finished_count_host, void* stream);

/* Waits until the work enqueued on `stream` so far is done (at most timeout_ms, FTB200_TIMEOUT after
 * that) and reports *should_stop = (finished_count_host[0] == batch_size*beam_width). */
int ftb200_wait_should_stop(const int* finished_count_host, int batch_size, int beam_width, void* stream,
                            int timeout_ms, int* should_stop);

/* ------------------------------------------------------------------------------------------
 * The fused decode-sampling step without a caller-provided workspace.
 * No counterpart in the reference: FasterTransformer always draws its buffers from an IAllocator.
 *
 * For hosts that cannot allocate device memory at the point of call - a server whose memory pool owns the
 * whole GPU, a plug-in callback that is forbidden to allocate - the scratch of ftb200_decode_step_sampling is
 * a fixed area of ftb200_static_scratch_bytes() (64 MiB) built into the library; every GPU that loads the
 * library holds it until the process exits.  `workspace` and `workspace_bytes` of the argument block are
 * ignored; everything else means what it means above and the results are the same.  No cudaMalloc, cudaFree
 * or other allocating call is made, and no stream or event is created: the kernels of the step run one
 * after the other on `stream`.
 *
 *   - A shape whose ftb200_sampling_workspace_bytes() exceeds the area is refused with
 *     FTB200_WORKSPACE_SMALL.  For local_batch_size up to twice the SM count the need is
 *     256 + ceil256(4 * rows) + rows * ceil256(vocab_size_padded) * 8 bytes, which admits 65 rows per call at
 *     vocab 128256 (66 are refused) and 262 at 32000: slice the batch with `ite` / `local_batch_size`.
 *   - The first call on each device looks up the device address of the area (cudaGetSymbolAddress), and the
 *     first call of each kernel variant on a device sets its shared-memory attribute and asks its occupancy.
 *     That set-up belongs before any stream capture on that device; whether the call itself can be recorded
 *     in a capture is not stated here either way.
 *   - All calls on a device share the one area.  Calls that may overlap on the GPU (different streams, or
 *     several host threads) race on it: serialise them, or give the overlapping ones their own workspace
 *     through ftb200_decode_step_sampling.
 * ------------------------------------------------------------------------------------------ */
size_t ftb200_static_scratch_bytes(void);
int    ftb200_decode_step_sampling_static(const ftb200_sampling_params* p);

/* ------------------------------------------------------------------------------------------
 * Beam search, one step (beam_width > 1), one launch.
 *
 * Replaces what OnlineBeamSearchLayer<T>::forward launches
 * (layers/beam_search_layers/BaseBeamSearchLayer.cu:181-289, OnlineBeamSearchLayer.cu:88-175):
 *   invokeAddBiasApplyPenalties   kernels/beam_search_penalty_kernels.cu:175-267
 *   invokeTopkSoftMax             kernels/online_softmax_beamsearch_kernels.cu:549-699
 *                                 (stage-1 / stage-2 online soft-max + top-2K, batch_topk_kernel)
 *   invokeUpdate                  layers/beam_search_layers/OnlineBeamSearchLayer.cu:24-86
 *   update_indir_cache_kernelLauncher   layers/beam_search_layers/BaseBeamSearchLayer.cu:23-79
 * Temperature, penalty, min_length, diversity and length penalty are scalars per call, as in the
 * reference (DynamicDecodeLayer.cc:286-386 loops over sub-batches when they differ per row).
 * The logits are read, never written.
 * sequence_length follows the parent beam as the reference's update_kernel does when the beams of a
 * batch entry run in lockstep (every length incremented, then gathered); the reference itself has no
 * barrier between the two (OnlineBeamSearchLayer.cu:40-46) and leaves timing-dependent lengths when
 * the beams of an entry span two warps (beam widths that do not divide 32).
 * ------------------------------------------------------------------------------------------ */

/* Mirrors BeamHypotheses, kernels/beam_search_topk_kernels.h:31-58 (device pointers; num_beams == null
 * switches the archive of finished beams off). */
typedef struct ftb200_beam_hyps {
    int*     output_ids_tgt;       /* [batch, 2K, max_seq_len] */
    int*     sequence_lengths_tgt; /* [batch, 2K] */
    float*   cum_log_probs;        /* [batch, 2K] */
    float*   normed_scores;        /* [batch, 2K] */
    float*   log_probs;            /* [batch, 2K, max_seq_len] or null */
    float*   min_normed_scores;    /* [batch] */
    int*     num_beams;            /* [batch] or null */
    uint8_t* is_done;              /* [batch] */
    int      early_stopping;
} ftb200_beam_hyps;

typedef struct ftb200_beam_params {
    int dtype, batch_size, local_batch_size, ite, beam_width;
    int vocab_size, vocab_size_padded, step, max_input_length, max_seq_len;

    const void* logits;         /* [local_batch_size, beam_width, vocab_size_padded] */
    const void* embedding_bias; /* [vocab_size_padded] or null */
    const int*  end_ids;        /* [local_batch_size] */
    const int*  input_lengths;  /* [local_batch_size * beam_width] or null */

    float temperature;
    float repetition_penalty;
    int   penalty_type;         /* ftb200_penalty_type */
    int   min_length;
    float diversity_rate;
    float length_penalty;

    int*     output_ids;        /* [max_seq_len, batch_size * beam_width], whole tensor */
    int*     parent_ids;        /* [max_seq_len, batch_size * beam_width], whole tensor */
    uint8_t* finished;          /* [local_batch_size * beam_width] */
    int*     sequence_length;   /* [local_batch_size * beam_width] */
    float*   cum_log_probs;     /* [local_batch_size * beam_width] */
    float*   output_log_probs;  /* [max_seq_len, batch_size * beam_width] whole tensor, or null */
    const int* src_cache_indirection; /* [local_batch_size, beam_width, max_seq_len] or null */
    int*       tgt_cache_indirection; /* same shape, or null */
    const ftb200_beam_hyps* beam_hyps; /* host pointer to the struct above, or null */

    void*  workspace;
    size_t workspace_bytes;
    void*  stream;
} ftb200_beam_params;

int ftb200_beam_workspace_bytes(int local_batch_size, int beam_width, size_t* bytes);
int ftb200_beam_search_step(const ftb200_beam_params* p);

/* ------------------------------------------------------------------------------------------
 * Vocabulary-parallel sampling: each GPU holds a column shard [local_batch, V/n] of the logits
 * (the tensor-parallel lm_head before FT's all-gather, models/multi_gpu_gpt/ParallelGpt.cc:1394-1435).
 * Instead of gathering the full fp32 logits and sampling redundantly on every rank, each rank
 *   1. ftb200_vocab_parallel_local: runs the fused penalties + selection on its shard and emits, per
 *      row, one record of (2 + cap) 64-bit words: the count, then up to cap (value, global column)
 *      entries, then one statistics word.  Top-k rows: every column whose value reaches the shard's
 *      k-th value (whole tie class included).  Top-p rows: the shard's largest columns (cap - 64 of
 *      them when cap > 128, else cap / 2) and, in the statistics word, two floats (maximum of the
 *      shard's final values << 32 | sum of exp(value - maximum));
 *   2. exchanges the records with ONE all-gather (ncclAllGather of local_batch*(2+cap)*8 bytes);
 *   3. ftb200_vocab_parallel_merge: merges the n records of a row and draws with the row's curand
 *      state.  All ranks hold the same states, so all ranks produce the same id - no broadcast.
 * Top-k rows: the ids equal what ftb200_decode_step_sampling returns on the gathered row (and
 * therefore the reference's).  Top-p rows: the (maximum, sum) pairs are combined as an online
 * soft-max combines them (reduce_md_op, kernels/online_softmax_beamsearch_kernels.cu:270-279), so the
 * denominator is not summed in the single-GPU order; a draw within rounding of a boundary may pick
 * the neighbouring column, everything else is the same id.
 * `p` is the same argument block; in step 1 `logits`/`vocab_size`/`vocab_size_padded` describe the
 * shard and token ids (history, bad words, end id) stay global; `vocab_offset` is the shard's first
 * column.  No log-probs.  A row that cannot be decided from the records - more than `cap` columns in
 * play on some shard, a top-p nucleus larger than the union of what the shards sent - is reported
 * through *overflow_count (device int, incremented) and gets id -1; its curand state, finished flag
 * and sequence length are left as they were, so the caller can repeat it - with a larger cap, or by
 * gathering that row's logits and calling ftb200_decode_step_sampling with ite = row,
 * local_batch_size = 1 (what fastertransformer_b200.VocabParallelSampler does) - and get the draw
 * the single-GPU path makes.
 * ------------------------------------------------------------------------------------------ */
int ftb200_vocab_parallel_local(const ftb200_sampling_params* p, int vocab_offset, int cap, uint64_t* records);
int ftb200_vocab_parallel_merge(const ftb200_sampling_params* p, const uint64_t* gathered, int n_ranks, int cap,
                                int* overflow_count);

/* ------------------------------------------------------------------------------------------------
 * Log-probability of given token ids under the soft-max of context logits, summed per sequence.
 * Replaces invokeLogProbFromLogits<T> (kernels/logprob_kernels.h:23-35, kernels/logprob_kernels.cu:142-183)
 * with the same argument order and meaning; `dtype` stands for the template parameter:
 *   cum_log_probs[b] = sum over step < input_lengths[b] - 1 of
 *                      log softmax(logits[step, b, :vocab_size])[input_ids[step + 1, b]]
 * logits:    [max_input_length, batch_size, vocab_size_padded], or batch-major when batch_first != 0;
 * input_ids: [max_input_length, batch_size], or [batch_size, max_input_length] when batch_first != 0;
 * workspace: device memory of at least sizeof(float) * max_input_length * batch_size bytes (the
 *            per-step log-probs land there in the reference's layout, log_probs_kernel :36-103).
 * Differences: row offsets are 64-bit (the reference's are int and wrap past 2^31 elements); an id
 * outside [0, vocab_size_padded) gives NaN instead of an unchecked read; bf16 is accepted.
 * ------------------------------------------------------------------------------------------ */
int ftb200_log_prob_from_logits(float* cum_log_probs, const void* logits, int dtype, const int* input_ids,
                                const int* input_lengths, size_t max_input_length, size_t batch_size,
                                size_t vocab_size, size_t vocab_size_padded, void* workspace, size_t workspace_size,
                                void* stream, int batch_first);

/* ------------------------------------------------------------------------------------------------
 * Caller-side steps either side of the per-step path (device pointers throughout).
 * ------------------------------------------------------------------------------------------ */

/* invokeDecodingInitialize<T> (kernels/decoding_kernels.h:25-34, decoding_kernels.cu:26-64): finished = 0,
 * sequence_length = max_input_length, word_ids[i] = sentence_ids[i / beam_width] (when word_ids is given),
 * cum_log_probs = 0 for beam 0 of each entry and -1e20 (-65504 for half) for the others.  `dtype` is the type
 * of cum_log_probs. */
int ftb200_decoding_initialize(uint8_t* finished, int* sequence_length, int* word_ids, void* cum_log_probs,
                               int dtype, const int* sentence_ids, int batch_size, int beam_width,
                               int max_input_length, void* stream);

/* Mirrors gatherTreeParam, kernels/decoding_kernels.h:123-145, field for field. */
typedef struct ftb200_gather_tree_params {
    int*       beams;                          /* [max_time, batch_size, beam_width] out */
    int*       max_sequence_lengths;           /* [batch_size, beam_width] in/out */
    int        max_sequence_length_final_step;
    const int* input_lengths;                  /* [batch_size, beam_width] or null */
    int*       response_input_lengths;         /* [batch_size, beam_width] out, or null */
    int        max_time;
    int        batch_size;
    int        beam_width;
    const int* step_ids;                       /* [max_time, batch_size, beam_width] */
    const int* parent_ids;                     /* same shape, or null (every parent 0) */
    const int* end_tokens;                     /* [batch_size] */
    int        max_input_length;
    const int* prefix_soft_prompt_lengths;     /* [batch_size] or null */
    const int* p_prompt_tuning_prompt_lengths; /* [batch_size] or null */
    int        max_input_without_prompt_length;
    int        max_prefix_soft_prompt_length;
    int*       output_ids;                     /* [batch_size, beam_width, out_len] out, or null */
    void*      stream;
} ftb200_gather_tree_params;

/* invokeGatherTree(gatherTreeParam) (kernels/decoding_kernels.cu:452-646): follows each beam's parents back
 * from its last step, drops prompt and padding positions, pads with the entry's end token, leaves nothing but
 * end tokens after the first one, and writes the transposed ids.  Set max_input_length = 1 and the prompt
 * fields to null/0 for the two short overloads (:585-634).
 * Differences: the reference lets every thread of an entry rewrite all of the entry's max_sequence_lengths
 * (racy once an entry's beams span two warps); here each length is updated once, which is what the lockstep
 * case gives, and response_input_lengths[i] uses beam i's own input length.  Writes at a negative time index
 * (sequence shorter than its padding) are skipped instead of issued.  beam_width <= 1024. */
int ftb200_gather_tree(const ftb200_gather_tree_params* p);

/* invokeFinalize (kernels/decoding_kernels.h:155-168, decoding_kernels.cu:698-804): ranks the archived
 * hypotheses of each entry by score (first index wins ties) and copies the best beam_width of them, without
 * the start token.  topk_output_ids / topk_log_probs: [batch, 2 * beam_width, max_seq_len + 1]; output_ids /
 * output_log_probs: [batch, beam_width, max_seq_len].  Entries past num_beams[b] resolve to archive slot 0
 * (what the reference finds once its candidates are used up). */
int ftb200_finalize(int* output_ids, int* sequence_lengths, float* cum_log_probs, float* output_log_probs,
                    const int* topk_output_ids, const int* topk_sequence_lengths, const float* scores,
                    const float* topk_cum_log_probs, const float* topk_log_probs, const int* num_beams,
                    int beam_width, int max_seq_len, int batch_size, void* stream);

/* invokeInsertUnfinishedPath (kernels/beam_search_topk_kernels.h:104-109, beam_search_topk_kernels.cu:788-843):
 * appends the beam_width live beams of every entry that is not done to its archive, following parent ids back
 * to step 0.  The BeamHypotheses fields the reference reads travel as arguments: `hyps` holds the archive
 * (rows of max_seq_len + 1 here, as the reference indexes them in this kernel), the *_src tables are
 * [step, batch_size * beam_width].  An out-of-range parent id is clamped instead of followed.
 * beam_width <= 512. */
int ftb200_insert_unfinished_path(const ftb200_beam_hyps* hyps, const int* output_ids_src, const int* parent_ids_src,
                                  const int* sequence_lengths_src, const float* log_probs_src, int max_seq_len,
                                  float length_penalty, const uint8_t* finished, const float* cum_log_probs,
                                  int batch_size, int beam_width, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FTB200_H */
