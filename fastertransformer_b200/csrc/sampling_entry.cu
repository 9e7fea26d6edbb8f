// extern "C" entry of the fused decode-sampling step: argument checks, shared-memory plan, launch.
#include <atomic>
#include <mutex>

#include "sampling_params.cuh"

namespace ftb200 {

template<int DT>
int sampling_occupancy(size_t smem, int* per_sm);
template<int DT>
int sampling_launch(const KParams& K, int grid, size_t smem, cudaStream_t st);
extern template int sampling_occupancy<FTB200_F32>(size_t, int*);
extern template int sampling_occupancy<FTB200_F16>(size_t, int*);
extern template int sampling_occupancy<FTB200_BF16>(size_t, int*);
extern template int sampling_launch<FTB200_F32>(const KParams&, int, size_t, cudaStream_t);
extern template int sampling_launch<FTB200_F16>(const KParams&, int, size_t, cudaStream_t);
extern template int sampling_launch<FTB200_BF16>(const KParams&, int, size_t, cudaStream_t);
template<int DT, bool TOPP, int VP = 0>
int fast_sampling_occupancy(size_t smem, int* per_sm);
template<int DT, bool TOPP, int VP = 0>
int fast_sampling_launch(const KParams& K, int grid, size_t smem, cudaStream_t st);
extern template int fast_sampling_occupancy<FTB200_F16, false, 1>(size_t, int*);
extern template int fast_sampling_occupancy<FTB200_BF16, false, 1>(size_t, int*);
extern template int fast_sampling_launch<FTB200_F16, false, 1>(const KParams&, int, size_t, cudaStream_t);
extern template int fast_sampling_launch<FTB200_BF16, false, 1>(const KParams&, int, size_t, cudaStream_t);
extern template int fast_sampling_occupancy<FTB200_F16, false>(size_t, int*);
extern template int fast_sampling_occupancy<FTB200_BF16, false>(size_t, int*);
extern template int fast_sampling_launch<FTB200_F16, false>(const KParams&, int, size_t, cudaStream_t);
extern template int fast_sampling_launch<FTB200_BF16, false>(const KParams&, int, size_t, cudaStream_t);
extern template int fast_sampling_occupancy<FTB200_F16, true>(size_t, int*);
extern template int fast_sampling_occupancy<FTB200_BF16, true>(size_t, int*);
extern template int fast_sampling_launch<FTB200_F16, true>(const KParams&, int, size_t, cudaStream_t);
extern template int fast_sampling_launch<FTB200_BF16, true>(const KParams&, int, size_t, cudaStream_t);
size_t fast_smem_for(int hash_slots, int vocab_padded, bool topp);
int    fast_max_history();
int    fast_max_words();
template<int DT>
int vp_merge_launch(const KParams& K, const u64* gathered, int nranks, int* overflow, int grid, cudaStream_t st);
extern template int vp_merge_launch<FTB200_F32>(const KParams&, const u64*, int, int*, int, cudaStream_t);
extern template int vp_merge_launch<FTB200_F16>(const KParams&, const u64*, int, int*, int, cudaStream_t);
extern template int vp_merge_launch<FTB200_BF16>(const KParams&, const u64*, int, int*, int, cudaStream_t);

static int sm_count()
{
    // per device (a process may drive several GPUs, one thread each)
    constexpr int           kMaxDev = 64;
    static std::atomic<int> n[kMaxDev];
    int                     dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDev) {
        dev = 0;
    }
    int v = n[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        if (v <= 0) {
            v = 148;
        }
        n[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

constexpr int kMaxCtasPerSm = 2;

static u64* g_row_trace = nullptr;  // diagnostic timeline buffer, see ftb200_set_row_trace

static size_t scratch_stride_for(int vocab_padded)
{
    return ((size_t)vocab_padded + 255) / 256 * 256;
}

// Workspace: 256-byte header (row tickets, length of the row list), the list of rows the single-pass kernel
// leaves to decode_sampling_kernel (one int per local row), then one candidate area per resident CTA.
static size_t redo_list_bytes(int local_batch)
{
    return ((size_t)local_batch * sizeof(int) + 255) / 256 * 256;
}

static int g_fast_path = 1;  // see ftb200_set_single_pass

// Second stream of the single-pass step (one per device, made on first use) with the two events of its fork and join.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t  fork = nullptr, join = nullptr;
    std::mutex   use;  // held from the record of `fork` to the wait on `join`: two host threads on one device
                       // share the stream and the events, and a wait takes the latest record of its event
};
static int side_stream(SideStream** out)
{
    constexpr int     kMaxDev = 64;
    static SideStream g_side[kMaxDev];
    static std::mutex g_mu;
    int               dev = 0;
    FTB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) {
        set_error("ftb200_decode_step_sampling: device ordinal out of range");
        return FTB200_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    SideStream& s = g_side[dev];
    if (s.stream == nullptr) {
        FTB_CUDA_CHECK(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
        FTB_CUDA_CHECK(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
        FTB_CUDA_CHECK(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
    }
    *out = &s;
    return FTB200_OK;
}

}  // namespace ftb200

using namespace ftb200;

extern "C" int ftb200_sampling_workspace_bytes(int dtype, int local_batch_size, int vocab_size_padded, size_t* bytes)
{
    if (bytes == nullptr || local_batch_size < 0 || vocab_size_padded <= 0 || dtype < 0 || dtype > 2) {
        set_error("ftb200_sampling_workspace_bytes: invalid argument");
        return FTB200_INVALID_ARG;
    }
    size_t ctas = (size_t)sm_count() * kMaxCtasPerSm;
    if ((size_t)local_batch_size < ctas) {
        ctas = (size_t)local_batch_size;
    }
    *bytes = 256 + redo_list_bytes(local_batch_size) + ctas * scratch_stride_for(vocab_size_padded) * sizeof(u64);
    return FTB200_OK;
}

// Argument checks, translation to the kernel argument block, shared-memory plan and grid size, shared by
// the entry points below.  `need_workspace` is false for the vocabulary-parallel merge.
static int plan_sampling(const ftb200_sampling_params* p, KParams& K, size_t& smem, int& grid, bool need_workspace)
{
    if (p == nullptr || p->logits == nullptr || p->end_ids == nullptr || p->output_ids == nullptr) {
        set_error("ftb200_decode_step_sampling: null logits / end_ids / output_ids");
        return FTB200_INVALID_ARG;
    }
    if (p->dtype < 0 || p->dtype > 2 || p->local_batch_size < 0 || p->vocab_size <= 0
        || p->vocab_size_padded < p->vocab_size || p->batch_size < p->local_batch_size || p->step < 0) {
        set_error("ftb200_decode_step_sampling: bad shape or dtype");
        return FTB200_INVALID_ARG;
    }
    if (p->vocab_size_padded > (1 << 21)) {
        set_error("ftb200_decode_step_sampling: vocab_size_padded above 2^21 is not supported");
        return FTB200_UNSUPPORTED;
    }
    if (p->topk_states == nullptr && p->topp_states == nullptr) {
        set_error("ftb200_decode_step_sampling: neither a top-k nor a top-p layer state was given");
        return FTB200_INVALID_ARG;
    }
    if (p->topk_states != nullptr) {
        if (p->topk_ks == nullptr || p->topk_ps == nullptr) {
            set_error("ftb200_decode_step_sampling: top-k layer needs topk_ks and topk_ps");
            return FTB200_INVALID_ARG;
        }
        if (p->max_top_k < 1 || p->max_top_k > kMaxTopK) {
            set_error("top-k kernel supports 1<=k<=1024 but got k=" + std::to_string(p->max_top_k));
            return FTB200_DOMAIN_ERROR;
        }
    }
    if (p->topp_states != nullptr && p->topp_ps == nullptr) {
        set_error("ftb200_decode_step_sampling: top-p layer needs topp_ps");
        return FTB200_INVALID_ARG;
    }
    if ((p->apply_temperature && p->temperature == nullptr) || (p->apply_repetition && p->repetition_penalty == nullptr)
        || (p->apply_min_length && (p->min_lengths == nullptr || p->sequence_length == nullptr))) {
        set_error("ftb200_decode_step_sampling: a penalty is switched on without its per-row array");
        return FTB200_INVALID_ARG;
    }
    size_t need = 0;
    ftb200_sampling_workspace_bytes(p->dtype, p->local_batch_size, p->vocab_size_padded, &need);
    if (need_workspace && (p->workspace == nullptr || p->workspace_bytes < need)) {
        set_error("ftb200_decode_step_sampling: workspace too small, need " + std::to_string(need) + " bytes");
        return FTB200_WORKSPACE_SMALL;
    }

    K.vp_out       = nullptr;
    K.vp_cap       = 0;
    K.vocab_offset = 0;
    K.dtype            = p->dtype;
    K.batch_size       = p->batch_size;
    K.local_batch      = p->local_batch_size;
    K.ite              = p->ite;
    K.vocab            = p->vocab_size;
    K.vocab_padded     = p->vocab_size_padded;
    K.step             = p->step;
    K.max_input_len    = p->max_input_length;
    K.logits           = p->logits;
    K.bias             = p->embedding_bias;
    K.end_ids          = p->end_ids;
    K.input_lengths    = p->input_lengths;
    K.output_ids       = p->output_ids;
    K.bad_words        = p->bad_words_len > 0 ? p->bad_words : nullptr;
    K.bad_words_len    = p->bad_words_len;
    K.bad_words_shared = p->bad_words_shared;
    K.temperature      = p->temperature;
    K.apply_temp       = p->apply_temperature ? 1 : 0;
    K.rep_penalty      = p->repetition_penalty;
    K.penalty_type     = p->penalty_type;
    K.apply_rep        = (p->apply_repetition && p->penalty_type != FTB200_PENALTY_NONE) ? 1 : 0;
    K.min_lengths      = p->min_lengths;
    K.apply_minlen     = p->apply_min_length ? 1 : 0;
    K.topk_states      = (curandState_t*)p->topk_states;
    K.topk_ks          = p->topk_ks;
    K.topk_ps          = p->topk_ps;
    K.topk_skip        = p->topk_skip;
    K.max_top_k        = p->topk_states != nullptr ? p->max_top_k : 1;
    K.topp_states      = (curandState_t*)p->topp_states;
    K.topp_ps          = p->topp_ps;
    K.topp_skip        = p->topp_skip;
    K.topp_initial     = p->topp_initial_ps;
    K.topp_decay       = (p->topp_decay && p->topp_min && p->topp_reset_ids && p->topp_initial_ps) ? p->topp_decay : nullptr;
    K.topp_min         = p->topp_min;
    K.topp_reset       = p->topp_reset_ids;
    K.seq_len          = p->sequence_length;
    K.finished         = p->finished;
    K.cum_log_probs    = p->cum_log_probs;
    K.out_log_probs    = p->output_log_probs;
    K.row_order        = p->row_order;
    K.trace            = g_row_trace;

    // shared-memory plan: candidates, histogram, 1024 floats, vector flags, token hash with two values per slot
    const int epv      = p->dtype == FTB200_F32 ? 4 : 8;
    K.flag_words       = ((p->vocab_size_padded / epv + 32) / 32 + 1) & ~1;  // even: what follows stays 8-byte aligned
    int specials       = (K.apply_rep ? p->step : 0) + (K.bad_words ? p->bad_words_len : 0) + 2;
    int slots          = 64;
    while (slots < 2 * specials) {
        slots <<= 1;
    }
    // (a large table costs the kernels resident CTAs: above 2048 slots it may be three quarters full)
    if (slots > 2048 && 3 * (slots / 2) >= 4 * specials) {
        slots /= 2;
    }
    K.hash_slots = slots;
    int lg       = 0;
    while ((1 << lg) < slots) {
        ++lg;
    }
    K.hash_shift = 32 - lg;
    smem         = (size_t)kCap * 8 + (size_t)kNB * 4 + 1024 * 4 + (size_t)K.flag_words * 4 + (size_t)slots * 12 + 32
                   + (size_t)kThreads * 16 * 2;
    if (smem > 200 * 1024 || specials > 4096) {
        set_error("ftb200_decode_step_sampling: token history too long for the shared-memory hash");
        return FTB200_UNSUPPORTED;
    }

    int per_sm = 0, rc;
    switch (p->dtype) {
        case FTB200_F32: rc = sampling_occupancy<FTB200_F32>(smem, &per_sm); break;
        case FTB200_F16: rc = sampling_occupancy<FTB200_F16>(smem, &per_sm); break;
        default: rc = sampling_occupancy<FTB200_BF16>(smem, &per_sm); break;
    }
    if (rc != FTB200_OK) {
        return rc;
    }
    if (per_sm < 1) {
        set_error("ftb200_decode_step_sampling: kernel does not fit on an SM");
        return FTB200_UNSUPPORTED;
    }
    if (per_sm > kMaxCtasPerSm) {
        per_sm = kMaxCtasPerSm;
    }
    grid = sm_count() * per_sm;
    if (grid > p->local_batch_size) {
        grid = p->local_batch_size;
    }
    K.ticket         = (u32*)p->workspace;
    K.redo_count     = nullptr;
    K.redo_rows      = nullptr;
    K.row_count_dev  = nullptr;
    K.scratch        = (u64*)((char*)p->workspace + 256 + redo_list_bytes(p->local_batch_size));
    K.scratch_stride = scratch_stride_for(p->vocab_size_padded);
    return FTB200_OK;
}

extern "C" int ftb200_set_row_trace(uint64_t* device_buf)
{
    g_row_trace = (u64*)device_buf;
    return FTB200_OK;
}

// One fused step.  `fork` allows the second stream of the single-pass kernels (made on first use); without it
// the same kernels run one after the other on the caller's stream and nothing is created.
namespace ftb200 {
int decode_step_sampling_impl(const ftb200_sampling_params* p, bool fork);
}

extern "C" int ftb200_decode_step_sampling(const ftb200_sampling_params* p)
{
    return decode_step_sampling_impl(p, true);
}

int ftb200::decode_step_sampling_impl(const ftb200_sampling_params* p, bool fork)
{
    reset_launch_count();
    KParams K;
    size_t  smem = 0;
    int     grid = 0;
    int     rc   = plan_sampling(p, K, smem, grid, true);
    if (rc != FTB200_OK) {
        return rc;
    }
    if (p->local_batch_size == 0) {
        return FTB200_OK;
    }
    cudaStream_t st = (cudaStream_t)p->stream;
    FTB_CUDA_CHECK(cudaMemsetAsync(K.ticket, 0, 256, st));
    // 16-bit logits without a bias, log-probs or timeline: the single-pass kernel serves the rows first and
    // leaves a list of the rows it does not cover; decode_sampling_kernel then works that list off.
    const bool single_pass = g_fast_path && p->dtype != FTB200_F32 && K.bias == nullptr && K.cum_log_probs == nullptr
                             && K.out_log_probs == nullptr && p->vocab_size_padded <= (1 << 20)
                             && p->vocab_size >= 16384 + 16 && (K.apply_rep ? p->step : 0) <= fast_max_history()
                             && (K.bad_words != nullptr ? K.bad_words_len : 0) <= fast_max_words();
    if (single_pass) {
        const size_t fsmem = fast_smem_for(K.hash_slots, p->vocab_size_padded, false);
        const size_t psmem = fast_smem_for(K.hash_slots, p->vocab_size_padded, true);
        const bool   f16   = p->dtype == FTB200_F16;
        int          fper = 0, pper = 0;
        rc = f16 ? fast_sampling_occupancy<FTB200_F16, false>(fsmem, &fper) :
                   fast_sampling_occupancy<FTB200_BF16, false>(fsmem, &fper);
        if (rc == FTB200_OK && K.topp_states != nullptr) {
            rc = f16 ? fast_sampling_occupancy<FTB200_F16, true>(psmem, &pper) :
                       fast_sampling_occupancy<FTB200_BF16, true>(psmem, &pper);
        }
        if (rc != FTB200_OK) {
            return rc;
        }
        if (fper >= 1 && (K.topp_states == nullptr || pper >= 1)) {
            KParams F    = K;
            F.redo_count = K.ticket + 1;
            F.redo_rows  = (int*)((char*)p->workspace + 256);
            // The rows of the top-p layer have a kernel of their own (it wants more registers than the top-k rows'
            // kernel can spare); the two run side by side, the top-p one on a second stream that forks from and
            // joins the caller's.  Each walks the row list and skips the other's rows.
            SideStream*                  side      = nullptr;
            std::unique_lock<std::mutex> side_use;
            const bool  topp_only = K.topp_states != nullptr && K.topk_states == nullptr;  // no fork, one launch
            if (K.topp_states != nullptr) {
                cudaStream_t pst = st;
                if (fork && !topp_only) {
                    rc = side_stream(&side);
                    if (rc != FTB200_OK) {
                        return rc;
                    }
                    side_use = std::unique_lock<std::mutex>(side->use);
                    FTB_CUDA_CHECK(cudaEventRecord(side->fork, st));
                    FTB_CUDA_CHECK(cudaStreamWaitEvent(side->stream, side->fork, 0));
                    pst = side->stream;
                }
                int pgrid = sm_count() * pper;
                pgrid     = pgrid < p->local_batch_size ? pgrid : p->local_batch_size;
                rc = f16 ? fast_sampling_launch<FTB200_F16, true>(F, pgrid, psmem, pst) :
                           fast_sampling_launch<FTB200_BF16, true>(F, pgrid, psmem, pst);
                if (rc != FTB200_OK) {
                    return rc;
                }
                note_launch(1);
                if (side != nullptr) {
                    FTB_CUDA_CHECK(cudaEventRecord(side->join, side->stream));
                }
            }
            if (!topp_only) {
                int fgrid = sm_count() * fper;
                fgrid     = fgrid < p->local_batch_size ? fgrid : p->local_batch_size;
                rc = f16 ? fast_sampling_launch<FTB200_F16, false>(F, fgrid, fsmem, st) :
                           fast_sampling_launch<FTB200_BF16, false>(F, fgrid, fsmem, st);
                if (rc != FTB200_OK) {
                    return rc;
                }
                note_launch(1);
            }
            if (side != nullptr) {
                FTB_CUDA_CHECK(cudaStreamWaitEvent(st, side->join, 0));
                side_use.unlock();
            }
            K.ticket        = K.ticket + 2;
            K.row_order     = F.redo_rows;
            K.row_count_dev = F.redo_count;
            if (K.trace != nullptr) {
                K.trace += (size_t)p->local_batch_size * 32;  // the general kernel's records follow the single-pass kernel's
            }
        }
    }
    switch (p->dtype) {
        case FTB200_F32: rc = sampling_launch<FTB200_F32>(K, grid, smem, st); break;
        case FTB200_F16: rc = sampling_launch<FTB200_F16>(K, grid, smem, st); break;
        default: rc = sampling_launch<FTB200_BF16>(K, grid, smem, st); break;
    }
    if (rc == FTB200_OK) {
        note_launch(1);
    }
    return rc;
}

extern "C" int ftb200_set_single_pass(int on)
{
    g_fast_path = on ? 1 : 0;
    return FTB200_OK;
}

// ---- vocabulary-parallel sampling (the logits of a row are split over several GPUs by column) ------
extern "C" int ftb200_vocab_parallel_local(const ftb200_sampling_params* p, int vocab_offset, int cap,
                                           uint64_t* records)
{
    reset_launch_count();
    if (records == nullptr || cap < 1 || cap > kCap || vocab_offset < 0) {
        set_error("ftb200_vocab_parallel_local: invalid argument");
        return FTB200_INVALID_ARG;
    }
    if (p != nullptr && (p->cum_log_probs != nullptr || p->output_log_probs != nullptr)) {
        set_error("ftb200_vocab_parallel_local: log-probs are not available with a sharded vocabulary");
        return FTB200_UNSUPPORTED;
    }
    KParams K;
    size_t  smem = 0;
    int     grid = 0;
    int     rc   = plan_sampling(p, K, smem, grid, true);
    if (rc != FTB200_OK) {
        return rc;
    }
    if (p->local_batch_size == 0) {
        return FTB200_OK;
    }
    K.vp_out       = (u64*)records;
    K.vp_cap       = cap;
    K.vocab_offset = vocab_offset;
    cudaStream_t st = (cudaStream_t)p->stream;
    FTB_CUDA_CHECK(cudaMemsetAsync(K.ticket, 0, 256, st));
    // 16-bit shards of at least 16 k columns: the single-pass kernel in its record form serves the top-k rows and
    // leaves a list of the others (top-p rows of the statistics form, rows it cannot decide) to the kernel below
    const bool single_pass = g_fast_path && p->dtype != FTB200_F32 && K.bias == nullptr && p->vocab_size_padded <= (1 << 20)
                             && p->vocab_size >= 16384 + 16 && (K.apply_rep ? p->step : 0) <= fast_max_history()
                             && (K.bad_words != nullptr ? K.bad_words_len : 0) <= fast_max_words();
    if (single_pass) {
        const size_t fsmem = fast_smem_for(K.hash_slots, p->vocab_size_padded, false);
        const bool   f16   = p->dtype == FTB200_F16;
        int          fper  = 0;
        rc = f16 ? fast_sampling_occupancy<FTB200_F16, false, 1>(fsmem, &fper) :
                   fast_sampling_occupancy<FTB200_BF16, false, 1>(fsmem, &fper);
        if (rc != FTB200_OK) {
            return rc;
        }
        if (fper >= 1) {
            KParams F    = K;
            F.redo_count = K.ticket + 1;
            F.redo_rows  = (int*)((char*)p->workspace + 256);
            int fgrid    = sm_count() * fper;
            fgrid        = fgrid < p->local_batch_size ? fgrid : p->local_batch_size;
            rc = f16 ? fast_sampling_launch<FTB200_F16, false, 1>(F, fgrid, fsmem, st) :
                       fast_sampling_launch<FTB200_BF16, false, 1>(F, fgrid, fsmem, st);
            if (rc != FTB200_OK) {
                return rc;
            }
            note_launch(1);
            K.ticket        = K.ticket + 2;
            K.row_order     = F.redo_rows;
            K.row_count_dev = F.redo_count;
        }
    }
    switch (p->dtype) {
        case FTB200_F32: rc = sampling_launch<FTB200_F32>(K, grid, smem, st); break;
        case FTB200_F16: rc = sampling_launch<FTB200_F16>(K, grid, smem, st); break;
        default: rc = sampling_launch<FTB200_BF16>(K, grid, smem, st); break;
    }
    if (rc == FTB200_OK) {
        note_launch(1);
    }
    return rc;
}

extern "C" int ftb200_vocab_parallel_merge(const ftb200_sampling_params* p, const uint64_t* gathered, int n_ranks,
                                           int cap, int* overflow_count)
{
    reset_launch_count();
    if (gathered == nullptr || overflow_count == nullptr || n_ranks < 1 || cap < 1 || cap > kCap) {
        set_error("ftb200_vocab_parallel_merge: invalid argument");
        return FTB200_INVALID_ARG;
    }
    KParams K;
    size_t  smem = 0;
    int     grid = 0;
    int     rc   = plan_sampling(p, K, smem, grid, false);
    if (rc != FTB200_OK) {
        return rc;
    }
    if (p->local_batch_size == 0) {
        return FTB200_OK;
    }
    K.vp_cap        = cap;
    cudaStream_t st = (cudaStream_t)p->stream;
    grid            = sm_count() * 3 < p->local_batch_size ? sm_count() * 3 : p->local_batch_size;  // (3 CTAs of 52 KB per SM)
    switch (p->dtype) {
        case FTB200_F32: rc = vp_merge_launch<FTB200_F32>(K, (const u64*)gathered, n_ranks, overflow_count, grid, st); break;
        case FTB200_F16: rc = vp_merge_launch<FTB200_F16>(K, (const u64*)gathered, n_ranks, overflow_count, grid, st); break;
        default: rc = vp_merge_launch<FTB200_BF16>(K, (const u64*)gathered, n_ranks, overflow_count, grid, st); break;
    }
    if (rc == FTB200_OK) {
        note_launch(1);
    }
    return rc;
}
