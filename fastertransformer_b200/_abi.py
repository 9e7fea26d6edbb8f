"""ctypes layouts of the structs in include/ftb200.h (no library is loaded here)."""
import ctypes as C


class SamplingParams(C.Structure):
    """ftb200_sampling_params, field for field."""
    _fields_ = [
        ("dtype", C.c_int), ("batch_size", C.c_int), ("local_batch_size", C.c_int), ("ite", C.c_int),
        ("vocab_size", C.c_int), ("vocab_size_padded", C.c_int), ("step", C.c_int), ("max_input_length", C.c_int),
        ("logits", C.c_void_p), ("embedding_bias", C.c_void_p), ("end_ids", C.c_void_p),
        ("input_lengths", C.c_void_p), ("output_ids", C.c_void_p), ("bad_words", C.c_void_p),
        ("bad_words_len", C.c_int), ("bad_words_shared", C.c_int),
        ("temperature", C.c_void_p), ("apply_temperature", C.c_int),
        ("repetition_penalty", C.c_void_p), ("penalty_type", C.c_int), ("apply_repetition", C.c_int),
        ("min_lengths", C.c_void_p), ("apply_min_length", C.c_int),
        ("topk_states", C.c_void_p), ("topk_ks", C.c_void_p), ("topk_ps", C.c_void_p), ("topk_skip", C.c_void_p),
        ("max_top_k", C.c_int),
        ("topp_states", C.c_void_p), ("topp_ps", C.c_void_p), ("topp_skip", C.c_void_p),
        ("topp_initial_ps", C.c_void_p), ("topp_decay", C.c_void_p), ("topp_min", C.c_void_p),
        ("topp_reset_ids", C.c_void_p),
        ("sequence_length", C.c_void_p), ("finished", C.c_void_p), ("cum_log_probs", C.c_void_p),
        ("output_log_probs", C.c_void_p),
        ("row_order", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class BeamHyps(C.Structure):
    """ftb200_beam_hyps."""
    _fields_ = [
        ("output_ids_tgt", C.c_void_p), ("sequence_lengths_tgt", C.c_void_p), ("cum_log_probs", C.c_void_p),
        ("normed_scores", C.c_void_p), ("log_probs", C.c_void_p), ("min_normed_scores", C.c_void_p),
        ("num_beams", C.c_void_p), ("is_done", C.c_void_p), ("early_stopping", C.c_int),
    ]


class BeamParams(C.Structure):
    """ftb200_beam_params."""
    _fields_ = [
        ("dtype", C.c_int), ("batch_size", C.c_int), ("local_batch_size", C.c_int), ("ite", C.c_int),
        ("beam_width", C.c_int), ("vocab_size", C.c_int), ("vocab_size_padded", C.c_int), ("step", C.c_int),
        ("max_input_length", C.c_int), ("max_seq_len", C.c_int),
        ("logits", C.c_void_p), ("embedding_bias", C.c_void_p), ("end_ids", C.c_void_p),
        ("input_lengths", C.c_void_p),
        ("temperature", C.c_float), ("repetition_penalty", C.c_float), ("penalty_type", C.c_int),
        ("min_length", C.c_int), ("diversity_rate", C.c_float), ("length_penalty", C.c_float),
        ("output_ids", C.c_void_p), ("parent_ids", C.c_void_p), ("finished", C.c_void_p),
        ("sequence_length", C.c_void_p), ("cum_log_probs", C.c_void_p), ("output_log_probs", C.c_void_p),
        ("src_cache_indirection", C.c_void_p), ("tgt_cache_indirection", C.c_void_p),
        ("beam_hyps", C.POINTER(BeamHyps)),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class GatherTreeParams(C.Structure):
    """ftb200_gather_tree_params (the fields of the reference's gatherTreeParam, in its order)."""
    _fields_ = [
        ("beams", C.c_void_p), ("max_sequence_lengths", C.c_void_p), ("max_sequence_length_final_step", C.c_int),
        ("input_lengths", C.c_void_p), ("response_input_lengths", C.c_void_p), ("max_time", C.c_int),
        ("batch_size", C.c_int), ("beam_width", C.c_int), ("step_ids", C.c_void_p), ("parent_ids", C.c_void_p),
        ("end_tokens", C.c_void_p), ("max_input_length", C.c_int), ("prefix_soft_prompt_lengths", C.c_void_p),
        ("p_prompt_tuning_prompt_lengths", C.c_void_p), ("max_input_without_prompt_length", C.c_int),
        ("max_prefix_soft_prompt_length", C.c_int), ("output_ids", C.c_void_p), ("stream", C.c_void_p),
    ]
