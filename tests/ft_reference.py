"""TEST INFRASTRUCTURE: ctypes driver of oracle/_ref/libft_decode_ref.so, the unmodified reference
DynamicDecodeLayer<T> compiled for sm_100a (see oracle/build_ref.sh, oracle/ref_harness.cu).
Same setup()/forward() surface as fastertransformer_b200.DynamicDecodeLayer so tests drive both alike."""
import ctypes as C
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libft_decode_ref.so")


class RuntimeArgs(C.Structure):
    _fields_ = [
        ("n_top_k", C.c_int), ("top_k", C.c_void_p), ("n_top_p", C.c_int), ("top_p", C.c_void_p),
        ("n_temperature", C.c_int), ("temperature", C.c_void_p),
        ("n_repetition_penalty", C.c_int), ("repetition_penalty", C.c_void_p),
        ("n_presence_penalty", C.c_int), ("presence_penalty", C.c_void_p),
        ("n_min_length", C.c_int), ("min_length", C.c_void_p),
        ("n_len_penalty", C.c_int), ("len_penalty", C.c_void_p),
        ("n_diversity", C.c_int), ("beam_search_diversity_rate", C.c_void_p),
        ("n_random_seed", C.c_int), ("random_seed", C.c_void_p),
        ("top_p_decay", C.c_void_p), ("top_p_min", C.c_void_p), ("top_p_reset_ids", C.c_void_p),
    ]


class StepArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("batch", C.c_int), ("beam", C.c_int), ("embedding_bias", C.c_void_p),
        ("step", C.c_int), ("max_input_length", C.c_int), ("ite", C.c_int), ("local_batch_size", C.c_int),
        ("end_id", C.c_void_p), ("input_lengths", C.c_void_p), ("sequence_limit_length", C.c_void_p),
        ("stop_words_list", C.c_void_p), ("stop_words_len", C.c_int),
        ("bad_words_list", C.c_void_p), ("bad_words_len", C.c_int), ("bad_words_shared", C.c_int),
        ("src_cache_indirection", C.c_void_p), ("max_seq_len", C.c_int),
        ("n_temperature", C.c_int), ("temperature", C.c_void_p),
        ("n_len_penalty", C.c_int), ("len_penalty", C.c_void_p),
        ("n_repetition_penalty", C.c_int), ("repetition_penalty", C.c_void_p),
        ("n_presence_penalty", C.c_int), ("presence_penalty", C.c_void_p),
        ("n_min_length", C.c_int), ("min_length", C.c_void_p),
        ("n_diversity", C.c_int), ("beam_search_diversity_rate", C.c_void_p),
        ("output_ids", C.c_void_p), ("finished", C.c_void_p), ("cum_log_probs", C.c_void_p),
        ("parent_ids", C.c_void_p), ("sequence_length", C.c_void_p), ("output_log_probs", C.c_void_p),
        ("output_log_probs_len", C.c_int), ("tgt_cache_indirection", C.c_void_p), ("beam_hyps", C.c_void_p),
        ("should_stop", C.c_void_p),
    ]


def available():
    return os.path.exists(REF_LIB)


_lib = None


def ref_lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(REF_LIB)
        _lib.ftref_create.restype = C.c_void_p
        _lib.ftref_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p]
        _lib.ftref_destroy.argtypes = [C.c_void_p]
        _lib.ftref_setup.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(RuntimeArgs)]
        _lib.ftref_forward.argtypes = [C.c_void_p, C.POINTER(StepArgs)]
        _lib.ftref_last_error.restype = C.c_char_p
        _lib.ftref_curand_init.argtypes = [C.c_void_p, C.c_int, C.c_ulonglong, C.c_void_p, C.c_void_p]
        _lib.ftref_curand_uniforms.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        V, Z = C.c_void_p, C.c_size_t
        _lib.ftref_log_prob_from_logits.argtypes = [V, V, C.c_int, V, V, Z, Z, Z, Z, V, Z, V, C.c_int]
        I = C.c_int
        _lib.ftref_decoding_initialize.argtypes = [V, V, V, V, I, V, I, I, I, V]
        _lib.ftref_gather_tree.argtypes = [V, V, I, V, V, I, I, I, V, V, V, I, V, V, I, I, V, V]
        _lib.ftref_finalize.argtypes = [V, V, V, V, V, V, V, V, V, V, I, I, I, V]
        _lib.ftref_insert_unfinished_path.argtypes = [V, V, V, V, V, V, V, V, V, V, V, I, C.c_float, V, V, I, I, V]
    return _lib


_HOST_KEYS = [
    ("runtime_top_k", "top_k", np.uint32), ("runtime_top_p", "top_p", np.float32),
    ("temperature", "temperature", np.float32), ("repetition_penalty", "repetition_penalty", np.float32),
    ("presence_penalty", "presence_penalty", np.float32), ("min_length", "min_length", np.int32),
    ("len_penalty", "len_penalty", np.float32),
    ("beam_search_diversity_rate", "beam_search_diversity_rate", np.float32),
    ("random_seed", "random_seed", np.uint64),
]


class RefDynamicDecodeLayer:
    """fastertransformer::DynamicDecodeLayer<float|half>, unmodified, through ref_harness.cu."""

    def __init__(self, vocab_size, vocab_size_padded, dtype=torch.float32, device="cuda:0"):
        if dtype == torch.bfloat16:
            raise ValueError("the reference has no bf16 instantiation of this path")
        self.lib = ref_lib()
        self.dtype = dtype
        self.vocab_size_padded = vocab_size_padded
        torch.cuda.set_device(torch.device(device))
        # the reference layer runs on the legacy default stream (stream 0)
        self.h = self.lib.ftref_create(0 if dtype == torch.float32 else 1, vocab_size, vocab_size_padded, None)
        if not self.h:
            raise RuntimeError(self.lib.ftref_last_error().decode())
        self._keep = []

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.lib.ftref_destroy(self.h)
        except Exception:
            pass

    def setup(self, batch_size, beam_width, runtime_args):
        A = RuntimeArgs()
        keep = []
        for key, field, dt in _HOST_KEYS:
            if key in runtime_args and runtime_args[key] is not None:
                arr = np.ascontiguousarray(np.atleast_1d(np.asarray(runtime_args[key])).astype(dt))
                keep.append(arr)
                setattr(A, "n_" + (field if field != "beam_search_diversity_rate" else "diversity"), arr.size)
                setattr(A, field, arr.ctypes.data)
        for key in ("top_p_decay", "top_p_min", "top_p_reset_ids"):
            t = runtime_args.get(key)
            if t is not None:
                setattr(A, key, t.data_ptr())
        self._keep = keep
        self.runtime_args = dict(runtime_args)
        torch.cuda.synchronize()
        if self.lib.ftref_setup(self.h, batch_size, beam_width, C.byref(A)) != 0:
            raise RuntimeError(self.lib.ftref_last_error().decode())
        torch.cuda.synchronize()

    def forward(self, outputs, inputs):
        S = StepArgs()
        logits = inputs["logits"]
        S.logits = logits.data_ptr()
        S.batch = logits.shape[0]
        S.beam = logits.shape[1] if logits.dim() == 3 else 1
        bias = inputs.get("embedding_bias")
        S.embedding_bias = None if bias is None else bias.data_ptr()
        S.step = int(inputs["step"])
        S.max_input_length = int(inputs["max_input_length"])
        S.ite = int(inputs.get("ite", 0))
        S.local_batch_size = int(inputs.get("local_batch_size", S.batch))
        S.end_id = inputs["end_id"].data_ptr()
        for key in ("input_lengths", "sequence_limit_length", "src_cache_indirection"):
            t = inputs.get(key)
            if t is not None:
                setattr(S, key, t.data_ptr())
        sw = inputs.get("stop_words_list")
        if sw is not None:
            S.stop_words_list, S.stop_words_len = sw.data_ptr(), sw.shape[-1]
        bw = inputs.get("bad_words_list")
        if bw is not None:
            S.bad_words_list, S.bad_words_len, S.bad_words_shared = bw.data_ptr(), bw.shape[-1], int(bw.dim() == 2)
        out_ids = outputs["output_ids"]
        S.max_seq_len = out_ids.shape[0]
        keep = []
        for key, field, dt in _HOST_KEYS:
            if field in ("top_k", "top_p", "random_seed"):
                continue
            v = inputs.get(key, None)
            if v is not None:
                arr = np.ascontiguousarray(np.atleast_1d(np.asarray(v)).astype(dt))
                keep.append(arr)
                setattr(S, "n_" + (field if field != "beam_search_diversity_rate" else "diversity"), arr.size)
                setattr(S, field, arr.ctypes.data)
        S.output_ids = out_ids.data_ptr()
        for key in ("finished", "cum_log_probs", "parent_ids", "sequence_length", "tgt_cache_indirection"):
            t = outputs.get(key)
            if t is not None:
                setattr(S, key, t.data_ptr())
        olp = outputs.get("output_log_probs")
        if olp is not None:
            S.output_log_probs, S.output_log_probs_len = olp.data_ptr(), olp.shape[0]
        bh = outputs.get("beam_hyps")
        if bh is not None:
            S.beam_hyps = bh
        stop = np.zeros(1, dtype=np.bool_)
        S.should_stop = stop.ctypes.data
        torch.cuda.synchronize()
        if self.lib.ftref_forward(self.h, C.byref(S)) != 0:
            raise RuntimeError(self.lib.ftref_last_error().decode())
        torch.cuda.synchronize()
        return bool(stop[0])
