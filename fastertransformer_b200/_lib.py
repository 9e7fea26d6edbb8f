"""ctypes binding of libftb200.so (include/ftb200.h)."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libftb200.so")


class FtbError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__("[FT][ERROR] ftb200 status %d: %s" % (status, msg))
        self.status = status


from ._abi import BeamHyps, BeamParams, GatherTreeParams, SamplingParams  # noqa: E402,F401


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libftb200.so is not built (%s). Run `python -m fastertransformer_b200.build`; "
            "there is no CPU fallback for the sampling kernels." % LIB_PATH)
    l = C.CDLL(LIB_PATH)
    l.ftb200_version.restype = C.c_char_p
    l.ftb200_last_error_string.restype = C.c_char_p
    l.ftb200_curand_init.argtypes = [C.c_void_p, C.c_int, C.c_ulonglong, C.c_void_p, C.c_void_p]
    l.ftb200_curand_peek_uniforms.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    l.ftb200_setup_topk_runtime_args.argtypes = [
        C.c_int, C.c_uint32, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    l.ftb200_setup_topp_runtime_args.argtypes = [
        C.c_int, C.c_uint32, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    l.ftb200_sampling_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_size_t)]
    l.ftb200_decode_step_sampling.argtypes = [C.POINTER(SamplingParams)]
    l.ftb200_decode_step_sampling_static.argtypes = [C.POINTER(SamplingParams)]
    l.ftb200_static_scratch_bytes.restype = C.c_size_t
    l.ftb200_set_row_trace.argtypes = [C.c_void_p]
    l.ftb200_beam_workspace_bytes.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_size_t)]
    l.ftb200_beam_search_step.argtypes = [C.POINTER(BeamParams)]
    l.ftb200_vocab_parallel_local.argtypes = [C.POINTER(SamplingParams), C.c_int, C.c_int, C.c_void_p]
    l.ftb200_vocab_parallel_merge.argtypes = [C.POINTER(SamplingParams), C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    V, I = C.c_void_p, C.c_int
    l.ftb200_ban_bad_words.argtypes = [V, I, V, V, I, I, I, V, I, I, I, I, I, V]
    l.ftb200_stop_criteria.argtypes = [V, V, V, I, V, V, I, I, I, I, I, V, V, V]
    l.ftb200_wait_should_stop.argtypes = [V, I, I, V, I, C.POINTER(C.c_int)]
    Z = C.c_size_t
    l.ftb200_log_prob_from_logits.argtypes = [V, V, I, V, V, Z, Z, Z, Z, V, Z, V, I]
    l.ftb200_decoding_initialize.argtypes = [V, V, V, V, I, V, I, I, I, V]
    l.ftb200_gather_tree.argtypes = [C.POINTER(GatherTreeParams)]
    l.ftb200_finalize.argtypes = [V, V, V, V, V, V, V, V, V, V, I, I, I, V]
    l.ftb200_insert_unfinished_path.argtypes = [C.POINTER(BeamHyps), V, V, V, V, I, C.c_float, V, V, I, I, V]
    return l


lib = _load()


def check(status):
    if status != 0:
        raise FtbError(status, lib.ftb200_last_error_string().decode())
