"""TEST INFRASTRUCTURE: ctypes driver of oracle/libft_oracle.so, the CPU restatement of the reference's
decode sampling path (oracle/ft_oracle.cpp).  Works on numpy arrays; uniforms are an input."""
import ctypes as C
import os
import subprocess

import numpy as np

from fastertransformer_b200._abi import BeamHyps, GatherTreeParams, SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_LIB = os.path.join(ROOT, "oracle", "libft_oracle.so")
_DT = {"float32": 0, "float16": 1, "bfloat16": 2}
_lib = None


def oracle_lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_LIB):
            subprocess.check_call([os.path.join(ROOT, "oracle", "build_oracle.sh")])
        _lib = C.CDLL(ORACLE_LIB)
        _lib.oracle_decode_step_sampling.argtypes = [C.POINTER(SamplingParams)]
        V = C.c_void_p
        _lib.oracle_setup_topk_runtime_args.argtypes = [C.c_int, C.c_uint32, V, C.c_int, C.c_float, V, C.c_int, V]
        _lib.oracle_setup_topp_runtime_args.argtypes = [C.c_int, C.c_uint32, V, C.c_int, C.c_float, V, C.c_int, V,
                                                        V, V, V, V, V, V, V]
        _lib.oracle_length_criterion.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.oracle_stop_words.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_int]
        Z = C.c_size_t
        _lib.oracle_log_prob_from_logits.argtypes = [V, V, V, C.c_int, V, V, Z, Z, Z, Z, C.c_int]
        I = C.c_int
        _lib.oracle_decoding_initialize.argtypes = [V, V, V, V, I, V, I, I, I]
        _lib.oracle_gather_tree.argtypes = [C.POINTER(GatherTreeParams)]
        _lib.oracle_finalize.argtypes = [V, V, V, V, V, V, V, V, V, V, I, I, I]
        _lib.oracle_insert_unfinished_path.argtypes = [C.POINTER(BeamHyps), V, V, V, V, I, C.c_float, V, V, I, I]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def bf16_bits(x):
    """float32 array -> bf16 bit patterns (round to nearest even), as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


class OracleDynamicDecodeLayer:
    """Same setup()/forward() surface as the CUDA layer, on host arrays.

    logits: float32 / float16 numpy arrays, or uint16 bf16 bit patterns with dtype_name='bfloat16'."""

    def __init__(self, vocab_size, vocab_size_padded, dtype_name="float32"):
        self.lib = oracle_lib()
        self.vocab_size, self.vocab_size_padded = vocab_size, vocab_size_padded
        self.dtype_name = dtype_name

    @staticmethod
    def _arg(a, key):
        v = a.get(key)
        return None if v is None else np.atleast_1d(np.asarray(v))

    @staticmethod
    def _bc(arr, B, dt, default):
        if arr is None:
            arr = np.asarray([default], dt)
        arr = arr.astype(dt)
        return np.full(B, arr[0], dt) if arr.size == 1 else arr.copy()

    def setup(self, batch_size, beam_width, a):
        B = batch_size
        self.B = B
        top_k, top_p = self._arg(a, "runtime_top_k"), self._arg(a, "runtime_top_p")
        self.temperature = self._bc(self._arg(a, "temperature"), B, np.float32, 1.0)
        if "repetition_penalty" in a:
            self.penalty_type, pen = 1, self._arg(a, "repetition_penalty")
        elif "presence_penalty" in a:
            self.penalty_type, pen = 0, self._arg(a, "presence_penalty")
        else:
            self.penalty_type, pen = 2, None
        self.penalty_default = 1.0 if self.penalty_type == 1 else 0.0
        self.penalty = self._bc(pen, B, np.float32, self.penalty_default)
        self.min_length = self._bc(self._arg(a, "min_length"), B, np.int32, 0)

        k_arr = top_k.astype(np.uint32) if top_k is not None else np.zeros(1, np.uint32)
        p_scalar = float(top_p[0]) if top_p is not None else 0.0
        self.topk_ks = np.zeros(B, np.uint32)
        self.topk_ps = np.zeros(B, np.float32)
        self.topk_skip = np.zeros(B, np.uint8)
        if k_arr.size > 1:
            self.topk_ks[:] = k_arr
        if top_p is not None and top_p.size > 1:
            self.topk_ps[:] = top_p
        self.lib.oracle_setup_topk_runtime_args(
            B, int(k_arr.max()), _p(self.topk_ks), int(k_arr.size), p_scalar,
            _p(self.topk_ps), 0 if top_p is None else int(top_p.size), _p(self.topk_skip))
        self.max_top_k = int(self.topk_ks.max())
        self.topp_active = top_p is not None
        self.topp_skip = np.ones(B, np.uint8)
        if self.topp_active:
            self.topp_ks = np.zeros(B, np.uint32)
            self.topp_ps = np.zeros(B, np.float32)
            self.topp_initial = np.zeros(B, np.float32)
            self.topp_decay = np.zeros(B, np.float32)
            self.topp_min = np.zeros(B, np.float32)
            self.topp_reset = np.zeros(B, np.int32)
            if k_arr.size > 1:
                self.topp_ks[:] = k_arr
            if top_p.size > 1:
                self.topp_ps[:] = top_p
            dec, mn, rs = a.get("top_p_decay"), a.get("top_p_min"), a.get("top_p_reset_ids")
            self.lib.oracle_setup_topp_runtime_args(
                B, int(k_arr[0]), _p(self.topp_ks), int(k_arr.size), p_scalar,
                _p(self.topp_ps), int(top_p.size), _p(self.topp_skip), _p(self.topp_initial), _p(self.topp_decay),
                _p(dec), _p(self.topp_min), _p(mn), _p(self.topp_reset), _p(rs))

    def forward(self, outputs, inputs, u_topk, u_topp):
        logits = np.ascontiguousarray(inputs["logits"])
        B = logits.shape[0]
        step, mil = int(inputs["step"]), int(inputs["max_input_length"])
        ite, lbs = int(inputs.get("ite", 0)), int(inputs.get("local_batch_size", B))
        lo, hi = ite * lbs, (ite + 1) * lbs
        topk_on = not self.topk_skip[lo:hi].all()
        topp_on = self.topp_active and not self.topp_skip[lo:hi].all()
        if not (topk_on or topp_on):
            return
        keep = []

        def sub(arr, width=1):
            if arr is None:
                return None
            v = np.ascontiguousarray(arr).reshape(-1)[lo * width:]
            keep.append(v)
            return v.ctypes.data

        P = SamplingParams()
        P.dtype = _DT[self.dtype_name]
        P.batch_size, P.local_batch_size, P.ite = B, lbs, ite
        P.vocab_size, P.vocab_size_padded = self.vocab_size, self.vocab_size_padded
        P.step, P.max_input_length = step, mil
        P.logits = sub(logits, self.vocab_size_padded)
        bias = inputs.get("embedding_bias")
        P.embedding_bias = None if bias is None else np.ascontiguousarray(bias).ctypes.data
        end = np.ascontiguousarray(inputs["end_id"], dtype=np.int32)
        P.end_ids = sub(end)
        il = inputs.get("input_lengths")
        P.input_lengths = sub(None if il is None else np.ascontiguousarray(il, dtype=np.int32))
        P.output_ids = outputs["output_ids"].ctypes.data
        bw = inputs.get("bad_words_list")
        if bw is not None:
            bw = np.ascontiguousarray(bw, dtype=np.int32)
            keep.append(bw)
            shared = bw.ndim == 2 or bw.shape[0] == 1
            L = bw.shape[-1]
            P.bad_words = bw.ctypes.data if shared else bw.ctypes.data + lo * 2 * L * 4
            P.bad_words_len, P.bad_words_shared = L, int(shared)
        P.temperature = sub(self.temperature)
        P.apply_temperature = int(bias is not None or bool((self.temperature[lo:hi] != 1.0).any()))
        P.repetition_penalty = sub(self.penalty)
        P.penalty_type = self.penalty_type
        P.apply_repetition = int(step > 1 and self.penalty_type != 2
                                 and bool((self.penalty[lo:hi] != self.penalty_default).any()))
        P.min_lengths = sub(self.min_length)
        P.apply_min_length = int(bool((self.min_length[lo:hi] > step - mil).any()))
        if topk_on:
            P.topk_states = sub(np.ascontiguousarray(u_topk, dtype=np.float32))
            P.topk_ks, P.topk_ps, P.topk_skip = sub(self.topk_ks), sub(self.topk_ps), sub(self.topk_skip)
            P.max_top_k = self.max_top_k
        if topp_on:
            P.topp_states = sub(np.ascontiguousarray(u_topp, dtype=np.float32))
            P.topp_ps, P.topp_skip = sub(self.topp_ps), sub(self.topp_skip)
            P.topp_initial_ps, P.topp_decay = sub(self.topp_initial), sub(self.topp_decay)
            P.topp_min, P.topp_reset_ids = sub(self.topp_min), sub(self.topp_reset)
        P.sequence_length = sub(outputs.get("sequence_length"))
        P.finished = sub(outputs.get("finished"))
        P.cum_log_probs = sub(outputs.get("cum_log_probs"))
        olp = outputs.get("output_log_probs")
        if olp is not None:
            P.output_log_probs = olp.ctypes.data + ((step - mil) * B + lo) * 4
        self.lib.oracle_decode_step_sampling(C.byref(P))


def oracle_log_prob_from_logits(logits, input_ids, input_lengths, vocab_size, batch_first=False,
                                dtype_name=None):
    """oracle_log_prob_from_logits on host arrays; returns (cum_log_probs [batch], log_probs in the
    reference's workspace layout).  bf16 logits come as uint16 bit patterns with dtype_name='bfloat16'."""
    lib = oracle_lib()
    logits = np.ascontiguousarray(logits)
    dtype_name = dtype_name or str(logits.dtype)
    if batch_first:
        batch, max_len, vp = logits.shape
    else:
        max_len, batch, vp = logits.shape
    ids = np.ascontiguousarray(input_ids, dtype=np.int32)
    lens = np.ascontiguousarray(input_lengths, dtype=np.int32)
    cum = np.zeros(batch, np.float32)
    lp = np.zeros(max(1, (max_len - 1) * batch), np.float32)
    rc = lib.oracle_log_prob_from_logits(_p(cum), _p(lp), _p(logits), _DT[dtype_name], _p(ids), _p(lens), max_len,
                                         batch, vocab_size, vp, int(batch_first))
    assert rc == 0
    shape = (batch, max_len - 1) if batch_first else (max_len - 1, batch)
    return cum, lp[:(max_len - 1) * batch].reshape(shape)
