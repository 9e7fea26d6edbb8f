"""Host-side mirror of FasterTransformer's DynamicDecodeLayer for the sampling path (beam_width == 1).

Same keys, dtypes and placement as the reference's TensorMap interface
(layers/DynamicDecodeLayer.cc:153-178 setup, :191-474 forward): runtime arguments are host arrays of
shape [1] or [batch]; logits, ids and state live on the GPU.  torch is used only to own device memory
and streams; every computation is a call into libftb200.so through the C ABI.
"""
import ctypes as C

import numpy as np
import torch

from ._lib import BeamHyps, BeamParams, SamplingParams, check, lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
CURAND_STATE_BYTES = 48  # sizeof(curandState_t), XORWOW


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class _SamplingLayerState:
    """Buffers one reference sampling layer keeps (BaseSamplingLayer.cc:29-53, TopK/TopP allocateBuffer)."""

    def __init__(self, batch, device):
        self.curand = torch.zeros(batch * CURAND_STATE_BYTES, dtype=torch.uint8, device=device)
        self.top_ks = torch.zeros(batch, dtype=torch.int32, device=device)  # uint32 payload
        self.top_ps = torch.zeros(batch, dtype=torch.float32, device=device)
        self.skip = torch.zeros(batch, dtype=torch.uint8, device=device)
        self.skip_host = np.ones(batch, dtype=bool)
        self.active = False


class DynamicDecodeLayer:
    """Drop-in for the sampling half of fastertransformer::DynamicDecodeLayer<T>."""

    def __init__(self, vocab_size, vocab_size_padded, dtype=torch.float32, device="cuda:0", stream=None):
        self.vocab_size = int(vocab_size)
        self.vocab_size_padded = int(vocab_size_padded)
        self.dtype = dtype
        self.device = torch.device(device)
        self.stream = stream
        self._workspace = None
        self._beam_ws = None
        self._gate = {}
        self.time_kernels = False   # when set, CUDA events bracket each fused launch (kernel_events)
        self.kernel_events = []
        self._count_dev = None
        self._count_host = None
        self.launches = 0

    # ---- helpers -------------------------------------------------------------------------------
    def _stream_ptr(self):
        s = self.stream if self.stream is not None else torch.cuda.current_stream(self.device)
        return C.c_void_p(s.cuda_stream)

    @staticmethod
    def _arg(args, key):
        v = args.get(key)
        if v is None:
            return None
        return np.atleast_1d(np.asarray(v))

    def _broadcast(self, arr, batch, dtype, default):
        if arr is None:
            arr = np.asarray([default], dtype=dtype)
        arr = arr.astype(dtype)
        if arr.size == 1:
            return np.full(batch, arr[0], dtype=dtype)
        if arr.size != batch:
            raise ValueError("runtime argument must have shape [1] or [batch_size]")
        return arr.copy()

    # ---- setup (DynamicDecodeLayer.cc:153-178 -> TopK/TopPSamplingLayer::setup) -------------------
    def setup(self, batch_size, beam_width, runtime_args):
        self.beam_width = int(beam_width)
        # hasDiffRuntimeArgs (DynamicDecodeLayer.cc:477-514): beam search then runs one batch entry at a time
        self.has_diff_runtime_args = False
        for key in ("beam_search_diversity_rate", "temperature", "len_penalty", "repetition_penalty",
                    "presence_penalty", "min_length"):
            v = self._arg(runtime_args, key)
            if v is not None and v.size > 1 and bool((v != v[0]).any()):
                self.has_diff_runtime_args = True
        if beam_width != 1:
            return  # the beam layers have no set-up (BaseBeamSearchLayer.cu:123-127)
        B, dev, st = int(batch_size), self.device, self._stream_ptr()
        self.batch_size = B
        self._gate = {}
        a = runtime_args
        top_k = self._arg(a, "runtime_top_k")
        top_p = self._arg(a, "runtime_top_p")
        seeds = self._arg(a, "random_seed")
        if "repetition_penalty" in a and "presence_penalty" in a:
            raise RuntimeError("[FT][ERROR] Found ambiguous parameters repetition_penalty and presence_penalty "
                               "which are mutually exclusive.")
        # BaseSamplingLayer::setup (BaseSamplingLayer.cc:112-206)
        self.temperature_host = self._broadcast(self._arg(a, "temperature"), B, np.float32, 1.0)
        if "repetition_penalty" in a:
            self.penalty_type, pen = 1, self._arg(a, "repetition_penalty")
        elif "presence_penalty" in a:
            self.penalty_type, pen = 0, self._arg(a, "presence_penalty")
        else:
            self.penalty_type, pen = 2, None
        default_pen = 1.0 if self.penalty_type == 1 else 0.0
        self.penalty_default = default_pen
        self.penalty_host = self._broadcast(pen, B, np.float32, default_pen)
        self.min_length_host = self._broadcast(self._arg(a, "min_length"), B, np.int32, 0)
        self.temperature = torch.from_numpy(self.temperature_host).to(dev)
        self.penalty = torch.from_numpy(self.penalty_host).to(dev)
        self.min_length = torch.from_numpy(self.min_length_host).to(dev)

        self.topk = _SamplingLayerState(B, dev)
        self.topp = _SamplingLayerState(B, dev)
        for layer in (self.topk, self.topp):
            if seeds is None:
                check(lib.ftb200_curand_init(_ptr(layer.curand), B, 0, None, st))
            elif seeds.size == 1:
                check(lib.ftb200_curand_init(_ptr(layer.curand), B, int(seeds[0]), None, st))
            else:
                if seeds.size != B:
                    raise RuntimeError("[FT][ERROR] random_seeds must be of shape [1] or [batch_size]")
                sd = torch.from_numpy(seeds.astype(np.uint64).view(np.int64)).to(dev)
                check(lib.ftb200_curand_init(_ptr(layer.curand), B, 0, _ptr(sd), st))
                torch.cuda.current_stream(dev).synchronize()

        # TopKSamplingLayer::setup (TopKSamplingLayer.cu:134-186)
        k_arr = top_k.astype(np.uint32) if top_k is not None else np.zeros(1, np.uint32)
        k_scalar = int(k_arr.max())
        p_scalar = float(top_p[0]) if top_p is not None else 0.0
        if k_arr.size > 1:
            self.topk.top_ks.copy_(torch.from_numpy(k_arr.view(np.int32)))
        if top_p is not None and top_p.size > 1:
            self.topk.top_ps.copy_(torch.from_numpy(top_p.astype(np.float32)))
        check(lib.ftb200_setup_topk_runtime_args(B, k_scalar, _ptr(self.topk.top_ks), int(k_arr.size), p_scalar,
                                                 _ptr(self.topk.top_ps), 0 if top_p is None else int(top_p.size),
                                                 _ptr(self.topk.skip), st))
        self.topk.skip_host = self.topk.skip.cpu().numpy().astype(bool)
        self.max_top_k = int(self.topk.top_ks.cpu().numpy().view(np.uint32).max())
        self.topk.active = True

        # TopPSamplingLayer::setup (TopPSamplingLayer.cu:184-253)
        if top_p is None:
            self.topp.skip_host[:] = True
            self.topp.active = False
        else:
            self.topp.initial = torch.zeros(B, dtype=torch.float32, device=dev)
            self.topp.decay = torch.zeros(B, dtype=torch.float32, device=dev)
            self.topp.min = torch.zeros(B, dtype=torch.float32, device=dev)
            self.topp.reset = torch.zeros(B, dtype=torch.int32, device=dev)
            if k_arr.size > 1:
                self.topp.top_ks.copy_(torch.from_numpy(k_arr.view(np.int32)))
            if top_p.size > 1:
                self.topp.top_ps.copy_(torch.from_numpy(top_p.astype(np.float32)))
            check(lib.ftb200_setup_topp_runtime_args(
                B, int(k_arr[0]), _ptr(self.topp.top_ks), int(k_arr.size), p_scalar, _ptr(self.topp.top_ps),
                int(top_p.size), _ptr(self.topp.skip), _ptr(self.topp.initial), _ptr(self.topp.decay),
                _ptr(a.get("top_p_decay")), _ptr(self.topp.min), _ptr(a.get("top_p_min")), _ptr(self.topp.reset),
                _ptr(a.get("top_p_reset_ids")), st))
            self.topp.skip_host = self.topp.skip.cpu().numpy().astype(bool)
            self.topp.active = True
        self._row_cost = self._estimate_row_cost()

    def _estimate_row_cost(self):
        """Relative cost of a row for the launch order: top-p rows cost most (three reads of the row and a
        sort of the nucleus), then top-k by k."""
        k = self.topk.top_ks.cpu().numpy().view(np.uint32).astype(np.float64)
        cost = 1.0 + k / 128.0
        if self.topp.active:
            p = self.topp.top_ps.cpu().numpy().astype(np.float64)
            cost = np.where(self.topk.skip_host, 10.0 + 8.0 * p, cost)
        return cost

    # ---- forward (DynamicDecodeLayer.cc:191-474, sampling branch) ---------------------------------
    def forward(self, outputs, inputs):
        logits = inputs["logits"]
        if logits.dim() == 3 and logits.shape[1] > 1:
            return self._forward_beam(outputs, inputs)
        B = logits.shape[0]
        step = int(inputs["step"])
        ite = int(inputs.get("ite", 0))
        lbs = int(inputs.get("local_batch_size", B))
        mil = int(inputs["max_input_length"])
        lo, hi = ite * lbs, (ite + 1) * lbs
        g = self._gate.get((lo, hi))
        if g is None:
            g = self._gate[(lo, hi)] = {
                "topk_on": self.topk.active and not self.topk.skip_host[lo:hi].all(),
                "topp_on": self.topp.active and not self.topp.skip_host[lo:hi].all(),
                "temp": bool((self.temperature_host[lo:hi] != 1.0).any()),
                "pen": bool((self.penalty_host[lo:hi] != self.penalty_default).any()),
                "minlen": int(self.min_length_host[lo:hi].max()),
                "order": torch.from_numpy(np.argsort(-self._row_cost[lo:hi], kind="stable").astype(np.int32))
                .to(self.device),
            }
        self._g = g
        self._stream = self._stream_ptr()  # one look-up per call, used by the sampling and the criteria launch
        topk_on, topp_on = g["topk_on"], g["topp_on"]
        if topk_on or topp_on:
            self._sample(outputs, inputs, logits, B, step, ite, lbs, mil, lo, hi, topk_on, topp_on)
        return self._stop_criteria(outputs, inputs, B, step, lbs, lo)

    # ---- beam search branch (DynamicDecodeLayer.cc:286-386 -> OnlineBeamSearchLayer::forward) -------
    def _forward_beam(self, outputs, inputs):
        logits = inputs["logits"]
        B, K, Vp = logits.shape
        step = int(inputs["step"])
        ite = int(inputs.get("ite", 0))
        lbs = int(inputs.get("local_batch_size", B))
        mil = int(inputs["max_input_length"])
        st = self._stream = self._stream_ptr()
        es = logits.element_size()
        out_ids = outputs["output_ids"]
        L = out_ids.shape[0]
        if "cum_log_probs" not in outputs:
            raise RuntimeError("[FT][ERROR] cum_log_probs should be provided in beam search.")
        bw = inputs.get("bad_words_list")
        if bw is not None:
            shared = bw.dim() == 2 or bw.shape[0] == 1
            Lw = bw.shape[-1]
            check(lib.ftb200_ban_bad_words(
                C.c_void_p(logits.data_ptr() + ite * lbs * K * Vp * es), _DT[logits.dtype],
                _ptr(out_ids), _ptr(outputs["parent_ids"]), B, lbs, K,
                C.c_void_p(bw.data_ptr() if shared else bw.data_ptr() + ite * lbs * 2 * Lw * 4), int(shared), Lw,
                ite * lbs, Vp, step, st))
            self.launches += 1

        def scalar(key, default):
            v = inputs.get(key)
            return default if v is None else np.atleast_1d(np.asarray(v)).reshape(-1)[0]

        sub = 1 if self.has_diff_runtime_args else lbs
        n_sub = lbs // sub
        need = C.c_size_t(0)
        check(lib.ftb200_beam_workspace_bytes(sub, K, C.byref(need)))
        if self._beam_ws is None or self._beam_ws.numel() < need.value:
            self._beam_ws = torch.empty(need.value, dtype=torch.uint8, device=self.device)
        hyps = outputs.get("beam_hyps")
        for d_ite in range(ite * n_sub, (ite + 1) * n_sub):
            row0 = d_ite * sub * K          # first batch-beam row of this sub-batch
            P = BeamParams()
            P.dtype = _DT[logits.dtype]
            P.batch_size, P.local_batch_size, P.ite, P.beam_width = B, sub, d_ite, K
            P.vocab_size, P.vocab_size_padded = self.vocab_size, Vp
            P.step, P.max_input_length, P.max_seq_len = step, mil, L
            P.logits = logits.data_ptr() + row0 * Vp * es
            bias = inputs.get("embedding_bias")
            P.embedding_bias = None if bias is None else bias.data_ptr()
            P.end_ids = inputs["end_id"].data_ptr() + d_ite * sub * 4
            il = inputs.get("input_lengths")
            P.input_lengths = None if il is None else il.data_ptr() + row0 * 4
            P.temperature = float(scalar("temperature", 1.0))
            if "repetition_penalty" in inputs and "presence_penalty" in inputs:
                raise RuntimeError("[FT][ERROR] Found ambiguous parameters repetition_penalty and "
                                   "presence_penalty which are mutually exclusive.")
            if inputs.get("repetition_penalty") is not None:
                P.penalty_type, P.repetition_penalty = 1, float(scalar("repetition_penalty", 1.0))
            elif inputs.get("presence_penalty") is not None:
                P.penalty_type, P.repetition_penalty = 0, float(scalar("presence_penalty", 0.0))
            else:
                P.penalty_type, P.repetition_penalty = 2, 1.0
            P.min_length = int(scalar("min_length", 0))
            P.diversity_rate = float(scalar("beam_search_diversity_rate", 0.0))
            P.length_penalty = float(scalar("len_penalty", 0.0))
            P.output_ids = out_ids.data_ptr()
            P.parent_ids = outputs["parent_ids"].data_ptr()
            P.finished = outputs["finished"].data_ptr() + row0
            P.sequence_length = outputs["sequence_length"].data_ptr() + row0 * 4
            P.cum_log_probs = outputs["cum_log_probs"].data_ptr() + row0 * 4
            olp = outputs.get("output_log_probs")
            P.output_log_probs = None if olp is None else olp.data_ptr()
            src, tgt = inputs.get("src_cache_indirection"), outputs.get("tgt_cache_indirection")
            P.src_cache_indirection = None if src is None else src.data_ptr()
            P.tgt_cache_indirection = None if tgt is None else tgt.data_ptr()
            if hyps is not None:
                H = BeamHyps()
                for f, _ in BeamHyps._fields_[:-1]:
                    t = hyps.get(f)
                    setattr(H, f, None if t is None else t.data_ptr())
                H.early_stopping = int(hyps.get("early_stopping", True))
                P.beam_hyps = C.pointer(H)
            P.workspace = self._beam_ws.data_ptr()
            P.workspace_bytes = self._beam_ws.numel()
            P.stream = st.value
            check(lib.ftb200_beam_search_step(C.byref(P)))
            self.launches += 1
        return self._stop_criteria(outputs, inputs, B, step, lbs, ite * lbs, beam=K)

    def _stop_criteria(self, outputs, inputs, B, step, lbs, lo, beam=1):
        """Stop words, length limit and should_stop (DynamicDecodeLayer.cc:447-473)."""
        sw = inputs.get("stop_words_list")
        lim = inputs.get("sequence_limit_length")
        if sw is None and lim is None:
            return False
        if self._count_dev is None:
            self._count_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._count_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        L = 0 if sw is None else sw.shape[-1]
        st = getattr(self, "_stream", None) or self._stream_ptr()
        check(lib.ftb200_stop_criteria(
            _ptr(outputs["output_ids"]), _ptr(outputs.get("parent_ids")),
            None if sw is None else C.c_void_p(sw.data_ptr() + lo * 2 * L * 4), L, _ptr(outputs["finished"]),
            _ptr(lim), lo * beam, lbs, B, beam, step, _ptr(self._count_dev),
            C.c_void_p(self._count_host.data_ptr()), st))
        self.launches += 1
        if lim is None:
            return False
        stop = C.c_int(0)
        check(lib.ftb200_wait_should_stop(C.c_void_p(self._count_host.data_ptr()), B, beam, st, 10000, C.byref(stop)))
        return bool(stop.value)

    def _sample(self, outputs, inputs, logits, B, step, ite, lbs, mil, lo, hi, topk_on, topp_on):
        Vp = self.vocab_size_padded
        es = logits.element_size()

        # The argument block of a slice is kept between steps: what setup() fixed (the layer's own buffers, the
        # launch order, the slice) is written once, the step's own values every time.
        P = self._g.get("params")
        if P is None or self._g["params_key"] != (B, lbs, ite, topk_on, topp_on):
            P = SamplingParams()
            P.batch_size, P.local_batch_size, P.ite = B, lbs, ite
            P.vocab_size, P.vocab_size_padded = self.vocab_size, Vp
            P.temperature = self.temperature.data_ptr() + lo * 4
            P.repetition_penalty = self.penalty.data_ptr() + lo * 4
            P.penalty_type = self.penalty_type
            P.min_lengths = self.min_length.data_ptr() + lo * 4
            if topk_on:
                P.topk_states = self.topk.curand.data_ptr() + lo * CURAND_STATE_BYTES
                P.topk_ks = self.topk.top_ks.data_ptr() + lo * 4
                P.topk_ps = self.topk.top_ps.data_ptr() + lo * 4
                P.topk_skip = self.topk.skip.data_ptr() + lo
                P.max_top_k = self.max_top_k
            if topp_on:
                P.topp_states = self.topp.curand.data_ptr() + lo * CURAND_STATE_BYTES
                P.topp_ps = self.topp.top_ps.data_ptr() + lo * 4
                P.topp_skip = self.topp.skip.data_ptr() + lo
                P.topp_initial_ps = self.topp.initial.data_ptr() + lo * 4
                P.topp_decay = self.topp.decay.data_ptr() + lo * 4
                P.topp_min = self.topp.min.data_ptr() + lo * 4
                P.topp_reset_ids = self.topp.reset.data_ptr() + lo * 4
            P.row_order = self._g["order"].data_ptr()
            self._g["params"], self._g["params_key"] = P, (B, lbs, ite, topk_on, topp_on)
        P.dtype = _DT[logits.dtype]
        P.step, P.max_input_length = step, mil
        P.logits = logits.data_ptr() + lo * Vp * es
        bias = inputs.get("embedding_bias")
        P.embedding_bias = None if bias is None else bias.data_ptr()
        P.end_ids = inputs["end_id"].data_ptr() + lo * 4
        il = inputs.get("input_lengths")
        P.input_lengths = None if il is None else il.data_ptr() + lo * 4
        P.output_ids = outputs["output_ids"].data_ptr()
        bw = inputs.get("bad_words_list")
        if bw is not None:
            shared = bw.dim() == 2 or bw.shape[0] == 1
            L = bw.shape[-1]
            P.bad_words = bw.data_ptr() if shared else bw.data_ptr() + lo * 2 * L * 4
            P.bad_words_len, P.bad_words_shared = L, int(shared)
        else:
            P.bad_words, P.bad_words_len, P.bad_words_shared = None, 0, 0
        # host-side gating of the penalty kernels (BaseSamplingLayer.cc:302-349)
        P.apply_temperature = int(bias is not None or self._g["temp"])
        P.apply_repetition = int(step > 1 and self.penalty_type != 2 and self._g["pen"])
        P.apply_min_length = int(self._g["minlen"] > step - mil)

        def sl(key, width):
            t = outputs.get(key)
            return None if t is None else t.data_ptr() + lo * width

        P.sequence_length = sl("sequence_length", 4)
        P.finished = sl("finished", 1)
        P.cum_log_probs = sl("cum_log_probs", 4)
        olp = outputs.get("output_log_probs")
        # [request_output_len, batch] sliced at (step - max_input_length) (DynamicDecodeLayer.cc:427-435)
        P.output_log_probs = None if olp is None else olp.data_ptr() + ((step - mil) * B + lo) * 4

        if self._workspace is None or self._ws_key != (P.dtype, lbs, Vp):
            need = C.c_size_t(0)
            check(lib.ftb200_sampling_workspace_bytes(P.dtype, lbs, Vp, C.byref(need)))
            if self._workspace is None or self._workspace.numel() < need.value:
                self._workspace = torch.empty(need.value, dtype=torch.uint8, device=self.device)
            self._ws_key = (P.dtype, lbs, Vp)
        P.workspace = self._workspace.data_ptr()
        P.workspace_bytes = self._workspace.numel()
        P.stream = self._stream.value
        if self.time_kernels:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            check(lib.ftb200_decode_step_sampling(C.byref(P)))
            e1.record()
            self.kernel_events.append((e0, e1))
        else:
            check(lib.ftb200_decode_step_sampling(C.byref(P)))
        self.launches += lib.ftb200_last_launch_count()
