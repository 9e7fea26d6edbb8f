"""`FasterTransformer.DynamicDecodeOp` as a Python class on the decode layers of this package.

Same constructor and the same positional argument lists for `setup` and `forward` as the torch custom class
the reference registers (th_op/common/DynamicDecodeOp.h:158-214, DynamicDecodeOp.cc:447-454), so that a script
written against `torch.classes.FasterTransformer.DynamicDecodeOp` runs unchanged with

    decode_op = fastertransformer_b200.th_decode_op.DynamicDecodeOp(vocab, vocab_padded, 1, 1, torch.float)

Runtime arguments arrive as torch tensors (host tensors of shape [batch] for everything `setup` takes, as in
the reference's own test, tests/unittests/th_op/test_th_decode_op.py:95-123); state tensors live on the GPU and
are updated in place; `forward` returns the `should_stop` flag as a one-element bool tensor on the host.
Tensor and pipeline parallel sizes other than 1 are refused: the reference uses them only to broadcast the
result from the last pipeline rank, which is the caller's collective, not part of the decode step.
"""
import numpy as np
import torch

from .decode_layer import DynamicDecodeLayer


def _host(t, dtype):
    if t is None:
        return None
    return np.ascontiguousarray(t.detach().cpu().numpy()).astype(dtype).reshape(-1)


class DynamicDecodeOp:
    def __init__(self, vocab_size, vocab_size_padded, tensor_para_size, pipeline_para_size, scalar_type):
        if int(tensor_para_size) != 1 or int(pipeline_para_size) != 1:
            raise RuntimeError("[FT][ERROR] DynamicDecodeOp of this package runs on one rank per GPU; "
                               "tensor_para_size and pipeline_para_size must be 1")
        if scalar_type not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError("[FT][ERROR] Wrong tensor type.")
        self.vocab_size = int(vocab_size)
        self.vocab_size_padded = int(vocab_size_padded)
        self.scalar_type = scalar_type
        self._layer = None
        self._beam_args = {}

    # th_op/common/DynamicDecodeOp.cc:63-103 (FtDynamicDecode<T>::setup)
    def setup(self, batch_size, beam_width, runtime_top_k_opt=None, runtime_top_p_opt=None, temperature_opt=None,
              repetition_penalty_opt=None, presence_penalty_opt=None, min_length_opt=None, length_penalty_opt=None,
              beam_search_diversity_rate_opt=None, random_seed_opt=None, top_p_decay_opt=None, top_p_min_opt=None,
              top_p_reset_ids_opt=None):
        device = torch.device("cuda", torch.cuda.current_device())
        self._layer = DynamicDecodeLayer(self.vocab_size, self.vocab_size_padded, self.scalar_type, device)
        args = {}
        for key, t, dt in (("runtime_top_k", runtime_top_k_opt, np.uint32), ("runtime_top_p", runtime_top_p_opt, np.float32),
                           ("temperature", temperature_opt, np.float32),
                           ("repetition_penalty", repetition_penalty_opt, np.float32),
                           ("presence_penalty", presence_penalty_opt, np.float32), ("min_length", min_length_opt, np.int32),
                           ("len_penalty", length_penalty_opt, np.float32),
                           ("beam_search_diversity_rate", beam_search_diversity_rate_opt, np.float32),
                           ("random_seed", random_seed_opt, np.uint64)):
            if t is not None:
                args[key] = _host(t, dt)
        for key, t in (("top_p_decay", top_p_decay_opt), ("top_p_min", top_p_min_opt), ("top_p_reset_ids", top_p_reset_ids_opt)):
            if t is not None:
                args[key] = t.to(device)
        self._layer.setup(int(batch_size), int(beam_width), args)

    # th_op/common/DynamicDecodeOp.cc:105-257 (FtDynamicDecode<T>::forward)
    def forward(self, logits, step, max_input_length, ite, local_batch_size, end_id, runtime_top_k_opt=None,
                runtime_top_p_opt=None, temperature_opt=None, repetition_penalty_opt=None, presence_penalty_opt=None,
                min_length_opt=None, length_penalty_opt=None, beam_search_diversity_rate_opt=None, top_p_decay_opt=None,
                top_p_min_opt=None, top_p_reset_ids_opt=None, embedding_bias_opt=None, input_lengths_opt=None,
                sequence_limit_length_opt=None, stop_words_list_opt=None, bad_words_list_opt=None,
                src_cache_indirection_opt=None, output_token_ids=None, finished_opt=None, sequence_lengths_opt=None,
                cum_log_probs_opt=None, output_log_probs_opt=None, parent_ids_opt=None, tgt_cache_indirection_opt=None):
        if self._layer is None:
            raise RuntimeError("[FT][ERROR] DynamicDecodeOp.forward called before setup")
        batch, beam = logits.shape[0], logits.shape[1]
        inputs = {"logits": logits.view(batch, -1) if beam == 1 else logits, "step": int(step),
                  "max_input_length": int(max_input_length), "ite": int(ite), "local_batch_size": int(local_batch_size),
                  "end_id": end_id}
        # the beam layers read their scalars from the forward arguments (BaseBeamSearchLayer.cu:220-258)
        for key, t, dt in (("temperature", temperature_opt, np.float32),
                           ("repetition_penalty", repetition_penalty_opt, np.float32),
                           ("presence_penalty", presence_penalty_opt, np.float32), ("min_length", min_length_opt, np.int32),
                           ("len_penalty", length_penalty_opt, np.float32),
                           ("beam_search_diversity_rate", beam_search_diversity_rate_opt, np.float32)):
            if t is not None and beam > 1:
                inputs[key] = _host(t, dt)
        for key, t in (("embedding_bias", embedding_bias_opt), ("input_lengths", input_lengths_opt),
                       ("sequence_limit_length", sequence_limit_length_opt), ("stop_words_list", stop_words_list_opt),
                       ("bad_words_list", bad_words_list_opt), ("src_cache_indirection", src_cache_indirection_opt)):
            if t is not None:
                inputs[key] = t
        ids = output_token_ids
        outputs = {"output_ids": ids.view(ids.shape[0], -1) if beam == 1 else ids}
        for key, t in (("finished", finished_opt), ("sequence_length", sequence_lengths_opt),
                       ("cum_log_probs", cum_log_probs_opt), ("output_log_probs", output_log_probs_opt),
                       ("parent_ids", parent_ids_opt), ("tgt_cache_indirection", tgt_cache_indirection_opt)):
            if t is not None:
                outputs[key] = t
        stop = self._layer.forward(outputs, inputs)
        return torch.tensor([bool(stop)], dtype=torch.bool)

    def broadcast_from_last_pipeline(self, tensors):
        """One rank per GPU and no pipeline inside the op: nothing to broadcast."""
        return None
