"""Context log-probabilities: host-side mirror of invokeLogProbFromLogits
(kernels/logprob_kernels.h:23-35) over the C-ABI entry ftb200_log_prob_from_logits."""
import torch

from ._lib import check, lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def log_prob_from_logits(logits, input_ids, input_lengths, vocab_size=None, batch_first=False, workspace=None):
    """cum_log_probs[b] = sum over step < input_lengths[b] - 1 of
    log softmax(logits[step, b, :vocab_size])[input_ids[step + 1, b]].

    logits: CUDA tensor [max_input_length, batch, vocab_size_padded] (batch-major when batch_first);
    input_ids: int32 [max_input_length, batch] (or [batch, max_input_length]); input_lengths: int32 [batch].
    workspace: optional float32 CUDA tensor with at least max_input_length * batch elements; it holds
    the per-step log-probs afterwards, as in the reference.  Returns float32 [batch]."""
    if not logits.is_cuda:
        raise ValueError("log_prob_from_logits needs CUDA tensors")
    logits = logits.contiguous()
    if batch_first:
        batch, max_len, vocab_padded = logits.shape
    else:
        max_len, batch, vocab_padded = logits.shape
    vocab_size = vocab_padded if vocab_size is None else vocab_size
    ids = input_ids.to(torch.int32).contiguous()
    lens = input_lengths.to(torch.int32).contiguous()
    if workspace is None:
        workspace = torch.empty(max_len * batch, dtype=torch.float32, device=logits.device)
    cum = torch.empty(batch, dtype=torch.float32, device=logits.device)
    check(lib.ftb200_log_prob_from_logits(cum.data_ptr(), logits.data_ptr(), _DT[logits.dtype], ids.data_ptr(),
                                          lens.data_ptr(), max_len, batch, vocab_size, vocab_padded,
                                          workspace.data_ptr(), workspace.numel() * 4,
                                          torch.cuda.current_stream().cuda_stream, int(batch_first)))
    return cum
