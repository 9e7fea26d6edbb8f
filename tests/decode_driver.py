"""TEST INFRASTRUCTURE: drives a DynamicDecodeLayer-like object (the CUDA one, the compiled reference
or the CPU oracle) through a SamplingWorkload and records what it produced."""
import numpy as np
import torch

from fastertransformer_b200.workloads import SamplingWorkload


def run_cuda_like(layer, w: SamplingWorkload, device, steps=None, want_log_probs=False, cast=None,
                  with_criteria=False, logits_hook=None):
    """layer: fastertransformer_b200.DynamicDecodeLayer or tests.ft_reference.RefDynamicDecodeLayer.
    cast: dtype the layer wants its logits in (the reference has no bf16: it gets the fp32 up-cast)."""
    steps = steps or w.steps
    st = w.initial_state(device)
    inputs = w.static_inputs(device)
    if not with_criteria:
        inputs.pop("sequence_limit_length", None)
    B = w.batch
    if want_log_probs:
        st["cum_log_probs"] = torch.zeros(B, dtype=torch.float32, device=device)
        st["output_log_probs"] = torch.zeros(w.steps, B, dtype=torch.float32, device=device)
    layer.setup(B, 1, w.runtime_args)
    rec = {"ids": [], "finished": [], "sequence_length": []}
    for s in range(steps):
        step = w.max_input_length + s
        logits = w.logits(step, device)
        if logits_hook is not None:
            logits = logits_hook(logits, step)
        if cast is not None and logits.dtype != cast:
            logits = logits.to(cast)
        inp = dict(inputs)
        inp["logits"] = logits.view(B, 1, w.vocab_padded) if hasattr(layer, "h") else logits
        inp["step"] = step
        layer.forward(st, inp)
        torch.cuda.synchronize()
        rec["ids"].append(st["output_ids"][step].cpu().numpy().copy())
        rec["finished"].append(st["finished"].cpu().numpy().copy())
        rec["sequence_length"].append(st["sequence_length"].cpu().numpy().copy())
    out = {k: np.stack(v) for k, v in rec.items()}
    if want_log_probs:
        out["cum_log_probs"] = st["cum_log_probs"].cpu().numpy()
        out["output_log_probs"] = st["output_log_probs"].cpu().numpy()[:steps]
    return out
