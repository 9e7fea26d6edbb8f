"""One process driving two GPUs in turn (needs at least two): the per-device state of the library - the shared-memory
opt-in and occupancy of every kernel variant, the SM count, the second stream of the single-pass step - must be set up
on each device on its own.  The same seeded workload runs on cuda:0, then on cuda:1, then on cuda:0 again, through the
general kernel (fp32) and through the single-pass kernels (bf16); all runs must give the same ids."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(device, dtype, vocab):
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", batch=24, steps=3, vocab=vocab)
    w.dtype = dtype
    torch.cuda.set_device(device)
    layer = DynamicDecodeLayer(w.vocab, w.vocab_padded, dtype, device)
    st = w.initial_state(device)
    inputs = w.static_inputs(device)
    layer.setup(w.batch, 1, w.runtime_args)
    for s in range(w.steps):
        step = w.max_input_length + s
        layer.forward(st, dict(inputs, logits=w.logits(step, torch.device("cpu")).to(device), step=step))
    torch.cuda.synchronize(device)
    return st["output_ids"].cpu().numpy()


@pytest.mark.parametrize("dtype,vocab", [(torch.float32, 8192), (torch.bfloat16, 32768)])
def test_same_ids_on_both_devices_from_one_process(dtype, vocab):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    a = _run(d0, dtype, vocab)
    b = _run(d1, dtype, vocab)
    c = _run(d0, dtype, vocab)
    assert np.array_equal(a, b), "the second device does not reproduce the first"
    assert np.array_equal(a, c)
