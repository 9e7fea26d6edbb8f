"""Two host threads driving one GPU at the same time, each with its own layer, state and CUDA stream (ctypes releases
the interpreter lock during the library calls, so the calls do overlap).  The per-device state the calls share - the
second stream of the single-pass step with its fork and join events, the occupancy caches - must not let one
thread's step see the other's: both threads must reproduce the ids of the same workloads run one after the other."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode(seed, device, stream, steps, out, key):
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", batch=48, steps=steps, vocab=32768, seed=seed)
    with torch.cuda.stream(stream):
        layer = DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, device)
        layer.stream = stream
        st = w.initial_state(device)
        inputs = w.static_inputs(device)
        layer.setup(w.batch, 1, w.runtime_args)
        logits = [w.logits(w.max_input_length + s, device) for s in range(steps)]
        stream.synchronize()
        for s in range(steps):
            layer.forward(st, dict(inputs, logits=logits[s], step=w.max_input_length + s))
        stream.synchronize()
    out[key] = st["output_ids"].cpu().numpy()


def test_two_threads_one_device(cuda_device):
    steps = 24
    alone, together = {}, {}
    for i, seed in enumerate((11, 12)):
        _decode(seed, cuda_device, torch.cuda.Stream(device=cuda_device), steps, alone, i)
    threads = [threading.Thread(target=_decode, args=(seed, cuda_device, torch.cuda.Stream(device=cuda_device), steps,
                                                      together, i)) for i, seed in enumerate((11, 12))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert set(together) == {0, 1}
    for i in (0, 1):
        assert np.array_equal(alone[i], together[i]), "thread %d differs from its run alone" % i
