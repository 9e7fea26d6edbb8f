"""The no-allocation entry point, ftb200_decode_step_sampling_static, against the ordinary one.

Some hosts of the library cannot hand it a scratch buffer (their memory pool owns the GPU, their step
callback may not allocate, or they are inside a stream capture), so that entry point keeps its scratch in
an area built into the library.  Here two identical decoders run the same steps, one through each entry
point, called through the C ABI; ids, finished flags and lengths must be equal and the log-probabilities
within 1e-3, on two calls in a row (the second call meets the scratch the first one left behind).
The file name makes pytest collect it last, so a failure here cannot hide the result of another test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


class _StaticEntry:
    """Forwards to libftb200 but sends the fused step through the no-allocation entry point."""

    def __init__(self, lib):
        self._lib = lib
        self.calls = 0

    def __getattr__(self, name):
        return getattr(self._lib, name)

    def ftb200_decode_step_sampling(self, params):
        self.calls += 1
        p = params._obj  # the argument block behind byref()
        p.workspace, p.workspace_bytes = None, 0  # prove the caller's workspace is not used
        return self._lib.ftb200_decode_step_sampling_static(params)


def _run(layer, w, device, steps):
    st = w.initial_state(device)
    st["cum_log_probs"] = torch.zeros(w.batch, device=device)
    st["output_log_probs"] = torch.zeros(w.steps, w.batch, device=device)
    inputs = w.static_inputs(device)
    inputs.pop("sequence_limit_length", None)
    layer.setup(w.batch, 1, w.runtime_args)
    for s in range(steps):
        step = w.max_input_length + s
        layer.forward(st, dict(inputs, logits=w.logits(step, device), step=step))
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in st.items()}


@pytest.mark.parametrize("name", ["c3", "c2"])
def test_static_scratch_matches_workspace_entry(name, cuda_device, monkeypatch):
    import fastertransformer_b200.decode_layer as dl
    from fastertransformer_b200.workloads import make_workload
    w = make_workload(name, batch=24, steps=2, vocab=16384)
    ref = _run(dl.DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, cuda_device), w, cuda_device, 2)
    shim = _StaticEntry(dl.lib)
    monkeypatch.setattr(dl, "lib", shim)
    got = _run(dl.DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, cuda_device), w, cuda_device, 2)
    assert shim.calls == 2
    for key in ("output_ids", "finished", "sequence_length"):
        assert (got[key] == ref[key]).all(), key
    np.testing.assert_allclose(got["cum_log_probs"], ref["cum_log_probs"], rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(got["output_log_probs"], ref["output_log_probs"], rtol=1e-3, atol=1e-4)


def test_static_scratch_refuses_oversized_shape(cuda_device):
    from fastertransformer_b200 import SamplingParams, lib
    P = SamplingParams()
    P.dtype, P.batch_size, P.local_batch_size, P.vocab_size, P.vocab_size_padded = 2, 1024, 1024, 128256, 128256
    rc = lib.ftb200_decode_step_sampling_static(C.byref(P))
    assert rc == 4  # FTB200_WORKSPACE_SMALL
    msg = lib.ftb200_last_error_string().decode()
    assert "built-in area" in msg and str(lib.ftb200_static_scratch_bytes()) in msg
