"""The no-allocation entry point, ftb200_decode_step_sampling_static, against the ordinary one.

Some hosts of the library cannot hand it a scratch buffer (their memory pool owns the GPU, or their step
callback may not allocate), so that entry point keeps its scratch in an area built into the library.  Here two identical decoders run the same steps, one through each entry
point, called through the C ABI; ids, finished flags and lengths must be equal and the log-probabilities
within 1e-3, on two calls in a row (the second call meets the scratch the first one left behind).  The
device's free memory must not move across the calls, and the row limit is checked at its exact boundary.
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


def _run(layer, w, device, steps, log_probs=True):
    st = w.initial_state(device)
    if log_probs:
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



@pytest.mark.parametrize("batch,vocab", [(24, 32768), (65, 128256)])
def test_static_entry_single_pass_rows_and_free_memory(batch, vocab, cuda_device, monkeypatch):
    """16-bit logits without log-probabilities take the single-pass kernels; through the static entry they run
    on the caller's stream alone.  65 rows at vocab 128256 is the largest shape the built-in area admits.
    Free device memory is read before and after the static calls (the logits of every step are made before
    the first reading) and must not move."""
    import fastertransformer_b200.decode_layer as dl
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", batch=batch, steps=3, vocab=vocab)
    ref = _run(dl.DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, cuda_device), w, cuda_device, 3, False)
    shim = _StaticEntry(dl.lib)
    monkeypatch.setattr(dl, "lib", shim)
    layer = dl.DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, cuda_device)
    _run(layer, w, cuda_device, 1, False)  # set-up of the device and of the kernel variants
    st = w.initial_state(cuda_device)
    inputs = w.static_inputs(cuda_device)
    inputs.pop("sequence_limit_length", None)
    layer.setup(w.batch, 1, w.runtime_args)
    steps = [dict(inputs, logits=w.logits(w.max_input_length + s, cuda_device), step=w.max_input_length + s)
             for s in range(3)]
    layer.forward(st, steps[0])
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info(cuda_device)[0]
    calls0 = shim.calls
    for s in (1, 2):
        layer.forward(st, steps[s])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_device)[0] == free0
    assert shim.calls == calls0 + 2
    for key in ("output_ids", "finished", "sequence_length"):
        assert (st[key].cpu().numpy() == ref[key]).all(), key


def test_static_scratch_row_limit_boundary(cuda_device):
    """The need is 256 + ceil256(4 rows) + rows * ceil256(vocab) * 8 bytes: 65 rows fit at vocab 128256, 66 do
    not.  The refusal comes before any pointer is read, so the refused side needs no buffers."""
    from fastertransformer_b200 import SamplingParams, lib
    area = lib.ftb200_static_scratch_bytes()

    def need(rows, vocab):
        n = C.c_size_t(0)
        assert lib.ftb200_sampling_workspace_bytes(2, rows, vocab, C.byref(n)) == 0
        return n.value

    assert need(65, 128256) == 256 + 512 + 65 * 128256 * 8 <= area
    assert need(66, 128256) > area
    assert need(262, 32000) <= area < need(263, 32000)
    P = SamplingParams()
    P.dtype, P.vocab_size, P.vocab_size_padded = 2, 128256, 128256
    P.batch_size = P.local_batch_size = 66
    assert lib.ftb200_decode_step_sampling_static(C.byref(P)) == 4  # FTB200_WORKSPACE_SMALL
