"""GPU parity of the features around the selection itself, each against the unmodified reference
DynamicDecodeLayer compiled for sm_100a (oracle/_ref), through the C ABI of libftb200.so:
  * embedding_bias (layers/sampling_layers/BaseSamplingLayer.cc:302-312, kernels/sampling_penalty_kernels.cu:117-147,
    kernels/sampling_topk_kernels.cu:67-110, kernels/sampling_topp_kernels.cu:1294-1345);
  * stop words and the length limit with the returned should_stop (kernels/stop_criteria_kernels.cu:24-157,
    layers/DynamicDecodeLayer.cc:447-473);
  * top_p_decay / top_p_min / top_p_reset_ids (kernels/sampling_topp_kernels.cu:1381-1427,
    layers/sampling_layers/TopPSamplingLayer.cu:30-109);
  * k above 1024 (kernels/sampling_topk_kernels.cu:394, pinned by tests/unittests/test_sampling_kernels.cu:431);
  * configuration 3 at its full size, bit for bit;
  * the bounded wait for should_stop running out."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import ft_reference

pytestmark = pytest.mark.gpu


def _layers(w, device):
    from fastertransformer_b200 import DynamicDecodeLayer
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    ref_dt = torch.float32 if w.dtype == torch.bfloat16 else w.dtype
    return (DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, device),
            ft_reference.RefDynamicDecodeLayer(w.vocab, w.vocab_padded, ref_dt, device), ref_dt)


def _run(layer, w, device, cast=None, extra_inputs=None, steps=None, is_ref=False):
    """Drives a layer through the workload with every input the workload has (length limit included) plus
    `extra_inputs`; records ids, finished, lengths and the returned should_stop of every step."""
    steps = steps or w.steps
    st = w.initial_state(device)
    inputs = w.static_inputs(device)
    for key, val in (extra_inputs or {}).items():
        if torch.is_tensor(val) and val.is_floating_point() and cast is not None and key == "embedding_bias":
            val = val.to(cast)
        inputs[key] = val
    B = w.batch
    if "stop_words_list" in inputs:
        # the reference looks the tensor up whenever stop words are given, whatever the beam width
        st["parent_ids"] = torch.zeros_like(st["output_ids"])
    layer.setup(B, 1, w.runtime_args)
    rec = {"ids": [], "finished": [], "sequence_length": [], "stop": []}
    for s in range(steps):
        step = w.max_input_length + s
        logits = w.logits(step, device)
        if cast is not None and logits.dtype != cast:
            logits = logits.to(cast)
        inp = dict(inputs)
        inp["logits"] = logits.view(B, 1, w.vocab_padded) if is_ref else logits
        inp["step"] = step
        stop = layer.forward(st, inp)
        torch.cuda.synchronize()
        rec["ids"].append(st["output_ids"][step].cpu().numpy().copy())
        rec["finished"].append(st["finished"].cpu().numpy().copy())
        rec["sequence_length"].append(st["sequence_length"].cpu().numpy().copy())
        rec["stop"].append(bool(stop))
    return {k: np.stack(v) for k, v in rec.items()}


def _same(mine, ref, what, keys=("ids", "finished", "sequence_length", "stop")):
    for key in keys:
        bad = np.argwhere(mine[key] != ref[key])
        assert bad.size == 0, "%s: %s differs at %d of %d entries, first %s (mine %s, reference %s)" % (
            what, key, len(bad), mine[key].size, bad[0], mine[key][tuple(bad[0])], ref[key][tuple(bad[0])])


# ---- embedding bias ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["f32", "f16", "bf16"])
@pytest.mark.parametrize("temperature", [False, True], ids=["t1", "temp"])
@pytest.mark.parametrize("vocab", [4099, 32000])
def test_embedding_bias_against_reference(dtype, temperature, vocab, cuda_device):
    from fastertransformer_b200.workloads import SamplingWorkload, _bad_words
    rng = np.random.default_rng(vocab + 17 * int(temperature))
    B, mil, steps = 24, 12, 4
    args = {"runtime_top_k": rng.choice(np.asarray([0, 1, 3, 40, 700], np.uint32), size=B),
            "runtime_top_p": rng.choice(np.asarray([0.0, 0.3, 0.9], np.float32), size=B),
            "repetition_penalty": np.asarray([1.25], np.float32),
            "random_seed": rng.integers(0, 2 ** 40, size=B).astype(np.uint64)}
    if temperature:
        args["temperature"] = rng.choice(np.asarray([0.6, 1.0, 1.4], np.float32), size=B)
    w = SamplingWorkload("bias", B, vocab, vocab, dtype, 2.0, steps, mil, vocab - 2, args, 600 + vocab,
                         bad_words=_bad_words(rng, B, vocab),
                         prompt=rng.integers(0, vocab, size=(mil, B)).astype(np.int32))
    g = torch.Generator(device=cuda_device)
    g.manual_seed(vocab)
    # values that every logits type holds exactly, so that the fp32 reference of a bf16 run sees the same bias
    bias = (torch.randn(vocab, generator=g, device=cuda_device) * 1.5).to(torch.bfloat16).to(dtype)
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, extra_inputs={"embedding_bias": bias.to(ref_dt)}, is_ref=True)
    mine = _run(mine_l, w, cuda_device, extra_inputs={"embedding_bias": bias})
    _same(mine, ref, "embedding_bias")


# ---- stop words, length limit, should_stop ----------------------------------------------------------------
@pytest.mark.parametrize("name,kw", [("c3", dict(batch=32, steps=8, vocab=8192)), ("c1", dict(batch=8, steps=8)),
                                     ("c2", dict(batch=16, steps=6))], ids=["c3", "c1", "c2"])
def test_stop_criteria_against_reference(name, kw, cuda_device):
    """Stop words are cut from what the rows really generate (a first run without them tells), so they fire;
    the length limit is ragged so that rows finish at different steps and should_stop turns true inside the run."""
    from fastertransformer_b200.workloads import make_workload
    w = make_workload(name, **kw)
    B, mil = w.batch, w.max_input_length
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    w.sequence_limit = None
    plain = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True)
    ids = plain["ids"]                                    # [steps, batch]
    L = 6
    sw = np.full((B, 2, L), -1, np.int32)
    sw[:, 0, :] = 0
    for b in range(B):
        if b % 3 == 0:       # one-token word: the token of step 2
            sw[b, 0, 0], sw[b, 1, 0] = ids[2, b], 1
        elif b % 3 == 1:     # two-token word ending at step 3, then a word that never matches
            sw[b, 0, 0:2], sw[b, 1, 0] = ids[2:4, b], 2
            sw[b, 0, 2:5], sw[b, 1, 1] = [1, 2, 3], 5
        else:                # three tokens reaching back into the prompt
            sw[b, 0, 0:3] = [w.prompt[mil - 1, b], ids[0, b], ids[1, b]]
            sw[b, 1, 0] = 3
    w.sequence_limit = (mil + 2 + (np.arange(B) % (w.steps - 2))).astype(np.uint32)
    extra = {"stop_words_list": torch.from_numpy(sw).to(cuda_device)}
    mine_l2, ref_l2, _ = _layers(w, cuda_device)
    ref = _run(ref_l2, w, cuda_device, cast=ref_dt, extra_inputs=extra, is_ref=True)
    mine = _run(mine_l2, w, cuda_device, extra_inputs=extra)
    assert ref["finished"][3].any() and not ref["finished"][0].all()
    assert ref["stop"][-1] and not ref["stop"][0], ref["stop"]
    _same(mine, ref, "stop criteria")


def test_length_limit_only_against_reference(cuda_device):
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", batch=20, steps=5, vocab=4099)
    w.sequence_limit = (w.max_input_length + 1 + (np.arange(w.batch) % 4)).astype(np.uint32)
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True)
    mine = _run(mine_l, w, cuda_device)
    assert ref["stop"][-1] and not ref["stop"][0]
    _same(mine, ref, "length limit")


def test_wait_should_stop_times_out(cuda_device):
    """The wait for the finished count gives up after its deadline with FTB200_TIMEOUT while the stream is
    still busy.  The stream is held by a host callback that sleeps (cudaLaunchHostFunc): nothing on the GPU
    waits, and the stream drains by itself afterwards."""
    from fastertransformer_b200 import lib
    rt = C.CDLL("libcudart.so.12")
    HOSTFN = C.CFUNCTYPE(None, C.c_void_p)
    slept = []

    def _sleep(_):
        time.sleep(0.25)
        slept.append(1)

    cb = HOSTFN(_sleep)
    rt.cudaLaunchHostFunc.argtypes = [C.c_void_p, HOSTFN, C.c_void_p]
    stream = torch.cuda.Stream(device=cuda_device)
    count = torch.zeros(1, dtype=torch.int32).pin_memory()
    assert rt.cudaLaunchHostFunc(C.c_void_p(stream.cuda_stream), cb, None) == 0
    stop = C.c_int(-7)
    rc = lib.ftb200_wait_should_stop(C.c_void_p(count.data_ptr()), 4, 1, C.c_void_p(stream.cuda_stream), 1,
                                     C.byref(stop))
    assert rc == 6, rc                          # FTB200_TIMEOUT
    assert stop.value == -7                     # untouched
    assert b"deadline" in lib.ftb200_last_error_string()
    stream.synchronize()
    assert slept == [1]
    # with the stream drained the same call answers
    count[0] = 4
    rc = lib.ftb200_wait_should_stop(C.c_void_p(count.data_ptr()), 4, 1, C.c_void_p(stream.cuda_stream), 1,
                                     C.byref(stop))
    assert rc == 0 and stop.value == 1


# ---- top-p decay ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["f32", "f16", "bf16"])
def test_top_p_decay_against_reference(dtype, cuda_device):
    from fastertransformer_b200.workloads import SamplingWorkload
    rng = np.random.default_rng(4242)
    B, V, mil, steps = 32, 1024, 4, 24
    p0 = rng.choice(np.asarray([0.95, 0.8, 0.6], np.float32), size=B)
    k = np.where(np.arange(B) % 8 == 7, 5, 0).astype(np.uint32)       # a few top-k rows in between
    decay = rng.choice(np.asarray([0.7, 0.9, 1.0], np.float32), size=B)
    pmin = rng.choice(np.asarray([0.05, 0.3], np.float32), size=B)
    reset = rng.integers(0, 12, size=B).astype(np.int32)             # small ids: the peaked rows draw them often
    args = {"runtime_top_k": k, "runtime_top_p": p0, "random_seed": rng.integers(0, 2 ** 40, size=B).astype(np.uint64),
            "top_p_decay": torch.from_numpy(decay).to(cuda_device), "top_p_min": torch.from_numpy(pmin).to(cuda_device),
            "top_p_reset_ids": torch.from_numpy(reset).to(cuda_device)}
    w = SamplingWorkload("decay", B, V, V, dtype, 1.0, steps, mil, V - 1, args, 99,
                         prompt=rng.integers(0, V, size=(mil, B)).astype(np.int32))
    base = w.logits

    def peaked(step, device, generator=None):
        x = base(step, device, generator).float()
        x[:, :12] += 5.0                      # the reset ids carry most of the mass
        return x.to(dtype)

    w.logits = peaked
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True)
    mine = _run(mine_l, w, cuda_device)
    _same(mine, ref, "top_p_decay")
    # the decayed runtime_top_p, recomputed from the ids (sampling_topp_kernels.cu:1381-1408, fp32)
    p = p0.copy()
    resets = 0
    for s in range(steps):
        hit = ref["ids"][s] == reset
        resets += int(hit[k == 0].sum())
        p = np.where(hit, p0, np.maximum((p * decay).astype(np.float32), pmin)).astype(np.float32)
    got = mine_l.topp.top_ps.cpu().numpy()
    rows = k == 0
    assert resets > 0 and (p[rows] != p0[rows]).any()
    np.testing.assert_array_equal(got[rows], p[rows])


# ---- k above the supported range ---------------------------------------------------------------------------
def test_top_k_above_1024_is_a_domain_error(cuda_device):
    """The kernel entry refuses k > 1024 the way invokeBatchTopKSampling does (std::domain_error there,
    FTB200_DOMAIN_ERROR with the same message here); the layer's set-up clips k to 1024 like the reference's."""
    from fastertransformer_b200 import DynamicDecodeLayer, lib
    from fastertransformer_b200._lib import SamplingParams
    B, V = 4, 4096
    layer = DynamicDecodeLayer(V, V, torch.float32, cuda_device)
    layer.setup(B, 1, {"runtime_top_k": np.asarray([1025], np.uint32), "random_seed": np.asarray([1], np.uint64)})
    assert layer.max_top_k == 1024            # TopKSamplingLayer.cu:52-56: clipped with a warning
    logits = torch.randn(B, V, device=cuda_device)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=cuda_device)
    ids = torch.zeros(2, B, dtype=torch.int32, device=cuda_device)
    end = torch.zeros(B, dtype=torch.int32, device=cuda_device)
    P = SamplingParams()
    P.dtype, P.batch_size, P.local_batch_size, P.vocab_size, P.vocab_size_padded, P.step = 0, B, B, V, V, 1
    P.logits, P.end_ids, P.output_ids = logits.data_ptr(), end.data_ptr(), ids.data_ptr()
    P.topk_states = layer.topk.curand.data_ptr()
    P.topk_ks, P.topk_ps, P.topk_skip = layer.topk.top_ks.data_ptr(), layer.topk.top_ps.data_ptr(), layer.topk.skip.data_ptr()
    P.workspace, P.workspace_bytes = ws.data_ptr(), ws.numel()
    for bad in (1025, 0, 5000):
        P.max_top_k = bad
        rc = lib.ftb200_decode_step_sampling(C.byref(P))
        assert rc == 2, (bad, rc)             # FTB200_DOMAIN_ERROR
        assert b"top-k kernel supports 1<=k<=1024 but got k=%d" % bad in lib.ftb200_last_error_string()
    P.max_top_k = 1024
    assert lib.ftb200_decode_step_sampling(C.byref(P)) == 0
    torch.cuda.synchronize()


# ---- configuration 3 at full size ------------------------------------------------------------------------------
def test_config3_full_size_bit_exact(cuda_device):
    """Batch 1024 x vocabulary 128256 bf16, three steps: ids, finished and lengths of every row equal the
    reference's (fed the fp32 up-cast, as it has no bf16 form)."""
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", steps=3)
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True)
    del ref_l
    torch.cuda.empty_cache()
    mine = _run(mine_l, w, cuda_device)
    _same(mine, ref, "config 3, 1024 x 128256")
    # banned words never come out: a one-token word bans its token outright
    bw = w.bad_words
    for b in range(w.batch):
        ends = bw[b, 1]
        start = 0
        for e in ends[ends >= 0]:
            if e - start == 1:
                assert (mine["ids"][:, b] != bw[b, 0, start]).all()
            start = e


# ---- longest token history the kernels take ------------------------------------------------------------------
def test_history_limit_against_reference(cuda_device):
    """With a repetition penalty on, the columns of the token history live in a shared-memory table of at most
    8192 slots (two per column): steps up to 4094 run and equal the reference, step 4095 is refused with
    FTB200_UNSUPPORTED and leaves the row state untouched."""
    from fastertransformer_b200 import FtbError
    from fastertransformer_b200.workloads import SamplingWorkload
    rng = np.random.default_rng(31)
    B, V, mil, steps = 2, 4099, 4091, 5                       # steps 4091 .. 4095
    args = {"runtime_top_k": np.asarray([3, 0], np.uint32), "runtime_top_p": np.asarray([0.0, 0.8], np.float32),
            "repetition_penalty": np.asarray([1.2], np.float32), "random_seed": np.asarray([3, 4], np.uint64)}
    w = SamplingWorkload("long", B, V, V, torch.float32, 2.0, steps, mil, V - 1, args, 12,
                         prompt=rng.integers(0, V, size=(mil, B)).astype(np.int32))
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True, steps=4)
    mine = _run(mine_l, w, cuda_device, steps=4)
    _same(mine, ref, "history of 4091..4094 tokens")
    with pytest.raises(FtbError) as e:
        _run(mine_l, w, cuda_device, steps=5)
    assert e.value.status == 5 and "history too long" in str(e.value)      # FTB200_UNSUPPORTED


@pytest.mark.parametrize("dtype,mil", [(torch.bfloat16, 1500), (torch.float16, 1100), (torch.bfloat16, 3000),
                                       (torch.float16, 4060)])
def test_long_history_single_pass_rows_against_reference(dtype, mil, cuda_device):
    """Histories of more than 1024 ids at a vocabulary the single-pass kernels serve: the ids come through the
    staging area a tile at a time and the table of special columns grows to 4096 / 8192 slots.  Mixed top-k and
    top-p rows, bad words, three steps, ids / flags / lengths equal to the reference."""
    from fastertransformer_b200.workloads import SamplingWorkload, _bad_words
    rng = np.random.default_rng(mil)
    B, V, steps = 10, 32768, 3
    args = {"runtime_top_k": np.asarray([1, 0, 40, 0, 8, 1024, 0, 2, 0, 64], np.uint32),
            "runtime_top_p": np.asarray([0.0, 0.5, 0.9, 0.95, 1.0, 0.7, 0.3, 0.0, 0.8, 0.6], np.float32),
            "repetition_penalty": np.asarray([1.15], np.float32),
            "random_seed": (np.arange(B) * 7 + 1).astype(np.uint64)}
    # (a prompt drawn from a part of the vocabulary, so that many ids repeat as they do in real text)
    prompt = rng.integers(0, 6000, size=(mil, B)).astype(np.int32)
    w = SamplingWorkload("longfast", B, V, V, dtype, 2.5, steps, mil, V - 1, args, 77,
                         bad_words=_bad_words(rng, B, V), prompt=prompt)
    mine_l, ref_l, ref_dt = _layers(w, cuda_device)
    ref = _run(ref_l, w, cuda_device, cast=ref_dt, is_ref=True)
    mine = _run(mine_l, w, cuda_device)
    _same(mine, ref, "history of %d ids" % mil)
