"""GPU parity of the one-launch beam-search step against the unmodified reference
(OnlineBeamSearchLayer through DynamicDecodeLayer, compiled for sm_100a) and the CPU restatement.
ids, parents, finished, lengths and the cache indirection must be identical; cum_log_probs within 1e-3
(the soft-max denominator is summed in a different order)."""
import ctypes as C

import numpy as np
import pytest
import torch

import ft_reference

pytestmark = pytest.mark.gpu


def make_state(B, K, V, L, mil, dtype, device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    st = {
        "output_ids": torch.zeros(L, B, K, dtype=torch.int32, device=device),
        "parent_ids": torch.zeros(L, B, K, dtype=torch.int32, device=device),
        "finished": torch.zeros(B * K, dtype=torch.bool, device=device),
        "sequence_length": torch.full((B * K,), mil, dtype=torch.int32, device=device),
        "cum_log_probs": (torch.randn(B * K, generator=g, device=device) - 5.0).float(),
        "tgt_cache_indirection": torch.zeros(B, K, L, dtype=torch.int32, device=device),
    }
    st["output_ids"][:mil] = torch.randint(3, V, (mil, B, 1), generator=g, device=device, dtype=torch.int32)
    return st


def run_beam(layer, is_ref, B, K, V, L, mil, steps, dtype, device, args, seed, end_id=2):
    st = make_state(B, K, V, L, mil, dtype, device, seed)
    src = torch.zeros(B, K, L, dtype=torch.int32, device=device)
    layer.setup(B, K, args)
    rec = []
    g = torch.Generator(device=device)
    for s in range(steps):
        step = mil + s
        g.manual_seed(seed * 7919 + step)
        logits = (torch.randn(B, K, V, generator=g, device=device) * 2.0).to(dtype)
        if s >= 2:
            logits[::3, :, end_id] += 9.0     # make some beams finish
        inp = dict(args)
        inp.update({"logits": logits.clone(), "step": step, "max_input_length": mil, "ite": 0, "local_batch_size": B,
                    "end_id": torch.full((B,), end_id, dtype=torch.int32, device=device),
                    "input_lengths": torch.full((B, K), mil, dtype=torch.int32, device=device),
                    "src_cache_indirection": src})
        layer.forward(st, inp)
        torch.cuda.synchronize()
        src, st["tgt_cache_indirection"] = st["tgt_cache_indirection"], src
        rec.append({k: v.clone().cpu().numpy() for k, v in st.items()})
    return rec


@pytest.mark.parametrize("B,K,V,dtype", [(8, 4, 32000, torch.float16), (5, 2, 1031, torch.float32),
                                         (3, 3, 4096, torch.float32), (2, 8, 5000, torch.float16)])
@pytest.mark.parametrize("args", [dict(), dict(len_penalty=np.asarray([1.0], np.float32)),
                                  dict(temperature=np.asarray([0.8], np.float32),
                                       repetition_penalty=np.asarray([1.3], np.float32),
                                       min_length=np.asarray([3], np.int32),
                                       beam_search_diversity_rate=np.asarray([0.2], np.float32))],
                         ids=["plain", "lenpen", "penalties"])
def test_beam_step_against_reference(B, K, V, dtype, args, cuda_device):
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    L, mil, steps = 12, 4, 6
    ref = run_beam(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps, dtype,
                   cuda_device, args, 11)
    mine = run_beam(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype, cuda_device,
                    args, 11)
    for s, (a, b) in enumerate(zip(mine, ref)):
        for key in ("output_ids", "parent_ids", "finished", "sequence_length"):
            assert (a[key] == b[key]).all(), (s, key, np.argwhere(a[key] != b[key])[:4])
        np.testing.assert_allclose(a["cum_log_probs"], b["cum_log_probs"], rtol=1e-3, atol=2e-3)


def test_beam_config4_shape(cuda_device):
    """Config 4: batch 64, beam 4, vocab 32000, fp16, length penalty 1.0, end id 2."""
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    B, K, V, L, mil, steps, dtype = 64, 4, 32000, 10, 2, 6, torch.float16
    args = dict(len_penalty=np.asarray([1.0], np.float32))
    ref = run_beam(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps, dtype,
                   cuda_device, args, 5)
    mine = run_beam(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype, cuda_device,
                    args, 5)
    for a, b in zip(mine, ref):
        for key in ("output_ids", "parent_ids", "finished", "sequence_length", "tgt_cache_indirection"):
            assert (a[key] == b[key]).all(), key


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("FTB200_RANDOM_CASES", "24")))))
def test_random_beam_configurations_against_reference(seed, cuda_device):
    """Random batch / beam / vocabulary / penalty combinations through several steps."""
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    rng = np.random.default_rng(31000 + seed)
    dtype = [torch.float32, torch.float16][seed % 2]
    B, K = int(rng.integers(1, 9)), int(rng.choice([2, 3, 4, 5, 8, 12]))
    V = int(rng.choice([257, 1031, 4096, 32000]))
    mil, steps = int(rng.integers(2, 6)), int(rng.integers(2, 6))
    L = mil + steps + 1
    if 32 % K != 0:
        # The reference's update_kernel adds 1 to sequence_length[index] and reads its parent's entry without a
        # barrier in between (layers/beam_search_layers/OnlineBeamSearchLayer.cu:40-46): the outcome is defined
        # only while the beams of an entry share a warp.  Here everything stays inside one warp; the library
        # gives the lockstep outcome for every shape.
        B = min(B, 32 // K)
    args = {}
    if seed % 3 == 0:
        args["len_penalty"] = np.asarray([float(rng.choice([0.5, 1.0, 2.0]))], np.float32)
    if seed % 4 == 1:
        args["beam_search_diversity_rate"] = np.asarray([0.3], np.float32)
    if seed % 5 == 2:
        args["temperature"] = np.asarray([0.7], np.float32)
        args["repetition_penalty"] = np.asarray([1.4], np.float32)
    if seed % 5 == 3:
        args["presence_penalty"] = np.asarray([0.5], np.float32)
        args["min_length"] = np.asarray([2], np.int32)
    ref = run_beam(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps, dtype,
                   cuda_device, args, 500 + seed)
    mine = run_beam(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype, cuda_device,
                    args, 500 + seed)
    for s, (a, b) in enumerate(zip(mine, ref)):
        for key in ("output_ids", "parent_ids", "finished", "sequence_length", "tgt_cache_indirection"):
            assert np.array_equal(a[key], b[key]), (seed, s, key)
        np.testing.assert_allclose(a["cum_log_probs"], b["cum_log_probs"], rtol=1e-3, atol=1e-3)


class _RefBeamHyps(C.Structure):
    """Field for field the reference's struct BeamHypotheses (kernels/beam_search_topk_kernels.h:31-58); the
    fields after is_done are filled in by OnlineBeamSearchLayer::invokeSoftMax on every step."""
    _fields_ = [(n, C.c_void_p) for n in
                ("output_ids_tgt", "sequence_lengths_tgt", "cum_log_probs", "normed_scores", "log_probs",
                 "min_normed_scores", "num_beams", "is_done", "output_ids_src", "parent_ids_src",
                 "sequence_lengths_src", "end_ids", "log_probs_src")] + [
        ("step", C.c_int), ("ite", C.c_int), ("batch_size", C.c_int), ("local_batch_size", C.c_int),
        ("max_seq_len", C.c_int), ("length_penalty", C.c_float), ("early_stopping", C.c_bool),
        ("is_return_normed_score", C.c_bool)]


def _archive(B, K, L, device, with_log_probs):
    t = {
        "output_ids_tgt": torch.zeros(B, 2 * K, L, dtype=torch.int32, device=device),
        "sequence_lengths_tgt": torch.zeros(B, 2 * K, dtype=torch.int32, device=device),
        "cum_log_probs": torch.zeros(B, 2 * K, dtype=torch.float32, device=device),
        "normed_scores": torch.zeros(B, 2 * K, dtype=torch.float32, device=device),
        "min_normed_scores": torch.zeros(B, dtype=torch.float32, device=device),
        "num_beams": torch.zeros(B, dtype=torch.int32, device=device),
        "is_done": torch.zeros(B, dtype=torch.bool, device=device),
    }
    if with_log_probs:
        t["log_probs"] = torch.zeros(B, 2 * K, L, dtype=torch.float32, device=device)
    return t


def run_beam_archive(layer, is_ref, B, K, V, L, mil, steps, dtype, device, args, seed, end_id=2, with_log_probs=False,
                     bad_words=None, finish_every=3):
    """Like run_beam, with a BeamHypotheses archive (and optionally output_log_probs and a bad-word list)."""
    st = make_state(B, K, V, L, mil, dtype, device, seed)
    arch = _archive(B, K, L, device, with_log_probs)
    if with_log_probs:
        st["output_log_probs"] = torch.zeros(L, B, K, dtype=torch.float32, device=device)
    if is_ref:
        assert ft_reference.ref_lib().ftref_sizeof_beam_hyps() == C.sizeof(_RefBeamHyps)
        h = _RefBeamHyps()
        for name, t in arch.items():
            setattr(h, name, t.data_ptr())
        h.early_stopping, h.is_return_normed_score = True, True
        st["beam_hyps"] = C.addressof(h)
    else:
        st["beam_hyps"] = dict(arch, early_stopping=True)
    src = torch.zeros(B, K, L, dtype=torch.int32, device=device)
    layer.setup(B, K, args)
    rec = []
    g = torch.Generator(device=device)
    for s in range(steps):
        step = mil + s
        g.manual_seed(seed * 7919 + step)
        logits = (torch.randn(B, K, V, generator=g, device=device) * 2.0).to(dtype)
        if s >= 2 and s % finish_every == 2:
            logits[::2, :, end_id] += 7.0     # every few steps the end token gets likely: beams finish over time
        inp = dict(args)
        inp.update({"logits": logits.clone(), "step": step, "max_input_length": mil, "ite": 0, "local_batch_size": B,
                    "end_id": torch.full((B,), end_id, dtype=torch.int32, device=device),
                    "input_lengths": torch.full((B, K), mil, dtype=torch.int32, device=device),
                    "src_cache_indirection": src})
        if bad_words is not None:
            inp["bad_words_list"] = bad_words
        layer.forward(st, inp)
        torch.cuda.synchronize()
        src, st["tgt_cache_indirection"] = st["tgt_cache_indirection"], src
        snap = {k: v.clone().cpu().numpy() for k, v in st.items() if torch.is_tensor(v)}
        snap.update({"hyps_" + k: v.clone().cpu().numpy() for k, v in arch.items()})
        rec.append(snap)
    return rec


def _compare_archive(mine, ref, K):
    for s, (a, b) in enumerate(zip(mine, ref)):
        for key in ("output_ids", "parent_ids", "finished", "sequence_length", "tgt_cache_indirection", "hyps_num_beams",
                    "hyps_sequence_lengths_tgt", "hyps_output_ids_tgt"):
            assert np.array_equal(a[key], b[key]), (s, key, np.argwhere(a[key] != b[key])[:4])
        np.testing.assert_allclose(a["cum_log_probs"], b["cum_log_probs"], rtol=1e-3, atol=2e-3)
        # only the first num_beams archive slots of an entry are defined
        n = b["hyps_num_beams"]
        used = np.arange(2 * K)[None, :] < n[:, None]
        for key in ("hyps_cum_log_probs", "hyps_normed_scores"):
            np.testing.assert_allclose(a[key][used], b[key][used], rtol=1e-3, atol=2e-3, err_msg="%s step %d" % (key, s))
        has = n > 0
        np.testing.assert_allclose(a["hyps_min_normed_scores"][has], b["hyps_min_normed_scores"][has], rtol=1e-3,
                                   atol=2e-3)
        if "hyps_log_probs" in a:
            np.testing.assert_allclose(a["hyps_log_probs"][used], b["hyps_log_probs"][used], rtol=1e-3, atol=2e-3)


def test_beam_config4_archive_64_steps(cuda_device):
    """Config 4 (batch 64, beam 4, vocab 32000, fp16, length penalty 1.0, end id 2) over its 64 steps with a
    BeamHypotheses archive: finished beams are traced into the archive, an entry with beam_width archived
    hypotheses stops (kernels/online_softmax_beamsearch_kernels.cu:134-237, OnlineBeamSearchLayer.cu:51-57)."""
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    B, K, V, mil, steps, dtype = 64, 4, 32000, 2, 64, torch.float16
    L = mil + steps
    args = dict(len_penalty=np.asarray([1.0], np.float32))
    ref = run_beam_archive(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps,
                           dtype, cuda_device, args, 5, finish_every=7)
    mine = run_beam_archive(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype,
                            cuda_device, args, 5, finish_every=7)
    nb = ref[-1]["hyps_num_beams"]
    assert nb.max() == K and (nb > 0).sum() >= B // 4, nb
    _compare_archive(mine, ref, K)


@pytest.mark.parametrize("B,K,V,dtype,lp", [(6, 4, 4096, torch.float32, True), (8, 2, 1031, torch.float16, False),
                                            (4, 8, 5000, torch.float32, False)])
def test_beam_archive_small_shapes(B, K, V, dtype, lp, cuda_device):
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    mil, steps = 3, 14
    L = mil + steps
    args = dict(len_penalty=np.asarray([0.6], np.float32))
    ref = run_beam_archive(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps,
                           dtype, cuda_device, args, 21, with_log_probs=lp)
    mine = run_beam_archive(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype,
                            cuda_device, args, 21, with_log_probs=lp)
    assert ref[-1]["hyps_num_beams"].max() > 0
    _compare_archive(mine, ref, K)


@pytest.mark.parametrize("shared", [True, False], ids=["shared-list", "per-row-list"])
def test_beam_bad_words_against_reference(shared, cuda_device):
    """The stand-alone bad-word ban in front of the beam step (layers/DynamicDecodeLayer.cc:247-283,
    kernels/ban_bad_words.cu:24-100): multi-token words follow the beams' parent chain."""
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    from fastertransformer_b200 import DynamicDecodeLayer
    B, K, V, mil, steps, dtype = 5, 4, 64, 3, 8, torch.float32
    L = mil + steps
    rng = np.random.default_rng(8)
    nw, Lw = 40, 80
    n_lists = 1 if shared else B
    bw = np.full((n_lists, 2, Lw), -1, np.int32)
    bw[:, 0, :] = 0
    for b in range(n_lists):
        pos = 0
        for i in range(nw):
            n = 1 if i < 6 else 2            # a vocabulary of 64: two-token words match often
            bw[b, 0, pos:pos + n] = rng.integers(3, V, size=n)
            pos += n
            bw[b, 1, i] = pos
    t = torch.from_numpy(bw[0] if shared else bw).to(cuda_device)
    ref = run_beam_archive(ft_reference.RefDynamicDecodeLayer(V, V, dtype, cuda_device), True, B, K, V, L, mil, steps,
                           dtype, cuda_device, {}, 33, bad_words=t)
    mine = run_beam_archive(DynamicDecodeLayer(V, V, dtype, cuda_device), False, B, K, V, L, mil, steps, dtype,
                            cuda_device, {}, 33, bad_words=t)
    one = set(int(x) for x in (bw[0, 0, :6] if shared else []))
    if shared:
        assert not (set(int(x) for x in ref[-1]["output_ids"][mil:].reshape(-1)) & one)
    _compare_archive(mine, ref, K)
