"""CPU checks of the oracle (oracle/ft_oracle.cpp) against the reference's own known answers.

  * tests/unittests/test_sampling_layer.cu (SamplingDecodeTest): 20 cases on a 3-step, 8-column toy
    distribution; every sampled id must fall in the expected set for 30 random streams
    (fixture tests/golden/sampling_layer_kat.json, made by tests/golden/make_sampling_layer_kat.py);
  * tests/unittests/th_op/test_th_decode_op.py:290-324: repetition / presence penalty must produce
    the id sequence [v-1, v-2, v-3, v-1, v-1]; :233-288: min_length must be honoured;
  * tests/unittests/test_penalty_kernels.cu:57-119, 450-495: host penalty loops (restated inline below).
"""
import json
import os

import numpy as np
import pytest

from ft_oracle import OracleDynamicDecodeLayer, oracle_lib

HERE = os.path.dirname(os.path.abspath(__file__))
KAT = json.load(open(os.path.join(HERE, "golden", "sampling_layer_kat.json")))
FLT_MAX = np.finfo(np.float32).max


def kat_logits(dtype):
    x = np.asarray([(-FLT_MAX if v == "-FLT_MAX" else v) for v in KAT["logits"]], dtype=np.float32).reshape(3, 8)
    if dtype == "float16":
        x = np.clip(x, -65504.0, 65504.0).astype(np.float16)
    return x


def kat_runtime_args(case):
    a = {}
    if "top_k" in case:
        a["runtime_top_k"] = np.asarray(case["top_k"], np.uint32)
    if "top_p" in case:
        a["runtime_top_p"] = np.asarray(case["top_p"], np.float32)
    return a


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("case", KAT["cases"], ids=[c["name"] for c in KAT["cases"]])
def test_sampling_layer_known_answers(case, dtype):
    B, V, steps = KAT["batch_size"], KAT["vocab_size"], KAT["steps"]
    toy = kat_logits(dtype)
    lbs, ite = (B // 3, 1) if case["use_local_batch"] else (B, 0)
    rng = np.random.default_rng(0)
    for seed in range(KAT["seeds"]):
        layer = OracleDynamicDecodeLayer(V, V, dtype)
        layer.setup(B, 1, kat_runtime_args(case))
        out = {
            "output_ids": np.zeros((steps, B), np.int32),
            "cum_log_probs": np.zeros(B, np.float32),
            "output_log_probs": np.zeros((steps, B), np.float32),
        }
        for step in range(steps):
            inp = {
                "logits": np.tile(toy[step], (B, 1)), "step": step, "max_input_length": 0, "ite": ite,
                "local_batch_size": lbs, "end_id": np.full(B, KAT["end_id"], np.int32),
            }
            u = 1.0 - rng.random(B, dtype=np.float32)  # (0, 1] like curand_uniform
            layer.forward(out, inp, u, u)
        for i, allowed in enumerate(case["expected"]):
            s, b = divmod(i, B)
            assert out["output_ids"][s, b] in allowed, (case["name"], seed, s, b, out["output_ids"][s, b], allowed)


@pytest.mark.parametrize("penalty", [("repetition_penalty", 2.0), ("presence_penalty", 0.5),
                                     ("presence_penalty", 1.0)])
def test_repetition_penalty_sequence(penalty):
    V, B, mil, gen = 1024, 4, 4, 5
    layer = OracleDynamicDecodeLayer(V, V, "float32")
    layer.setup(B, 1, {"runtime_top_k": np.asarray([1], np.uint32), "runtime_top_p": np.asarray([0.0], np.float32),
                       penalty[0]: np.asarray([penalty[1]], np.float32)})
    out = {"output_ids": np.zeros((mil + gen, B), np.int32), "finished": np.zeros(B, np.bool_),
           "sequence_length": np.full(B, mil - 1, np.int32)}
    out["output_ids"][:mil] = 1
    input_lengths = np.asarray([4, 1, 2, 3], np.int32)
    for b in range(B):
        out["output_ids"][input_lengths[b]:mil, b] = 0
    logits = np.zeros((B, V), np.float32)
    logits[:, V - 1], logits[:, V - 2], logits[:, V - 3] = 2.0, 1.8, 1.6
    for step in range(mil, mil + gen):
        inp = {"logits": logits.copy(), "step": step, "max_input_length": mil, "end_id": np.zeros(B, np.int32),
               "input_lengths": input_lengths}
        layer.forward(out, inp, np.ones(B, np.float32), np.ones(B, np.float32))
    expect = np.asarray([V - 1, V - 2, V - 3, V - 1, V - 1], np.int32)
    assert (out["output_ids"][mil:] == expect[:, None]).all()


@pytest.mark.parametrize("method", [dict(top_k=1, top_p=0.0), dict(top_k=0, top_p=0.8)])
@pytest.mark.parametrize("tc", [dict(batch_size=4, mil=4, min_length=2, gen=4),
                                dict(batch_size=4, mil=4, min_length=12, gen=16)])
def test_min_length_honoured(tc, method):
    V, B, mil, gen = 256, tc["batch_size"], tc["mil"], tc["gen"]
    rng = np.random.default_rng(3)
    layer = OracleDynamicDecodeLayer(V, V, "float32")
    layer.setup(B, 1, {"runtime_top_k": np.asarray([method["top_k"]], np.uint32),
                       "runtime_top_p": np.asarray([method["top_p"]], np.float32),
                       "min_length": np.asarray([tc["min_length"]], np.int32)})
    out = {"output_ids": np.ones((mil + gen, B), np.int32), "finished": np.zeros(B, np.bool_),
           "sequence_length": np.full(B, mil - 1, np.int32)}
    for step in range(mil, mil + gen):
        logits = rng.standard_normal((B, V)).astype(np.float32)
        logits[:, 0] = logits.max(axis=1) + 1  # the end token is the most probable
        inp = {"logits": logits, "step": step, "max_input_length": mil, "end_id": np.zeros(B, np.int32)}
        u = 1.0 - rng.random(B, dtype=np.float32)
        layer.forward(out, inp, u, u)
    assert ((out["sequence_length"] + 1) >= mil + tc["min_length"]).all()


def test_penalty_kernels_host_reference():
    """Temperature and repetition penalty against plain numpy restatements of the reference's host
    loops (test_penalty_kernels.cu:188-208 temperature, :57-119 repetition)."""
    import ctypes as C
    from fastertransformer_b200._abi import SamplingParams
    rng = np.random.default_rng(5)
    B, V, Vp, step, mil = 3, 37, 40, 9, 4
    logits = rng.uniform(-5, 5, size=(B, Vp)).astype(np.float32)
    bias = rng.uniform(-5, 5, size=Vp).astype(np.float32)
    temps = np.asarray([2.0, 0.5, 1.0], np.float32)
    pens = np.asarray([1.7, 0.4, 1.0], np.float32)
    out_ids = rng.integers(0, V, size=(step + 1, B)).astype(np.int32)
    in_len = np.asarray([4, 2, 3], np.int32)
    # host reference: (x + bias) / T, then penalise each distinct history id once
    ref = (logits[:, :V] + bias[:V]) * (1.0 / (temps[:, None] + np.float32(1e-6))).astype(np.float32)
    ref = ref.astype(np.float32)
    for b in range(B):
        seen = set()
        for t in range(step):
            if in_len[b] <= t < mil:
                continue
            tok = int(out_ids[t, b])
            if tok in seen:
                continue
            seen.add(tok)
            v = ref[b, tok]
            ref[b, tok] = v * pens[b] if v < 0 else v / pens[b]
    # argmax sampling (k=1) must pick the arg-max of the penalised logits
    layer = OracleDynamicDecodeLayer(V, Vp, "float32")
    layer.setup(B, 1, {"runtime_top_k": np.asarray([1], np.uint32), "temperature": temps,
                       "repetition_penalty": pens})
    out = {"output_ids": out_ids.copy()}
    layer.forward(out, {"logits": logits, "embedding_bias": bias, "step": step, "max_input_length": mil,
                        "end_id": np.zeros(B, np.int32), "input_lengths": in_len},
                  np.ones(B, np.float32), None)
    assert (out["output_ids"][step] == ref.argmax(axis=1)).all()


def test_length_and_stop_criteria():
    lib = oracle_lib()
    B, step = 4, 5
    fin = np.asarray([0, 1, 0, 0], np.uint8)
    limit = np.asarray([6, 6, 5, 3], np.uint32)
    stop = lib.oracle_length_criterion(fin.ctypes.data, limit.ctypes.data, B, 1, step)
    assert fin.tolist() == [0, 1, 1, 1] and stop == 0
    ids = np.zeros((8, B), np.int32)
    ids[4, :] = [7, 7, 9, 7]
    ids[5, :] = [8, 3, 8, 8]
    words = np.full((B, 2, 4), -1, np.int32)
    words[:, 0, :3] = [7, 8, 3]
    words[:, 1, :2] = [2, 3]   # words: (7, 8) and (3)
    fin = np.zeros(B, np.uint8)
    lib.oracle_stop_words(ids.ctypes.data, words.ctypes.data, fin.ctypes.data, 0, 4, B, B, step)
    assert fin.tolist() == [1, 1, 0, 1]
