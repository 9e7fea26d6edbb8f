"""CPU checks of the log-prob restatement (oracle_log_prob_from_logits): against the outputs of the
reference's own kernel on seeded inputs (tests/golden/logprob_ref.json) and against a float64
restatement of the reference test's host check (tests/unittests/test_logprob_kernels.cu:38-122)."""
import json
import os
import sys

import numpy as np
import pytest

from ft_oracle import oracle_log_prob_from_logits

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from make_logprob_fixture import CASES, logprob_case  # noqa: E402

with open(os.path.join(HERE, "golden", "logprob_ref.json")) as f:
    GOLDEN = json.load(f)


def host_cum_log_probs(logits, ids, lengths, vocab, batch_first):
    """float64 form of computeCumLogProbs / computeCumLogProbsBatchFirst."""
    x = np.asarray(logits, dtype=np.float64)
    if batch_first:
        x = x.transpose(1, 0, 2)
        ids = ids.T
    max_len, batch, _ = x.shape
    x = x[:, :, :vocab]
    m = x.max(axis=2, keepdims=True)
    lse = np.log(np.exp(x - m).sum(axis=2)) + m[:, :, 0]
    cum = np.zeros(batch)
    lp = np.zeros((max_len - 1, batch))
    for step in range(1, max_len):
        for b in range(batch):
            if step < lengths[b]:
                lp[step - 1, b] = x[step - 1, b, ids[step, b]] - lse[step - 1, b]
                cum[b] += lp[step - 1, b]
    return cum, (lp.T if batch_first else lp)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_reference_kernel_outputs(case):
    name, max_len, batch, vocab, vp, dtype, bf = case
    logits, ids, lengths = logprob_case(*case)
    cum, lp = oracle_log_prob_from_logits(logits, ids, lengths, vocab, batch_first=bf)
    g = GOLDEN[name]
    steps = np.arange(max_len - 1)
    valid = steps[None, :] < (lengths[:, None] - 1) if bf else steps[:, None] < (lengths[None, :] - 1)
    # __expf / __logf of the fast-math build against libm: a few ulp per term
    np.testing.assert_allclose(np.where(valid, lp, 0.0).ravel(), np.array(g["log_probs"], np.float32),
                               rtol=0, atol=2e-5)
    np.testing.assert_allclose(cum, np.array(g["cum_log_probs"], np.float32), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_host_check(case):
    name, max_len, batch, vocab, vp, dtype, bf = case
    logits, ids, lengths = logprob_case(*case)
    cum, lp = oracle_log_prob_from_logits(logits, ids, lengths, vocab, batch_first=bf)
    want_cum, want_lp = host_cum_log_probs(logits, ids, lengths, vocab, bf)
    steps = np.arange(max_len - 1)
    valid = steps[None, :] < (lengths[:, None] - 1) if bf else steps[:, None] < (lengths[None, :] - 1)
    np.testing.assert_allclose(np.where(valid, lp, 0.0), np.where(valid, want_lp, 0.0), rtol=0, atol=2e-5)
    # the reference's own tolerance is atol 1e-4 + rtol 1e-2 (fp32), 1e-3 + 1e-1 (half) (gtest_utils.h:78-80)
    np.testing.assert_allclose(cum, want_cum, rtol=1e-5, atol=1e-4)


def test_bf16_rows_and_first_step_only():
    rng = np.random.default_rng(5)
    from ft_oracle import bf16_bits
    x = rng.uniform(-3, 3, size=(4, 2, 40)).astype(np.float32)
    bits = bf16_bits(x)
    up = (bits.astype(np.uint32) << 16).view(np.float32)
    ids = rng.integers(0, 33, size=(4, 2)).astype(np.int32)
    lengths = np.array([1, 4], np.int32)
    cum, _ = oracle_log_prob_from_logits(bits, ids, lengths, 33, dtype_name="bfloat16")
    want, _ = host_cum_log_probs(up, ids, lengths, 33, False)
    assert cum[0] == 0.0          # a sequence of length 1 has no scored token
    np.testing.assert_allclose(cum, want, rtol=1e-5, atol=1e-4)
