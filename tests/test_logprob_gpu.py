"""ftb200_log_prob_from_logits against the reference's invokeLogProbFromLogits (oracle/_ref), the CPU
restatement and the committed outputs of the reference kernel.  Shapes are the reference test's own
(tests/unittests/test_logprob_kernels.cu:265-303) plus ragged, padded and unaligned rows."""
import json
import os
import sys

import numpy as np
import pytest
import torch

import ft_reference
from ft_oracle import oracle_log_prob_from_logits

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from make_logprob_fixture import CASES, logprob_case  # noqa: E402

# log-probs are floating point: 1e-3 absolute per scored token is the bar; sums over n tokens get n times that
TOL = 1e-3


def run_ours(logits, ids, lengths, vocab, bf):
    from fastertransformer_b200 import log_prob_from_logits
    max_len = logits.shape[1] if bf else logits.shape[0]
    batch = logits.shape[0] if bf else logits.shape[1]
    ws = torch.zeros(max_len * batch, dtype=torch.float32, device="cuda")
    cum = log_prob_from_logits(logits, ids, lengths, vocab_size=vocab, batch_first=bf, workspace=ws)
    torch.cuda.synchronize()
    return cum.cpu().numpy(), ws[:(max_len - 1) * batch].cpu().numpy()


def run_ref(logits, ids, lengths, vocab, bf):
    lib = ft_reference.ref_lib()
    max_len = logits.shape[1] if bf else logits.shape[0]
    batch = logits.shape[0] if bf else logits.shape[1]
    ws = torch.zeros(max_len * batch, dtype=torch.float32, device="cuda")
    cum = torch.zeros(batch, dtype=torch.float32, device="cuda")
    rc = lib.ftref_log_prob_from_logits(cum.data_ptr(), logits.data_ptr(), 0 if logits.dtype == torch.float32 else 1,
                                        ids.data_ptr(), lengths.data_ptr(), max_len, batch, vocab,
                                        logits.shape[2], ws.data_ptr(), ws.numel() * 4, None, int(bf))
    torch.cuda.synchronize()
    assert rc == 0
    return cum.cpu().numpy(), ws[:(max_len - 1) * batch].cpu().numpy()


def valid_mask(lengths, max_len, bf):
    steps = np.arange(max_len - 1)
    m = steps[None, :] < (lengths[:, None] - 1) if bf else steps[:, None] < (lengths[None, :] - 1)
    return m.ravel()


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_committed_reference_outputs(case):
    name, max_len, batch, vocab, vp, dtype, bf = case
    with open(os.path.join(HERE, "golden", "logprob_ref.json")) as f:
        g = json.load(f)[name]
    logits, ids, lengths = logprob_case(*case)
    cum, lp = run_ours(torch.from_numpy(logits).cuda(), torch.from_numpy(ids).cuda(),
                       torch.from_numpy(lengths).cuda(), vocab, bf)
    m = valid_mask(lengths, max_len, bf)
    np.testing.assert_allclose(np.where(m, lp, 0.0), np.array(g["log_probs"], np.float32), rtol=0, atol=TOL)
    np.testing.assert_allclose(cum, np.array(g["cum_log_probs"], np.float32), rtol=0, atol=TOL * max_len)


REF_SHAPES = [(1, 32, 16), (129, 8, 50211), (1023, 8, 5001), (4096, 8, 5001)]


@pytest.mark.skipif(not ft_reference.available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("bf", [False, True], ids=["step_major", "batch_first"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("shape", REF_SHAPES, ids=[f"len{s[0]}_b{s[1]}_v{s[2]}" for s in REF_SHAPES])
def test_reference_test_shapes(shape, dtype, bf):
    max_input_length, batch, vocab = shape
    max_len = max_input_length + 1        # the reference test scores max_input_length tokens (:140)
    g = torch.Generator(device="cuda").manual_seed(max_len * 7 + batch)
    full = (batch, max_len, vocab) if bf else (max_len, batch, vocab)
    logits = (torch.rand(full, generator=g, device="cuda") * 6 - 3).to(dtype)
    ids = torch.randint(0, vocab, (batch, max_len) if bf else (max_len, batch), generator=g, device="cuda",
                        dtype=torch.int32)
    lengths = torch.randint(1, max_len + 1, (batch,), generator=g, device="cuda", dtype=torch.int32)
    lengths[0] = max_len
    cum, lp = run_ours(logits, ids, lengths, vocab, bf)
    rcum, rlp = run_ref(logits, ids, lengths, vocab, bf)
    m = valid_mask(lengths.cpu().numpy(), max_len, bf)
    assert np.abs(np.where(m, lp - rlp, 0.0)).max() <= 2e-5       # same arithmetic up to summation order
    n = lengths.cpu().numpy().astype(np.float64)
    assert (np.abs(cum - rcum) <= 1e-6 * np.abs(rcum) + 2e-5 * np.sqrt(n) + 1e-4).all()
    # the reference test's own check, against its host computation (gtest_utils.h:39-102)
    atol, rtol = (1e-4, 1e-2) if dtype == torch.float32 else (1e-3, 1e-1)
    x = logits.float().double()
    if bf:
        x = x.transpose(0, 1)
        idm = ids.t()
    else:
        idm = ids
    lsm = torch.log_softmax(x[:-1], dim=2)
    tok = torch.gather(lsm, 2, idm[1:].long().unsqueeze(2))[:, :, 0]
    steps = torch.arange(max_len - 1, device="cuda")[:, None]
    want = torch.where(steps < (lengths[None, :] - 1), tok, torch.zeros_like(tok)).sum(0).cpu().numpy()
    assert (np.abs(cum - want) <= atol + rtol * np.abs(want)).all()


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("bf", [False, True], ids=["step_major", "batch_first"])
def test_padded_unaligned_rows_against_restatement(dtype, bf):
    # vocab_padded odd: rows start at every 2- or 4-byte phase of a 16-byte line; vocab < padded
    max_len, batch, vocab, vp = 7, 5, 1003, 1011
    rng = np.random.default_rng(17)
    shape = (batch, max_len, vp) if bf else (max_len, batch, vp)
    x = rng.uniform(-6, 6, size=shape).astype(np.float32)
    x[..., vocab:] = 50.0                       # padding must not be counted
    ids = rng.integers(0, vocab, size=(batch, max_len) if bf else (max_len, batch)).astype(np.int32)
    lengths = np.array([7, 1, 2, 5, 7], np.int32)
    tdt = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    d = torch.from_numpy(x).cuda().to(tdt)
    if dtype == "bfloat16":
        host = d.view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        host = d.cpu().numpy()
    cum, lp = run_ours(d, torch.from_numpy(ids).cuda(), torch.from_numpy(lengths).cuda(), vocab, bf)
    ocum, olp = oracle_log_prob_from_logits(host, ids, lengths, vocab, batch_first=bf, dtype_name=dtype)
    m = valid_mask(lengths, max_len, bf)
    np.testing.assert_allclose(np.where(m, lp, 0.0), np.where(m, olp.ravel(), 0.0), rtol=0, atol=2e-5)
    np.testing.assert_allclose(cum, ocum, rtol=0, atol=1e-4)
    assert cum[1] == 0.0


def test_argument_checks():
    from fastertransformer_b200 import lib
    x = torch.zeros(2, 2, 8, device="cuda")
    i = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    n = torch.ones(2, dtype=torch.int32, device="cuda")
    c = torch.zeros(2, device="cuda")
    ws = torch.zeros(4, device="cuda")
    f = lib.ftb200_log_prob_from_logits
    assert f(c.data_ptr(), x.data_ptr(), 0, i.data_ptr(), n.data_ptr(), 2, 2, 8, 8, ws.data_ptr(), 8, None, 0) == 4
    assert f(c.data_ptr(), x.data_ptr(), 0, i.data_ptr(), n.data_ptr(), 2, 2, 9, 8, ws.data_ptr(), 16, None, 0) == 1
    assert f(c.data_ptr(), x.data_ptr(), 9, i.data_ptr(), n.data_ptr(), 2, 2, 8, 8, ws.data_ptr(), 16, None, 0) == 1
    assert f(c.data_ptr(), None, 0, i.data_ptr(), n.data_ptr(), 2, 2, 8, 8, ws.data_ptr(), 16, None, 0) == 1


def test_single_position_sequences_score_nothing():
    from fastertransformer_b200 import log_prob_from_logits
    x = torch.randn(1, 5, 64, device="cuda")
    ids = torch.zeros(1, 5, dtype=torch.int32, device="cuda")
    n = torch.ones(5, dtype=torch.int32, device="cuda")
    cum = log_prob_from_logits(x, ids, n)
    assert cum.shape == (5,) and bool((cum == 0).all())
