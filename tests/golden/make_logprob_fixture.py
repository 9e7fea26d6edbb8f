"""Generates tests/golden/logprob_ref.json: outputs of the reference's own invokeLogProbFromLogits
(kernels/logprob_kernels.cu:142-183, compiled into oracle/_ref/libft_decode_ref.so) on seeded inputs.
Needs a GPU.  The inputs are not stored: logprob_case() rebuilds them from the seed.

usage: python tests/golden/make_logprob_fixture.py [OUT.json]
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

CASES = [
    # name, max_input_length, batch, vocab, vocab_padded, dtype, batch_first
    ("f32_small", 6, 3, 50, 56, "float32", False),
    ("f32_small_bf", 6, 3, 50, 56, "float32", True),
    ("f16_small", 6, 3, 50, 56, "float16", False),
    ("f16_small_bf", 6, 3, 50, 56, "float16", True),
    ("f32_odd_vocab", 9, 4, 5001, 5001, "float32", False),
    ("f16_odd_vocab", 9, 4, 5001, 5001, "float16", True),
    ("f32_long", 130, 2, 1031, 1040, "float32", True),
    ("f16_tiny_vocab", 2, 32, 16, 16, "float16", False),
]


def logprob_case(name, max_len, batch, vocab, vocab_padded, dtype, batch_first):
    """Seeded inputs: logits uniform in [-3, 3] like the reference's test (test_logprob_kernels.cu:143),
    ragged lengths in [1, max_len], ids below vocab."""
    rng = np.random.default_rng(abs(hash_name(name)))
    shape = (batch, max_len, vocab_padded) if batch_first else (max_len, batch, vocab_padded)
    logits = rng.uniform(-3.0, 3.0, size=shape).astype(np.float32).astype(dtype)
    ids = rng.integers(0, vocab, size=(batch, max_len) if batch_first else (max_len, batch)).astype(np.int32)
    lengths = rng.integers(1, max_len + 1, size=batch).astype(np.int32)
    lengths[0] = max_len
    return logits, ids, lengths


def hash_name(name):
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


def main():
    import torch
    from ft_reference import ref_lib
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "logprob_ref.json")
    lib = ref_lib()
    out = {}
    for case in CASES:
        name, max_len, batch, vocab, vp, dtype, bf = case
        logits, ids, lengths = logprob_case(*case)
        d_logits = torch.from_numpy(logits).cuda()
        d_ids = torch.from_numpy(ids).cuda()
        d_len = torch.from_numpy(lengths).cuda()
        ws = torch.zeros(max_len * batch, dtype=torch.float32, device="cuda")
        cum = torch.zeros(batch, dtype=torch.float32, device="cuda")
        rc = lib.ftref_log_prob_from_logits(cum.data_ptr(), d_logits.data_ptr(), 0 if dtype == "float32" else 1,
                                            d_ids.data_ptr(), d_len.data_ptr(), max_len, batch, vocab, vp,
                                            ws.data_ptr(), ws.numel() * 4, None, int(bf))
        torch.cuda.synchronize()
        assert rc == 0
        lp = ws[:(max_len - 1) * batch].cpu().numpy().reshape((batch, max_len - 1) if bf else (max_len - 1, batch))
        # entries the kernel does not write (step >= length - 1) are left out
        steps = np.arange(max_len - 1)
        valid = steps[None, :] < (lengths[:, None] - 1) if bf else steps[:, None] < (lengths[None, :] - 1)
        out[name] = {"cum_log_probs": [float(x) for x in cum.cpu().numpy()],
                     "log_probs": [float(x) for x in np.where(valid, lp, 0.0).ravel()]}
    with open(out_path, "w") as f:
        json.dump(out, f)
    print("wrote", out_path, len(out), "cases")


if __name__ == "__main__":
    main()
