"""Seeded synthetic decode workloads with the shapes, sizes and value distributions of the five
benchmark configurations (no public dataset is involved; logits are random draws):

  c1  top-k, batch 8, vocab 50257, fp32 N(0, 2^2), k=50, T=1.0, repetition 1.2 over a 64-id prompt
  c2  top-p, batch 256, vocab 51200, fp16 N(0, 3^2) + 4 spikes of +8 per row, p=0.9, T=0.8,
      presence 0.5 over a 128-id prompt, min_length 16
  c3  mixed per-row k in {0,1,40,1024} / p in {0,0.5,0.95}, batch 1024, vocab 128256, bf16 N(0, 2.5^2),
      repetition 1.1 over a 512-id prompt, 8 bad words of 1-3 tokens per row, end id 128001
  (c4 beam search and c5 vocab-parallel live in their own modules.)

Host-side arguments are numpy arrays (the reference takes them as CPU tensors); logits are drawn on
the device with a torch generator seeded by (seed + step) so every implementation sees the same bits.
"""
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class SamplingWorkload:
    name: str
    batch: int
    vocab: int
    vocab_padded: int
    dtype: torch.dtype
    sigma: float
    steps: int
    max_input_length: int
    end_id: int
    runtime_args: dict
    seed: int
    spikes: int = 0
    spike_height: float = 0.0
    bad_words: np.ndarray = None          # [batch, 2, L] int32 or None
    sequence_limit: np.ndarray = None     # [batch] uint32 or None
    prompt: np.ndarray = field(default=None, repr=False)  # [max_input_length, batch] int32

    @property
    def max_seq_len(self):
        return self.max_input_length + self.steps

    def logits(self, step, device, generator=None):
        """Logits of one step: [batch, vocab_padded] in the workload dtype, same bits on every call."""
        g = generator or torch.Generator(device=device)
        g.manual_seed(self.seed * 100003 + step)
        x = torch.randn(self.batch, self.vocab_padded, generator=g, device=device, dtype=torch.float32)
        x.mul_(self.sigma)
        if self.spikes:
            cols = torch.randint(0, self.vocab, (self.batch, self.spikes), generator=g, device=device)
            x.scatter_add_(1, cols, torch.full_like(cols, self.spike_height, dtype=torch.float32))
        return x.to(self.dtype)

    def initial_state(self, device):
        """output_ids [max_seq_len, batch] holding the prompt, plus the per-row state tensors."""
        B = self.batch
        out_ids = torch.zeros(self.max_seq_len, B, dtype=torch.int32, device=device)
        out_ids[: self.max_input_length] = torch.from_numpy(self.prompt).to(device)
        st = {
            "output_ids": out_ids,
            "finished": torch.zeros(B, dtype=torch.bool, device=device),
            "sequence_length": torch.full((B,), self.max_input_length, dtype=torch.int32, device=device),
        }
        return st

    def static_inputs(self, device):
        B = self.batch
        d = {
            "end_id": torch.full((B,), self.end_id, dtype=torch.int32, device=device),
            "input_lengths": torch.full((B,), self.max_input_length, dtype=torch.int32, device=device),
            "max_input_length": self.max_input_length,
            "ite": 0,
            "local_batch_size": B,
        }
        if self.bad_words is not None:
            d["bad_words_list"] = torch.from_numpy(self.bad_words).to(device)
        if self.sequence_limit is not None:
            d["sequence_limit_length"] = torch.from_numpy(self.sequence_limit.view(np.int32)).to(device)
        return d


def _bad_words(rng, batch, vocab, n_words=8, max_len=3):
    L = n_words * max_len
    out = np.full((batch, 2, L), -1, dtype=np.int32)
    out[:, 0, :] = 0
    for b in range(batch):
        pos = 0
        for w in range(n_words):
            n = int(rng.integers(1, max_len + 1))
            out[b, 0, pos:pos + n] = rng.integers(1, vocab, size=n)
            pos += n
            out[b, 1, w] = pos
    return out


def make_workload(name, batch=None, steps=None, vocab=None, seed=None):
    """One of 'c1', 'c2', 'c3'; batch / steps / vocab override the full-size defaults."""
    if name == "c1":
        B, V, S, mil = batch or 8, vocab or 50257, steps or 32, 64
        sd = 1235 if seed is None else seed
        rng = np.random.Generator(np.random.PCG64(sd))
        args = {
            "runtime_top_k": np.asarray([50], np.uint32),
            "temperature": np.asarray([1.0], np.float32),
            "repetition_penalty": np.asarray([1.2], np.float32),
            "random_seed": (np.arange(B) + 7).astype(np.uint64),
        }
        return SamplingWorkload("c1", B, V, (V + 7) // 8 * 8, torch.float32, 2.0, S, mil, V - 1, args, sd,
                                prompt=rng.integers(0, V, size=(mil, B)).astype(np.int32))
    if name == "c2":
        B, V, S, mil = batch or 256, vocab or 51200, steps or 64, 128
        sd = 1236 if seed is None else seed
        rng = np.random.Generator(np.random.PCG64(sd))
        args = {
            "runtime_top_p": np.asarray([0.9], np.float32),
            "temperature": np.asarray([0.8], np.float32),
            "presence_penalty": np.asarray([0.5], np.float32),
            "min_length": np.asarray([16], np.int32),
            "random_seed": np.asarray([11], np.uint64),
        }
        return SamplingWorkload("c2", B, V, (V + 7) // 8 * 8, torch.float16, 3.0, S, mil, V - 1, args, sd,
                                spikes=4, spike_height=8.0,
                                prompt=rng.integers(0, V, size=(mil, B)).astype(np.int32))
    if name == "c3":
        B, V, S, mil = batch or 1024, vocab or 128256, steps or 128, 512
        sd = 1237 if seed is None else seed
        rng = np.random.Generator(np.random.PCG64(sd))
        end_id = 128001 if V > 128001 else V - 1
        args = {
            "runtime_top_k": rng.choice(np.asarray([0, 1, 40, 1024], np.uint32), size=B),
            "runtime_top_p": rng.choice(np.asarray([0.0, 0.5, 0.95], np.float32), size=B),
            "repetition_penalty": np.asarray([1.1], np.float32),
            "random_seed": (np.arange(B) * 3 + 1).astype(np.uint64),
        }
        return SamplingWorkload("c3", B, V, (V + 7) // 8 * 8, torch.bfloat16, 2.5, S, mil, end_id, args, sd,
                                bad_words=_bad_words(rng, B, V),
                                sequence_limit=np.full(B, mil + S, dtype=np.uint32),
                                prompt=rng.integers(0, V, size=(mil, B)).astype(np.int32))
    raise ValueError("unknown workload " + name)


def algorithmic_bytes_per_step(w, step):
    """HBM bytes the path has to move for one step: every logit once, the token history and word
    lists of each row, the per-row state (curand state in and out, ids, flags, arguments)."""
    es = torch.empty(0, dtype=w.dtype).element_size()
    hist = step if ("repetition_penalty" in w.runtime_args or "presence_penalty" in w.runtime_args) else 0
    words = 0 if w.bad_words is None else w.bad_words.shape[-1] * 2
    per_row = w.vocab_padded * es + 4 * hist + 4 * words + 96 + 32
    return w.batch * per_row
