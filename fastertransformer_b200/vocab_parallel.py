"""Vocabulary-parallel sampling over a column-sharded lm_head (host side).

Each rank holds logits[:, rank*V/n : (rank+1)*V/n].  Instead of FasterTransformer's all-gather of the full
fp32 logits followed by redundant sampling on every rank (models/multi_gpu_gpt/ParallelGpt.cc:1394-1435),
each rank selects candidates on its shard, ONE all-gather exchanges a few hundred bytes per row, and every
rank merges and draws with identical curand states - same id on every rank, equal to the single-GPU result.

Top-k rows (k > 0, with or without p) are exact: the union of the shards' candidates holds every column the
selection can touch.  Pure top-p rows (k = 0) need the soft-max denominator of the whole row summed in the
single-GPU order, which no combination of per-shard partial sums reproduces (float addition does not
associate), so by default (`top_p="exact"`) their shard rows - and only theirs - are all-gathered and sampled by
the unsharded kernel: identical to the single-GPU result, no host synchronisation (which rows are top-p rows is
known from the runtime arguments).  `top_p="statistics"` is the cheaper approximate form: each shard sends its
largest columns plus its (maximum, sum of exponentials), the ranks combine the pairs like an online soft-max, a
draw within rounding of a boundary may pick the neighbouring column, and a nucleus larger than the union is
reported (and, with `resolve_undecided`, repeated on gathered rows after a read of the overflow counter).

`VocabParallelSampler` reuses DynamicDecodeLayer for the set-up (runtime arguments, curand states).  The
exchange goes through torch.distributed (NCCL) when a process group is given; `forward_shards` runs all
shards on one device, which is how the single-GPU tests check the merge.
"""
import ctypes as C

import torch

from ._lib import SamplingParams, check, lib
from .decode_layer import CURAND_STATE_BYTES, DynamicDecodeLayer, _DT
from .parallel import gather_rows


class VocabParallelSampler(DynamicDecodeLayer):
    def __init__(self, vocab_size, shard_size, n_shards, dtype, device, cap_extra=64, group=None, topp_candidates=448,
                 resolve_undecided=True, top_p="exact"):
        """`top_p`: "exact" (default) gathers the shard rows of the pure top-p rows and samples them unsharded;
        "statistics" exchanges candidates and soft-max statistics instead, for which the next arguments are:
        `topp_candidates`: columns every shard sends for a top-p row (its largest ones, plus its soft-max
        statistics).  A row whose nucleus needs more than the union holds comes back from the merge with id -1,
        its generator untouched, and is counted by overflow_count().  With `resolve_undecided` such rows get a
        second round in the same call: their shard rows are gathered (one more all-gather, of the undecided rows
        only) and sampled by the unsharded kernel - the id the single-GPU path gives.  Without it the caller
        repeats them."""
        super().__init__(vocab_size, shard_size * n_shards, dtype, device)
        self.shard_size, self.n_shards, self.cap_extra, self.group = shard_size, n_shards, cap_extra, group
        if top_p not in ("exact", "statistics"):
            raise ValueError("top_p must be 'exact' or 'statistics'")
        self.exact_top_p = top_p == "exact"
        self.topp_candidates = int(topp_candidates)
        self.resolve_undecided = bool(resolve_undecided)
        self._topp_rows = None   # device indices of the pure top-p rows (exact mode), set by setup()
        self._full_rows = None   # [batch, vocab_padded] scratch; only the top-p rows are ever written or read
        self.resolved_rows = 0
        self._seen_overflow = 0
        self._records = None
        self._gathered = None
        self._overflow = torch.zeros(1, dtype=torch.int32, device=self.device)

    def setup(self, batch_size, beam_width, runtime_args):
        super().setup(batch_size, beam_width, runtime_args)
        self._topp_rows = None
        if self.exact_top_p and self._has_topp():
            rows = (~self.topp.skip_host).nonzero()[0]
            self._topp_rows = torch.from_numpy(rows.astype("int64")).to(self.device)
        self._all_top_p = self._topp_rows is not None and bool(self.topk.skip_host.all())

    def _params(self, outputs, inputs, logits, vocab, vocab_padded, halves="both"):
        B = logits.shape[0]
        step, mil = int(inputs["step"]), int(inputs["max_input_length"])
        P = SamplingParams()
        P.dtype = _DT[logits.dtype]
        P.batch_size = P.local_batch_size = B
        P.vocab_size, P.vocab_size_padded = vocab, vocab_padded
        P.step, P.max_input_length = step, mil
        P.logits = logits.data_ptr()
        P.end_ids = inputs["end_id"].data_ptr()
        il = inputs.get("input_lengths")
        P.input_lengths = None if il is None else il.data_ptr()
        P.output_ids = outputs["output_ids"].data_ptr()
        bw = inputs.get("bad_words_list")
        if bw is not None:
            P.bad_words, P.bad_words_len = bw.data_ptr(), bw.shape[-1]
            P.bad_words_shared = int(bw.dim() == 2 or bw.shape[0] == 1)
        P.temperature = self.temperature.data_ptr()
        P.apply_temperature = int(bool((self.temperature_host != 1.0).any()))
        P.repetition_penalty = self.penalty.data_ptr()
        P.penalty_type = self.penalty_type
        P.apply_repetition = int(step > 1 and self.penalty_type != 2
                                 and bool((self.penalty_host != self.penalty_default).any()))
        P.min_lengths = self.min_length.data_ptr()
        P.apply_min_length = int(bool((self.min_length_host > step - mil).any()))
        if halves != "top_p":
            P.topk_states = self.topk.curand.data_ptr()
            P.topk_ks, P.topk_ps = self.topk.top_ks.data_ptr(), self.topk.top_ps.data_ptr()
            P.topk_skip, P.max_top_k = self.topk.skip.data_ptr(), self.max_top_k
        if self._has_topp() and halves != "top_k":
            P.topp_states = self.topp.curand.data_ptr()
            P.topp_ps, P.topp_skip = self.topp.top_ps.data_ptr(), self.topp.skip.data_ptr()
            P.topp_initial_ps, P.topp_decay = self.topp.initial.data_ptr(), self.topp.decay.data_ptr()
            P.topp_min, P.topp_reset_ids = self.topp.min.data_ptr(), self.topp.reset.data_ptr()
        for key, width in (("sequence_length", 4), ("finished", 1)):
            t = outputs.get(key)
            setattr(P, key, None if t is None else t.data_ptr())
        need = C.c_size_t(0)
        check(lib.ftb200_sampling_workspace_bytes(P.dtype, B, vocab_padded, C.byref(need)))
        if self._workspace is None or self._workspace.numel() < need.value:
            self._workspace = torch.empty(need.value, dtype=torch.uint8, device=self.device)
        P.workspace, P.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        P.stream = self._stream_ptr().value
        return P

    def _has_topp(self):
        return self.topp.active and not bool(self.topp.skip_host.all())

    @property
    def _record_halves(self):
        """Which half of the argument block the record exchange serves: in exact mode the top-p rows stay out."""
        return "top_k" if self.exact_top_p else "both"

    @property
    def cap(self):
        k = max(self.max_top_k, self.topp_candidates) if self._has_topp() and not self.exact_top_p else self.max_top_k
        return min(k, 1024) + self.cap_extra

    def local_pass(self, outputs, inputs, shard_logits, shard_index, records):
        """Candidates of one shard -> records [batch, 2 + cap] (int64 view of the 64-bit words: count, entries,
        and for top-p rows the shard's soft-max statistics in the last word)."""
        off = shard_index * self.shard_size
        vocab = max(0, min(self.shard_size, self.vocab_size - off))
        P = self._params(outputs, inputs, shard_logits, max(vocab, 1), self.shard_size, self._record_halves)
        check(lib.ftb200_vocab_parallel_local(C.byref(P), off, self.cap, C.c_void_p(records.data_ptr())))
        self.launches += 1

    def merge(self, outputs, inputs, gathered, logits_like):
        P = self._params(outputs, inputs, logits_like, self.vocab_size, self.shard_size * self.n_shards,
                         self._record_halves)
        check(lib.ftb200_vocab_parallel_merge(C.byref(P), C.c_void_p(gathered.data_ptr()), self.n_shards, self.cap,
                                              C.c_void_p(self._overflow.data_ptr())))
        self.launches += 1

    def _buffers(self, B):
        shape = (B, 2 + self.cap)
        if self._records is None or tuple(self._records.shape) != shape:
            self._records = torch.zeros(shape, dtype=torch.int64, device=self.device)
            self._gathered = torch.zeros((self.n_shards,) + shape, dtype=torch.int64, device=self.device)
        return self._records, self._gathered

    def forward_rank(self, outputs, inputs, shard_logits, rank):
        """One rank of a tensor-parallel group: local pass, one all-gather, merge; then, if rows stayed
        undecided, their logits are gathered and they are sampled unsharded (every rank gets the same rows: the
        merge is the same computation everywhere)."""
        import torch.distributed as dist
        if not self._all_top_p:
            rec, gathered = self._buffers(shard_logits.shape[0])
            self.local_pass(outputs, inputs, shard_logits, rank, rec)
            dist.all_gather_into_tensor(gathered.view(-1), rec.view(-1), group=self.group)
            self.merge(outputs, inputs, gathered, shard_logits)
        if self._topp_rows is not None:
            # the pure top-p rows: their shard rows from every rank, side by side, then the unsharded kernel
            mine = shard_logits.index_select(0, self._topp_rows)
            parts = torch.empty((self.n_shards,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
            dist.all_gather_into_tensor(parts.view(-1), mine.view(-1), group=self.group)
            self._sample_top_p_rows(outputs, inputs, parts)
            return
        rows = self._undecided_rows(outputs, inputs)
        if rows is not None:
            self._resolve(outputs, inputs, rows, gather_rows(shard_logits, rows, self.n_shards, self.group))

    def forward_shards(self, outputs, inputs, shards):
        """All shards on this device (no communication): the arithmetic of forward_rank on every rank."""
        if not self._all_top_p:
            rec, gathered = self._buffers(shards[0].shape[0])
            for i, sh in enumerate(shards):
                self.local_pass(outputs, inputs, sh, i, rec)
                gathered[i].copy_(rec)
            self.merge(outputs, inputs, gathered, shards[0])
        if self._topp_rows is not None:
            self._sample_top_p_rows(outputs, inputs, torch.stack([sh.index_select(0, self._topp_rows) for sh in shards]))
            return
        rows = self._undecided_rows(outputs, inputs)
        if rows is not None:
            self._resolve(outputs, inputs, rows, torch.cat([sh.index_select(0, rows) for sh in shards], dim=1).contiguous())

    def _sample_top_p_rows(self, outputs, inputs, parts):
        """`parts` [n_shards, n_rows, shard]: the shard rows of the pure top-p rows from every rank.  They are put
        side by side at their own row of a [batch, vocab_padded] scratch (the other rows of it are never touched)
        and the unsharded step runs with the top-p half of the argument block alone, so that every other row is
        skipped: one call, the ids and generator states of the single-GPU path."""
        B = outputs["output_ids"].shape[-1]
        Vp = self.shard_size * self.n_shards
        if self._full_rows is None or tuple(self._full_rows.shape) != (B, Vp) or self._full_rows.dtype != parts.dtype:
            self._full_rows = torch.empty(B, Vp, dtype=parts.dtype, device=self.device)
        self._full_rows.view(B, self.n_shards, self.shard_size).index_copy_(0, self._topp_rows, parts.permute(1, 0, 2))
        P = self._params(outputs, inputs, self._full_rows, self.vocab_size, Vp, "top_p")
        check(lib.ftb200_decode_step_sampling(C.byref(P)))
        self.launches += lib.ftb200_last_launch_count()

    def _undecided_rows(self, outputs, inputs):
        """Row indices (device tensor) the merge of this step left undecided, or None.  Reads the overflow
        counter, which synchronises the stream - the price of the second round; switch it off with
        resolve_undecided=False."""
        if not self.resolve_undecided or not self._has_topp():
            return None  # (top-k rows overflow only on tie classes wider than the record: reported, not repeated)
        total = int(self._overflow.item())
        new, self._seen_overflow = total - self._seen_overflow, total
        if new == 0:
            return None
        ids = outputs["output_ids"][int(inputs["step"])].reshape(-1)
        return (ids == -1).nonzero().reshape(-1)

    def _resolve(self, outputs, inputs, rows, full_rows):
        """Sample the given rows from their full-vocabulary logits [len(rows), vocab_padded] with the unsharded
        kernel, one call per row (ite = row, local batch 1: every per-row array is entered at that row)."""
        Vp = self.shard_size * self.n_shards
        B = outputs["output_ids"].shape[-1]
        for j, r in enumerate(rows.tolist()):
            P = self._params(outputs, inputs, full_rows[j:j + 1], self.vocab_size, Vp)
            P.batch_size, P.local_batch_size, P.ite = B, 1, r
            for name, width in (("end_ids", 4), ("input_lengths", 4), ("temperature", 4), ("repetition_penalty", 4),
                                ("min_lengths", 4), ("topk_states", CURAND_STATE_BYTES), ("topk_ks", 4), ("topk_ps", 4),
                                ("topk_skip", 1), ("topp_states", CURAND_STATE_BYTES), ("topp_ps", 4), ("topp_skip", 1),
                                ("topp_initial_ps", 4), ("topp_decay", 4), ("topp_min", 4), ("topp_reset_ids", 4),
                                ("sequence_length", 4), ("finished", 1)):
                base = getattr(P, name)
                if base:
                    setattr(P, name, base + r * width)
            if P.bad_words and not P.bad_words_shared:
                P.bad_words = P.bad_words + r * 2 * P.bad_words_len * 4
            check(lib.ftb200_decode_step_sampling(C.byref(P)))
            self.launches += 1
            self.resolved_rows += 1

    def overflow_count(self):
        return int(self._overflow.item())
