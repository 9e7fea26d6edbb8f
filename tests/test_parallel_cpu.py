"""World-size-2 checks of the multi-GPU host logic on CPU (gloo):
  * forward_rank of the vocabulary-parallel sampler, its control flow and collectives unchanged, with the three
    kernel calls replaced by the CPU oracle: top-k rows through records and merge, pure top-p rows through the
    gather of their shard rows and the unsharded step; every rank must end with the oracle's ids of the full rows;
  * batch sharding: two ranks each decode their block of rows with the CPU oracle; the concatenation equals
    the single-process result (rows are independent - no collective on the data path);
  * vocabulary-parallel protocol: each rank packs candidate records of its column shard, one all_gather
    exchanges them, and the oracle run on the merged (sparse) rows returns the ids of the full rows."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastertransformer_b200.parallel import gather_rows, shard_rows
from vp_records import merge_records, pack_record
from ft_oracle import OracleDynamicDecodeLayer

B, V, K, MIL = 6, 512, 7, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs():
    rng = np.random.default_rng(42)
    logits = (rng.standard_normal((B, V)) * 2).astype(np.float32)
    logits = np.round(logits * 4) / 4          # tie classes at the k-th value
    prompt = rng.integers(0, V, size=(MIL, B)).astype(np.int32)
    u = (1.0 - rng.random(B)).astype(np.float32)
    return logits, prompt, u


def _decode(logits, prompt, u, rows):
    args = {"runtime_top_k": np.asarray([K], np.uint32), "random_seed": np.asarray([1], np.uint64)}
    n = len(rows)
    layer = OracleDynamicDecodeLayer(V, V, "float32")
    layer.setup(n, 1, args)
    out = {"output_ids": np.zeros((MIL + 1, n), np.int32), "finished": np.zeros(n, np.bool_),
           "sequence_length": np.full(n, MIL, np.int32)}
    out["output_ids"][:MIL] = prompt[:, rows]
    layer.forward(out, {"logits": np.ascontiguousarray(logits[rows]), "step": MIL, "max_input_length": MIL,
                        "end_id": np.full(n, V - 1, np.int32)}, u[rows], None)
    return out["output_ids"][MIL].copy()


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    logits, prompt, u = _inputs()
    # (1) batch sharding
    first, n = shard_rows(B, world, rank)
    mine = _decode(logits, prompt, u, list(range(first, first + n)))
    parts = [torch.zeros(shard_rows(B, world, r)[1], dtype=torch.int32) for r in range(world)]
    dist.all_gather(parts, torch.from_numpy(mine))
    batch_ids = torch.cat(parts).numpy()
    # (2) vocabulary-parallel records
    shard, cap = V // world, K + 32
    rec = np.stack([pack_record(logits[b, rank * shard:(rank + 1) * shard], K, cap, rank * shard) for b in range(B)])
    gathered = [torch.zeros(B, 2 + cap, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(rec.view(np.int64)))
    merged = np.stack([merge_records([g.numpy().view(np.uint64)[b] for g in gathered], V) for b in range(B)])
    vp_ids = _decode(merged, prompt, u, list(range(B)))
    # (3) second round: full rows of the rows a merge would leave undecided (same list on every rank)
    rows = torch.tensor([1, B - 1, 4])
    full = gather_rows(torch.from_numpy(np.ascontiguousarray(logits[:, rank * shard:(rank + 1) * shard])), rows, world)
    assert np.array_equal(full.numpy(), logits[rows.numpy()]), "gathered rows are not the full rows"
    q.put((rank, batch_ids, vp_ids))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_rows_partition():
    for batch in (1, 7, 64, 1024):
        for world in (1, 2, 3, 8):
            blocks = [shard_rows(batch, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and sum(n for _, n in blocks) == batch
            for (f0, n0), (f1, _) in zip(blocks, blocks[1:]):
                assert f0 + n0 == f1


def test_two_ranks_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    logits, prompt, u = _inputs()
    expect = _decode(logits, prompt, u, list(range(B)))
    for rank, batch_ids, vp_ids in results:
        assert (batch_ids == expect).all(), ("batch sharding", rank)
        assert (vp_ids == expect).all(), ("vocabulary parallel", rank)


# ---- forward_rank with the kernels replaced by the CPU oracle -------------------------------------------------
VB, VV, VMIL = 10, 1024, 3
V_KS = np.asarray([0, 5, 0, 7, 7, 0, 3, 0, 5, 0], np.uint32)          # 0: a pure top-p row
V_PS = np.asarray([0.6, 1.0, 0.9, 0.8, 1.0, 0.3, 1.0, 0.95, 0.5, 0.7], np.float32)


def _vp_inputs():
    rng = np.random.default_rng(7)
    logits = (rng.standard_normal((VB, VV)) * 3).astype(np.float32)
    prompt = rng.integers(0, VV, size=(VMIL, VB)).astype(np.int32)
    u = (1.0 - rng.random(VB)).astype(np.float32)
    return logits, prompt, u


def _oracle_step(logits, prompt, u, ks, ps):
    """Ids of the full rows from the CPU oracle (top-k rows draw from u, top-p rows from the same u)."""
    args = {"runtime_top_k": ks, "runtime_top_p": ps, "random_seed": np.asarray([1], np.uint64)}
    n = logits.shape[0]
    layer = OracleDynamicDecodeLayer(logits.shape[1], logits.shape[1], "float32")
    layer.setup(n, 1, args)
    out = {"output_ids": np.zeros((VMIL + 1, n), np.int32), "finished": np.zeros(n, np.bool_),
           "sequence_length": np.full(n, VMIL, np.int32)}
    out["output_ids"][:VMIL] = prompt
    layer.forward(out, {"logits": np.ascontiguousarray(logits), "step": VMIL, "max_input_length": VMIL,
                        "end_id": np.full(n, logits.shape[1] - 1, np.int32)}, u, u)
    return out["output_ids"][VMIL].copy()


def _vp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    logits, prompt, u = _vp_inputs()
    shard = VV // world
    is_topp = V_KS == 0
    kmax = int(V_KS.max())

    class OracleBacked(VocabParallelSampler):
        """forward_rank, _buffers and the collectives are the class's own; the kernel calls are the oracle."""

        def __init__(self):  # (no device, no library call)
            self.device = torch.device("cpu")
            self.vocab_size, self.shard_size, self.n_shards, self.cap_extra, self.group = VV, shard, world, 32, None
            self.exact_top_p, self.max_top_k, self.topp_candidates = True, kmax, 0
            self._records = self._gathered = self._full_rows = None
            self._topp_rows = torch.from_numpy(np.flatnonzero(is_topp).astype(np.int64))
            self._all_top_p = False
            self.launches = 0
            self.seen = {}

        def _has_topp(self):
            return True

        def local_pass(self, outputs, inputs, shard_logits, shard_index, records):
            x = shard_logits.numpy()
            rec = np.zeros((VB, 2 + self.cap), np.uint64)
            for b in np.flatnonzero(~is_topp):
                rec[b] = pack_record(x[b], int(V_KS[b]), self.cap, shard_index * shard)
            records.copy_(torch.from_numpy(rec.view(np.int64)))

        def merge(self, outputs, inputs, gathered, logits_like):
            g = gathered.numpy().view(np.uint64)
            rows = np.flatnonzero(~is_topp)
            merged = np.stack([merge_records([g[s][b] for s in range(world)], VV) for b in rows])
            outputs["output_ids"][VMIL, rows] = _oracle_step(merged, prompt[:, rows], u[rows], V_KS[rows], V_PS[rows])

        def _sample_top_p_rows(self, outputs, inputs, parts):
            rows = self._topp_rows.numpy()
            full = parts.permute(1, 0, 2).reshape(len(rows), VV).numpy()
            self.seen["full_rows_equal"] = bool(np.array_equal(full, logits[rows]))
            outputs["output_ids"][VMIL, rows] = _oracle_step(full, prompt[:, rows], u[rows], V_KS[rows], V_PS[rows])

    vp = OracleBacked()
    outputs = {"output_ids": np.zeros((VMIL + 1, VB), np.int32)}
    outputs["output_ids"][:VMIL] = prompt
    mine = torch.from_numpy(np.ascontiguousarray(logits[:, rank * shard:(rank + 1) * shard]))
    vp.forward_rank(outputs, {"step": VMIL, "max_input_length": VMIL}, mine, rank)
    q.put((rank, outputs["output_ids"][VMIL].copy(), vp.seen.get("full_rows_equal", False), vp.cap))
    dist.barrier()
    dist.destroy_process_group()


def test_forward_rank_control_flow_two_ranks_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_vp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    logits, prompt, u = _vp_inputs()
    expect = _oracle_step(logits, prompt, u, V_KS, V_PS)
    for rank, ids, full_ok, cap in results:
        assert full_ok, ("the gathered top-p rows are not the full rows", rank)
        assert cap == int(V_KS.max()) + 32  # (the records of the exact form carry top-k candidates only)
        assert (ids == expect).all(), ("vocabulary parallel, exact top-p", rank, ids, expect)
