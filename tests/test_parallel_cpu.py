"""World-size-2 checks of the multi-GPU host logic on CPU (gloo):
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
