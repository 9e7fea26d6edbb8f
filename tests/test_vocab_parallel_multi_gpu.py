"""forward_rank of the vocabulary-parallel sampler over NCCL, one process per GPU (needs at least two GPUs): every
rank holds its column shard of the same seeded logits, and after each step every rank's ids, flags, lengths and
generator states must equal those of the unsharded layer run on the full rows in the same process - top-k rows
through the record exchange, pure top-p rows through the gather of their shard rows (the default, exact form)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
B, MIL, STEPS = 48, 5, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, shard, dtype_name, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    dtype = getattr(torch, dtype_name)
    V = shard * world
    rng = np.random.default_rng(5)
    args = {"runtime_top_k": rng.choice(np.asarray([0, 0, 8, 40], np.uint32), size=B),
            "runtime_top_p": rng.choice(np.asarray([0.3, 0.6, 0.9, 0.97], np.float32), size=B),
            "temperature": np.asarray([0.9], np.float32), "repetition_penalty": np.asarray([1.2], np.float32),
            "random_seed": (np.arange(B) * 5 + 3).astype(np.uint64)}
    prompt = torch.from_numpy(rng.integers(0, V, size=(MIL, B)).astype(np.int32)).to(dev)

    def state():
        ids = torch.zeros(MIL + STEPS, B, dtype=torch.int32, device=dev)
        ids[:MIL] = prompt
        return {"output_ids": ids, "finished": torch.zeros(B, dtype=torch.bool, device=dev),
                "sequence_length": torch.full((B,), MIL, dtype=torch.int32, device=dev)}

    full = DynamicDecodeLayer(V, V, dtype, dev)
    full.setup(B, 1, args)
    vp = VocabParallelSampler(V, shard, world, dtype, dev)
    vp.setup(B, 1, args)
    st_a, st_b = state(), state()
    end = torch.full((B,), V - 1, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev)
    ok = True
    for s in range(STEPS):
        g.manual_seed(900 + s)  # the same logits on every rank
        x = (torch.randn(B, V, generator=g, device=dev) * 2.5).to(dtype)
        inp = {"step": MIL + s, "max_input_length": MIL, "end_id": end, "ite": 0, "local_batch_size": B}
        full.forward(st_a, dict(inp, logits=x))
        vp.forward_rank(st_b, inp, x[:, rank * shard:(rank + 1) * shard].contiguous(), rank)
        torch.cuda.synchronize()
        for key in ("output_ids", "finished", "sequence_length"):
            ok = ok and torch.equal(st_a[key], st_b[key])
        ok = ok and torch.equal(vp.topp.curand, full.topp.curand) and torch.equal(vp.topk.curand, full.topk.curand)
    q.put((rank, bool(ok), int(vp.overflow_count())))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shard,dtype_name", [(8192, "bfloat16"), (5000, "float16")])
def test_forward_rank_over_nccl(shard, dtype_name):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, shard, dtype_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, overflow in results:
        assert ok, ("rank differs from the unsharded layer", rank)
        assert overflow == 0
