"""Vocabulary-parallel top-k sampling: shards + merge must give the ids of the single-GPU fused step on the
gathered row (which the other tests tie to the reference), for plain, penalised and tie-heavy logits."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_shards,shard,k", [(8, 4000, 64), (4, 2560, 5), (2, 8192, 1), (8, 1024, 40)])
@pytest.mark.parametrize("coarse", [False, True], ids=["distinct", "ties"])
def test_shards_match_full_row(n_shards, shard, k, coarse, cuda_device):
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    B, V, mil, steps = 12, n_shards * shard, 6, 3
    rng = np.random.default_rng(n_shards * 100 + k)
    args = {"runtime_top_k": np.asarray([k], np.uint32), "runtime_top_p": np.asarray([0.92], np.float32),
            "temperature": np.asarray([0.7], np.float32), "repetition_penalty": np.asarray([1.2], np.float32),
            "random_seed": np.asarray([9], np.uint64)}
    prompt = torch.from_numpy(rng.integers(0, V, size=(mil, B)).astype(np.int32)).to(cuda_device)

    def state():
        out = torch.zeros(mil + steps, B, dtype=torch.int32, device=cuda_device)
        out[:mil] = prompt
        return {"output_ids": out, "finished": torch.zeros(B, dtype=torch.bool, device=cuda_device),
                "sequence_length": torch.full((B,), mil, dtype=torch.int32, device=cuda_device)}

    full = DynamicDecodeLayer(V, V, torch.bfloat16, cuda_device)
    vp = VocabParallelSampler(V, shard, n_shards, torch.bfloat16, cuda_device)
    full.setup(B, 1, args)
    vp.setup(B, 1, args)
    s_full, s_vp = state(), state()
    g = torch.Generator(device=cuda_device)
    for s in range(steps):
        step = mil + s
        g.manual_seed(1000 + step)
        x = torch.randn(B, V, generator=g, device=cuda_device) * 3.0
        if coarse:
            x = (x * 2).round() / 2
        x = x.to(torch.bfloat16)
        inp = {"step": step, "max_input_length": mil, "end_id": torch.full((B,), V - 1, dtype=torch.int32, device=cuda_device),
               "input_lengths": torch.full((B,), mil, dtype=torch.int32, device=cuda_device)}
        full.forward(s_full, dict(inp, logits=x))
        shards = [x[:, i * shard:(i + 1) * shard].contiguous() for i in range(n_shards)]
        vp.forward_shards(s_vp, inp, shards)
        torch.cuda.synchronize()
        assert vp.overflow_count() == 0
        for key in ("output_ids", "finished", "sequence_length"):
            assert torch.equal(s_full[key], s_vp[key]), (s, key)
