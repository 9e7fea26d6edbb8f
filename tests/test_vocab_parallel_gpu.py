"""Vocabulary-parallel top-k sampling: shards + merge must give the ids of the single-GPU fused step on the
gathered row (which the other tests tie to the reference), for plain, penalised and tie-heavy logits."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


# (shards of 16400 columns and more of 16-bit logits take the single-pass kernel in its record form)
@pytest.mark.parametrize("n_shards,shard,k", [(8, 4000, 64), (4, 2560, 5), (2, 8192, 1), (8, 1024, 40), (2, 32000, 64),
                                              (4, 16448, 40), (2, 20000, 1), (2, 32768, 300), (3, 17000, 1000)])
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
    # (room in the records for the tie classes of the coarse case: about a hundred columns share a value there)
    vp = VocabParallelSampler(V, shard, n_shards, torch.bfloat16, cuda_device, cap_extra=512 if coarse else 64)
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


@pytest.mark.parametrize("dtype,n_shards,shard,sigma", [(torch.bfloat16, 4, 4096, 4.0), (torch.float16, 2, 5000, 5.0),
                                                        (torch.float32, 8, 2048, 6.0), (torch.bfloat16, 4, 8192, 1.2),
                                                        (torch.bfloat16, 2, 16448, 2.5), (torch.float16, 4, 8200, 1.0)])
@pytest.mark.parametrize("all_top_p", [False, True], ids=["mixed", "all_top_p"])
def test_vocab_parallel_top_p_rows_exact(dtype, n_shards, shard, sigma, all_top_p, cuda_device):
    """The default form: pure top-p rows are gathered and sampled unsharded.  Everything - ids of every row,
    finished flags, lengths and both layers' generator states - must EQUAL the unsharded layer's over several
    steps, on peaked and on deliberately flat rows (sigma 1.0 - 1.2), with shards that are and are not a
    multiple of 1024 columns, and nothing may be reported as overflow."""
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    B, mil, steps = 64, 6, 4
    V = shard * n_shards
    rng = np.random.default_rng(170 + n_shards)
    ks = np.zeros(B, np.uint32) if all_top_p else rng.choice(np.asarray([0, 0, 8, 40], np.uint32), size=B)
    args = {"runtime_top_k": ks, "runtime_top_p": rng.choice(np.asarray([0.3, 0.6, 0.9, 0.97], np.float32), size=B),
            "temperature": np.asarray([0.9], np.float32), "repetition_penalty": np.asarray([1.2], np.float32),
            "random_seed": (np.arange(B) * 5 + 3).astype(np.uint64)}
    prompt = torch.from_numpy(rng.integers(0, V, size=(mil, B)).astype(np.int32)).to(cuda_device)

    def state():
        ids = torch.zeros(mil + steps, B, dtype=torch.int32, device=cuda_device)
        ids[:mil] = prompt
        return {"output_ids": ids, "finished": torch.zeros(B, dtype=torch.bool, device=cuda_device),
                "sequence_length": torch.full((B,), mil, dtype=torch.int32, device=cuda_device)}

    full = DynamicDecodeLayer(V, V, dtype, cuda_device)
    full.setup(B, 1, args)
    vp = VocabParallelSampler(V, shard, n_shards, dtype, cuda_device)
    vp.setup(B, 1, args)
    st_a, st_b = state(), state()
    end = torch.full((B,), V - 1, dtype=torch.int32, device=cuda_device)
    g = torch.Generator(device=cuda_device)
    for s in range(steps):
        g.manual_seed(900 + s)
        x = (torch.randn(B, V, generator=g, device=cuda_device) * sigma).to(dtype)
        inp = {"step": mil + s, "max_input_length": mil, "end_id": end, "ite": 0, "local_batch_size": B}
        full.forward(st_a, dict(inp, logits=x))
        vp.forward_shards(st_b, inp, [x[:, i * shard:(i + 1) * shard].contiguous() for i in range(n_shards)])
        torch.cuda.synchronize()
        for key in ("output_ids", "finished", "sequence_length"):
            assert torch.equal(st_a[key], st_b[key]), (s, key)
        assert torch.equal(vp.topp.curand, full.topp.curand) and torch.equal(vp.topk.curand, full.topk.curand)
        assert vp.overflow_count() == 0


@pytest.mark.parametrize("resolve", [True, False], ids=["second_round", "report_only"])
@pytest.mark.parametrize("dtype,n_shards,sigma,max_undecided", [(torch.bfloat16, 4, 4.0, 0.2), (torch.float16, 2, 5.0, 0.2),
                                                                (torch.float32, 8, 6.0, 0.2), (torch.bfloat16, 4, 1.2, 1.0),
                                                                (torch.bfloat16, 2, 4.0, 0.2)])
def test_vocab_parallel_top_p_rows(dtype, n_shards, sigma, max_undecided, resolve, cuda_device):
    """The approximate form (top_p="statistics"): mixed top-k / top-p rows over a sharded vocabulary against the
    unsharded kernel.  Top-k rows must be identical.  Top-p rows combine per-shard soft-max statistics, so their denominator is summed in another
    order: ids are compared.  The rows the exchange cannot decide either get a second round on their gathered
    logits (then they are the unsharded kernel's ids, and no -1 is left) or are reported with id -1 and an
    untouched generator."""
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    # (two shards: wide ones, which take the single-pass kernel for the top-k rows and leave the top-p rows to the
    #  general kernel's statistics form)
    B, shard, mil, steps = 96, (4096 if n_shards > 2 or dtype != torch.bfloat16 else 17408), 6, 4
    V = shard * n_shards
    rng = np.random.default_rng(17 + n_shards)
    args = {"runtime_top_k": rng.choice(np.asarray([0, 0, 8, 40], np.uint32), size=B),
            "runtime_top_p": rng.choice(np.asarray([0.3, 0.6, 0.9], np.float32), size=B),
            "temperature": np.asarray([0.9], np.float32), "repetition_penalty": np.asarray([1.2], np.float32),
            "random_seed": (np.arange(B) * 5 + 3).astype(np.uint64)}
    prompt = rng.integers(0, V, size=(mil, B)).astype(np.int32)

    def state():
        ids = torch.zeros(mil + steps, B, dtype=torch.int32, device=cuda_device)
        ids[:mil] = torch.from_numpy(prompt).to(cuda_device)
        return {"output_ids": ids, "finished": torch.zeros(B, dtype=torch.bool, device=cuda_device),
                "sequence_length": torch.full((B,), mil, dtype=torch.int32, device=cuda_device)}

    full = DynamicDecodeLayer(V, V, dtype, cuda_device)
    full.setup(B, 1, args)
    vp = VocabParallelSampler(V, shard, n_shards, dtype, cuda_device, resolve_undecided=resolve, top_p="statistics")
    vp.setup(B, 1, args)
    st_a, st_b = state(), state()
    end = torch.full((B,), V - 1, dtype=torch.int32, device=cuda_device)
    is_topp = (args["runtime_top_k"] == 0)
    g = torch.Generator(device=cuda_device)
    same_topp = total_topp = undecided = 0
    for s in range(steps):
        g.manual_seed(900 + s)
        x = (torch.randn(B, V, generator=g, device=cuda_device) * sigma).to(dtype)
        inp = {"step": mil + s, "max_input_length": mil, "end_id": end, "ite": 0, "local_batch_size": B}
        before = vp.topp.curand.clone()
        full.forward(st_a, dict(inp, logits=x))
        vp.forward_shards(st_b, inp, [x[:, i * shard:(i + 1) * shard].contiguous() for i in range(n_shards)])
        a = st_a["output_ids"][mil + s].cpu().numpy()
        b = st_b["output_ids"][mil + s].cpu().numpy()
        assert np.array_equal(a[~is_topp], b[~is_topp]), "top-k rows must not depend on the sharding"
        und = b == -1
        assert not und[~is_topp].any()
        if resolve:
            assert not und.any()
            # every row drew exactly once: the generators march in step with the unsharded layer's
            assert torch.equal(vp.topp.curand, full.topp.curand)
        else:
            # an undecided row keeps the generator it had, so that its repetition draws the same number
            rows = torch.from_numpy(np.nonzero(und)[0]).to(cuda_device)
            assert torch.equal(vp.topp.curand.view(B, -1)[rows], before.view(B, -1)[rows])
            vp.topp.curand.copy_(full.topp.curand)
        undecided += int(und.sum())
        ok = is_topp & ~und
        same_topp += int((a[ok] == b[ok]).sum())
        total_topp += int(ok.sum())
        # keep both histories identical so that later steps stay comparable
        st_b["output_ids"][mil + s].copy_(st_a["output_ids"][mil + s])
        st_b["finished"].copy_(st_a["finished"])
        st_b["sequence_length"].copy_(st_a["sequence_length"])
    print("top-p rows: %d of %d ids equal to the unsharded kernel, %d undecided, %d given a second round"
          % (same_topp, total_topp, undecided, vp.resolved_rows))
    if resolve:
        assert undecided == 0 and vp.overflow_count() == vp.resolved_rows
        if max_undecided >= 1.0:
            assert vp.resolved_rows > 0
    else:
        assert vp.overflow_count() == undecided and vp.resolved_rows == 0
        # (flat logits: the nucleus outgrows what the shards send - those rows have to come back undecided, not wrong)
        assert undecided <= max_undecided * is_topp.sum() * steps
        if max_undecided < 1.0:
            assert total_topp > 0
        else:
            assert undecided > 0
    assert same_topp >= 0.97 * total_topp, (same_topp, total_topp)
