"""GPU parity tests of the fused decode-sampling kernel (through the C ABI of libftb200.so) against
  (1) the unmodified reference DynamicDecodeLayer compiled for sm_100a (oracle/_ref), same logits,
      same seeds: ids, finished and sequence_length must be bit-identical, log-probs within 1e-3;
  (2) the reference's known-answer sets (tests/golden/sampling_layer_kat.json);
  (3) the CPU oracle fed the uniforms the kernel will draw."""
import json
import os

import numpy as np
import pytest
import torch

import ft_reference
from decode_driver import run_cuda_like
from ft_oracle import OracleDynamicDecodeLayer, bf16_bits

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
KAT = json.load(open(os.path.join(HERE, "golden", "sampling_layer_kat.json")))
FLT_MAX = np.finfo(np.float32).max


def _layer(w, device):
    from fastertransformer_b200 import DynamicDecodeLayer
    return DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, device)


def _ref_layer(w, device):
    if not ft_reference.available():
        pytest.skip("oracle/_ref/libft_decode_ref.so not built")
    dt = torch.float32 if w.dtype == torch.bfloat16 else w.dtype
    return ft_reference.RefDynamicDecodeLayer(w.vocab, w.vocab_padded, dt, device), dt


def _compare(mine, ref, what=""):
    for key in ("ids", "finished", "sequence_length"):
        bad = np.argwhere(mine[key] != ref[key])
        assert bad.size == 0, "%s %s differs at %d of %d (first %s: mine %s ref %s)" % (
            what, key, len(bad), mine[key].size, bad[0], mine[key][tuple(bad[0])], ref[key][tuple(bad[0])])
    if "cum_log_probs" in mine:
        np.testing.assert_allclose(mine["cum_log_probs"], ref["cum_log_probs"], rtol=1e-3, atol=1e-4)
        np.testing.assert_allclose(mine["output_log_probs"], ref["output_log_probs"], rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", KAT["cases"], ids=[c["name"] for c in KAT["cases"]])
def test_known_answers(case, dtype, cuda_device):
    from fastertransformer_b200 import DynamicDecodeLayer
    B, V, steps = KAT["batch_size"], KAT["vocab_size"], KAT["steps"]
    toy = np.asarray([(-FLT_MAX if v == "-FLT_MAX" else v) for v in KAT["logits"]], np.float32).reshape(3, 8)
    if dtype == torch.float16:
        toy = np.clip(toy, -65504.0, 65504.0)
    toy_t = torch.from_numpy(toy).to(cuda_device).to(dtype)
    args = {}
    if "top_k" in case:
        args["runtime_top_k"] = np.asarray(case["top_k"], np.uint32)
    if "top_p" in case:
        args["runtime_top_p"] = np.asarray(case["top_p"], np.float32)
    lbs, ite = (B // 3, 1) if case["use_local_batch"] else (B, 0)
    for seed in range(KAT["seeds"]):
        layer = DynamicDecodeLayer(V, V, dtype, cuda_device)
        a = dict(args)
        a["random_seed"] = np.asarray([seed], np.uint64)
        layer.setup(B, 1, a)
        out = {"output_ids": torch.zeros(steps, B, dtype=torch.int32, device=cuda_device),
               "cum_log_probs": torch.zeros(B, device=cuda_device),
               "output_log_probs": torch.zeros(steps, B, device=cuda_device)}
        for step in range(steps):
            layer.forward(out, {"logits": toy_t[step].repeat(B, 1).contiguous(), "step": step,
                                "max_input_length": 0, "ite": ite, "local_batch_size": lbs,
                                "end_id": torch.full((B,), KAT["end_id"], dtype=torch.int32, device=cuda_device)})
        ids = out["output_ids"].cpu().numpy()
        for i, allowed in enumerate(case["expected"]):
            s, b = divmod(i, B)
            assert ids[s, b] in allowed, (case["name"], seed, s, b, ids[s, b], allowed)


SMALL = [
    ("c1", dict(batch=8, steps=6)),
    ("c1", dict(batch=5, steps=3, vocab=50251)),      # odd vocab: rows not 16-byte aligned
    ("c2", dict(batch=16, steps=5)),
    ("c3", dict(batch=48, steps=4)),
    ("c3", dict(batch=24, steps=3, vocab=32003)),
    ("c3", dict(batch=32, steps=40)),                 # long enough for sampled tokens to come back penalised
    ("c2", dict(batch=24, steps=40)),
]


@pytest.mark.parametrize("name,kw", SMALL, ids=["%s-%s" % (n, "-".join(str(v) for v in k.values())) for n, k in SMALL])
@pytest.mark.parametrize("log_probs", [False, True], ids=["ids", "logprobs"])
def test_against_reference(name, kw, log_probs, cuda_device):
    from fastertransformer_b200.workloads import make_workload
    w = make_workload(name, **kw)
    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, want_log_probs=log_probs, cast=ref_dt, with_criteria=False)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device, want_log_probs=log_probs)
    _compare(mine, ref, name)


def test_against_reference_with_ties(cuda_device):
    """bf16-quantised logits on a small vocabulary: most top-k boundaries fall inside a tie class."""
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", batch=32, steps=3, vocab=4099)
    w.sigma = 0.7

    def coarse(x, step):
        return (x.float() * 4).round().div(4).to(x.dtype)

    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, cast=ref_dt, logits_hook=coarse)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device, logits_hook=coarse)
    _compare(mine, ref, "ties")


@pytest.mark.parametrize("name,kw", [("c1", dict(batch=4, steps=3, vocab=2048)),
                                     ("c2", dict(batch=4, steps=3, vocab=4096)),
                                     ("c3", dict(batch=16, steps=2, vocab=4096))])
def test_against_cpu_oracle(name, kw, cuda_device):
    """Kernel vs the CPU restatement, fed the uniforms the kernel is about to draw."""
    import ctypes as C
    from fastertransformer_b200 import lib, check
    from fastertransformer_b200.workloads import make_workload
    w = make_workload(name, **kw)
    B = w.batch
    layer = _layer(w, cuda_device)
    dname = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16"}[w.dtype]
    orc = OracleDynamicDecodeLayer(w.vocab, w.vocab_padded, dname)
    st = w.initial_state(cuda_device)
    inputs = w.static_inputs(cuda_device)
    inputs.pop("sequence_limit_length", None)
    layer.setup(B, 1, w.runtime_args)
    orc.setup(B, 1, w.runtime_args)
    ost = {k: v.cpu().numpy().copy() for k, v in st.items()}
    oin = {k: (v.cpu().numpy() if torch.is_tensor(v) else v) for k, v in inputs.items()}
    mismatches = 0
    for s in range(w.steps):
        step = w.max_input_length + s
        logits = w.logits(step, cuda_device)
        u = torch.zeros(2, B, device=cuda_device)
        check(lib.ftb200_curand_peek_uniforms(C.c_void_p(layer.topk.curand.data_ptr()), B, 1,
                                               C.c_void_p(u[0].data_ptr()), None))
        check(lib.ftb200_curand_peek_uniforms(C.c_void_p(layer.topp.curand.data_ptr()), B, 1,
                                               C.c_void_p(u[1].data_ptr()), None))
        torch.cuda.synchronize()
        inp = dict(inputs, logits=logits, step=step)
        layer.forward(st, inp)
        torch.cuda.synchronize()
        if w.dtype == torch.bfloat16:
            host_logits = bf16_bits(logits.float().cpu().numpy())
        else:
            host_logits = logits.cpu().numpy()
        un = u.cpu().numpy()
        orc.forward(ost, dict(oin, logits=host_logits, step=step), un[0], un[1])
        got = st["output_ids"][step].cpu().numpy()
        mismatches += int((got != ost["output_ids"][step]).sum())
        # keep both histories identical so later steps stay comparable
        ost["output_ids"][step] = got
        ost["finished"][:] = st["finished"].cpu().numpy()
        ost["sequence_length"][:] = st["sequence_length"].cpu().numpy()
    # libm exp/log vs the GPU's approximate instructions: a draw within a few ulp of a boundary may flip
    assert mismatches <= max(1, int(0.01 * B * w.steps)), mismatches


@pytest.mark.parametrize("vocab,batch", [(8, 1), (33, 3), (1025, 2), (7, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_small_shapes_against_reference(vocab, batch, dtype, cuda_device):
    from fastertransformer_b200.workloads import SamplingWorkload
    rng = np.random.default_rng(vocab * 131 + batch)
    mil, steps = 3, 4
    args = {"runtime_top_k": rng.choice(np.asarray([0, 1, 2, 5], np.uint32), size=batch),
            "runtime_top_p": rng.choice(np.asarray([0.0, 0.4, 0.9], np.float32), size=batch),
            "temperature": np.asarray([0.7], np.float32), "repetition_penalty": np.asarray([1.3], np.float32),
            "random_seed": np.asarray([5], np.uint64)}
    w = SamplingWorkload("tiny", batch, vocab, vocab, dtype, 1.5, steps, mil, vocab - 1, args, 77,
                         prompt=rng.integers(0, vocab, size=(mil, batch)).astype(np.int32))
    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, cast=ref_dt)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device)
    _compare(mine, ref, "tiny")


def test_full_size_properties(cuda_device):
    """Config 3 at full size (1024 x 128256 bf16): every id is a legal draw for its row."""
    from fastertransformer_b200.workloads import make_workload
    w = make_workload("c3", steps=2)
    layer = _layer(w, cuda_device)
    out = run_cuda_like(layer, w, cuda_device)
    k = w.runtime_args["runtime_top_k"].astype(np.int64)
    p = w.runtime_args["runtime_top_p"]
    for s in range(2):
        step = w.max_input_length + s
        logits = w.logits(step, cuda_device).float()
        ids = torch.from_numpy(out["ids"][s]).to(cuda_device).long()
        assert ((ids >= 0) & (ids < w.vocab)).all()
        val = logits.gather(1, ids[:, None])[:, 0]
        rank = (logits > val[:, None]).sum(dim=1).cpu().numpy()   # number of strictly larger logits
        kk = np.where((k == 0) & (p == 0), 1, k)
        topk_rows = kk > 0
        # penalties only lower history tokens, so a sampled token's rank can only improve
        assert (rank[topk_rows] < kk[topk_rows] + w.max_input_length + s + 24).all()
        greedy = kk == 1
        assert (rank[greedy] <= w.max_input_length + s + 24).all()
        # a one-token bad word bans its token outright
        ends = w.bad_words[:, 1, :]
        starts = np.concatenate([np.zeros((w.batch, 1), np.int32), ends[:, :-1]], axis=1)
        single = (ends >= 0) & (ends - starts == 1)
        tok = np.take_along_axis(w.bad_words[:, 0, :], np.clip(starts, 0, None), axis=1)
        assert single.any()
        assert not ((tok == out["ids"][s][:, None]) & single).any()
    # a row's length grows by one per step until the row has drawn its end id
    done_before = np.concatenate([np.zeros((1, w.batch), bool), out["finished"][:-1].astype(bool)])
    grow = np.diff(np.concatenate([np.full((1, w.batch), w.max_input_length), out["sequence_length"]]), axis=0)
    topk_rows = kk > 0
    assert (grow[:, topk_rows][~done_before[:, topk_rows]] == 1).all()
    assert (grow[:, topk_rows][done_before[:, topk_rows]] == 0).all()
    assert (out["finished"].astype(bool) == (out["ids"] == w.end_id))[:, topk_rows][~done_before[:, topk_rows]].all()


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["topk", "topp"])
def test_draw_distribution_chi_square(kind, cuda_device):
    """10^6 draws from one logits row against the analytic distribution of the reference's draw rule
    (sampling_topk_kernels.cu:276-287: r = u * sum of the k exponentials, first index whose running difference
    is <= 0; sampling_topp_kernels.cu:910-960: first sorted index whose inclusive cumulative probability
    reaches u * p).  Every row has its own curand stream."""
    from scipy.stats import chisquare
    from fastertransformer_b200 import DynamicDecodeLayer
    B, V, steps = 8192, 64, 123
    rng = np.random.Generator(np.random.PCG64(77))
    row = rng.normal(0.0, 1.5, size=V).astype(np.float32)
    order = np.argsort(-row, kind="stable")
    e = np.exp((row - row.max()).astype(np.float64))
    if kind == "topk":
        k = 12
        args = {"runtime_top_k": np.asarray([k], np.uint32), "runtime_top_p": np.asarray([1.0], np.float32)}
        expect = np.zeros(V)
        expect[order[:k]] = e[order[:k]] / e[order[:k]].sum()
    else:
        p = 0.8
        args = {"runtime_top_k": np.asarray([0], np.uint32), "runtime_top_p": np.asarray([p], np.float32)}
        prob = e / e.sum()
        c = np.cumsum(prob[order])
        lo = np.concatenate([[0.0], c[:-1]])
        width = np.clip(np.minimum(c, p) - lo, 0.0, None) / p
        expect = np.zeros(V)
        expect[order] = width
    args["random_seed"] = (np.arange(B) * 11 + 5).astype(np.uint64)
    layer = DynamicDecodeLayer(V, V, torch.float32, cuda_device)
    layer.setup(B, 1, args)
    st = {"output_ids": torch.zeros(steps + 1, B, dtype=torch.int32, device=cuda_device)}
    logits = torch.from_numpy(np.tile(row, (B, 1))).to(cuda_device)
    end = torch.full((B,), V + 5, dtype=torch.int32, device=cuda_device)  # never drawn: rows never finish
    for s in range(steps):
        layer.forward(st, {"logits": logits, "step": s + 1, "max_input_length": 1, "ite": 0, "local_batch_size": B,
                           "end_id": end})
    ids = st["output_ids"][1:].cpu().numpy().reshape(-1)
    assert ids.size >= 10 ** 6
    counts = np.bincount(ids, minlength=V).astype(np.float64)
    assert counts[expect == 0].sum() == 0, "a column outside the top-k / nucleus was drawn"
    sel = expect > 0
    stat, pval = chisquare(counts[sel], expect[sel] * ids.size)
    assert pval > 1e-4, (stat, pval)


def _random_workload(seed):
    """A random decode configuration: logits type, shape, per-row k / p mix, temperature, penalty kind, bad words,
    spread of the logits (flat rows make large top-p nuclei, peaked rows make small ones)."""
    from fastertransformer_b200.workloads import SamplingWorkload, _bad_words
    rng = np.random.default_rng(9000 + seed)
    dtype = [torch.float32, torch.float16, torch.bfloat16][seed % 3]
    vocab = int(rng.choice([1536, 4099, 8192, 20011, 32000, 50257]))
    vpad = vocab if seed % 4 else (vocab + 7) // 8 * 8 + 8 * int(rng.integers(0, 3))
    batch = int(rng.integers(3, 40))
    mil, steps = int(rng.integers(2, 40)), int(rng.integers(2, 5))
    ks = np.asarray([0, 1, 2, 17, 64, 300, 1024], np.uint32)
    ps = np.asarray([0.0, 0.05, 0.3, 0.7, 0.95, 1.0], np.float32)
    args = {"runtime_top_k": rng.choice(ks, size=batch), "runtime_top_p": rng.choice(ps, size=batch),
            "random_seed": rng.integers(0, 2 ** 40, size=batch).astype(np.uint64)}
    if seed % 2:
        args["temperature"] = rng.choice(np.asarray([0.5, 0.8, 1.0, 1.7], np.float32), size=batch)
    kind = seed % 5
    if kind in (0, 1):
        args["repetition_penalty"] = rng.choice(np.asarray([0.8, 1.0, 1.3, 2.0], np.float32), size=batch)
    elif kind == 2:
        args["presence_penalty"] = np.asarray([0.6], np.float32)
    if seed % 3 == 1:
        args["min_length"] = np.asarray([2], np.int32)
    w = SamplingWorkload("rand%d" % seed, batch, vocab, vpad, dtype, float(rng.choice([0.4, 1.5, 3.0, 6.0])), steps, mil,
                         int(rng.integers(0, vocab)), args, 4000 + seed,
                         bad_words=_bad_words(rng, batch, vocab) if seed % 2 == 0 else None,
                         prompt=rng.integers(0, vocab, size=(mil, batch)).astype(np.int32))
    return w


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("FTB200_RANDOM_CASES", "30")))))
def test_random_configurations_against_reference(seed, cuda_device):
    w = _random_workload(seed)
    log_probs = seed % 7 == 3
    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, want_log_probs=log_probs, cast=ref_dt, with_criteria=False)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device, want_log_probs=log_probs)
    _compare(mine, ref, w.name)


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("FTB200_RANDOM_LARGE_CASES", "9")))))
def test_random_large_vocabularies_against_reference(seed, cuda_device):
    """The same random mix at the vocabulary sizes of current models (aligned and odd), where the two-pass
    top-k, the dense class count and the wide candidate sets come into play."""
    from fastertransformer_b200.workloads import SamplingWorkload, _bad_words
    rng = np.random.default_rng(777 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    vocab = [128256, 100003, 151936][(seed // 3) % 3]
    batch, mil, steps = 40, int(rng.integers(20, 200)), 3
    args = {"runtime_top_k": rng.choice(np.asarray([0, 1, 5, 40, 512, 1024], np.uint32), size=batch),
            "runtime_top_p": rng.choice(np.asarray([0.0, 0.2, 0.6, 0.9, 0.99], np.float32), size=batch),
            "random_seed": rng.integers(0, 2 ** 40, size=batch).astype(np.uint64),
            "repetition_penalty": np.asarray([1.15], np.float32)}
    if seed % 2:
        args["temperature"] = rng.choice(np.asarray([0.6, 1.0, 1.3], np.float32), size=batch)
    w = SamplingWorkload("large%d" % seed, batch, vocab, vocab, dtype, float(rng.choice([1.0, 2.5, 5.0])), steps, mil,
                         vocab - 3, args, 5000 + seed, bad_words=_bad_words(rng, batch, vocab),
                         prompt=rng.integers(0, vocab, size=(mil, batch)).astype(np.int32))
    log_probs = seed % 4 == 2
    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, want_log_probs=log_probs, cast=ref_dt, with_criteria=False)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device, want_log_probs=log_probs)
    _compare(mine, ref, w.name)


@pytest.mark.parametrize("name,kw", [("c3", dict(batch=48, steps=3)), ("c3", dict(batch=24, steps=3, vocab=32003)),
                                     ("c2", dict(batch=32, steps=3))],
                         ids=["c3", "c3-odd-vocab", "c2"])
@pytest.mark.parametrize("n_top", [1, 12, 200], ids=["top1", "top12", "top200"])
def test_largest_columns_in_history_against_reference(name, kw, n_top, cuda_device):
    """The prompt of every row holds the row's largest columns of every step (what a long generation does to
    itself): the row maximum is a penalised column, so the maximum over the other columns has to be found, and
    many of the per-slot maxima of the first pass belong to penalised columns."""
    from fastertransformer_b200.workloads import make_workload
    w = make_workload(name, **kw)
    mil = w.max_input_length
    assert mil >= 3 * n_top or n_top == 200
    prompt = w.prompt.copy()
    pos = 0
    for s in range(w.steps):
        x = w.logits(mil + s, cuda_device).float()[:, :w.vocab]
        top = torch.topk(x, n_top, dim=1).indices.cpu().numpy().astype(np.int32)       # [batch, n_top]
        take = min(n_top, (mil - pos))
        prompt[pos:pos + take] = top[:, :take].T
        pos += take
    w.prompt = prompt
    ref_layer, ref_dt = _ref_layer(w, cuda_device)
    ref = run_cuda_like(ref_layer, w, cuda_device, cast=ref_dt, with_criteria=False)
    mine = run_cuda_like(_layer(w, cuda_device), w, cuda_device)
    _compare(mine, ref, name)
