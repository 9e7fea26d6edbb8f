"""The cases of the reference's own test of its torch op (tests/unittests/th_op/test_th_decode_op.py: minimum
length at sampling and at beam search, the id sequence under repetition / presence penalty), re-driven through
the compiled torch custom class torch.classes.FasterTransformer.DynamicDecodeOp of this package
(fastertransformer_b200/th_op, lib/libth_ftb200.so) and through its Python twin
fastertransformer_b200.th_decode_op.DynamicDecodeOp, with the same positional argument lists."""
import itertools
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
VOCAB, END_ID = 1024, 0
TH_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fastertransformer_b200", "lib",
                      "libth_ftb200.so")
IMPL = "python"


@pytest.fixture(params=["torch_class", "python"], autouse=True)
def op_impl(request):
    global IMPL
    IMPL = request.param
    yield
    IMPL = "python"


def make_op(dtype=torch.float):
    if IMPL == "torch_class":
        if not os.path.exists(TH_LIB):
            pytest.fail("lib/libth_ftb200.so is not built: run python -m fastertransformer_b200.build")
        torch.classes.load_library(TH_LIB)
        return torch.classes.FasterTransformer.DynamicDecodeOp(VOCAB, VOCAB, 1, 1, dtype)
    from fastertransformer_b200.th_decode_op import DynamicDecodeOp
    return DynamicDecodeOp(VOCAB, VOCAB, 1, 1, dtype)


def _vec(batch, value, dtype, cpu):
    if value is None:
        return None
    return value * torch.ones(batch, dtype=dtype, device="cpu" if cpu else "cuda")


def run_decode(batch_size=4, beam_width=1, max_input_length=4, gen_length=3, top_k=None, top_p=None, temperature=None,
               repetition_penalty=None, presence_penalty=None, min_length=None, len_penalty=None,
               beam_search_diversity_rate=None, random_seed=None, logit_fn=None, use_random_input_tokens=True,
               dtype=torch.float):
    op = make_op(dtype)
    dev = torch.device("cuda", torch.cuda.current_device())
    ite, lbs, L = 0, batch_size, max_input_length + gen_length
    eos = _vec(batch_size, END_ID, torch.int, False)
    a = dict(top_ks=_vec(batch_size, top_k, torch.int, True), top_ps=_vec(batch_size, top_p, torch.float, True),
             temps=_vec(batch_size, temperature, torch.float, True),
             reps=_vec(batch_size, repetition_penalty, torch.float, True),
             pres=_vec(batch_size, presence_penalty, torch.float, True), mins=_vec(batch_size, min_length, torch.int, True),
             lens=_vec(batch_size, len_penalty, torch.float, True),
             divs=_vec(batch_size, beam_search_diversity_rate, torch.float, True),
             seeds=_vec(batch_size, random_seed, torch.int64, True))
    if beam_width > 1:
        parent_ids = torch.zeros(L, batch_size * beam_width, dtype=torch.int32, device=dev)
        cache = torch.zeros(2, batch_size, beam_width, L, dtype=torch.int32, device=dev)
        cum = torch.zeros(batch_size * beam_width, device=dev)
    else:
        parent_ids = cache = cum = None
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    if use_random_input_tokens:
        tokens = torch.randint(1, VOCAB, (batch_size, max_input_length), dtype=torch.int, device=dev, generator=g)
    else:
        tokens = torch.ones(batch_size, max_input_length, dtype=torch.int, device=dev)
    in_len = torch.randint(1, max_input_length + 1, (batch_size,), dtype=torch.int, device=dev, generator=g)
    in_len[0] = max_input_length
    steps = torch.arange(0, max_input_length, device=dev).unsqueeze(0).tile(batch_size, 1)
    tokens[in_len.unsqueeze(1) <= steps] = END_ID
    tokens = tokens.repeat(1, beam_width).view(batch_size * beam_width, -1)
    in_len = in_len.view(-1, 1).repeat(1, beam_width).view(-1)
    op.setup(batch_size, beam_width, a["top_ks"], a["top_ps"], a["temps"], a["reps"], a["pres"], a["mins"], a["lens"],
             a["divs"], a["seeds"], None, None, None)
    finished = torch.zeros_like(in_len).bool()
    seq_len = (max_input_length - 1) * torch.ones_like(in_len)
    out_ids = torch.zeros(L, batch_size * beam_width, dtype=torch.int32, device=dev)
    out_ids[:max_input_length] = tokens.T
    src = tgt = None
    for step in range(max_input_length, L):
        if cache is not None:
            s = (step - max_input_length) % 2
            src, tgt = cache[s], cache[1 - s]
        logits = (torch.randn(batch_size, beam_width, VOCAB, device=dev, generator=g) if logit_fn is None
                  else logit_fn(batch_size, beam_width, dev, g)).to(dtype)
        stop = op.forward(logits, step, max_input_length, ite, lbs, eos, a["top_ks"], a["top_ps"], a["temps"], a["reps"],
                          a["pres"], a["mins"], a["lens"], a["divs"], None, None, None, None, in_len, None, None, None, src,
                          out_ids.view(-1, batch_size, beam_width), finished, seq_len, cum, None, parent_ids, tgt)
        if bool(stop):
            break
    return dict(output_token_ids=out_ids.T, output_sequence_lengths=seq_len + 1)


def _eos_most_probable(batch, beam, dev, g):
    logits = torch.randn(batch, beam, VOCAB, device=dev, generator=g)
    logits[..., END_ID] = logits.max(dim=-1)[0] + 1
    return logits


@pytest.mark.parametrize("tc,method", list(itertools.product(
    [dict(batch_size=4, max_input_length=4, min_length=2, gen_length=4),
     dict(batch_size=4, max_input_length=4, min_length=32, gen_length=64),
     dict(batch_size=2048, max_input_length=6, min_length=4, gen_length=8)],   # batch exceeds 1024
    [dict(top_k=1, top_p=0.0), dict(top_k=0, top_p=0.8)])))
def test_min_length_correctness_at_sampling(tc, method):
    out = run_decode(beam_width=1, logit_fn=_eos_most_probable, **tc, **method)
    assert bool((out["output_sequence_lengths"] >= tc["max_input_length"] + tc["min_length"]).all())


@pytest.mark.parametrize("tc", [dict(batch_size=4, beam_width=2, max_input_length=4, min_length=2, gen_length=4),
                                dict(batch_size=1024, beam_width=2, max_input_length=4, min_length=4, gen_length=8),
                                dict(batch_size=4, beam_width=60, max_input_length=4, min_length=4, gen_length=8)])
def test_min_length_correctness_at_beamsearch(tc):
    out = run_decode(logit_fn=_eos_most_probable, **tc)
    assert bool((out["output_sequence_lengths"] >= tc["max_input_length"] + tc["min_length"]).all())


def _descending_three(batch, beam, dev, g):
    # token v-1 is the most probable unless penalised: the expected ids are v-1, v-2, v-3, v-1, v-1, ...
    logits = torch.zeros(batch, beam, VOCAB, device=dev)
    logits[..., VOCAB - 1], logits[..., VOCAB - 2], logits[..., VOCAB - 3] = 2.0, 1.8, 1.6
    return logits


@pytest.mark.parametrize("tc,method", list(itertools.product(
    [dict(batch_size=4, max_input_length=4, repetition_penalty=2), dict(batch_size=2048, max_input_length=4, repetition_penalty=2),
     dict(batch_size=4, max_input_length=4, presence_penalty=0.5), dict(batch_size=4, max_input_length=4, presence_penalty=1.0),
     dict(batch_size=2048, max_input_length=4, presence_penalty=0.5)],
    [dict(top_k=1, top_p=0.0), dict(beam_width=2)])))
def test_repetition_penalty_correctness(tc, method):
    gen = 5
    beam = method.get("beam_width", 1)
    expect = (VOCAB - 1) * torch.ones(tc["batch_size"] * beam, gen, dtype=torch.int32)
    expect[:, 1], expect[:, 2] = VOCAB - 2, VOCAB - 3
    out = run_decode(gen_length=gen, use_random_input_tokens=False, logit_fn=_descending_three, **tc, **method)
    got = out["output_token_ids"][:, tc["max_input_length"]:]
    assert bool((expect.to(got.device) == got).all())


def test_compiled_class_and_python_twin_draw_the_same_ids():
    global IMPL
    if IMPL != "torch_class":
        pytest.skip("runs once")
    outs = []
    for impl in ("torch_class", "python"):
        IMPL = impl
        outs.append(run_decode(batch_size=64, max_input_length=5, gen_length=12, top_k=20, top_p=0.7, temperature=0.8,
                               repetition_penalty=1.3, random_seed=11))
        outs.append(run_decode(batch_size=8, beam_width=4, max_input_length=5, gen_length=12, len_penalty=1.0,
                               beam_search_diversity_rate=0.2))
    IMPL = "torch_class"
    for a, b in ((outs[0], outs[2]), (outs[1], outs[3])):
        assert bool((a["output_token_ids"] == b["output_token_ids"]).all())
        assert bool((a["output_sequence_lengths"] == b["output_sequence_lengths"]).all())


def test_compiled_class_argument_checks():
    if IMPL != "torch_class":
        pytest.skip("the compiled class's own checks")
    op = make_op()
    with pytest.raises(RuntimeError):      # runtime arguments are host tensors (CHECK_OPTIONAL_CPU_INPUT)
        op.setup(2, 1, torch.ones(2, dtype=torch.int, device="cuda"), None, None, None, None, None, None, None, None,
                 None, None, None)
    with pytest.raises(RuntimeError):      # tensor / pipeline parallel sizes other than 1
        torch.classes.FasterTransformer.DynamicDecodeOp(VOCAB, VOCAB, 2, 1, torch.float)
    with pytest.raises(RuntimeError):      # logits of another type than the op's
        op.setup(2, 1, torch.ones(2, dtype=torch.int), None, None, None, None, None, None, None, None, None, None, None)
        ids = torch.zeros(3, 2, 1, dtype=torch.int32, device="cuda")
        op.forward(torch.zeros(2, 1, VOCAB, dtype=torch.half, device="cuda"), 1, 1, 0, 2,
                   torch.zeros(2, dtype=torch.int32, device="cuda"), None, None, None, None, None, None, None, None, None,
                   None, None, None, None, None, None, None, None, ids, None, None, None, None, None, None)


@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16], ids=["half", "bfloat16"])
def test_compiled_class_16_bit_logits(dtype):
    global IMPL
    if IMPL != "torch_class":
        pytest.skip("runs once")
    outs = []
    for impl in ("torch_class", "python"):
        IMPL = impl
        outs.append(run_decode(batch_size=32, max_input_length=5, gen_length=10, top_k=0, top_p=0.8, temperature=0.9,
                               presence_penalty=0.3, random_seed=5, dtype=dtype))
    IMPL = "torch_class"
    assert bool((outs[0]["output_token_ids"] == outs[1]["output_token_ids"]).all())
    assert bool((outs[0]["output_sequence_lengths"] == outs[1]["output_sequence_lengths"]).all())

