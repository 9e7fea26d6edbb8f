"""ftb200_decoding_initialize / ftb200_gather_tree / ftb200_finalize / ftb200_insert_unfinished_path against
the reference's kernels (oracle/_ref), their committed outputs, and the CPU restatement.  Integer outputs are
compared bit for bit; normalised scores to 2e-6 relative (powf under the reference's fast-math build)."""
import json
import os

import numpy as np
import pytest

import decoding_cases as dc
import ft_reference

pytestmark = pytest.mark.gpu
needs_ref = pytest.mark.skipif(not ft_reference.available(), reason="oracle/_ref not built")

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoding_ref.json")) as f:
    GOLDEN = json.load(f)


def check_gold(res, gold, float_keys=()):
    for k, v in res.items():
        if v is None:
            assert gold[k] is None
            continue
        want = np.array(gold[k], dtype=v.dtype).reshape(v.shape)
        if k in float_keys:
            np.testing.assert_allclose(v, want, rtol=2e-6, atol=0, err_msg=k)
        else:
            np.testing.assert_array_equal(v, want, err_msg=k)


@pytest.mark.parametrize("name", list(dc.GOLDEN_GATHER))
def test_gather_tree_committed_reference_outputs(name):
    check_gold(dc.run_gather_tree("ours", dc.gather_tree_case(**dc.GOLDEN_GATHER[name])),
               GOLDEN["gather_tree"][name])


@pytest.mark.parametrize("name", list(dc.GOLDEN_FINALIZE))
def test_finalize_committed_reference_outputs(name):
    check_gold(dc.run_finalize("ours", dc.finalize_case(**dc.GOLDEN_FINALIZE[name])), GOLDEN["finalize"][name])


@pytest.mark.parametrize("name", list(dc.GOLDEN_INSERT))
def test_insert_committed_reference_outputs(name):
    check_gold(dc.run_insert("ours", dc.insert_case(**dc.GOLDEN_INSERT[name])), GOLDEN["insert"][name],
               float_keys=("normed",))


# Entries whose beams share a warp in the reference's launch (beam_width divides 32, or everything in one warp):
# there its length update is well defined.
GATHER_LIVE = [
    dict(seed=31, B=64, K=4, T=600, M=40, final_step=1, with_response=True),
    dict(seed=32, B=300, K=4, T=90, M=12, final_step=1),                      # two blocks in the reference
    dict(seed=33, B=10, K=3, T=50, M=7, final_step=1),
    dict(seed=34, B=5, K=16, T=2100, M=100, final_step=1, bad_parents=True),  # 128 levels per tile here
    dict(seed=35, B=9, K=1, T=3000, M=900, final_step=1),
    dict(seed=36, B=7, K=1, T=40, M=0, with_output=False),
    dict(seed=37, B=33, K=8, T=300, M=0, with_output=False),
    dict(seed=38, B=12, K=2, T=700, M=64, prefix=True, final_step=1, with_response=True),
    dict(seed=39, B=12, K=8, T=260, M=33, virtual=True, final_step=1),
    dict(seed=40, B=6, K=4, T=130, M=20, prefix=True, virtual=True, final_step=1, bad_parents=True),
    dict(seed=41, B=2, K=32, T=64, M=5, final_step=0),
]


@needs_ref
@pytest.mark.parametrize("kw", GATHER_LIVE, ids=[f"b{k['B']}_k{k['K']}_t{k['T']}_s{k['seed']}" for k in GATHER_LIVE])
def test_gather_tree_against_reference(kw):
    c = dc.gather_tree_case(**kw)
    ours, ref = dc.run_gather_tree("ours", c), dc.run_gather_tree("ref", c)
    dc.same(ours, ref)
    dc.same(ours, dc.run_gather_tree("oracle", c))


@pytest.mark.parametrize("kw", [
    dict(seed=51, B=40, K=3, T=80, M=9, final_step=1),        # beams of an entry span two warps in the reference
    dict(seed=52, B=2, K=300, T=70, M=6, final_step=1),       # more beams than threads
    dict(seed=53, B=1, K=1024, T=30, M=4, final_step=1),
    dict(seed=54, B=3, K=5, T=10, M=0, with_output=False),
], ids=["k3_two_warps", "k300", "k1024", "k5_short"])
def test_gather_tree_against_restatement(kw):
    c = dc.gather_tree_case(**kw)
    dc.same(dc.run_gather_tree("ours", c), dc.run_gather_tree("oracle", c))


def test_gather_tree_empty_sequences_leave_buffers_alone():
    c = dc.gather_tree_case(seed=3, B=3, K=2, T=8, with_output=False)
    c["seq_lengths"][:] = 0
    r = dc.run_gather_tree("ours", c)
    assert (r["beams"] == dc.SENTINEL).all()
    dc.same(r, dc.run_gather_tree("oracle", c))


FINALIZE_LIVE = [dict(seed=61, B=64, K=4, L=500), dict(seed=62, B=3, K=64, L=40),
                 dict(seed=63, B=2, K=200, L=9, with_log_probs=False), dict(seed=64, B=128, K=1, L=33),
                 dict(seed=65, B=5, K=495, L=4)]


@needs_ref
@pytest.mark.parametrize("kw", FINALIZE_LIVE, ids=[f"b{k['B']}_k{k['K']}_l{k['L']}" for k in FINALIZE_LIVE])
def test_finalize_against_reference(kw):
    c = dc.finalize_case(**kw)
    ours, ref = dc.run_finalize("ours", c), dc.run_finalize("ref", c)
    # positions past a hypothesis' length are not written by either
    dc.same(ours, ref)
    dc.same(ours, dc.run_finalize("oracle", c))


def test_finalize_short_archives_against_restatement():
    c = dc.finalize_case(seed=66, B=40, K=6, L=12, short_archives=True)
    dc.same(dc.run_finalize("ours", c), dc.run_finalize("oracle", c))


def test_finalize_refuses_what_the_reference_asserts():
    import torch
    from fastertransformer_b200 import lib
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    f = torch.zeros(8, device="cuda")
    rc = lib.ftb200_finalize(z.data_ptr(), z.data_ptr(), None, None, z.data_ptr(), z.data_ptr(), f.data_ptr(), None,
                             None, z.data_ptr(), 497, 1, 1, None)
    assert rc == 5      # 994 threads round up to 1024, where FT_CHECK(block.x < 1024) fires
    assert lib.ftb200_finalize(None, z.data_ptr(), None, None, z.data_ptr(), z.data_ptr(), f.data_ptr(), None,
                               None, z.data_ptr(), 4, 1, 1, None) == 1


INSERT_LIVE = [dict(seed=71, B=32, K=4, L=700), dict(seed=72, B=3, K=100, L=50, length_penalty=1.0),
               dict(seed=73, B=64, K=1, L=90, with_log_probs=False, length_penalty=0.6),
               dict(seed=74, B=2, K=512, L=9), dict(seed=75, B=5, K=8, L=3000, with_log_probs=False)]


@needs_ref
@pytest.mark.parametrize("kw", INSERT_LIVE, ids=[f"b{k['B']}_k{k['K']}_l{k['L']}" for k in INSERT_LIVE])
def test_insert_unfinished_path_against_reference(kw):
    c = dc.insert_case(**kw)
    ours, ref = dc.run_insert("ours", c), dc.run_insert("ref", c)
    dc.same(ours, ref, float_keys=("normed",))
    dc.same(ours, dc.run_insert("oracle", c), float_keys=("normed",))


def test_insert_then_finalize_round_trip():
    """Archive K live beams into empty archives, rank them: the best-scoring live beam comes out first with the
    ids its parent chain spells."""
    B, K, L = 4, 4, 11
    c = dc.insert_case(seed=81, B=B, K=K, L=L, length_penalty=1.0)
    c["num_beams"][:] = 0
    c["is_done"][:] = 0
    a = dc.run_insert("ours", c)
    assert (a["num_beams"] == K).all()
    f = dc.finalize_case(seed=82, B=B, K=K, L=L)
    f["topk_output_ids"], f["topk_sequence_lengths"] = a["output_ids_tgt"], a["lengths_tgt"]
    f["scores"], f["topk_cum_log_probs"], f["topk_log_probs"] = a["normed"], a["cum_tgt"], a["log_probs_tgt"]
    f["num_beams"] = a["num_beams"]
    r = dc.run_finalize("ours", f)
    for b in range(B):
        best = int(np.argmax(a["normed"][b, :K]))
        n = int(a["lengths_tgt"][b, best])
        assert r["lengths"][b, 0] == n
        np.testing.assert_array_equal(r["output_ids"][b, 0, :n], a["output_ids_tgt"][b, best, 1:n + 1])
        # the chain, by hand
        col, want = b * K + best, []
        want.append(c["output_ids_src"][n, col])
        prev = c["parent_ids_src"][n, col]
        for j in range(n - 1, -1, -1):
            want.append(c["output_ids_src"][j, b * K + prev])
            prev = c["parent_ids_src"][j, b * K + prev]
        np.testing.assert_array_equal(a["output_ids_tgt"][b, best, :n + 1], want[::-1])


@needs_ref
@pytest.mark.parametrize("dtype", [0, 1, 2], ids=["f32", "f16", "bf16"])
@pytest.mark.parametrize("with_word_ids", [True, False])
def test_decoding_initialize_against_reference(dtype, with_word_ids):
    ours = dc.run_initialize("ours", 37, 5, 123, dtype, with_word_ids)
    dc.same(ours, dc.run_initialize("ref", 37, 5, 123, dtype, with_word_ids))
    dc.same(ours, dc.run_initialize("oracle", 37, 5, 123, dtype, with_word_ids))
    check_gold(dc.run_initialize("ours", 3, 4, 17, dtype), GOLDEN["initialize"][str(dtype)])


def test_argument_checks():
    import ctypes as C
    import torch
    from fastertransformer_b200 import GatherTreeParams, lib
    z = torch.zeros(16, dtype=torch.int32, device="cuda")
    P = GatherTreeParams(beams=z.data_ptr(), max_sequence_lengths=z.data_ptr(), max_time=1, batch_size=1,
                         beam_width=2000, step_ids=z.data_ptr(), parent_ids=z.data_ptr(), end_tokens=z.data_ptr(),
                         max_input_length=1)
    assert lib.ftb200_gather_tree(C.byref(P)) == 5          # more beams than the kernel serves
    P.beam_width, P.step_ids = 2, None
    assert lib.ftb200_gather_tree(C.byref(P)) == 1
    assert lib.ftb200_gather_tree(None) == 1
    assert lib.ftb200_decoding_initialize(None, z.data_ptr(), None, z.data_ptr(), 0, None, 1, 1, 1, None) == 1
    assert lib.ftb200_decoding_initialize(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 0, None, 1, 1, 1,
                                          None) == 1      # word_ids without sentence_ids
    assert lib.ftb200_insert_unfinished_path(None, z.data_ptr(), z.data_ptr(), z.data_ptr(), None, 4, 0.0,
                                             z.data_ptr(), z.data_ptr(), 1, 1, None) == 1
