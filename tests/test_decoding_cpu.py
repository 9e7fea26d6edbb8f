"""CPU checks of the restated caller-side kernels (oracle_gather_tree, oracle_finalize,
oracle_insert_unfinished_path, oracle_decoding_initialize) against the committed outputs of the reference's
own kernels (tests/golden/decoding_ref.json, made by tests/golden/make_decoding_fixture.py)."""
import json
import os

import numpy as np
import pytest

import decoding_cases as dc

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoding_ref.json")) as f:
    GOLDEN = json.load(f)


def check(res, gold, float_keys=()):
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
def test_gather_tree(name):
    check(dc.run_gather_tree("oracle", dc.gather_tree_case(**dc.GOLDEN_GATHER[name])), GOLDEN["gather_tree"][name])


@pytest.mark.parametrize("name", list(dc.GOLDEN_FINALIZE))
def test_finalize(name):
    check(dc.run_finalize("oracle", dc.finalize_case(**dc.GOLDEN_FINALIZE[name])), GOLDEN["finalize"][name])


@pytest.mark.parametrize("name", list(dc.GOLDEN_INSERT))
def test_insert_unfinished_path(name):
    check(dc.run_insert("oracle", dc.insert_case(**dc.GOLDEN_INSERT[name])), GOLDEN["insert"][name],
          float_keys=("normed",))


@pytest.mark.parametrize("dtype", [0, 1, 2])
def test_decoding_initialize(dtype):
    check(dc.run_initialize("oracle", 3, 4, 17, dtype), GOLDEN["initialize"][str(dtype)])


def test_gather_tree_follows_parents_by_hand():
    # T=3, one entry, two beams: beam 0 ends on token 30 whose parent chain is 1 -> 0
    c = dc.gather_tree_case(seed=0, B=1, K=2, T=3, with_output=False)
    c["step_ids"] = np.array([[[10, 11]], [[20, 21]], [[30, 31]]], np.int32)
    c["parent_ids"] = np.array([[[0, 0]], [[0, 0]], [[1, 0]]], np.int32)
    c["end_tokens"] = np.array([99], np.int32)
    c["seq_lengths"] = np.array([[3, 3]], np.int32)
    r = dc.run_gather_tree("oracle", c)
    assert r["beams"][:, 0, 0].tolist() == [10, 21, 30]
    assert r["beams"][:, 0, 1].tolist() == [10, 20, 31]
