"""Generates tests/golden/decoding_ref.json: outputs of the reference's own invokeGatherTree, invokeFinalize,
invokeInsertUnfinishedPath and invokeDecodingInitialize (compiled into oracle/_ref/libft_decode_ref.so) on the
seeded cases of tests/decoding_cases.py.  Needs a GPU.

usage: python tests/golden/make_decoding_fixture.py [OUT.json]
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def pack(res):
    return {k: None if v is None else np.asarray(v).ravel().tolist() for k, v in res.items()}


def main():
    import decoding_cases as dc
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "decoding_ref.json")
    out = {"gather_tree": {}, "finalize": {}, "insert": {}, "initialize": {}}
    for name, kw in dc.GOLDEN_GATHER.items():
        out["gather_tree"][name] = pack(dc.run_gather_tree("ref", dc.gather_tree_case(**kw)))
    for name, kw in dc.GOLDEN_FINALIZE.items():
        out["finalize"][name] = pack(dc.run_finalize("ref", dc.finalize_case(**kw)))
    for name, kw in dc.GOLDEN_INSERT.items():
        out["insert"][name] = pack(dc.run_insert("ref", dc.insert_case(**kw)))
    for dtype in (0, 1, 2):
        out["initialize"][str(dtype)] = pack(dc.run_initialize("ref", 3, 4, 17, dtype))
    with open(out_path, "w") as f:
        json.dump(out, f)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
