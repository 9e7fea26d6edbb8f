"""Extracts the known-answer cases of the reference's sampling layer test into JSON.

Reads tests/unittests/test_sampling_layer.cu of a FasterTransformer checkout as TEXT (nothing is
compiled or run): the 3x8 toy logits (probabilities 0.4/0.3/0.2/0.1 on four columns per step) and, for
every TYPED_TEST(SamplingDecodeTest, ...), the runtime top-k / top-p arguments and the set of ids each
(step, row) may produce.  Output: tests/golden/sampling_layer_kat.json.

usage: python tests/golden/make_sampling_layer_kat.py [FT_ROOT]     (default: $FT_REFERENCE_ROOT)
"""
import json
import os
import re
import sys

root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FT_REFERENCE_ROOT", "")
if not root:
    sys.exit("usage: make_sampling_layer_kat.py REFERENCE_ROOT   (or set FT_REFERENCE_ROOT)")
src = open(os.path.join(root, "tests/unittests/test_sampling_layer.cu")).read()

m = re.search(r"test_input_logits = new T\[24\]\{(.*?)\};", src, re.S)
body = re.sub(r"//.*", "", m.group(1))
logits = [("-FLT_MAX" if "FLT_MAX" in t else float(t)) for t in (x.strip() for x in body.split(",")) if t]
assert len(logits) == 24

cases = []
for tm in re.finditer(r"TYPED_TEST\(SamplingDecodeTest,\s*(\w+)\)\s*\{(.*?)\n\}", src, re.S):
    name, b = tm.group(1), tm.group(2)
    call = re.search(r"this->runTest\((.*?)\);", b, re.S).group(1)
    argv = [a.strip() for a in call.split(",")]
    case = {"name": name, "use_local_batch": len(argv) > 7 and argv[7] == "true"}
    k1 = re.search(r"int\s+top_k\s*=\s*(\d+)\s*;", b)
    kn = re.search(r"int\*\s*top_ks\s*=\s*new int\[batch_size\]\{(.*?)\}", b)
    p1 = re.search(r"float\s+top_p\s*=\s*([0-9.]+)f?\s*;", b)
    pn = re.search(r"float\*\s*top_ps\s*=\s*new float\[batch_size\]\{(.*?)\}", b)
    if argv[1] != "nullptr":
        case["top_k"] = [int(k1.group(1))] if argv[1] == "&top_k" else [int(x) for x in kn.group(1).split(",")]
    if argv[3] != "nullptr":
        case["top_p"] = ([float(p1.group(1))] if argv[3] == "&top_p" else
                         [float(x.strip().rstrip("f")) for x in pn.group(1).split(",")])
    em = re.search(r"expected_output_ids\s*\{(.*?)\};", b, re.S)
    ebody = re.sub(r"//.*", "", em.group(1))
    sets = [[int(x) for x in s.split(",") if x.strip()] for s in re.findall(r"\{([^{}]*)\}", ebody)]
    assert len(sets) == 18, (name, len(sets))
    case["expected"] = sets
    cases.append(case)

out = {
    "source": "tests/unittests/test_sampling_layer.cu (SamplingDecodeTest)",
    "batch_size": 6, "vocab_size": 8, "end_id": 7, "max_input_len": 0, "steps": 3, "seeds": 30,
    "logits": logits, "cases": cases,
}
dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampling_layer_kat.json")
json.dump(out, open(dst, "w"), indent=1)
print("wrote", dst, len(cases), "cases")
