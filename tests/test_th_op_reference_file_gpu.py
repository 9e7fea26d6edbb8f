"""The reference's own test of its torch op, run as it stands against this package's torch custom class
(fastertransformer_b200/th_op, lib/libth_ftb200.so registers torch.classes.FasterTransformer.DynamicDecodeOp with the
reference's constructor and forward argument lists, th_op/dynamic_decode/DynamicDecodeOp.h:64-124)."""
import os

import pytest

pytestmark = pytest.mark.gpu
TH_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fastertransformer_b200", "lib",
                      "libth_ftb200.so")


def test_reference_test_file_runs_unmodified(tmp_path):
    """The reference's tests/unittests/th_op/test_th_decode_op.py, byte for byte, run by unittest from a directory
    whose lib/libth_transformer.so is this package's libth_ftb200.so.  The file comes from a FasterTransformer
    checkout ($FT_REFERENCE_ROOT) or from where oracle/build_ref.sh placed it next to the compiled reference."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    places = [os.path.join(os.environ.get("FT_REFERENCE_ROOT", ""), "tests", "unittests", "th_op", "test_th_decode_op.py"),
              os.path.join(root, "oracle", "_ref", "th_op", "test_th_decode_op.py")]
    src = next((p for p in places if os.path.isfile(p)), None)
    if src is None:
        pytest.skip("the reference's test file is not at hand: run oracle/build_ref.sh on a FasterTransformer checkout")
    assert os.path.exists(TH_LIB), "lib/libth_ftb200.so is not built: run python -m fastertransformer_b200.build"
    (tmp_path / "lib").mkdir()
    os.symlink(TH_LIB, tmp_path / "lib" / "libth_transformer.so")
    os.symlink(src, tmp_path / "test_th_decode_op.py")
    r = subprocess.run([sys.executable, "-m", "unittest", "-v", "test_th_decode_op"], cwd=tmp_path, capture_output=True,
                       text=True, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "skipped" not in tail and "OK" in tail, tail
    assert all(name in tail for name in ("test_min_length_correctness_at_sampling",
                                         "test_min_length_correctness_at_beamsearch",
                                         "test_repetition_penalty_correctness")), tail
