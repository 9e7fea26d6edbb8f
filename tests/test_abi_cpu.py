"""The C-ABI library loads without a GPU and exports every function include/ftb200.h declares.
No kernel is launched here; argument checks that need no device are exercised."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "ftb200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ftb200_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from fastertransformer_b200 import lib
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), "libftb200.so does not export " + n


def test_version_and_error_string():
    from fastertransformer_b200 import lib
    assert b"sm_100a" in lib.ftb200_version()
    assert lib.ftb200_last_error_string() is not None


def test_argument_checks_need_no_device():
    from fastertransformer_b200 import SamplingParams, lib
    assert lib.ftb200_decode_step_sampling(None) == 1                      # FTB200_INVALID_ARG
    P = SamplingParams()
    assert lib.ftb200_decode_step_sampling(C.byref(P)) == 1
    assert b"null" in lib.ftb200_last_error_string()
    n = C.c_size_t(0)
    assert lib.ftb200_sampling_workspace_bytes(7, 1, 8, C.byref(n)) == 1   # bad dtype
    assert lib.ftb200_curand_init(None, 4, 0, None, None) == 1
    assert lib.ftb200_stop_criteria(None, None, None, 0, None, None, 0, 0, 0, 1, 0, None, None, None) == 1


def test_struct_layout_matches_header():
    """Field order of the ctypes mirror follows the header (names in declaration order)."""
    from fastertransformer_b200._abi import SamplingParams
    src = open(os.path.join(ROOT, "include", "ftb200.h")).read()
    body = src[src.index("typedef struct ftb200_sampling_params {"):src.index("} ftb200_sampling_params;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"(\w+)\s*;", body)
    assert fields == [f[0] for f in SamplingParams._fields_]
