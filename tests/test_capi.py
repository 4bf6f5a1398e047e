"""The C-ABI library loads and exports every function that include/aprnet_b200.h declares, and the
argument checks that need no GPU answer with a status code instead of crashing."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "aprnet_b200.h")
LIB = os.path.join(ROOT, "apr-cnn_b200", "libaprnet_b200.so")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aprnet_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_set():
    names = declared_functions()
    for must in ("aprnet_apr_create", "aprnet_conv333_forward", "aprnet_conv333_backward_input",
                 "aprnet_conv333_backward_weights", "aprnet_conv111_forward", "aprnet_maxpool_forward",
                 "aprnet_upsample_forward", "aprnet_fill_tree_mean_forward", "aprnet_fill_tree_max",
                 "aprnet_restrict333_forward"):
        assert must in names
    assert len(names) >= 30


def test_library_exports_every_declared_symbol():
    assert os.path.isfile(LIB), "build the library first: python apr-cnn_b200/build.py"
    lib = C.CDLL(LIB)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_argument_errors_are_status_codes():
    lib = C.CDLL(LIB)
    lib.aprnet_last_error.restype = C.c_char_p
    lib.aprnet_number_parts.restype = C.c_int64
    assert lib.aprnet_number_parts(None, 0) == -1
    rc = lib.aprnet_restrict333_forward(0, 3, 2, C.c_int64(4), None, None, None)       # num_levels < num_stencils
    assert rc == -1 and b"num_levels" in lib.aprnet_last_error()
    rc = lib.aprnet_conv111_forward(None, 0, 0, 1, 1, 1, None, C.c_int64(0), None, None, C.c_int64(0), None)
    assert rc == -1
    assert lib.aprnet_conv333_partial_elems(32, 32) >= 27 * 32 * 32 * 4
