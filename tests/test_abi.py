"""The C-ABI library loads without a GPU and exports every function the public header declares."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mggb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mggb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from mgg_osdi23_b200._lib import lib, SIGNATURES
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mggb200.h but not exported"
    # every bound signature is declared, and the other way round (except the two non-status queries)
    assert set(SIGNATURES) | {"mggb_version", "mggb_last_error"} == set(names)


def test_version_and_error_string():
    from mgg_osdi23_b200._lib import lib
    assert lib.mggb_version() >= 100
    assert isinstance(lib.mggb_last_error(), bytes)


def test_compute_entry_points_validate_before_touching_the_gpu():
    """Bad arguments are rejected on the host (no CUDA call is made, so this runs without a GPU)."""
    from mgg_osdi23_b200._lib import lib, ERR_INVALID_ARG
    assert lib.mggb_dense_forward(None, None, None, 4, 4, 4, None, 0, None, 0, None) == ERR_INVALID_ARG
    assert lib.mggb_softmax_forward(None, None, 4, 4, None) == ERR_INVALID_ARG
    assert lib.mggb_row_scale(None, None, None, 4, 4, None) == ERR_INVALID_ARG
    table = (C.c_void_p * 1)(0)
    assert lib.mggb_sag_np_div(None, table, 1, None, None, None, None, 0, 4, 16, 4, 0, 16, 4, 1, None, 0, None, 0, None) == ERR_INVALID_ARG
    one = C.c_void_p(16)
    table = (C.c_void_p * 1)(16)
    # knob validation: warp_per_block out of range, zero part size, too many PEs
    for ps, wpb, dist, npes in ((16, 0, 1, 1), (16, 17, 1, 1), (0, 4, 1, 1), (16, 4, 0, 1), (16, 4, 1, 17)):
        st = lib.mggb_sag_np_div(one, table, npes, one, one, one, one, 0, 4, 16, 4, 0, ps, wpb, dist, None, 0, None, 0, None)
        assert st == ERR_INVALID_ARG, (ps, wpb, dist, npes)
    # GIN output must not alias the PE's own input
    st = lib.mggb_gin_np_div(one, table, 1, one, one, one, one, 0, 4, 16, 4, 0, 16, 4, 1, 0.0, 0, None)
    assert st == ERR_INVALID_ARG and b"alias" in lib.mggb_last_error()


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    """Without the built library the package refuses to import (there is no fallback path)."""
    import importlib
    import mgg_osdi23_b200._lib as real
    monkeypatch.setattr(real, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        real._load()
    except ImportError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("expected ImportError")
