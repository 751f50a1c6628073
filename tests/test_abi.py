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


def test_flag_constants_match_the_header():
    """The Python constants are the header's enumerators (a mismatch would silently select another kernel)."""
    from mgg_osdi23_b200 import _lib
    text = open(os.path.join(ROOT, "include", "mggb200.h")).read()
    enums = {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(MGGB_[A-Z0-9_]+)\s*=\s*(-?\d+)", text)}
    for name in ("AGG_ACCUMULATE", "AGG_NO_HUB_SPLIT", "AGG_GROUP_PER_NODE", "AGG_STAGE_ROWS", "AGG_GIN_COMBINE", "AGG_NO_REMOTE",
                 "DENSE_RELU", "DENSE_TF32", "DENSE_SIMT", "DENSE_TENSOR"):
        assert "MGGB_" + name in enums, name
        assert getattr(_lib, name) == enums["MGGB_" + name], name
    flags = [enums[k] for k in enums if k.startswith("MGGB_AGG_")]
    assert len(set(flags)) == len(flags) and all(f & (f - 1) == 0 for f in flags)      # distinct single bits


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


def test_hub_threshold_follows_the_documented_rule():
    """max(16384, 64*ps*dist*wpb) for the block-per-node kernels, 1024 for the group-per-node kernel at
    dim 16, -1 (no hub list) for wide blocks, the no-split flag, or rows too wide for the 16-warp block."""
    from mgg_osdi23_b200 import api, _lib
    assert api.hub_threshold(16, 4, 1, 16) == 16384
    assert api.hub_threshold(32, 4, 2, 16) == 64 * 64 * 4
    assert api.hub_threshold(32, 8, 16, 64) == 64 * 512 * 8
    assert api.hub_threshold(16, 16, 1, 16) == -1
    assert api.hub_threshold(16, 4, 1, 16, _lib.AGG_NO_HUB_SPLIT) == -1
    assert api.hub_threshold(16, 4, 1, 16, _lib.AGG_GROUP_PER_NODE) == 1024
    assert api.hub_threshold(16, 4, 1, 64, _lib.AGG_GROUP_PER_NODE) == 16384
    assert api.hub_threshold(16, 4, 1, 4000) == -1
    assert api.hub_threshold(1 << 20, 8, 1 << 10, 16) == 64 * (1 << 24) * 8          # computed in 64 bits


def test_shard_tells_the_aggregation_when_it_has_no_hub_rows():
    import numpy as np
    from mgg_osdi23_b200 import drivers, _lib
    rp = np.array([0, 3, 5, 40000], np.int32)
    col = np.zeros(40000, np.int32)
    sh = drivers.Shard(rp, col, 0, 1, device="cpu")
    assert sh.max_degree == 39995
    assert sh.agg_flags(drivers.Knobs(16, 4, 1), 16) == 0                                 # a row above 16384: keep the hub kernel
    assert sh.agg_flags(drivers.Knobs(32, 8, 8), 16) == _lib.AGG_NO_HUB_SPLIT             # threshold 131072: nothing reaches it
    assert sh.agg_flags(drivers.Knobs(16, 4, 1, _lib.AGG_GROUP_PER_NODE), 16) == _lib.AGG_GROUP_PER_NODE
