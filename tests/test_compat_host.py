"""The C++ shim's host half (split_CSR<int>, build_part<int>) compiled and run without a GPU."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import mgg_osdi23_b200 as mgg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _arrays(stdout):
    out = {}
    for line in stdout.splitlines():
        parts = line.split()
        if parts and parts[0].split("_")[0] in ("split", "part", "lcg"):
            out[parts[0]] = np.array([int(x) for x in parts[1:]], dtype=np.int32)
    return out


def test_cpp_shim_partitioner_matches_the_python_api_and_the_known_answers(tmp_path, oracle):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    exe = str(tmp_path / "compat_host_check")
    pkg = os.path.join(ROOT, "mgg_osdi23_b200")
    cmd = [nvcc, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "compat_host_check.cu"),
           "-o", exe, "-L", pkg, "-lmggb200", "-Xlinker", "-rpath", "-Xlinker", pkg]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    a = _arrays(r.stdout)

    # known answers (outputs of the reference's own host functions on these inputs)
    assert a["split_small_local_ptr"].tolist() == [0, 1, 2] and a["split_small_remote_ptr"].tolist() == [0, 1, 1]
    assert a["split_small_local_col"].tolist() == [1, 0] and a["split_small_remote_col"].tolist() == [2]
    assert a["part_small_partPtr"].tolist() == [0, 2, 3, 5, 6] and a["part_small_part2Node"].tolist() == [0, 0, 1, 2]
    assert a["part_small_node2Part"].tolist() == [0, 2, 3, 4, 4]
    assert a["part_corner_partPtr"].tolist() == [0, 2, 3, 0]            # the sentinel the reference leaves at 0
    assert a["part_corner_part2Node"].tolist() == [0, 0, 1] and a["part_corner_node2Part"].tolist() == [0, 2, 3, 3, 3]
    # the reference's one summary line per build_part call
    assert "part, num_nodes: 3, part_size, 2, num_parts, 4" in r.stdout

    # the seeded graph: same arrays as the Python API and the oracle give
    ptr, col = a["lcg_ptr"], a["lcg_col"]
    assert len(ptr) == 61 and ptr[-1] == len(col)
    for got, want, orc in zip(("local_ptr", "remote_ptr", "local_col", "remote_col"), mgg.split_CSR(ptr, col, 20, 40),
                              oracle.split_csr(ptr, col, 20, 40)):
        assert np.array_equal(a["split_lcg_" + got], want) and np.array_equal(want, orc)
    for got, want, orc in zip(("partPtr", "part2Node", "node2Part"), mgg.build_part("lcg", ptr, 60, 4), oracle.build_part(ptr, 60, 4)):
        assert np.array_equal(a["part_lcg_" + got], want) and np.array_equal(want, orc)
