"""Host-side checks of bench.py that need no GPU."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_traffic_figures_belong_to_the_committed_kernel_sources():
    """Every ncu traffic figure is stamped with the hash of the kernel source it was captured from;
    a figure whose source has changed since would be printed as null."""
    assert bench.NCU_TRAFFIC, "no traffic figures"
    for (workload, tokens, kernel), (nbytes, source, src_file, stamp) in bench.NCU_TRAFFIC.items():
        assert bench.file_stamp(src_file) == stamp, f"{workload}/{kernel}: {src_file} changed since the capture in {source}"
        assert os.path.exists(os.path.join(ROOT, source.split(" ")[0])), source
        got, _ = bench.ncu_traffic(workload, tokens, kernel)
        assert got == nbytes > 0


def test_workload_names_resolve():
    for name, T in (("c0", 128), ("c1_t1", 1), ("c1_t4", 4), ("c1_t8", 8), ("c2", 512), ("c3", 4096), ("c4", 16384), ("c3s", 512), ("c4s", 2048)):
        assert bench.shape_named(name).T == T
    assert bench.shape_named("c3", 77).T == 77


def test_c3_traffic_is_the_small_case_times_eight():
    for kernel in ("gate_up", "down"):
        small, _ = bench.ncu_traffic("c3s", 512, kernel)
        full, src = bench.ncu_traffic("c3", 4096, kernel)
        assert full == 8 * small and "x 8" in src
