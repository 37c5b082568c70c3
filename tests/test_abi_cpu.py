"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU, exports
every symbol include/coli_b200.h declares, and fails loudly (no fallback) when asked to compute."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "coli_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(coli_(?:cuda|b200)_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_all_exported_and_bound():
    from speedycolibri_b200 import _lib

    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"libcoli_b200.so does not export {n}"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"


def test_struct_layout_matches_header():
    """ColiMoeLayer: 11 ints/floats, padding to 8, 9 pointers, 2 ints, padding, 1 pointer."""
    from speedycolibri_b200 import _lib

    assert C.sizeof(_lib.ColiMoeLayer) == 48 + 9 * 8 + 8 + 8
    assert _lib.ColiMoeLayer.router_w.offset == 48
    assert _lib.ColiMoeLayer.ep_rank.offset == 48 + 72
    assert _lib.ColiMoeLayer.expert_owner.offset == 48 + 72 + 8


def test_no_gpu_means_error_not_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from speedycolibri_b200 import backend

    with pytest.raises(backend.CudaError):
        backend.init([0])
    assert backend.device_count() == 0
    x = np.zeros((1, 64), np.float32)
    with pytest.raises(backend.CudaError, match="not initialised"):
        backend.F32Matmul(np.zeros((4, 64), np.float32))(x)


def test_fingerprint_matches_reference_formula():
    """FNV-1a over (nodes, experts, owners) — crates/colibri-cluster/src/sharding.rs:251-265 —
    in the C library, in the Python mirror and in the oracle."""
    from oracle import oracle
    from speedycolibri_b200 import backend
    from speedycolibri_b200.cluster import ExpertSharding

    for nodes, E in [(1, 4), (2, 32), (8, 256), (3, 10)]:
        sh = ExpertSharding.new(nodes, E)
        assert sh.fingerprint() == backend.sharding_fingerprint(nodes, E)
        assert sh.fingerprint() == oracle.lib().orc_sharding_fingerprint(nodes, E, None)
    bal = ExpertSharding.balanced(4, 16, [16 - e for e in range(16)])
    assert bal.fingerprint() == backend.sharding_fingerprint(4, 16, bal.owner_table())
    assert bal.fingerprint() != ExpertSharding.new(4, 16).fingerprint()


def test_shape_work_figures():
    """The per-config byte and flop figures used for the roofline (quant.rs:762-766 for bytes)."""
    from speedycolibri_b200.configs import CONFIGS

    c1 = CONFIGS["c1"]
    assert c1.matrix_bytes(768, 2048) == 768 * 1024 + 768 * 128 + 4
    assert abs(c1.expert_bytes() / 1e6 - 2.654) < 0.01
    c3 = CONFIGS["c3"]
    assert abs(c3.expert_bytes() / 1e6 - 24.77) < 0.01
    assert abs(c3.flops() / 1e9 - 3262) < 5
    c2 = CONFIGS["c2"]
    assert abs(c2.expert_bytes() / 1e6 - 4.72) < 0.01
