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
    """ColiMoeLayer: 11 ints/floats, padding to 8, 9 pointers, 2 ints, 2 pointers."""
    from speedycolibri_b200 import _lib

    assert C.sizeof(_lib.ColiMoeLayer) == 48 + 9 * 8 + 8 + 8 + 8
    assert _lib.ColiMoeLayer.nccl_comm.offset == 48 + 72 + 16
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


def test_init_refuses_a_repeated_ordinal():
    """crates/colibri-backend/cuda/backend_cuda.cu:2636-2640: a device listed twice is refused before
    anything is created (checked ahead of the device query, so it answers the same without a GPU)."""
    from speedycolibri_b200 import _lib

    lib = _lib.load()
    devs = (C.c_int * 2)(0, 0)
    assert lib.coli_cuda_init(devs, 2) == 0
    assert b"listed twice" in lib.coli_cuda_last_error()


def test_b200_answers_of_the_residency_calls():
    """The symbols the engine's expert dispatch links against besides the compute calls
    (crates/colibri-backend/src/cuda.rs:78-82,393): no pageable access, switches without effect."""
    from speedycolibri_b200 import _lib

    lib = _lib.load()
    assert lib.coli_cuda_pageable_access(0) == 0
    lib.coli_cuda_set_weight_zerocopy(1)
    lib.coli_cuda_set_ffn_devcopy(0)
    assert lib.coli_cuda_scratch_bytes(-1) == 0  # nothing initialised, nothing reserved
    vals = [C.c_uint64(7) for _ in range(3)] + [C.c_double(7.0) for _ in range(3)]
    lib.coli_cuda_group_stats(*[C.byref(v) for v in vals])
    assert [v.value for v in vals] == [0, 0, 0, 0.0, 0.0, 0.0]


def test_mxfp4_resident_scales_decode_to_the_same_weights(orc):
    """An MXFP4 matrix is held in the NVFP4 resident form.  E2M1 x 2^e x g (linear.rs:134-175, the
    oracle's fmt-6 arm) must equal E2M1 x ue4m3(code) x g' for every weight: the scales spread over
    15 binades, a zero block with a huge scale byte is ignored when the shift is chosen, a NaN byte
    stays NaN, and a block more than 17 binades below the largest decodes as zero."""
    from speedycolibri_b200 import _lib

    lib = _lib.load()
    rng = np.random.default_rng(11)
    O, I = 12, 160  # 5 blocks of 32 per row
    nib = rng.integers(0, 256, (O, I // 2), dtype=np.uint8)
    bs = rng.integers(100, 116, (O, I // 32), dtype=np.uint8)
    nib[3, 16:32] = 0x80  # block (3, 1): only -0.0 / +0.0 nibbles ...
    bs[3, 1] = 250        # ... under an enormous scale: must not set the shift
    bs16 = np.zeros((O, I // 16), np.uint8)
    g2 = C.c_float()
    assert lib.coli_b200_mxfp4_resident_scales(nib.ctypes.data, bs.ctypes.data, C.c_float(1.0), I, O, bs16.ctypes.data, C.byref(g2)) == 1
    want = orc.dequant(orc.FMT_MXFP4, nib, bs, 1.0, O, I)
    got = orc.dequant(orc.FMT_NVFP4, nib, bs16, g2.value, O, I)
    assert np.array_equal(want.view(np.uint32) & 0x7FFFFFFF, got.view(np.uint32) & 0x7FFFFFFF)  # bit-equal magnitudes
    assert np.array_equal(np.signbit(want), np.signbit(got))
    assert np.all(bs16[:, 0::2] == bs16[:, 1::2])  # both halves of a 32-block share its scale
    # out-of-range and NaN blocks
    bs2 = bs.copy()
    bs2[0, 0] = 60    # 2^-67: far more than 17 binades below the largest block
    bs2[1, 2] = 0xFF  # NaN
    assert lib.coli_b200_mxfp4_resident_scales(nib.ctypes.data, bs2.ctypes.data, C.c_float(1.0), I, O, bs16.ctypes.data, C.byref(g2)) == 1
    got = orc.dequant(orc.FMT_NVFP4, nib, bs16, g2.value, O, I)
    assert np.all(got[0, :32] == 0.0)
    # 0x7F is the NaN code of the hardware's e4m3 -> f16 conversion (the reference's CPU decoder of
    # linear.rs:188-197 has no NaN case, so the oracle cannot show it)
    assert np.all(bs16[1, 4:6] == 0x7F)
    keep = np.ones((O, I), bool)
    keep[0, :32] = False
    keep[1, 64:96] = False
    assert np.array_equal(np.abs(want)[keep], np.abs(got)[keep])
