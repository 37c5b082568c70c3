"""GPU parity of the pieces around the main block tests: MXFP4 experts (fmt 6) through both kernel
families, the reference-named host calls at prefill sizes (tcgen05 path), degenerate inputs
(all-zero FP8 blocks, a row of NaN logits) and two devices in one process."""
import ctypes as C

import numpy as np
import pytest

from speedycolibri_b200 import synth
from speedycolibri_b200.configs import CONFIGS, FMT_FP8_B128, FMT_MXFP4
from tests.helpers import host_layer, rel_l2, upload_layer

pytestmark = pytest.mark.gpu


def make_block(shape, layer, max_tokens=None, **kw):
    from speedycolibri_b200.moe import Config, MoeBlock

    return MoeBlock(Config.from_shape(shape), layer, max_tokens or shape.T, **kw)


def bf16_valued(rng, shape):
    return synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal(shape).astype(np.float32)))


# ---- MXFP4 ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,T", [("tiny_mx", 21), ("tiny_mx", 1), ("mid_mx", 512), ("mid_mx", 77)])
def test_block_mxfp4(gpu_backend, orc, name, T):
    """E2M1 nibbles with an E8M0 scale per 32 (linear.rs:134-175): register-level kernel (tiny) and
    tcgen05 kernels (mid, block magnitudes spread over several binades)."""
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, T)
    out, idx, w = blk.moe(x, want_routing=True)
    blk.check()
    want = L.moe_block(x)
    assert np.array_equal(idx, want["idx"]) and np.array_equal(w.view(np.uint32), want["w"].view(np.uint32))
    err = rel_l2(out, want["out"])
    assert err <= 5e-3, err
    blk.close()


def test_mxfp4_handles_export_and_host_calls(gpu_backend, orc):
    from speedycolibri_b200 import _lib
    from speedycolibri_b200.backend import CudaError, CudaTensor

    shape = CONFIGS["tiny_mx"]
    L, packed = host_layer(shape)
    layer = upload_layer(shape, packed)
    # export returns the container's own bytes (E8M0 scales included) although HBM holds another form
    for e in (0, 5):
        for t, (q, s, g) in zip((layer.experts[e].gate, layer.experts[e].up, layer.experts[e].down), packed["experts"][e]):
            assert t.fmt == FMT_MXFP4
            q2, s2, g2 = t.export()
            assert np.array_equal(q2, q) and np.array_equal(s2, s) and g2 == g
    rng = np.random.default_rng(3)
    for S in (1, 7, 40):  # 40 rows: the tcgen05 path
        x = bf16_valued(rng, (S, shape.H))
        e = layer.experts[2]
        y = gpu_backend.expert_mlp_mxfp4(e.gate, e.up, e.down, x)
        want = L.expert_ffn(2, x)
        assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()
    rows = [5, 1, 12]
    x = bf16_valued(rng, (sum(rows), shape.H))
    es = [layer.experts[i] for i in (1, 4, 7)]
    y = gpu_backend.expert_group_mxfp4([e.gate for e in es], [e.up for e in es], [e.down for e in es], rows, x)
    off = 0
    for ei, r in zip((1, 4, 7), rows):
        want = L.expert_ffn(ei, x[off:off + r])
        assert np.abs(y[off:off + r] - want).max() <= 1e-2 * np.abs(want).max()
        off += r
    # the situ activation is declined, and an NVFP4 tensor is not accepted as MXFP4
    lib = _lib.load()
    e = layer.experts[0]
    yb = np.empty((1, shape.H), np.float32)
    assert lib.coli_cuda_expert_mlp_mxfp4_situ(e.gate.handle, e.up.handle, e.down.handle, yb.ctypes.data, x.ctypes.data, 1,
                                               C.c_float(1.0), C.c_float(0.0)) == 0
    assert b"situ" in lib.coli_cuda_last_error()
    nv = CONFIGS["tiny"]
    _, nv_packed = host_layer(nv)
    q, s, g = nv_packed["experts"][0][0]
    t = CudaTensor.wrap_nvfp4(q, s, g, nv.H, nv.I)
    with pytest.raises(CudaError):
        gpu_backend.expert_mlp_mxfp4(t, t, t, np.zeros((1, nv.H), np.float32))


# ---- reference-named host calls at prefill sizes -----------------------------------------------------------
def test_expert_group_nvfp4_prefill_rows_take_the_tcgen05_path(gpu_backend, orc):
    """rows = [150, 40, 300]: the reference switches kernels above 32 rows (backend_cuda.cu:4738-4783);
    here such a group runs on the tcgen05 kernels (two launches for the whole group)."""
    from speedycolibri_b200 import _lib

    lib = _lib.load()
    shape = CONFIGS["mid"]
    L, packed = host_layer(shape)
    layer = upload_layer(shape, packed)
    rng = np.random.default_rng(21)
    rows, ids = [150, 40, 300], (6, 0, 3)
    x = bf16_valued(rng, (sum(rows), shape.H))
    es = [layer.experts[i] for i in ids]
    before = gpu_backend.group_stats()
    n0 = lib.coli_b200_launch_count()
    y = gpu_backend.expert_group_nvfp4([e.gate for e in es], [e.up for e in es], [e.down for e in es], rows, x)
    assert lib.coli_b200_launch_count() - n0 == 5  # f32->f16, work list, gate+up, down, bf16->f32
    after = gpu_backend.group_stats()
    assert after["calls"] == before["calls"] + 1 and after["rows"] == before["rows"] + sum(rows)
    assert after["experts"] == before["experts"] + 3 and after["kernel_ms"] > before["kernel_ms"]
    off = 0
    for ei, r in zip(ids, rows):
        want = L.expert_ffn(ei, x[off:off + r])
        err = np.linalg.norm(y[off:off + r] - want) / np.linalg.norm(want)
        assert err <= 5e-3, (ei, err)
        assert np.abs(y[off:off + r] - want).max() <= 2e-2 * np.abs(want).max()
        off += r
    # one expert, 200 rows, through the single-expert call
    x1 = bf16_valued(rng, (200, shape.H))
    e = layer.experts[5]
    y1 = gpu_backend.expert_mlp_nvfp4(e.gate, e.up, e.down, x1)
    want = L.expert_ffn(5, x1)
    assert np.linalg.norm(y1 - want) / np.linalg.norm(want) <= 5e-3
    assert gpu_backend.scratch_bytes() > 0


def test_host_calls_take_genuine_f32_activations(gpu_backend, orc):
    """The host-f32 calls round x to f16 (11 significant bits), not to bf16 (8): a one-hot x of
    1 + 2^-9 — exact in f16, rounded to 1.0 by bf16 — must come back as that multiple of the weight
    column; and an expert call on x that is not bf16-representable stays inside the bar."""
    shape = CONFIGS["tiny_sig"]
    L, packed = host_layer(shape)
    q, s, g = packed["experts"][1][0]  # gate of expert 1: [I, H]
    W = orc.dequant(orc.FMT_NVFP4, q, s, g, shape.I, shape.H)
    mm = gpu_backend.Nvfp4Matmul(q, s, g, shape.I, shape.H)
    scale = np.float32(1.0 + 2.0 ** -9)
    x = np.zeros((4, shape.H), np.float32)
    cols = [0, 17, 64, shape.H - 1]
    for r, c in enumerate(cols):
        x[r, c] = scale
    y = mm(x)
    for r, c in enumerate(cols):
        assert np.allclose(y[r], W[:, c] * scale, rtol=1e-6, atol=0.0), (r, c)
        nz = np.abs(W[:, c]) > 0
        assert nz.any() and not np.allclose(y[r][nz], W[:, c][nz], rtol=1e-4, atol=0.0)  # a bf16 rounding would give exactly W
    mm.free()
    layer = upload_layer(shape, packed)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((16, shape.H)).astype(np.float32)
    e = layer.experts[1]
    y = gpu_backend.expert_mlp_nvfp4(e.gate, e.up, e.down, x)
    want = L.expert_ffn(1, x)
    assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 3e-3


# ---- degenerate inputs --------------------------------------------------------------------------------------
@pytest.mark.parametrize("T", [19, 300])
def test_fp8_all_zero_blocks_decode_to_zero(gpu_backend, orc, T):
    """A 128x128 block of zeros has scale amax/448 = 0; code x 0 = 0 in the reference's decoder
    (convert.rs:731-741).  One row block of every expert's gate is zero over all of K, one k-tile of
    a down block is zero: the output must stay finite and equal to the oracle's on both kernel families."""
    shape = CONFIGS["mid_fp8"].with_tokens(T)
    _, packed = host_layer(shape)
    for ex in packed["experts"] + [packed["shared"]]:
        (gq, gs, _), _, (dq, ds, _) = ex
        gq[128:256, :] = 0
        gs[1, :] = 0.0
        dq[0:128, 128:256] = 0
        ds[0, 1] = 0.0
    from oracle.layers import make_layer

    L = make_layer(shape, packed["router"], packed["experts"], packed["shared"], packed["select_bias"], packed["logit_bias"])
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, T)
    out = blk.moe(x)
    blk.check()
    got = synth.bf16_bits_to_f32(out)
    assert np.isfinite(got).all()
    assert rel_l2(out, L.moe_block(x)["out"]) <= 5e-3
    blk.close()


def test_nan_logits_row_repeats_expert_zero_and_keeps_rows_apart(gpu_backend, orc):
    """A token whose activations are NaN gets NaN logits; the reference's scan then picks expert 0 in
    every round (moe.rs:1075-1088).  The k pairs of that token all land in expert 0's segment: each
    must get a row of its own, and the other tokens' outputs must be untouched."""
    shape = CONFIGS["tiny"].with_tokens(9)
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, 9)
    clean = blk.moe(x)
    xn = x.copy()
    xn[4, :] = 0x7FC0  # bf16 NaN
    out, idx, _ = blk.moe(xn, want_routing=True)
    blk.check()
    assert np.all(idx[4] == 0)
    want_idx, _ = L.route_tokens(xn)
    assert np.array_equal(idx, want_idx)
    keep = [t for t in range(9) if t != 4]
    assert np.array_equal(out[keep], clean[keep])
    blk.close()


def test_two_devices_in_one_process():
    """Kernel attributes belong to a device: a process that drives two GPUs must be able to run the
    large-shared-memory kernels (tcgen05 experts, decode front end) on both."""
    import subprocess
    import sys
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    code = r"""
import numpy as np
from speedycolibri_b200 import backend, synth
from speedycolibri_b200.configs import CONFIGS
from speedycolibri_b200.moe import Config, MoeBlock
from oracle.layers import host_layer, rel_l2
backend.init([0, 1])
for name, T in (("mid", 300), ("tiny_sig", 5)):
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    x = synth.host_tokens(shape, T)
    want = L.moe_block(x)["out"]
    for dev in (0, 1):
        blk = MoeBlock(Config.from_shape(shape), synth.upload_packed_layer(shape, packed, device=dev), T, device=dev)
        err = rel_l2(blk.moe(x), want)
        assert err <= 5e-3, (name, dev, err)
        blk.close()
print("TWO_DEVICES_OK")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert "TWO_DEVICES_OK" in r.stdout, r.stdout + r.stderr
