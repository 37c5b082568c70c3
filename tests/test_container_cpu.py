"""Container format of block-scaled FP4 experts (host logic only): names, blob split, sidecars, refusals."""
import numpy as np
import pytest

from speedycolibri_b200 import container
from speedycolibri_b200.configs import CONFIGS
from tests.helpers import host_packed_expert


def test_weight_name_matches_the_loader():
    # crates/colibri-engine/src/moe.rs:331-336
    assert container.weight_name(3, 17, "gate_proj") == "model.layers.3.mlp.experts.17.gate_proj.weight"
    assert container.weight_name(0, 2, "down_proj", prefix="block_sparse_moe") == \
        "model.layers.0.block_sparse_moe.experts.2.down_proj.weight"


def test_roundtrip_two_shards(tmp_path, orc):
    shape = CONFIGS["tiny"]
    packed = {e: host_packed_expert(shape, e) for e in range(3)}
    a, b = {}, {}
    for e, p in packed.items():
        (a if e < 2 else b).update(container.expert_tensors(5, e, p))
    a["model.layers.5.mlp.gate.weight"] = np.arange(12, dtype=np.uint16).reshape(3, 4)  # an unrelated bf16 tensor
    container.write_safetensors(str(tmp_path / "model-00001.safetensors"), a)
    container.write_safetensors(str(tmp_path / "model-00002.safetensors"), b)
    sh = container.Shards(str(tmp_path))
    assert sh.has("model.layers.5.mlp.experts.2.up_proj.weight.g")
    assert np.array_equal(sh.read("model.layers.5.mlp.gate.weight"), a["model.layers.5.mlp.gate.weight"])
    for e, p in packed.items():
        fmt, got = container.read_expert(sh, 5, e, shape.H, shape.I)
        assert fmt == 5
        for (nib, bs, g), (wn, wb, wg) in zip(got, p):
            assert np.array_equal(nib, wn) and np.array_equal(bs, wb) and g == np.float32(wg)
    # the blob is nibbles then scales, in that order (moe.rs:793-812)
    blob = sh.read(container.weight_name(5, 0, "gate_proj"))
    nb = shape.I * ((shape.H + 1) // 2)
    assert np.array_equal(blob[:nb].reshape(shape.I, -1), packed[0][0][0])


def test_refusals(tmp_path, orc):
    shape = CONFIGS["tiny"]
    t = container.expert_tensors(0, 0, host_packed_expert(shape, 0))
    name = container.weight_name(0, 0, "up_proj")
    mx = dict(t)
    mx[name + ".mx"] = mx.pop(name + ".g")  # one projection marked MXFP4: its blob has NVFP4's scale count
    container.write_safetensors(str(tmp_path / "mx.safetensors"), mx)
    with pytest.raises(ValueError, match="does not match MXFP4"):
        container.read_expert(container.Shards(str(tmp_path / "mx.safetensors")), 0, 0, shape.H, shape.I)
    qs = {k: v for k, v in t.items() if not k.endswith(".g")}
    qs[name + ".qs"] = np.ones(4, np.float32)
    container.write_safetensors(str(tmp_path / "qs.safetensors"), qs)
    with pytest.raises(ValueError, match="no block-scaled FP4 sidecar"):
        container.read_expert(container.Shards(str(tmp_path / "qs.safetensors")), 0, 0, shape.H, shape.I)
    container.write_safetensors(str(tmp_path / "ok.safetensors"), t)
    sh = container.Shards(str(tmp_path / "ok.safetensors"))
    with pytest.raises(ValueError, match="does not match"):
        container.read_expert(sh, 0, 0, shape.H + 16, shape.I)  # wrong shape for the blob
    with pytest.raises(KeyError):
        sh.read("model.layers.9.mlp.experts.0.gate_proj.weight")
    with pytest.raises(ValueError):
        container.split_nvfp4_blob(np.zeros(7, np.uint8), 2, 16)


def test_mxfp4_expert_loads_as_fmt6_with_the_right_block_stride(tmp_path):
    """crates/colibri-engine/src/moe.rs:3468-3560: nibbles ++ E8M0 scales with an `.mx` sidecar of 1.0
    load as fmt 6 with O*I/32 scale bytes (NVFP4's stride of 16 would give twice as many)."""
    O = I = 64  # square, so gate, up and down share one blob shape; 2 MXFP4 blocks per row
    nib_bytes, bs_bytes = O * I // 2, O * I // 32
    blob = np.empty(nib_bytes + bs_bytes, np.uint8)
    blob[:nib_bytes] = (np.arange(nib_bytes) * 7 + 3) % 256
    blob[nib_bytes:] = 127  # 2^0
    t = {}
    for proj in container.PROJS:
        name = container.weight_name(0, 0, proj)
        t[name] = blob.copy()
        t[name + ".mx"] = np.array([1.0], np.float32)
    container.write_safetensors(str(tmp_path / "model.safetensors"), t)
    sh = container.Shards(str(tmp_path))
    assert container.fp4_sidecar(sh, container.weight_name(0, 0, "up_proj")) == (container.weight_name(0, 0, "up_proj") + ".mx", 6, 32)
    fmt, packed = container.read_expert(sh, 0, 0, I, O)
    assert fmt == 6
    for nib, bs, g in packed:
        assert nib.size == nib_bytes and bs.size == bs_bytes and g == 1.0
        assert np.array_equal(nib.reshape(-1), blob[:nib_bytes]) and np.all(bs == 127)
    # what the writer emits for an MXFP4 expert is what the reader looks up
    again = container.expert_tensors(0, 0, packed, fmt=6)
    assert set(again) == set(t) and all(np.array_equal(again[k], t[k]) for k in t)
