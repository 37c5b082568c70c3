"""Container format of NVFP4 experts (host logic only): names, blob split, sidecars, refusals."""
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
        got = container.read_expert(sh, 5, e, shape.H, shape.I)
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
    mx[name + ".mx"] = mx.pop(name + ".g")  # MXFP4 marker instead of NVFP4
    container.write_safetensors(str(tmp_path / "mx.safetensors"), mx)
    with pytest.raises(ValueError, match="not a resident format"):
        container.read_expert(container.Shards(str(tmp_path / "mx.safetensors")), 0, 0, shape.H, shape.I)
    container.write_safetensors(str(tmp_path / "ok.safetensors"), t)
    sh = container.Shards(str(tmp_path / "ok.safetensors"))
    with pytest.raises(ValueError, match="does not match"):
        container.read_expert(sh, 0, 0, shape.H + 16, shape.I)  # wrong shape for the blob
    with pytest.raises(KeyError):
        sh.read("model.layers.9.mlp.experts.0.gate_proj.weight")
    with pytest.raises(ValueError):
        container.split_nvfp4_blob(np.zeros(7, np.uint8), 2, 16)
