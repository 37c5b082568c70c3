"""Container -> HBM loader for NVFP4 expert weights.

Mirrors how the reference's loader finds and splits an expert's tensors
(crates/colibri-engine/src/moe.rs:326-360 names and sidecars, 770-815 the blob split):

* one U8 tensor per projection, named ``model.layers.{L}.{prefix}.experts.{E}.{proj}.weight`` with
  proj in gate_proj / up_proj / down_proj, holding ``nibbles ++ block scales``:
  ``O * ceil(I/2)`` bytes of E2M1 pairs (low nibble = even column) followed by
  ``O * ceil(I/16)`` ue4m3 block-scale bytes;
* an F32 sidecar of one element, ``<name>.g``, the per-tensor scale (its presence marks NVFP4;
  ``.mx`` would mark MXFP4, which is not a resident format of this library).

The files are safetensors shards: an 8-byte little-endian header length, a JSON header mapping
tensor names to ``{"dtype", "shape", "data_offsets"}``, then the raw bytes.  Only what the expert
path needs is implemented: U8 / F32 / BF16 tensors, reading by name, and a writer so that tests
and tools can produce a container without any third-party package.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

import numpy as np

PROJS = ("gate_proj", "up_proj", "down_proj")
_DTYPES = {"U8": np.uint8, "F32": np.float32, "BF16": np.uint16, "I32": np.int32}


def weight_name(layer: int, eid, proj: str, prefix: str = "mlp") -> str:
    """moe.rs:331-336; ``eid`` may be an expert id or ``"shared"`` style suffix given by the caller."""
    return f"model.layers.{layer}.{prefix}.experts.{eid}.{proj}.weight"


def write_safetensors(path: str, tensors: dict) -> None:
    """tensors: name -> numpy array (uint8 / float32 / uint16 holding bf16 bits / int32)."""
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        code = next(k for k, v in _DTYPES.items() if v == arr.dtype.type)
        raw = arr.tobytes()
        header[name] = {"dtype": code, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


@dataclass
class _Entry:
    path: str
    dtype: str
    shape: tuple
    begin: int
    end: int


class Shards:
    """Index over one or more safetensors files (a directory of ``*.safetensors`` or explicit paths)."""

    def __init__(self, paths):
        if isinstance(paths, str):
            if os.path.isdir(paths):
                paths = sorted(os.path.join(paths, f) for f in os.listdir(paths) if f.endswith(".safetensors"))
            else:
                paths = [paths]
        self.index: dict[str, _Entry] = {}
        for p in paths:
            with open(p, "rb") as f:
                (n,) = struct.unpack("<Q", f.read(8))
                header = json.loads(f.read(n))
            base = 8 + n
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                b, e = meta["data_offsets"]
                self.index[name] = _Entry(p, meta["dtype"], tuple(meta["shape"]), base + b, base + e)

    def has(self, name: str) -> bool:
        return name in self.index

    def read(self, name: str) -> np.ndarray:
        ent = self.index.get(name)
        if ent is None:
            raise KeyError(f"tensor {name!r} is not in the container")
        if ent.dtype not in _DTYPES:
            raise ValueError(f"tensor {name!r} has unsupported dtype {ent.dtype}")
        with open(ent.path, "rb") as f:
            f.seek(ent.begin)
            raw = f.read(ent.end - ent.begin)
        return np.frombuffer(raw, dtype=_DTYPES[ent.dtype]).reshape(ent.shape)


def split_nvfp4_blob(blob: np.ndarray, O: int, I: int):
    """``nibbles ++ block scales`` -> (nibbles [O, ceil(I/2)], scales [O, ceil(I/16)]); moe.rs:793-812."""
    nib_bytes, bs_bytes = O * ((I + 1) // 2), O * ((I + 15) // 16)
    blob = np.ascontiguousarray(blob, dtype=np.uint8).reshape(-1)
    if blob.size != nib_bytes + bs_bytes:
        raise ValueError(f"blob of {blob.size} bytes does not match [O={O}, I={I}]: want {nib_bytes} + {bs_bytes}")
    return blob[:nib_bytes].reshape(O, (I + 1) // 2), blob[nib_bytes:].reshape(O, (I + 15) // 16)


def read_expert(shards: Shards, layer: int, eid, H: int, I: int, prefix: str = "mlp"):
    """One expert as ((nib, bs, g) for gate [I,H], up [I,H], down [H,I]).  A missing ``.g`` sidecar
    means the expert is not NVFP4 and is refused (``.mx`` = MXFP4, ``.qs`` = int / e4m3 rows)."""
    out = []
    for proj, (O, K) in zip(PROJS, ((I, H), (I, H), (H, I))):
        name = weight_name(layer, eid, proj, prefix)
        if not shards.has(name + ".g"):
            other = [s for s in (".mx", ".qs") if shards.has(name + s)]
            raise ValueError(f"{name}: no NVFP4 sidecar (.g)" + (f"; found {other[0]}, which is not a resident format" if other else ""))
        nib, bs = split_nvfp4_blob(shards.read(name), O, K)
        g = float(shards.read(name + ".g").reshape(-1)[0])
        out.append((nib, bs, g))
    return tuple(out)


def expert_tensors(layer: int, eid, packed, prefix: str = "mlp") -> dict:
    """The container entries of one expert given its (nib, bs, g) triples: what convert writes."""
    t = {}
    for proj, (nib, bs, g) in zip(PROJS, packed):
        name = weight_name(layer, eid, proj, prefix)
        t[name] = np.concatenate([np.ascontiguousarray(nib, np.uint8).reshape(-1), np.ascontiguousarray(bs, np.uint8).reshape(-1)])
        t[name + ".g"] = np.array([g], np.float32)
    return t


def load_layer(shards: Shards, layer: int, H: int, I: int, E: int, device: int = 0, shared_id=None, prefix: str = "mlp",
               local=None):
    """Upload the experts of one layer into HBM: a speedycolibri_b200.moe.Layer-compatible list of
    resident handles.  ``local``: ids to load (expert parallelism), default all."""
    from .backend import CudaTensor
    from .configs import FMT_NVFP4
    from .moe import Expert

    def up(packed):
        ts = []
        for (nib, bs, g), (O, K) in zip(packed, ((I, H), (I, H), (H, I))):
            ts.append(CudaTensor.wrap_nvfp4(nib, bs, g, K, O, device))
        return Expert(*ts)

    experts = [up(read_expert(shards, layer, e, H, I, prefix)) if (local is None or e in local) else None for e in range(E)]
    shared = up(read_expert(shards, layer, shared_id, H, I, prefix)) if shared_id is not None else None
    return experts, shared, FMT_NVFP4
