"""Container -> HBM loader for block-scaled FP4 expert weights (NVFP4 and MXFP4).

Mirrors how the reference's loader finds and splits an expert's tensors
(crates/colibri-engine/src/moe.rs:326-360 names and sidecars, 770-815 the blob split):

* one U8 tensor per projection, named ``model.layers.{L}.{prefix}.experts.{E}.{proj}.weight`` with
  proj in gate_proj / up_proj / down_proj, holding ``nibbles ++ block scales``:
  ``O * ceil(I/2)`` bytes of E2M1 pairs (low nibble = even column) followed by
  ``O * ceil(I/16)`` ue4m3 block-scale bytes;
* an F32 sidecar of one element that names the format (moe.rs:338-360 ``fp4_sidecar``):
  ``<name>.g`` = NVFP4, the per-tensor scale; ``<name>.mx`` = MXFP4, whose block scales are
  ``O * ceil(I/32)`` OCP E8M0 bytes and whose sidecar holds the identity scale 1.0.

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


def split_mxfp4_blob(blob: np.ndarray, O: int, I: int):
    """``nibbles ++ E8M0 block scales`` -> (nibbles [O, ceil(I/2)], scales [O, ceil(I/32)]); the block
    stride is 32, half as many scale bytes as NVFP4 (moe.rs:3468-3560)."""
    nib_bytes, bs_bytes = O * ((I + 1) // 2), O * ((I + 31) // 32)
    blob = np.ascontiguousarray(blob, dtype=np.uint8).reshape(-1)
    if blob.size != nib_bytes + bs_bytes:
        raise ValueError(f"blob of {blob.size} bytes does not match MXFP4 [O={O}, I={I}]: want {nib_bytes} + {bs_bytes}")
    return blob[:nib_bytes].reshape(O, (I + 1) // 2), blob[nib_bytes:].reshape(O, (I + 31) // 32)


def fp4_sidecar(shards: Shards, base: str):
    """(sidecar name, fmt code, block size) of the block-scaled FP4 tensor `base`, or None — moe.rs:349-360."""
    if shards.has(base + ".g"):
        return base + ".g", 5, 16
    if shards.has(base + ".mx"):
        return base + ".mx", 6, 32
    return None


def read_expert(shards: Shards, layer: int, eid, H: int, I: int, prefix: str = "mlp"):
    """One expert as (fmt, ((nib, bs, g) for gate [I,H], up [I,H], down [H,I])), fmt 5 (NVFP4, ``.g``
    sidecar) or 6 (MXFP4, ``.mx``).  An expert with neither sidecar (``.qs`` = int / e4m3 rows) is
    not a block-scaled FP4 expert and is refused, as is one whose projections disagree."""
    out, fmts = [], set()
    for proj, (O, K) in zip(PROJS, ((I, H), (I, H), (H, I))):
        name = weight_name(layer, eid, proj, prefix)
        side = fp4_sidecar(shards, name)
        if side is None:
            raise ValueError(f"{name}: no block-scaled FP4 sidecar (.g / .mx)" + ("; found .qs, which this loader does not read" if shards.has(name + ".qs") else ""))
        sname, fmt, _ = side
        nib, bs = (split_nvfp4_blob if fmt == 5 else split_mxfp4_blob)(shards.read(name), O, K)
        g = float(shards.read(sname).reshape(-1)[0])
        out.append((nib, bs, g))
        fmts.add(fmt)
    if len(fmts) != 1:
        raise ValueError(f"expert {eid} of layer {layer} mixes NVFP4 and MXFP4 projections")
    return fmts.pop(), tuple(out)


def expert_tensors(layer: int, eid, packed, prefix: str = "mlp", fmt: int = 5) -> dict:
    """The container entries of one expert given its (nib, bs, g) triples: what convert writes
    (``.g`` sidecar for NVFP4, ``.mx`` holding 1.0 for an MXFP4 passthrough, convert.rs:2822-2870)."""
    t = {}
    for proj, (nib, bs, g) in zip(PROJS, packed):
        name = weight_name(layer, eid, proj, prefix)
        t[name] = np.concatenate([np.ascontiguousarray(nib, np.uint8).reshape(-1), np.ascontiguousarray(bs, np.uint8).reshape(-1)])
        t[name + (".g" if fmt == 5 else ".mx")] = np.array([g], np.float32)
    return t


def load_layer(shards: Shards, layer: int, H: int, I: int, E: int, device: int = 0, shared_id=None, prefix: str = "mlp",
               local=None):
    """Upload the experts of one layer into HBM: a speedycolibri_b200.moe.Layer-compatible list of
    resident handles.  ``local``: ids to load (expert parallelism), default all."""
    from .backend import CudaTensor
    from .moe import Expert

    fmts = set()

    def up(fmt_packed):
        fmt, packed = fmt_packed
        fmts.add(fmt)
        wrap = CudaTensor.wrap_nvfp4 if fmt == 5 else CudaTensor.wrap_mxfp4
        return Expert(*[wrap(nib, bs, g, K, O, device) for (nib, bs, g), (O, K) in zip(packed, ((I, H), (I, H), (H, I)))])

    experts = [up(read_expert(shards, layer, e, H, I, prefix)) if (local is None or e in local) else None for e in range(E)]
    shared = up(read_expert(shards, layer, shared_id, H, I, prefix)) if shared_id is not None else None
    if len(fmts) != 1:
        raise ValueError(f"layer {layer} mixes expert formats {sorted(fmts)}; a ColiMoe handle takes one format")
    return experts, shared, fmts.pop()
