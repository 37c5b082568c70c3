"""Writes the committed fixtures of this folder: for each small shape, a digest of the seeded inputs
and the CPU oracle's routing and block output on them.

    python tests/golden/make_golden.py

The oracle (oracle/moe_oracle.cpp) is pinned to the reference's own known-answer vectors by
tests/test_oracle_pins.py; these fixtures freeze what that pinned oracle answers on whole layers,
so that a later change to the oracle, to the synthetic generators or to the quantisers shows up as
a difference against committed bytes, and so that the GPU parity tests have a fixed target that does
not depend on the oracle being rebuilt the same way.  The reference itself is a Rust workspace and
cannot run where these fixtures are made (no cargo), which is why its outputs are not the source."""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = ("tiny", "tiny_sig", "tiny_fp8", "tiny_mx", "tiny_zipf", "mid_ragged")


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def golden_of(name: str) -> dict:
    from oracle.layers import host_layer
    from speedycolibri_b200 import synth
    from speedycolibri_b200.configs import CONFIGS

    shape = CONFIGS[name]
    L, packed = host_layer(shape)
    x = synth.host_tokens(shape)
    want = L.moe_block(x)
    weights = []
    for tri in packed["experts"] + ([packed["shared"]] if packed["shared"] is not None else []):
        for m in tri:  # (q, s, g) per matrix
            weights += [np.asarray(v) for v in m]
    return dict(x_sha=np.array(digest(x)), weights_sha=np.array(digest(*weights)), router_sha=np.array(digest(packed["router"])),
                idx=want["idx"].astype(np.int32), w_bits=want["w"].view(np.uint32).copy(), out_bits=want["out"].view(np.uint16).copy())


def main() -> None:
    for name in SHAPES:
        g = golden_of(name)
        np.savez_compressed(os.path.join(HERE, f"block_{name}.npz"), **g)
        print(name, g["idx"].shape, g["out_bits"].shape, str(g["x_sha"])[:12])


if __name__ == "__main__":
    main()
