"""B200 (sm_100a) backend for the routed-expert MoE block of GriffinPilz/SpeedyColibri.

The compute lives in ``libcoli_b200.so`` (CUDA, built from ``csrc/``) behind the C ABI of
``include/coli_b200.h``; this package is the host-side mirror of the reference's operator
interface for that path:

* :mod:`.backend`  — safe wrappers over the C ABI (the role of crates/colibri-backend/src/cuda.rs)
* :mod:`.moe`      — ``Config`` / ``Expert`` / ``Layer`` / ``moe`` / ``route`` (crates/colibri-engine/src/moe.rs)
* :mod:`.cluster`  — ``ExpertSharding`` and ``ShardedMoe``, the expert-parallel block
  (crates/colibri-cluster/src/sharding.rs, moe.rs:1620-1794): one library call per rank that
  dispatches token rows to the experts' owners and brings the result rows back
* :mod:`.configs`, :mod:`.synth` — the benchmark shapes and their seeded synthetic tensors

There is no CPU fallback: importing :mod:`.backend` without the built library raises.
"""
from .configs import CONFIGS, MoeShape  # noqa: F401

__all__ = ["CONFIGS", "MoeShape"]
