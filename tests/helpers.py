"""Shared test plumbing: build the same layer for the CPU oracle and for the CUDA library."""
from __future__ import annotations

from oracle.layers import (host_layer, host_packed_expert, host_sample_layer, oracle_layer_from_device,  # noqa: F401
                           quantize_host, rel_l2)
from speedycolibri_b200.synth import upload_packed_layer as upload_layer  # noqa: F401
