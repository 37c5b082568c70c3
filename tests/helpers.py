"""Shared test plumbing: build the same layer for the CPU oracle and for the CUDA library."""
from __future__ import annotations

import numpy as np

from oracle import oracle
from speedycolibri_b200 import synth
from speedycolibri_b200.configs import FMT_E4M3_ROW, FMT_NVFP4, MoeShape


def quantize_host(shape: MoeShape, w: np.ndarray):
    """(q, s, g) in the reference's container layout, via the oracle's quantisers."""
    if shape.fmt == FMT_NVFP4:
        return oracle.quantize_nvfp4(w)
    if shape.fmt == FMT_E4M3_ROW:
        # per-row scaled e4m3 (linear.rs:93-109); the reference holds no encoder for it, so the rule
        # of the 128x128 form is applied per row: scale = amax / 448, code = e4m3(w / scale)
        sc = np.maximum(np.abs(w).max(axis=1) / 448.0, 1e-30).astype(np.float32)
        enc = np.frompyfunc(lambda v: oracle.lib().orc_f32_to_e4m3(float(v)), 1, 1)
        codes = enc((w / sc[:, None]).astype(np.float32)).astype(np.uint8)
        return codes, sc, 1.0
    codes, sc = oracle.quantize_fp8_b128(w)
    return codes, sc, 1.0


def host_packed_expert(shape: MoeShape, e: int):
    return tuple(quantize_host(shape, synth.host_dense_weight(shape, which, e)) for which in ("gate", "up", "down"))


def host_layer(shape: MoeShape):
    """Numpy-generated, oracle-quantised layer: returns (oracle.Layer, packed dict)."""
    experts = [host_packed_expert(shape, e) for e in range(shape.E)]
    shared = host_packed_expert(shape, shape.E) if shape.shared else None
    router = synth.host_router(shape)
    sb, lb = synth.select_bias(shape), synth.zipf_logit_bias(shape)
    L = oracle.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale,
                     shape.n_group, shape.topk_group, shape.fmt, router, experts, shared, sb, lb)
    return L, dict(experts=experts, shared=shared, router=router, select_bias=sb, logit_bias=lb)


def upload_layer(shape: MoeShape, packed, device: int = 0, local=None):
    """The packed host layer as resident handles (speedycolibri_b200.moe.Layer)."""
    from speedycolibri_b200.backend import CudaTensor
    from speedycolibri_b200.moe import Expert, Layer

    def up(ex):
        out = []
        for mi, which in enumerate(("gate", "up", "down")):
            O, K = (shape.H, shape.I) if which == "down" else (shape.I, shape.H)
            q, s, g = ex[mi]
            if shape.fmt == FMT_NVFP4:
                out.append(CudaTensor.wrap_nvfp4(q, s, g, K, O, device))
            else:
                out.append(CudaTensor.upload(q, s, shape.fmt, K, O, device))
        return Expert(*out)

    experts = [up(ex) if (local is None or e in local) else None for e, ex in enumerate(packed["experts"])]
    shared = up(packed["shared"]) if packed["shared"] is not None else None
    return Layer(router=packed["router"], experts=experts, router_bias=packed["select_bias"],
                 logit_bias=packed["logit_bias"], shared=shared)


def oracle_layer_from_device(shape: MoeShape, layer, needed):
    """Export the resident experts in `needed` (plus the shared expert) back to host and wrap
    them for the oracle; experts that are not needed stay NULL."""
    def ex(e):
        return tuple(t.export() for t in (e.gate, e.up, e.down))

    experts = [ex(layer.experts[e]) if e in needed else None for e in range(shape.E)]
    shared = ex(layer.shared) if layer.shared is not None else None
    return oracle.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale,
                        shape.n_group, shape.topk_group, shape.fmt, layer.router, experts, shared,
                        layer.router_bias, layer.logit_bias)


def rel_l2(a_bits: np.ndarray, b_bits: np.ndarray) -> float:
    a = synth.bf16_bits_to_f32(a_bits).astype(np.float64)
    b = synth.bf16_bits_to_f32(b_bits).astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
