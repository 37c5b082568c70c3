"""TEST INFRASTRUCTURE — host-side layer builders on top of the CPU oracle: quantise seeded dense
weights with the oracle's (reference-exact) quantisers, wrap them as an ``oracle.Layer``, or rebuild
such a layer from weights exported from the GPU.  Used by tests/, the smoke check and bench.py's
CPU-baseline / reference arm only."""
from __future__ import annotations

import numpy as np

from oracle import oracle
from speedycolibri_b200 import synth
from speedycolibri_b200.configs import FMT_E4M3_ROW, FMT_MXFP4, FMT_NVFP4, MoeShape


def quantize_host(shape: MoeShape, w: np.ndarray):
    """(q, s, g) in the reference's container layout, via the oracle's quantisers."""
    if shape.fmt == FMT_NVFP4:
        return oracle.quantize_nvfp4(w)
    if shape.fmt == FMT_MXFP4:
        return oracle.quantize_mxfp4(w)
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


def make_layer(shape: MoeShape, router, experts, shared, select_bias, logit_bias):
    return oracle.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale,
                        shape.n_group, shape.topk_group, shape.fmt, router, experts, shared, select_bias, logit_bias)


def host_layer(shape: MoeShape):
    """Numpy-generated, oracle-quantised layer: returns (oracle.Layer, packed dict)."""
    experts = [host_packed_expert(shape, e) for e in range(shape.E)]
    shared = host_packed_expert(shape, shape.E) if shape.shared else None
    router = synth.host_router(shape)
    sb, lb = synth.select_bias(shape), synth.zipf_logit_bias(shape)
    return make_layer(shape, router, experts, shared, sb, lb), dict(experts=experts, shared=shared, router=router,
                                                                    select_bias=sb, logit_bias=lb)


def host_sample_layer(shape: MoeShape, x_bits, cache: dict | None = None):
    """Oracle layer holding only the experts the sample tokens route to (generated on the host, several
    experts at a time on host threads).  `cache` (expert id -> packed triple) carries experts over
    from an earlier, smaller sample.  Returns (layer, number of routed experts touched)."""
    from concurrent.futures import ThreadPoolExecutor

    router = synth.host_router(shape)
    sb, lb = synth.select_bias(shape), synth.zipf_logit_bias(shape)
    probe = make_layer(shape, router, [None] * shape.E, None, sb, lb)
    idx, _ = probe.route_tokens(x_bits)
    needed = sorted(set(idx.reshape(-1).tolist()))
    cache = {} if cache is None else cache
    todo = [e for e in needed + ([shape.E] if shape.shared else []) if e not in cache]
    with ThreadPoolExecutor(max_workers=max(1, min(8, oracle.hardware_threads()))) as pool:
        for e, packed in zip(todo, pool.map(lambda e: host_packed_expert(shape, e), todo)):
            cache[e] = packed
    experts = [cache[e] if e in needed else None for e in range(shape.E)]
    shared = cache[shape.E] if shape.shared else None
    return make_layer(shape, router, experts, shared, sb, lb), len(needed)


def oracle_layer_from_device(shape: MoeShape, layer, needed):
    """Export the resident experts in `needed` (plus the shared expert) back to host and wrap
    them for the oracle; experts that are not needed (or not resident on this rank) stay NULL."""
    def ex(e):
        return tuple(t.export() for t in (e.gate, e.up, e.down))

    experts = [ex(layer.experts[e]) if (e in needed and layer.experts[e] is not None) else None for e in range(shape.E)]
    shared = ex(layer.shared) if layer.shared is not None else None
    return make_layer(shape, layer.router, experts, shared, layer.router_bias, layer.logit_bias)


def rel_l2(a_bits: np.ndarray, b_bits: np.ndarray) -> float:
    a = synth.bf16_bits_to_f32(a_bits).astype(np.float64)
    b = synth.bf16_bits_to_f32(b_bits).astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
