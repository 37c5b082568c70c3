"""Seeded synthetic tensors for the benchmark shapes.  They stand in for model checkpoints and
datasets (none is used): expert weights ~N(0, 0.02) quantised with the reference's own rules,
router ~N(0, 1/sqrt(H)) in bf16 (so logits ~N(0,1)), activations ~N(0,1) in bf16.

Every tensor has its own seed derived from (base seed, shape name, tensor name, expert id), so
a rank that owns a subset of the experts generates exactly the bytes the single-GPU run has."""
from __future__ import annotations

import hashlib
import math
from typing import Optional, Sequence

import numpy as np

from .configs import FMT_MXFP4, FMT_NVFP4, MoeShape

BASE_SEED = 20261125
WEIGHT_STD = 0.02


def tensor_seed(shape_name: str, tensor: str, index: int = 0, base: int = BASE_SEED) -> int:
    h = hashlib.sha256(f"{base}/{shape_name}/{tensor}/{index}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (crates/colibri-core/src/dtype.rs:176-194)."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = b + 0x7FFF + ((b >> 16) & 1)
    return (r >> 16).astype(np.uint16)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def zipf_logit_bias(shape: MoeShape) -> Optional[np.ndarray]:
    """Additive logit bias that makes expert popularity follow Zipf(s) over a seeded
    permutation of the expert ids: bias[pi(r)] = -s*ln(r+1), shifted to zero mean."""
    if shape.zipf_s <= 0:
        return None
    rng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, "zipf_perm")))
    perm = rng.permutation(shape.E)
    b = np.empty(shape.E, np.float32)
    b[perm] = (-shape.zipf_s * np.log(np.arange(shape.E) + 1.0)).astype(np.float32)
    return (b - b.mean()).astype(np.float32)


def select_bias(shape: MoeShape) -> Optional[np.ndarray]:
    if shape.select_bias_std <= 0:
        return None
    rng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, "select_bias")))
    return (rng.standard_normal(shape.E) * shape.select_bias_std).astype(np.float32)


# ---- host (numpy) generation: small shapes, CPU tests -------------------------------------------
def host_router(shape: MoeShape) -> np.ndarray:
    rng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, "router")))
    return f32_to_bf16_bits(rng.standard_normal((shape.E, shape.H)).astype(np.float32) / math.sqrt(shape.H))


def host_tokens(shape: MoeShape, T: Optional[int] = None, index: int = 0) -> np.ndarray:
    T = shape.T if T is None else T
    rng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, "x", index)))
    return f32_to_bf16_bits(rng.standard_normal((T, shape.H)).astype(np.float32))


def host_dense_weight(shape: MoeShape, which: str, expert: int) -> np.ndarray:
    """f32 [O,K] ~N(0, 0.02): gate/up are [I,H], down is [H,I] (convert.rs expert_oi)."""
    O, K = (shape.H, shape.I) if which == "down" else (shape.I, shape.H)
    rng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, which, expert)))
    w = rng.standard_normal((O, K), dtype=np.float32) * np.float32(WEIGHT_STD)
    if shape.block_spread > 0.0:
        # magnitudes that differ from one 128x128 block to the next (quantisation scales then do too)
        srng = np.random.Generator(np.random.Philox(tensor_seed(shape.name, which + "_spread", expert)))
        nb_o, nb_k = (O + 127) // 128, (K + 127) // 128
        mult = np.exp(shape.block_spread * srng.standard_normal((nb_o, nb_k))).astype(np.float32)
        w = w * np.repeat(np.repeat(mult, 128, axis=0), 128, axis=1)[:O, :K]
    return w


# ---- device (torch) generation: any shape, needs the GPU ------------------------------------------
def device_tokens(shape: MoeShape, T: Optional[int] = None, index: int = 0, device: int = 0):
    import torch

    T = shape.T if T is None else T
    g = torch.Generator(device=f"cuda:{device}")
    g.manual_seed(tensor_seed(shape.name, "x_dev", index))
    return torch.randn((T, shape.H), generator=g, device=f"cuda:{device}", dtype=torch.float32).to(torch.bfloat16)


def device_router_bits(shape: MoeShape, device: int = 0) -> np.ndarray:
    import torch

    g = torch.Generator(device=f"cuda:{device}")
    g.manual_seed(tensor_seed(shape.name, "router_dev"))
    r = torch.randn((shape.E, shape.H), generator=g, device=f"cuda:{device}", dtype=torch.float32) / math.sqrt(shape.H)
    return r.to(torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)


def device_expert(shape: MoeShape, expert: int, device: int = 0):
    """Generate one expert's three matrices on the GPU, quantise them there with the library's
    (reference-exact) quantiser and return an ``Expert`` of resident handles."""
    import torch

    from . import backend
    from .moe import Expert

    out = []
    for which in ("gate", "up", "down"):
        O, K = (shape.H, shape.I) if which == "down" else (shape.I, shape.H)
        g = torch.Generator(device=f"cuda:{device}")
        g.manual_seed(tensor_seed(shape.name, which + "_dev", expert))
        w = torch.randn((O, K), generator=g, device=f"cuda:{device}", dtype=torch.float32) * WEIGHT_STD
        if shape.fmt == FMT_NVFP4:
            nib, bs, gs = backend.quantize_nvfp4_dev(w, device)
            out.append(backend.CudaTensor.from_device(shape.fmt, nib, bs, gs, K, O, device))
        else:
            codes, sc = backend.quantize_fp8_b128_dev(w, device)
            out.append(backend.CudaTensor.from_device(shape.fmt, codes, sc, 1.0, K, O, device))
        del w
    return Expert(*out)


def device_layer(shape: MoeShape, device: int = 0, local_experts: Optional[Sequence[int]] = None):
    """A ``Layer`` with resident synthetic weights.  `local_experts` (default: all) lists the
    routed experts this rank holds; the shared expert (index E) is always generated."""
    from .moe import Layer

    local = set(range(shape.E)) if local_experts is None else set(local_experts)
    experts = [device_expert(shape, e, device) if e in local else None for e in range(shape.E)]
    shared = device_expert(shape, shape.E, device) if shape.shared else None
    return Layer(router=device_router_bits(shape, device), experts=experts, router_bias=select_bias(shape),
                 logit_bias=zipf_logit_bias(shape), shared=shared)


def upload_packed_layer(shape: MoeShape, packed, device: int = 0, local=None):
    """A ``Layer`` of resident handles from host arrays in the reference's container layout:
    packed = dict(experts=[(gate, up, down) triples of (q, s, g)], shared=triple or None, router=bf16
    bits, select_bias, logit_bias).  `local`: the expert ids this rank holds (default all)."""
    from .backend import CudaTensor
    from .moe import Expert, Layer

    def up(ex):
        out = []
        for mi, which in enumerate(("gate", "up", "down")):
            O, K = (shape.H, shape.I) if which == "down" else (shape.I, shape.H)
            q, s, g = ex[mi]
            if shape.fmt == FMT_NVFP4:
                out.append(CudaTensor.wrap_nvfp4(q, s, g, K, O, device))
            elif shape.fmt == FMT_MXFP4:
                out.append(CudaTensor.wrap_mxfp4(q, s, g, K, O, device))
            else:
                out.append(CudaTensor.upload(q, s, shape.fmt, K, O, device))
        return Expert(*out)

    experts = [up(ex) if (local is None or e in local) else None for e, ex in enumerate(packed["experts"])]
    shared = up(packed["shared"]) if packed["shared"] is not None else None
    return Layer(router=packed["router"], experts=experts, router_bias=packed["select_bias"],
                 logit_bias=packed["logit_bias"], shared=shared)
