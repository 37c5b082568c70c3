"""Locate, build and load ``libcoli_b200.so`` and declare its C ABI for ctypes."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libcoli_b200.so")
SOURCES = ["abi.cu", "ep.cu", "routing.cu", "layout.cu", "expert_small.cu", "expert_tc.cu", "expert_tc_tmem.cu", "combine.cu"]
HEADERS = ["internal.cuh", "host_state.cuh", "tc_common.cuh", "coli_math.h", os.path.join("..", "..", "include", "coli_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off", "-shared",
]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(os.path.join(_CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library for sm_100a with nvcc (cross-compiles without a GPU): one object per
    source, compiled side by side, then one link."""
    if not force and not _stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    objdir = os.path.join(_HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + os.environ.get("COLI_NVCC_EXTRA", "").split()

    def compile_one(src):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = ["nvcc", *flags, *(["-Xptxas=-v"] if verbose else []), "-c", "-o", obj, src]
        r = subprocess.run(cmd, cwd=_CSRC, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + r.stdout + r.stderr)
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    r = subprocess.run(["nvcc", "-shared", "-o", LIB_PATH, *objs], cwd=_CSRC, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB_PATH


class ColiMoeLayer(C.Structure):
    """``ColiMoeLayer`` of include/coli_b200.h."""

    _fields_ = [
        ("H", C.c_int32), ("E", C.c_int32), ("k", C.c_int32), ("I", C.c_int32),
        ("score", C.c_int32), ("norm_topk", C.c_int32), ("routed_scale", C.c_float),
        ("n_group", C.c_int32), ("topk_group", C.c_int32), ("fmt", C.c_int32), ("device", C.c_int32),
        ("router_w", C.c_void_p), ("select_bias", C.c_void_p), ("logit_bias", C.c_void_p),
        ("gate", C.POINTER(C.c_void_p)), ("up", C.POINTER(C.c_void_p)), ("down", C.POINTER(C.c_void_p)),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
        ("ep_rank", C.c_int32), ("ep_world", C.c_int32), ("expert_owner", C.c_void_p),
        ("nccl_comm", C.c_void_p),
    ]


_P = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_i = C.c_int
_f = C.c_float
_sz = C.c_size_t

# name -> (restype, argtypes); every symbol include/coli_b200.h declares
SIGNATURES = {
    "coli_cuda_init": (_i, [C.POINTER(_i), _i]),
    "coli_cuda_shutdown": (None, []),
    "coli_cuda_device_count": (_i, []),
    "coli_cuda_device_at": (_i, [_i]),
    "coli_cuda_mem_info": (_i, [_i, C.POINTER(_sz), C.POINTER(_sz)]),
    "coli_cuda_device_sync": (_i, [_i]),
    "coli_cuda_set_activation": (None, [_i, _f, _f]),
    "coli_cuda_stats": (None, [_i, C.POINTER(_sz), C.POINTER(_sz)]),
    "coli_cuda_last_error": (C.c_char_p, []),
    "coli_cuda_scratch_bytes": (_sz, [_i]),
    "coli_cuda_group_stats": (None, [_P, _P, _P, _P, _P, _P]),
    "coli_cuda_pageable_access": (_i, [_i]),
    "coli_cuda_set_weight_zerocopy": (None, [_i]),
    "coli_cuda_set_ffn_devcopy": (None, [_i]),
    "coli_cuda_host_register": (_i, [_P, _sz]),
    "coli_cuda_host_unregister": (None, [_P]),
    "coli_cuda_tensor_wrap_mxfp4": (_i, [_PP, _P, _P, _f, _i, _i, _i]),
    "coli_b200_mxfp4_resident_scales": (_i, [_P, _P, _f, _i, _i, _P, C.POINTER(_f)]),
    "coli_cuda_expert_mlp_mxfp4": (_i, [_P, _P, _P, _P, _P, _i]),
    "coli_cuda_expert_group_mxfp4": (_i, [_PP, _PP, _PP, C.POINTER(_i), _i, _P, _P]),
    "coli_cuda_expert_mlp_mxfp4_situ": (_i, [_P, _P, _P, _P, _P, _i, _f, _f]),
    "coli_cuda_tensor_upload": (_i, [_PP, _P, _P, _i, _i, _i, _i]),
    "coli_cuda_tensor_wrap": (_i, [_PP, _P, _P, _i, _i, _i, _i]),
    "coli_cuda_tensor_wrap_nvfp4": (_i, [_PP, _P, _P, _f, _i, _i, _i]),
    "coli_cuda_tensor_free": (None, [_P]),
    "coli_cuda_tensor_bytes": (_sz, [_P]),
    "coli_cuda_tensor_device": (_i, [_P]),
    "coli_b200_tensor_from_device": (_i, [_PP, _i, _P, _P, _f, _i, _i, _i]),
    "coli_b200_tensor_export": (_i, [_P, _P, _P, C.POINTER(_f)]),
    "coli_b200_quantize_nvfp4": (_i, [_i, _P, _i, _i, _P, _P, C.POINTER(_f)]),
    "coli_b200_quantize_fp8_b128": (_i, [_i, _P, _i, _i, _P, _P]),
    "coli_cuda_expert_mlp_nvfp4": (_i, [_P, _P, _P, _P, _P, _i]),
    "coli_cuda_expert_mlp_fp8": (_i, [_P, _P, _P, _P, _P, _i]),
    "coli_cuda_expert_group_nvfp4": (_i, [_PP, _PP, _PP, C.POINTER(_i), _i, _P, _P]),
    "coli_cuda_matmul": (_i, [_PP, _P, _P, _P, _P, _i, _i, _i, _i, _i]),
    "coli_cuda_expert_mlp": (_i, [_P, _P, _P, _P, _P, _i]),
    "coli_cuda_expert_group": (_i, [_PP, _PP, _PP, C.POINTER(_i), _i, _P, _P]),
    "coli_cuda_matmul_nvfp4": (_i, [_PP, _P, _P, _P, _P, _f, _i, _i, _i, _i]),
    "coli_cuda_expert_mlp_nvfp4_relu2": (_i, [_P, _P, _P, _P, _i, _i]),
    "coli_cuda_expert_group_nvfp4_relu2": (_i, [_PP, _PP, C.POINTER(_i), _i, _P, _P]),
    "coli_cuda_expert_seg_nvfp4_relu2": (_i, [_PP, _PP, C.POINTER(_i), _i, _P, _P]),
    "coli_b200_moe_create": (_i, [_PP, C.POINTER(ColiMoeLayer), _i]),
    "coli_b200_moe_destroy": (None, [_P]),
    "coli_b200_moe_workspace_bytes": (_sz, [_P]),
    "coli_b200_moe_block": (_i, [_P, _P, _P, _i, _P, _P]),
    "coli_b200_moe_block_dev": (_i, [_P, _P, _P, _i, _P]),
    "coli_b200_moe_layer_step_dev": (_i, [_P, _P, _P, _f, _i, _P]),
    "coli_b200_moe_check": (_i, [_P]),
    "coli_b200_moe_last_routing": (_i, [_P, _i, _P, _P]),
    "coli_b200_moe_local_experts": (_i, [_P]),
    "coli_b200_moe_topk_dev": (_i, [_P, _P, _i, _P, _P, _P]),
    "coli_b200_moe_gather_local_dev": (_i, [_P, _P, _P, _i, _P, _P, _P, _P]),
    "coli_b200_moe_experts_dev": (_i, [_P, _P, _P, _i, _i, _P, _P]),
    "coli_b200_moe_shared_dev": (_i, [_P, _P, _i, _P, _P]),
    "coli_b200_moe_combine_partial_dev": (_i, [_P, _P, _P, _P, _P, _i, _P]),
    "coli_b200_moe_finish_dev": (_i, [_P, _P, _P, _P, _i, _P]),
    "coli_b200_moe_block_ep_dev": (_i, [_P, _P, _P, _i, _P]),
    "coli_b200_moe_block_ep_emulate": (_i, [_PP, _i, _PP, _PP, C.POINTER(_i), _P]),
    "coli_b200_ep_barrier_probe": (_i, [_P, _i, _P]),
    "coli_b200_nccl_unique_id": (_i, [_P]),
    "coli_b200_nccl_comm_create": (_i, [_PP, _P, _i, _i, _i]),
    "coli_b200_nccl_comm_destroy": (None, [_P]),
    "coli_b200_ep_layout": (_i, [_P, _i, _i, _P]),
    "coli_b200_ep_profile": (_i, [_P, _i]),
    "coli_b200_ep_stage_ms": (_i, [_P, C.POINTER(_f), C.POINTER(_i)]),
    "coli_b200_ep_last_counts": (_i, [_P, _P]),
    "coli_b200_moe_profile": (_i, [_P, _i]),
    "coli_b200_moe_phase_ms": (_i, [_P, C.POINTER(_f), C.POINTER(_i)]),
    "coli_b200_moe_stream": (_P, [_P]),
    "coli_b200_launch_count": (C.c_uint64, []),
    "coli_b200_route_noalloc": (_i, [_P, _P, _P, _P, _i, _i, _i, _i, _i, _i, _f, _i, _i, _P, _P, _P]),
    "coli_b200_sharding_fingerprint": (C.c_uint64, [C.c_uint32, C.c_uint32, _P]),
}

_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Load the library (building it first if the sources are newer).  Raises if that fails:
    there is no other implementation to fall back to."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if _stale():
            try:
                build()
            except Exception as e:  # no nvcc on the box and no prebuilt library
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"libcoli_b200.so is missing and could not be built ({e}); "
                        "the MoE block has no CPU fallback"
                    ) from e
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the ABI lost a symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib
