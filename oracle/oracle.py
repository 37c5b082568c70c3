"""TEST INFRASTRUCTURE — ctypes wrapper over oracle/liboracle.so (the CPU restatement of the
reference's MoE block, see moe_oracle.cpp).  Imported only by tests/, by the smoke check and by
bench.py's CPU-baseline / reference arm; the product package never imports it."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")

FMT_E4M3_ROW, FMT_NVFP4, FMT_MXFP4, FMT_FP8_B128 = 4, 5, 6, 8


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "moe_oracle.cpp")
    hdr = os.path.join(_HERE, "..", "speedycolibri_b200", "csrc", "coli_math.h")
    stale = (not os.path.exists(LIB_PATH)) or any(os.path.getmtime(f) > os.path.getmtime(LIB_PATH) for f in (src, hdr))
    if force or stale:
        r = subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    return LIB_PATH


class OrcLayer(C.Structure):
    _fields_ = [
        ("H", C.c_int32), ("E", C.c_int32), ("k", C.c_int32), ("I", C.c_int32),
        ("score", C.c_int32), ("norm_topk", C.c_int32), ("routed_scale", C.c_float),
        ("n_group", C.c_int32), ("topk_group", C.c_int32), ("fmt", C.c_int32), ("has_shared", C.c_int32),
        ("router_w", C.c_void_p), ("select_bias", C.c_void_p), ("logit_bias", C.c_void_p),
        ("gate_q", C.POINTER(C.c_void_p)), ("up_q", C.POINTER(C.c_void_p)), ("down_q", C.POINTER(C.c_void_p)),
        ("gate_s", C.POINTER(C.c_void_p)), ("up_s", C.POINTER(C.c_void_p)), ("down_s", C.POINTER(C.c_void_p)),
        ("gate_g", C.c_void_p), ("up_g", C.c_void_p), ("down_g", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        P, i, f = C.c_void_p, C.c_int, C.c_float
        L.orc_f32_to_e4m3.restype, L.orc_f32_to_e4m3.argtypes = C.c_uint8, [f]
        L.orc_e4m3_to_f32.restype, L.orc_e4m3_to_f32.argtypes = f, [C.c_uint8]
        L.orc_e2m1_code.restype, L.orc_e2m1_code.argtypes = C.c_uint8, [f]
        L.orc_e2m1_to_f32.restype, L.orc_e2m1_to_f32.argtypes = f, [C.c_uint8]
        L.orc_f32_to_bf16.restype, L.orc_f32_to_bf16.argtypes = C.c_uint16, [f]
        L.orc_bf16_to_f32.restype, L.orc_bf16_to_f32.argtypes = f, [C.c_uint16]
        L.orc_expf.restype, L.orc_expf.argtypes = f, [f]
        L.orc_sigmoidf.restype, L.orc_sigmoidf.argtypes = f, [f]
        L.orc_siluf.restype, L.orc_siluf.argtypes = f, [f]
        L.orc_rmsnorm.restype, L.orc_rmsnorm.argtypes = None, [P, P, P, i, f]
        L.orc_set_activation.restype, L.orc_set_activation.argtypes = None, [i, f, f]
        L.orc_act_combine.restype, L.orc_act_combine.argtypes = f, [f, f, i, f, f]
        L.orc_expf_array.restype, L.orc_expf_array.argtypes = None, [P, P, C.c_int64]
        L.orc_quantize_nvfp4.restype, L.orc_quantize_nvfp4.argtypes = None, [P, i, i, P, P, C.POINTER(f)]
        L.orc_quantize_fp8_b128.restype, L.orc_quantize_fp8_b128.argtypes = None, [P, i, i, P, P]
        L.orc_quantize_mxfp4.restype, L.orc_quantize_mxfp4.argtypes = None, [P, i, i, P, P]
        L.orc_e8m0_to_f32.restype, L.orc_e8m0_to_f32.argtypes = f, [C.c_uint8]
        L.orc_matmul_qt.restype, L.orc_matmul_qt.argtypes = None, [i, P, P, f, P, P, i, i, i]
        L.orc_expert_ffn.restype, L.orc_expert_ffn.argtypes = None, [C.POINTER(OrcLayer), i, P, i, P]
        L.orc_route.restype, L.orc_route.argtypes = None, [C.POINTER(OrcLayer), P, P, P]
        L.orc_router_logits.restype, L.orc_router_logits.argtypes = None, [C.POINTER(OrcLayer), P, i, P]
        L.orc_route_tokens.restype, L.orc_route_tokens.argtypes = None, [C.POINTER(OrcLayer), P, i, P, P]
        L.orc_moe_block.restype, L.orc_moe_block.argtypes = i, [C.POINTER(OrcLayer), P, P, i, P, P, P, i, P]
        L.orc_set_threads.restype, L.orc_set_threads.argtypes = None, [i]
        L.orc_get_threads.restype, L.orc_get_threads.argtypes = i, []
        L.orc_hardware_threads.restype, L.orc_hardware_threads.argtypes = i, []
        L.orc_sharding_fingerprint.restype, L.orc_sharding_fingerprint.argtypes = C.c_uint64, [C.c_uint32, C.c_uint32, P]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def set_activation(oai: int = 0, alpha: float = 1.702, limit: float = 0.0) -> None:
    """Process-wide gate/up combine, as the reference keeps it (moe.rs:92-103): plain SwiGLU,
    clamped SwiGLU (oai = 0, limit > 0) or clamped OpenAI-SwiGLU (oai = 1)."""
    lib().orc_set_activation(int(oai), float(alpha), float(limit))


def act_combine(g: float, u: float, oai: int, alpha: float, limit: float) -> float:
    return float(lib().orc_act_combine(float(g), float(u), int(oai), float(alpha), float(limit)))


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """Row-wise RMSNorm, math.rs:8-20."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        lib().orc_rmsnorm(out[r].ctypes.data, x[r].ctypes.data, w.ctypes.data, x.shape[1], float(eps))
    return out


def hardware_threads() -> int:
    return lib().orc_hardware_threads()


# ---- codecs / quantisers ---------------------------------------------------------------------
def quantize_nvfp4(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    O, I = w.shape
    nib = np.zeros((O, (I + 1) // 2), np.uint8)
    bs = np.zeros((O, (I + 15) // 16), np.uint8)
    g = C.c_float()
    lib().orc_quantize_nvfp4(_p(w), O, I, _p(nib), _p(bs), C.byref(g))
    return nib, bs, g.value


def quantize_fp8_b128(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    O, I = w.shape
    codes = np.zeros((O, I), np.uint8)
    sc = np.zeros(((O + 127) // 128, (I + 127) // 128), np.float32)
    lib().orc_quantize_fp8_b128(_p(w), O, I, _p(codes), _p(sc))
    return codes, sc


def quantize_mxfp4(w: np.ndarray):
    """(nibbles [O, I/2], E8M0 block scales [O, ceil(I/32)], 1.0) — gpubench.rs:84-119."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    O, I = w.shape
    nib = np.zeros((O, (I + 1) // 2), np.uint8)
    bs = np.zeros((O, (I + 31) // 32), np.uint8)
    lib().orc_quantize_mxfp4(_p(w), O, I, _p(nib), _p(bs))
    return nib, bs, 1.0


def matmul_qt(fmt: int, q: np.ndarray, s: np.ndarray, g: float, x: np.ndarray, O: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    S, K = x.shape
    y = np.empty((S, O), np.float32)
    lib().orc_matmul_qt(fmt, _p(q), _p(s), float(g), _p(x), _p(y), S, K, O)
    return y


def dequant(fmt: int, q: np.ndarray, s: np.ndarray, g: float, O: int, K: int) -> np.ndarray:
    """Dense f32 W[O,K] as the reference's matmul sees it (one-hot probe, linear.rs:449-485)."""
    return matmul_qt(fmt, q, s, g, np.eye(K, dtype=np.float32), O).T.copy()


class Layer:
    """Holds the numpy arrays of one layer and the C struct that points into them."""

    def __init__(self, H, E, k, I, score, norm_topk, routed_scale, n_group, topk_group, fmt, router_w,
                 experts, shared=None, select_bias=None, logit_bias=None):
        """experts: list of E entries, each None or ((gq,gs,gg),(uq,us,ug),(dq,ds,dg)); shared alike."""
        self.keep = []
        L = OrcLayer()
        L.H, L.E, L.k, L.I = H, E, k, I
        L.score, L.norm_topk, L.routed_scale = score, int(norm_topk), routed_scale
        L.n_group, L.topk_group, L.fmt, L.has_shared = n_group, topk_group, fmt, int(shared is not None)
        self.router_w = np.ascontiguousarray(router_w, dtype=np.uint16)
        L.router_w = self.router_w.ctypes.data
        if select_bias is not None:
            self.select_bias = np.ascontiguousarray(select_bias, dtype=np.float32)
            L.select_bias = self.select_bias.ctypes.data
        if logit_bias is not None:
            self.logit_bias = np.ascontiguousarray(logit_bias, dtype=np.float32)
            L.logit_bias = self.logit_bias.ctypes.data
        allx = list(experts) + ([shared] if shared is not None else [])
        n = len(allx)
        sdt = np.uint8 if fmt in (FMT_NVFP4, FMT_MXFP4) else np.float32
        tabs = {}
        for mi, name in enumerate(("gate", "up", "down")):
            qs, ss = (C.c_void_p * n)(), (C.c_void_p * n)()
            gs = np.ones(n, np.float32)
            for e, ex in enumerate(allx):
                if ex is None:
                    continue
                q, s, g = ex[mi]
                q = np.ascontiguousarray(q, dtype=np.uint8)
                s = np.ascontiguousarray(s, dtype=sdt)
                self.keep += [q, s]
                qs[e], ss[e], gs[e] = q.ctypes.data, s.ctypes.data, g
            tabs[name] = (qs, ss, gs)
            self.keep += [qs, ss, gs]
        L.gate_q, L.gate_s, L.gate_g = C.cast(tabs["gate"][0], C.POINTER(C.c_void_p)), C.cast(tabs["gate"][1], C.POINTER(C.c_void_p)), tabs["gate"][2].ctypes.data
        L.up_q, L.up_s, L.up_g = C.cast(tabs["up"][0], C.POINTER(C.c_void_p)), C.cast(tabs["up"][1], C.POINTER(C.c_void_p)), tabs["up"][2].ctypes.data
        L.down_q, L.down_s, L.down_g = C.cast(tabs["down"][0], C.POINTER(C.c_void_p)), C.cast(tabs["down"][1], C.POINTER(C.c_void_p)), tabs["down"][2].ctypes.data
        self.c = L
        self.H, self.E, self.k, self.I = H, E, min(k, E), I

    def route_logits(self, logits: np.ndarray):
        """One token: f32 logits [E] -> (idx [k], w [k])  (moe.rs:1047 `route`)."""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        idx = np.empty(self.k, np.int32)
        w = np.empty(self.k, np.float32)
        lib().orc_route(C.byref(self.c), _p(logits), _p(idx), _p(w))
        return idx, w

    def router_logits(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.uint16)
        out = np.empty((x.shape[0], self.E), np.float32)
        lib().orc_router_logits(C.byref(self.c), _p(x), x.shape[0], _p(out))
        return out

    def route_tokens(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.uint16)
        T = x.shape[0]
        idx = np.empty((T, self.k), np.int32)
        w = np.empty((T, self.k), np.float32)
        lib().orc_route_tokens(C.byref(self.c), _p(x), T, _p(idx), _p(w))
        return idx, w

    def expert_ffn(self, ei: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        lib().orc_expert_ffn(C.byref(self.c), ei, _p(x), x.shape[0], _p(out))
        return out

    def moe_block(self, x: np.ndarray, world: int = 1, owner=None):
        """bf16 bits [T,H] -> dict(out=bf16 bits, out_f32, idx, w)."""
        x = np.ascontiguousarray(x, dtype=np.uint16)
        T = x.shape[0]
        out = np.empty_like(x)
        out32 = np.empty((T, self.H), np.float32)
        idx = np.empty((T, self.k), np.int32)
        w = np.empty((T, self.k), np.float32)
        own = None if owner is None else np.ascontiguousarray(owner, dtype=np.int32)
        lib().orc_moe_block(C.byref(self.c), _p(x), _p(out), T, _p(idx), _p(w), _p(out32), world, _p(own))
        return dict(out=out, out_f32=out32, idx=idx, w=w)
