"""Safe wrappers over the C ABI of libcoli_b200.so — the role crates/colibri-backend/src/cuda.rs
plays for the reference (same call names, argument meaning and 1/0 return convention turned
into exceptions).  Host arrays are numpy, device arrays are torch CUDA tensors used purely as
memory (their ``data_ptr()`` is what crosses the ABI)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .configs import FMT_E4M3_ROW, FMT_FP8_B128, FMT_MXFP4, FMT_NVFP4


class CudaError(RuntimeError):
    """A C-ABI call returned 0; the message is coli_cuda_last_error()."""


def _lib_():
    return _lib.load()


def _check(ok: int, what: str) -> None:
    if not ok:
        msg = _lib_().coli_cuda_last_error().decode(errors="replace")
        raise CudaError(f"{what}: {msg}")


def _np_ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "host arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def init(devices=None) -> None:
    """coli_cuda_init (crates/colibri-backend/src/cuda.rs:400-430): idempotent per device set."""
    devices = [0] if devices is None else list(devices)
    arr = (C.c_int * len(devices))(*devices)
    _check(_lib_().coli_cuda_init(arr, len(devices)), "coli_cuda_init")


def shutdown() -> None:
    _lib_().coli_cuda_shutdown()


def device_count() -> int:
    return _lib_().coli_cuda_device_count()


def mem_info(device: int = 0):
    f, t = C.c_size_t(), C.c_size_t()
    _check(_lib_().coli_cuda_mem_info(device, C.byref(f), C.byref(t)), "coli_cuda_mem_info")
    return f.value, t.value


def stats(device: int = -1):
    n, b = C.c_size_t(), C.c_size_t()
    _lib_().coli_cuda_stats(device, C.byref(n), C.byref(b))
    return n.value, b.value


def device_sync(device: int = 0) -> None:
    _check(_lib_().coli_cuda_device_sync(device), "coli_cuda_device_sync")


def set_activation(oai: int = 0, alpha: float = 0.0, limit: float = 0.0) -> None:
    _lib_().coli_cuda_set_activation(oai, alpha, limit)


def sharding_fingerprint(num_nodes: int, n_experts: int, owner=None) -> int:
    if owner is None:
        return _lib_().coli_b200_sharding_fingerprint(num_nodes, n_experts, None)
    arr = np.ascontiguousarray(owner, dtype=np.uint32)
    return _lib_().coli_b200_sharding_fingerprint(num_nodes, n_experts, _np_ptr(arr))


class CudaTensor:
    """Persistent HBM copy of one quantised matrix W[O,I] (``ColiCudaTensor``)."""

    def __init__(self, handle: int, fmt: int, I: int, O: int, device: int):
        self.handle, self.fmt, self.I, self.O, self.device = handle, fmt, I, O, device

    # -- constructors ------------------------------------------------------------------
    @classmethod
    def wrap_nvfp4(cls, nibbles: np.ndarray, bscale: np.ndarray, gscale: float, I: int, O: int, device: int = 0):
        """coli_cuda_tensor_wrap_nvfp4: nibbles [O, ceil(I/2)] u8, bscale [O, ceil(I/16)] u8."""
        nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
        bscale = np.ascontiguousarray(bscale, dtype=np.uint8)
        assert nibbles.size == O * ((I + 1) // 2) and bscale.size == O * ((I + 15) // 16)
        h = C.c_void_p()
        _check(_lib_().coli_cuda_tensor_wrap_nvfp4(C.byref(h), _np_ptr(nibbles), _np_ptr(bscale), float(gscale), I, O, device),
               "coli_cuda_tensor_wrap_nvfp4")
        return cls(h.value, FMT_NVFP4, I, O, device)

    @classmethod
    def wrap_mxfp4(cls, nibbles: np.ndarray, bscale: np.ndarray, gscale: float, I: int, O: int, device: int = 0):
        """coli_cuda_tensor_wrap_mxfp4: nibbles [O, ceil(I/2)] u8, bscale [O, ceil(I/32)] E8M0 bytes."""
        nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
        bscale = np.ascontiguousarray(bscale, dtype=np.uint8)
        assert nibbles.size == O * ((I + 1) // 2) and bscale.size == O * ((I + 31) // 32)
        h = C.c_void_p()
        _check(_lib_().coli_cuda_tensor_wrap_mxfp4(C.byref(h), _np_ptr(nibbles), _np_ptr(bscale), float(gscale), I, O, device),
               "coli_cuda_tensor_wrap_mxfp4")
        return cls(h.value, FMT_MXFP4, I, O, device)

    @classmethod
    def upload(cls, codes: np.ndarray, scales: np.ndarray, fmt: int, I: int, O: int, device: int = 0):
        """coli_cuda_tensor_upload for the FP8 forms (fmt 4: row scales [O]; fmt 8: [ceil(O/128), ceil(I/128)])."""
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        assert codes.size == O * I
        want = O if fmt == FMT_E4M3_ROW else ((O + 127) // 128) * ((I + 127) // 128)
        assert scales.size == want
        h = C.c_void_p()
        _check(_lib_().coli_cuda_tensor_upload(C.byref(h), _np_ptr(codes), _np_ptr(scales), fmt, I, O, device),
               "coli_cuda_tensor_upload")
        return cls(h.value, fmt, I, O, device)

    @classmethod
    def from_device(cls, fmt: int, q, s, gscale: float, I: int, O: int, device: int = 0):
        """coli_b200_tensor_from_device: q, s are torch CUDA tensors in the reference layouts."""
        h = C.c_void_p()
        _check(_lib_().coli_b200_tensor_from_device(C.byref(h), fmt, q.data_ptr(), s.data_ptr(), float(gscale), I, O, device),
               "coli_b200_tensor_from_device")
        return cls(h.value, fmt, I, O, device)

    # -- accessors ---------------------------------------------------------------------
    def export(self):
        """Back to host in the reference layouts: (q u8, s u8|f32, gscale)."""
        I, O = self.I, self.O
        if self.fmt == FMT_NVFP4:
            q = np.empty((O, (I + 1) // 2), np.uint8)
            s = np.empty((O, (I + 15) // 16), np.uint8)
        elif self.fmt == FMT_MXFP4:
            q = np.empty((O, (I + 1) // 2), np.uint8)
            s = np.empty((O, (I + 31) // 32), np.uint8)
        elif self.fmt == FMT_FP8_B128:
            q = np.empty((O, I), np.uint8)
            s = np.empty(((O + 127) // 128, (I + 127) // 128), np.float32)
        else:
            q = np.empty((O, I), np.uint8)
            s = np.empty((O,), np.float32)
        g = C.c_float()
        _check(_lib_().coli_b200_tensor_export(self.handle, _np_ptr(q), _np_ptr(s), C.byref(g)), "coli_b200_tensor_export")
        return q, s, g.value

    def nbytes(self) -> int:
        return _lib_().coli_cuda_tensor_bytes(self.handle)

    def free(self) -> None:
        if self.handle:
            _lib_().coli_cuda_tensor_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# ---- device-side quantisers ------------------------------------------------------------------
def quantize_nvfp4_dev(w, device: int = 0):
    """f32 CUDA tensor [O,I] -> (nibbles u8 [O,ceil(I/2)], bscale u8 [O,ceil(I/16)], gscale)."""
    import torch

    O, I = w.shape
    assert w.dtype == torch.float32 and w.is_contiguous()
    nib = torch.empty((O, (I + 1) // 2), dtype=torch.uint8, device=w.device)
    bs = torch.empty((O, (I + 15) // 16), dtype=torch.uint8, device=w.device)
    g = C.c_float()
    _check(_lib_().coli_b200_quantize_nvfp4(device, w.data_ptr(), O, I, nib.data_ptr(), bs.data_ptr(), C.byref(g)),
           "coli_b200_quantize_nvfp4")
    return nib, bs, g.value


def quantize_fp8_b128_dev(w, device: int = 0):
    import torch

    O, I = w.shape
    assert w.dtype == torch.float32 and w.is_contiguous()
    codes = torch.empty((O, I), dtype=torch.uint8, device=w.device)
    sc = torch.empty(((O + 127) // 128, (I + 127) // 128), dtype=torch.float32, device=w.device)
    _check(_lib_().coli_b200_quantize_fp8_b128(device, w.data_ptr(), O, I, codes.data_ptr(), sc.data_ptr()),
           "coli_b200_quantize_fp8_b128")
    return codes, sc


# ---- the reference's host-pointer expert calls ---------------------------------------------------
def expert_mlp_nvfp4(gate: CudaTensor, up: CudaTensor, down: CudaTensor, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_mlp_nvfp4 (cuda.rs:833-880): x, y host f32 [S, D]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    _check(_lib_().coli_cuda_expert_mlp_nvfp4(gate.handle, up.handle, down.handle, _np_ptr(y), _np_ptr(x), x.shape[0]),
           "coli_cuda_expert_mlp_nvfp4")
    return y


def expert_mlp_fp8(gate: CudaTensor, up: CudaTensor, down: CudaTensor, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    _check(_lib_().coli_cuda_expert_mlp_fp8(gate.handle, up.handle, down.handle, _np_ptr(y), _np_ptr(x), x.shape[0]),
           "coli_cuda_expert_mlp_fp8")
    return y


def expert_group_nvfp4(gates, ups, downs, rows, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_group_nvfp4 (cuda.rs:1020-1067): x holds sum(rows) rows in expert order."""
    n = len(rows)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    mk = lambda ts: (C.c_void_p * n)(*[t.handle for t in ts])
    r = (C.c_int * n)(*[int(v) for v in rows])
    _check(_lib_().coli_cuda_expert_group_nvfp4(mk(gates), mk(ups), mk(downs), r, n, _np_ptr(y), _np_ptr(x)),
           "coli_cuda_expert_group_nvfp4")
    return y


def expert_mlp_mxfp4(gate: CudaTensor, up: CudaTensor, down: CudaTensor, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_mlp_mxfp4 (cuda.rs:92-99): fmt 6 on all three; x, y host f32 [S, D]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    _check(_lib_().coli_cuda_expert_mlp_mxfp4(gate.handle, up.handle, down.handle, _np_ptr(y), _np_ptr(x), x.shape[0]),
           "coli_cuda_expert_mlp_mxfp4")
    return y


def expert_group_mxfp4(gates, ups, downs, rows, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_group_mxfp4 (cuda.rs:212-220): x holds sum(rows) rows in expert order."""
    n = len(rows)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    mk = lambda ts: (C.c_void_p * n)(*[t.handle for t in ts])
    r = (C.c_int * n)(*[int(v) for v in rows])
    _check(_lib_().coli_cuda_expert_group_mxfp4(mk(gates), mk(ups), mk(downs), r, n, _np_ptr(y), _np_ptr(x)),
           "coli_cuda_expert_group_mxfp4")
    return y


def scratch_bytes(device: int = -1) -> int:
    """coli_cuda_scratch_bytes (backend_cuda.h:48-51)."""
    return int(_lib_().coli_cuda_scratch_bytes(device))


def group_stats() -> dict:
    """coli_cuda_group_stats (backend_cuda.h:52-53): totals over the grouped expert calls since load."""
    c, e, r = C.c_uint64(), C.c_uint64(), C.c_uint64()
    a, b, d = C.c_double(), C.c_double(), C.c_double()
    _lib_().coli_cuda_group_stats(C.byref(c), C.byref(e), C.byref(r), C.byref(a), C.byref(b), C.byref(d))
    return dict(calls=c.value, experts=e.value, rows=r.value, h2d_ms=a.value, kernel_ms=b.value, d2h_ms=d.value)


class F32Matmul:
    """coli_cuda_matmul with fmt 0 — the router GEMM of crates/colibri-engine/src/gpu.rs:2219-2249.
    Keeps the ``slot`` the reference threads through the call so W is uploaded once."""

    def __init__(self, w: np.ndarray, device: int = 0):
        self.w = np.ascontiguousarray(w, dtype=np.float32)
        self.O, self.I = self.w.shape
        self.device = device
        self.slot = C.c_void_p()

    def __call__(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty((x.shape[0], self.O), np.float32)
        _check(_lib_().coli_cuda_matmul(C.byref(self.slot), _np_ptr(y), _np_ptr(x), _np_ptr(self.w), None, 0,
                                        x.shape[0], self.I, self.O, self.device), "coli_cuda_matmul")
        return y

    def free(self):
        if self.slot.value:
            _lib_().coli_cuda_tensor_free(self.slot)
            self.slot = C.c_void_p()


def expert_mlp(gate: CudaTensor, up: CudaTensor, down: CudaTensor, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_mlp (backend_cuda.h:107-109): any resident expert format."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    _check(_lib_().coli_cuda_expert_mlp(gate.handle, up.handle, down.handle, _np_ptr(y), _np_ptr(x), x.shape[0]),
           "coli_cuda_expert_mlp")
    return y


def expert_group(gates, ups, downs, rows, x: np.ndarray) -> np.ndarray:
    """coli_cuda_expert_group (backend_cuda.h:136-140): x holds sum(rows) rows in expert order."""
    n = len(rows)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    mk = lambda ts: (C.c_void_p * n)(*[t.handle for t in ts])
    r = (C.c_int * n)(*[int(v) for v in rows])
    _check(_lib_().coli_cuda_expert_group(mk(gates), mk(ups), mk(downs), r, n, _np_ptr(y), _np_ptr(x)), "coli_cuda_expert_group")
    return y


class Nvfp4Matmul:
    """coli_cuda_matmul_nvfp4 (backend_cuda.h:127-129): y = x @ W^T for one NVFP4 matrix given as the
    container's host arrays; the slot keeps the HBM copy between calls."""

    def __init__(self, nibbles: np.ndarray, bscale: np.ndarray, gscale: float, O: int, I: int, device: int = 0):
        self.nib = np.ascontiguousarray(nibbles, dtype=np.uint8)
        self.bs = np.ascontiguousarray(bscale, dtype=np.uint8)
        self.g, self.O, self.I, self.device = float(gscale), O, I, device
        self.slot = C.c_void_p()

    def __call__(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty((x.shape[0], self.O), np.float32)
        _check(_lib_().coli_cuda_matmul_nvfp4(C.byref(self.slot), _np_ptr(y), _np_ptr(x), _np_ptr(self.nib), _np_ptr(self.bs),
                                              self.g, x.shape[0], self.I, self.O, self.device), "coli_cuda_matmul_nvfp4")
        return y

    def free(self):
        if self.slot.value:
            _lib_().coli_cuda_tensor_free(self.slot)
            self.slot = C.c_void_p()


def expert_group_relu2(ups, downs, rows, x: np.ndarray, seg: bool = False) -> np.ndarray:
    """coli_cuda_expert_group_nvfp4_relu2 / coli_cuda_expert_seg_nvfp4_relu2 (backend_cuda.h:152-160):
    gateless experts, y = down(relu(up x)^2); x holds sum(rows) rows in expert order."""
    n = len(rows)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    mk = lambda ts: (C.c_void_p * n)(*[t.handle for t in ts])
    r = (C.c_int * n)(*[int(v) for v in rows])
    fn = _lib_().coli_cuda_expert_seg_nvfp4_relu2 if seg else _lib_().coli_cuda_expert_group_nvfp4_relu2
    _check(fn(mk(ups), mk(downs), r, n, _np_ptr(y), _np_ptr(x)), "coli_cuda_expert_group_nvfp4_relu2")
    return y


def expert_mlp_relu2(up: CudaTensor, down: CudaTensor, x: np.ndarray, exact: bool = False) -> np.ndarray:
    """coli_cuda_expert_mlp_nvfp4_relu2 (backend_cuda.h:131-132)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    _check(_lib_().coli_cuda_expert_mlp_nvfp4_relu2(up.handle, down.handle, _np_ptr(y), _np_ptr(x), x.shape[0], int(exact)),
           "coli_cuda_expert_mlp_nvfp4_relu2")
    return y
