"""Host-side mirror of the reference's MoE layer interface (crates/colibri-engine/src/moe.rs):
``Config`` (the routing fields of colibri_core::Config), ``Expert``, ``Layer`` and ``MoeBlock`` with
``moe`` / ``route``.  The arithmetic runs in libcoli_b200.so; nothing here computes."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import _lib
from .backend import CudaTensor, _check, _lib_, _np_ptr
from .configs import FMT_NVFP4, SCORE_SIGMOID, SCORE_SOFTMAX, MoeShape


@dataclass
class Config:
    """The fields of colibri_core::Config the block reads (crates/colibri-core/src/config.rs:177-)."""

    hidden: int
    n_experts: int
    topk: int
    moe_inter: int
    router_score: int = SCORE_SIGMOID   # RouterScore::{Softmax, Sigmoid}
    norm_topk: bool = False
    routed_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    fmt: int = FMT_NVFP4

    @classmethod
    def from_shape(cls, s: MoeShape) -> "Config":
        return cls(s.H, s.E, s.k, s.I, s.score, s.norm_topk, s.routed_scale, s.n_group, s.topk_group, s.fmt)


@dataclass
class Expert:
    """crates/colibri-engine/src/moe.rs:233-241."""

    gate: CudaTensor
    up: CudaTensor
    down: CudaTensor


@dataclass
class Layer:
    """The MoE fields of the reference's Layer (crates/colibri-engine/src/model.rs:129-131):
    router weights (bf16 bit patterns, [E,H]), the sigmoid selection bias, the experts, the
    shared expert.  ``logit_bias`` is the one extension (added to the logits before scoring)."""

    router: np.ndarray                       # uint16 (bf16 bits) [E,H]
    experts: Sequence[Optional[Expert]]      # E entries; None = not resident on this rank
    router_bias: Optional[np.ndarray] = None # f32 [E]
    logit_bias: Optional[np.ndarray] = None  # f32 [E]
    shared: Optional[Expert] = None


class MoeBlock:
    """One layer's device-resident tables and workspace (``ColiMoe``)."""

    def __init__(self, cfg: Config, layer: Layer, max_tokens: int, device: int = 0, ep_rank: int = 0,
                 ep_world: int = 1, expert_owner: Optional[Sequence[int]] = None, nccl_comm: Optional[int] = None):
        self.cfg, self.device, self.max_tokens = cfg, device, max_tokens
        self.ep_rank, self.ep_world = ep_rank, ep_world
        E = cfg.n_experts
        assert len(layer.experts) == E
        router = np.ascontiguousarray(layer.router, dtype=np.uint16)
        assert router.shape == (E, cfg.hidden)
        L = _lib.ColiMoeLayer()
        L.H, L.E, L.k, L.I = cfg.hidden, E, cfg.topk, cfg.moe_inter
        L.score, L.norm_topk, L.routed_scale = cfg.router_score, int(cfg.norm_topk), cfg.routed_scale
        L.n_group, L.topk_group, L.fmt, L.device = cfg.n_group, cfg.topk_group, cfg.fmt, device
        L.router_w = router.ctypes.data
        keep = [router]
        if layer.router_bias is not None:
            b = np.ascontiguousarray(layer.router_bias, dtype=np.float32)
            keep.append(b)
            L.select_bias = b.ctypes.data
        if layer.logit_bias is not None:
            b = np.ascontiguousarray(layer.logit_bias, dtype=np.float32)
            keep.append(b)
            L.logit_bias = b.ctypes.data
        tabs = []
        for name in ("gate", "up", "down"):
            arr = (C.c_void_p * E)(*[(getattr(e, name).handle if e is not None else None) for e in layer.experts])
            tabs.append(arr)
        L.gate, L.up, L.down = (C.cast(t, C.POINTER(C.c_void_p)) for t in tabs)
        if layer.shared is not None:
            L.sh_gate, L.sh_up, L.sh_down = layer.shared.gate.handle, layer.shared.up.handle, layer.shared.down.handle
        L.ep_rank, L.ep_world = ep_rank, ep_world
        if expert_owner is not None:
            own = np.ascontiguousarray(expert_owner, dtype=np.int32)
            keep.append(own)
            L.expert_owner = own.ctypes.data
        if nccl_comm:
            L.nccl_comm = nccl_comm
        h = C.c_void_p()
        _check(_lib_().coli_b200_moe_create(C.byref(h), C.byref(L), max_tokens), "coli_b200_moe_create")
        self.handle = h.value
        self.layer = layer  # keeps the weight handles alive
        self.has_shared = layer.shared is not None

    # -- reference-style host call: moe(cfg, l, layer, x, s_len, out, with_shared, provider) ----
    def moe(self, x: np.ndarray, want_routing: bool = False):
        """Host bf16 bits [T,H] in -> host bf16 bits [T,H] out (synchronous, copies inside)."""
        x = np.ascontiguousarray(x, dtype=np.uint16)
        T = x.shape[0]
        out = np.empty_like(x)
        idx = np.empty((T, self.cfg.topk), np.int32) if want_routing else None
        w = np.empty((T, self.cfg.topk), np.float32) if want_routing else None
        _check(_lib_().coli_b200_moe_block(self.handle, _np_ptr(x), _np_ptr(out), T,
                                           _np_ptr(idx) if want_routing else None,
                                           _np_ptr(w) if want_routing else None), "coli_b200_moe_block")
        return (out, idx, w) if want_routing else out

    # -- device-resident call ------------------------------------------------------------------
    def forward(self, x, out=None, stream=None):
        """torch bf16 CUDA [T,H] -> torch bf16 CUDA [T,H], asynchronous on the current torch stream."""
        import torch

        assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        st = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        _check(_lib_().coli_b200_moe_block_dev(self.handle, x.data_ptr(), out.data_ptr(), x.shape[0], st),
               "coli_b200_moe_block_dev")
        return out

    def layer_step(self, resid, post_ln_w, eps: float, stream=None):
        """The layer step around the block (forward.rs:376-393), in place on the f32 residual stream:
        resid += moe_block(bf16(rmsnorm(resid, post_ln_w, eps))).  torch f32 CUDA [T,H] and [H]."""
        import torch

        assert resid.dtype == torch.float32 and resid.is_cuda and resid.is_contiguous()
        assert post_ln_w.dtype == torch.float32 and post_ln_w.is_cuda and post_ln_w.numel() == resid.shape[1]
        st = torch.cuda.current_stream(resid.device).cuda_stream if stream is None else stream
        _check(_lib_().coli_b200_moe_layer_step_dev(self.handle, resid.data_ptr(), post_ln_w.data_ptr(), float(eps), resid.shape[0], st),
               "coli_b200_moe_layer_step_dev")
        return resid

    def check(self) -> None:
        """Synchronise and raise if a kernel of this handle abandoned a bounded device-side wait."""
        _check(_lib_().coli_b200_moe_check(self.handle), "coli_b200_moe_check")

    def last_routing(self, T: int):
        idx = np.empty((T, self.cfg.topk), np.int32)
        w = np.empty((T, self.cfg.topk), np.float32)
        _check(_lib_().coli_b200_moe_last_routing(self.handle, T, _np_ptr(idx), _np_ptr(w)), "coli_b200_moe_last_routing")
        return idx, w

    def moe_ptr(self, x_ptr: int, out_ptr: int, T: int) -> None:
        """coli_b200_moe_block on raw HOST addresses (e.g. pinned buffers): bf16 [T,H] each."""
        _check(_lib_().coli_b200_moe_block(self.handle, x_ptr, out_ptr, T, None, None), "coli_b200_moe_block")

    def stream(self) -> int:
        """The cudaStream_t the host-pointer call runs on."""
        return _lib_().coli_b200_moe_stream(self.handle)

    PHASES = ("router", "permute", "gate_up", "down", "combine")

    def profile(self, enable: bool) -> None:
        """Per-phase CUDA-event timing inside forward() (synchronises each call while on)."""
        _check(_lib_().coli_b200_moe_profile(self.handle, int(enable)), "coli_b200_moe_profile")

    def phase_ms(self):
        """(dict phase -> accumulated ms, number of calls) since profile(True)."""
        ms = (C.c_float * len(self.PHASES))()
        n = C.c_int()
        _check(_lib_().coli_b200_moe_phase_ms(self.handle, ms, C.byref(n)), "coli_b200_moe_phase_ms")
        return dict(zip(self.PHASES, [float(v) for v in ms])), n.value

    def workspace_bytes(self) -> int:
        return _lib_().coli_b200_moe_workspace_bytes(self.handle)

    # -- expert-parallel call (one per rank; the role of moe.rs:1737 `moe_sharded`) ---------------
    def forward_ep(self, x, out=None, stream=None):
        """torch bf16 CUDA [T_local,H] -> [T_local,H]; every rank of the communicator calls it."""
        import torch

        assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        st = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        _check(_lib_().coli_b200_moe_block_ep_dev(self.handle, x.data_ptr(), out.data_ptr(), x.shape[0], st),
               "coli_b200_moe_block_ep_dev")
        return out

    EP_STAGES = ("route", "plan_pack", "counts", "dispatch", "permute", "experts", "return_pack", "return", "combine")

    def ep_profile(self, enable: bool) -> None:
        _check(_lib_().coli_b200_ep_profile(self.handle, int(enable)), "coli_b200_ep_profile")

    def ep_stage_ms(self):
        """(dict stage -> accumulated ms, calls) since ep_profile(True)."""
        ms = (C.c_float * len(self.EP_STAGES))()
        n = C.c_int()
        _check(_lib_().coli_b200_ep_stage_ms(self.handle, ms, C.byref(n)), "coli_b200_ep_stage_ms")
        return dict(zip(self.EP_STAGES, [float(v) for v in ms])), n.value

    def ep_last_counts(self) -> np.ndarray:
        """int32 [world, 2, world]: [s, 0, d] tokens rank s sent to rank d, [s, 1, d] pairs of s owned by d."""
        tab = np.zeros((self.ep_world, 2, self.ep_world), np.int32)
        _check(_lib_().coli_b200_ep_last_counts(self.handle, _np_ptr(tab)), "coli_b200_ep_last_counts")
        return tab

    # -- stages (the pieces the block is made of, callable one by one) ----------------------------
    def local_experts(self) -> int:
        return _lib_().coli_b200_moe_local_experts(self.handle)

    def topk_dev(self, x, idx, w, stream):
        _check(_lib_().coli_b200_moe_topk_dev(self.handle, x.data_ptr(), x.shape[0], idx.data_ptr(), w.data_ptr(), stream),
               "coli_b200_moe_topk_dev")

    def gather_local_dev(self, x, idx, rows, seg_count, slot, stream):
        _check(_lib_().coli_b200_moe_gather_local_dev(self.handle, x.data_ptr(), idx.data_ptr(), x.shape[0], rows.data_ptr(),
                                                      seg_count.data_ptr(), slot.data_ptr(), stream), "coli_b200_moe_gather_local_dev")

    def experts_dev(self, rows, seg_count, rows_expected, y, stream):
        _check(_lib_().coli_b200_moe_experts_dev(self.handle, rows.data_ptr(), seg_count.data_ptr(), rows.shape[0], rows_expected,
                                                 y.data_ptr(), stream), "coli_b200_moe_experts_dev")

    def shared_dev(self, x, y, stream):
        _check(_lib_().coli_b200_moe_shared_dev(self.handle, x.data_ptr(), x.shape[0], y.data_ptr(), stream),
               "coli_b200_moe_shared_dev")

    def combine_partial_dev(self, y_rows, slot, w, partial, stream):
        _check(_lib_().coli_b200_moe_combine_partial_dev(self.handle, y_rows.data_ptr(), slot.data_ptr(), w.data_ptr(),
                                                         partial.data_ptr(), partial.shape[0], stream), "coli_b200_moe_combine_partial_dev")

    def finish_dev(self, partial, shared_y, out, stream):
        _check(_lib_().coli_b200_moe_finish_dev(self.handle, partial.data_ptr(), shared_y.data_ptr() if shared_y is not None else None,
                                                out.data_ptr(), out.shape[0], stream), "coli_b200_moe_finish_dev")

    def close(self):
        if self.handle:
            _lib_().coli_b200_moe_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
