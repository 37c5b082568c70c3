"""The allocation-free routing entry point (coli_b200_route_noalloc) against the handle-based
path.  It exists for callers that cannot allocate device memory — servers whose HBM is fully
committed to weight/KV pools, decode loops that cannot take cudaMalloc's device-wide stall — so
its only scratch is a fixed device array inside the library.  Collected last on purpose: a run
that stops at the first failure has then already exercised every other test."""
import ctypes as C

import numpy as np
import pytest

from speedycolibri_b200 import synth
from speedycolibri_b200.configs import CONFIGS
from tests.helpers import host_layer, upload_layer

pytestmark = pytest.mark.gpu


def route_noalloc(lib, shape, x_dev, router_dev, sb_dev, lb_dev, T, stream=None):
    import torch

    idx = torch.full((T, shape.k), -1, dtype=torch.int32, device="cuda")
    w = torch.full((T, shape.k), float("nan"), dtype=torch.float32, device="cuda")
    ok = lib.coli_b200_route_noalloc(x_dev.data_ptr(), router_dev.data_ptr(),
                                     sb_dev.data_ptr() if sb_dev is not None else None,
                                     lb_dev.data_ptr() if lb_dev is not None else None,
                                     T, shape.H, shape.E, shape.k, shape.score, int(shape.norm_topk),
                                     C.c_float(shape.routed_scale), shape.n_group, shape.topk_group,
                                     idx.data_ptr(), w.data_ptr(), stream)
    assert ok == 1, lib.coli_cuda_last_error().decode()
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy()


@pytest.mark.parametrize("name,T", [("tiny_sig", 37), ("tiny_zipf", 70), ("c1", 8)])
def test_noalloc_routing_matches_handle_path_twice(gpu_backend, orc, name, T):
    import torch

    from speedycolibri_b200 import _lib
    from speedycolibri_b200.moe import Config, MoeBlock

    lib = _lib.load()
    shape = CONFIGS[name].with_tokens(T)
    if name == "c1":  # device-generated weights; only the router matters here
        layer = synth.device_layer(shape.with_tokens(T))
        L = orc.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale, shape.n_group,
                      shape.topk_group, shape.fmt, layer.router, [None] * shape.E, None, layer.router_bias, layer.logit_bias)
    else:
        L, packed = host_layer(shape)
        layer = upload_layer(shape, packed)
    blk = MoeBlock(Config.from_shape(shape), layer, T)
    router_dev = torch.from_numpy(np.ascontiguousarray(layer.router).view(np.int16)).cuda()
    sb = torch.from_numpy(layer.router_bias).cuda() if layer.router_bias is not None else None
    lb = torch.from_numpy(layer.logit_bias).cuda() if layer.logit_bias is not None else None
    for call in range(2):  # two calls in a row share the built-in scratch; the second sees the first's leftovers
        xh = synth.host_tokens(shape, T, index=call)
        _, want_idx, want_w = blk.moe(xh, want_routing=True)  # the existing entry point
        xd = torch.from_numpy(xh.view(np.int16)).cuda()
        idx, w = route_noalloc(lib, shape, xd, router_dev, sb, lb, T)
        assert np.array_equal(idx, want_idx), f"call {call}: indices differ"
        assert np.array_equal(w.view(np.uint32), want_w.view(np.uint32)), f"call {call}: weights differ"
        # and against the CPU oracle, so that the check is not one CUDA path against another
        o_idx, o_w = L.route_tokens(xh)
        assert np.array_equal(idx, o_idx), f"call {call}: indices differ from the oracle"
        assert np.array_equal(w.view(np.uint32), o_w.view(np.uint32)), f"call {call}: weights differ from the oracle"
    blk.close()


def test_noalloc_at_the_exact_limit_on_a_side_stream(gpu_backend, orc):
    """T*E == COLI_ROUTE_NOALLOC_MAX_LOGITS (E=512, T=256) fills the built-in scratch to its last
    word; launched on a stream of its own and compared with the oracle's routing."""
    import torch

    from speedycolibri_b200 import _lib
    from speedycolibri_b200.configs import MoeShape

    lib = _lib.load()
    shape = MoeShape("noalloc_limit", H=64, E=512, k=8, I=32, T=256, shared=False)
    assert shape.T * shape.E == 131072
    router = synth.host_router(shape)
    xh = synth.host_tokens(shape)
    L = orc.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale, shape.n_group,
                  shape.topk_group, shape.fmt, router, [None] * shape.E, None, None, None)
    want_idx, want_w = L.route_tokens(xh)
    router_dev = torch.from_numpy(router.view(np.int16)).cuda()
    xd = torch.from_numpy(xh.view(np.int16)).cuda()
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    for call in range(2):
        idx, w = route_noalloc(lib, shape, xd, router_dev, None, None, shape.T, stream=side.cuda_stream)
        assert np.array_equal(idx, want_idx), f"call {call}: indices differ from the oracle"
        assert np.array_equal(w.view(np.uint32), want_w.view(np.uint32)), f"call {call}: weights differ from the oracle"


def test_noalloc_rejects_oversize_and_bad_arguments(gpu_backend):
    import torch

    from speedycolibri_b200 import _lib

    lib = _lib.load()
    buf = torch.zeros(16, dtype=torch.int32, device="cuda")
    E, T = 512, 300  # 153600 logits > 131072
    ok = lib.coli_b200_route_noalloc(buf.data_ptr(), buf.data_ptr(), None, None, T, 64, E, 8, 0, 0, C.c_float(1.0), 1, 1,
                                     buf.data_ptr(), buf.data_ptr(), None)
    assert ok == 0 and b"exceeds the built-in scratch" in lib.coli_cuda_last_error()
    ok = lib.coli_b200_route_noalloc(None, buf.data_ptr(), None, None, 1, 64, 8, 2, 0, 0, C.c_float(1.0), 1, 1,
                                     buf.data_ptr(), buf.data_ptr(), None)
    assert ok == 0
