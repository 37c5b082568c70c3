"""Parity of the CUDA path against the CPU oracle, through the C ABI.  Bars: routing indices and
weights bit-exact; quantised bytes bit-exact; block output relative L2 <= 1e-2 on bf16 (the
tolerance the task states), rows compared on the same seeded inputs and quantised weights."""
import numpy as np
import pytest

from speedycolibri_b200 import synth
from speedycolibri_b200.configs import CONFIGS, FMT_E4M3_ROW, FMT_FP8_B128, FMT_NVFP4
from tests.helpers import host_layer, oracle_layer_from_device, rel_l2, upload_layer

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-2


def make_block(shape, layer, max_tokens=None, **kw):
    from speedycolibri_b200.moe import Config, MoeBlock

    return MoeBlock(Config.from_shape(shape), layer, max_tokens or shape.T, **kw)


# ---- byte-exact pieces ------------------------------------------------------------------------------
@pytest.mark.parametrize("O,I", [(48, 256), (16, 16), (33, 200), (128, 2048), (7, 24)])
def test_device_quantiser_nvfp4_bit_exact(gpu_backend, orc, O, I):
    import torch

    rng = np.random.default_rng(O * 1000 + I)
    w = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    w[0, : min(16, I)] = 0.0                    # an all-zero block (scale code 0)
    w[-1, -1] = 0.5                             # an outlier that sets the tensor scale
    nib, bs, g = gpu_backend.quantize_nvfp4_dev(torch.from_numpy(w).cuda())
    wn, wb, wg = orc.quantize_nvfp4(w)
    assert g == wg
    assert np.array_equal(bs.cpu().numpy(), wb)
    assert np.array_equal(nib.cpu().numpy(), wn)


@pytest.mark.parametrize("O,I", [(128, 128), (200, 300), (768, 2048)])
def test_device_quantiser_fp8_bit_exact(gpu_backend, orc, O, I):
    import torch

    rng = np.random.default_rng(O + I)
    w = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    codes, sc = gpu_backend.quantize_fp8_b128_dev(torch.from_numpy(w).cuda())
    wc, ws = orc.quantize_fp8_b128(w)
    assert np.array_equal(sc.cpu().numpy(), ws)
    assert np.array_equal(codes.cpu().numpy(), wc)


@pytest.mark.parametrize("O,I", [(32, 128), (40, 200), (768, 2048), (5, 24)])
def test_upload_export_roundtrip(gpu_backend, orc, O, I):
    """The HBM repack is a permutation: what went in comes back out, for every format."""
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    nib, bs, g = orc.quantize_nvfp4(w)
    t = gpu_backend.CudaTensor.wrap_nvfp4(nib, bs, g, I, O)
    q2, s2, g2 = t.export()
    assert np.array_equal(q2, nib) and np.array_equal(s2, bs) and g2 == np.float32(g)
    assert t.nbytes() >= nib.size + bs.size
    codes, sc = orc.quantize_fp8_b128(w)
    t8 = gpu_backend.CudaTensor.upload(codes, sc, FMT_FP8_B128, I, O)
    q3, s3, _ = t8.export()
    assert np.array_equal(q3, codes) and np.array_equal(s3, sc)
    n0, _ = gpu_backend.stats(0)
    t.free(); t8.free()
    assert gpu_backend.stats(0)[0] == n0 - 2


def test_router_matmul_f32_bit_exact(gpu_backend, orc):
    """coli_cuda_matmul fmt 0 == the reference's sequential matmul_f32 (linear.rs:209-220)."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, 200)).astype(np.float32)
    w = rng.standard_normal((33, 200)).astype(np.float32)
    mm = gpu_backend.F32Matmul(w)
    y = mm(x)
    want = orc.matmul_qt(0, w.view(np.uint8), np.zeros(1, np.uint8), 1.0, x, 33)
    assert np.array_equal(y, want)
    assert np.array_equal(mm(x[:2]), want[:2])  # cached device copy of W is reused
    mm.free()


# ---- routing ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,T", [("tiny", 5), ("tiny_sig", 37), ("tiny_zipf", 70), ("tiny_fp8", 19), ("c0", 128),
                                    ("c1", 1), ("c1", 8), ("c1", 77), ("tiny_sig", 300)])
def test_routing_bit_exact(gpu_backend, orc, name, T):
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape) if shape.E * shape.H * shape.I < 2e7 else (None, None)
    if L is None:
        pytest.skip("shape too large for host generation")
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, T)
    out, idx, w = blk.moe(x, want_routing=True)
    widx, ww = L.route_tokens(x)
    assert np.array_equal(idx, widx)
    assert np.array_equal(w.view(np.uint32), ww.view(np.uint32)), float(np.abs(w - ww).max())
    blk.close()


def test_routing_near_ties_and_extremes(gpu_backend, orc):
    """Ties (duplicate router rows => equal logits) go to the lowest id; huge logits survive."""
    shape = CONFIGS["tiny"]
    L, packed = host_layer(shape)
    router = packed["router"].copy()
    router[3] = router[1]
    router[6] = router[1]                                   # experts 1, 3, 6 always tie
    packed = dict(packed, router=router)
    from oracle import oracle
    Lt = oracle.Layer(shape.H, shape.E, shape.k, shape.I, shape.score, shape.norm_topk, shape.routed_scale, 1, 1,
                      shape.fmt, router, packed["experts"], packed["shared"], None, None)
    blk = make_block(shape, upload_layer(shape, packed), max_tokens=64)
    x = synth.host_tokens(shape, 64)
    x[0] = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x[0]) * 300.0)   # logits in the hundreds
    _, idx, w = blk.moe(x, want_routing=True)
    widx, ww = Lt.route_tokens(x)
    assert np.array_equal(idx, widx) and np.array_equal(w.view(np.uint32), ww.view(np.uint32))
    for row in idx.tolist():
        if 3 in row:
            assert 1 in row and row.index(1) < row.index(3)
    assert np.isfinite(w).all()
    blk.close()


# ---- whole block ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,T", [("tiny", 5), ("tiny", 1), ("tiny_sig", 37), ("tiny_fp8", 19), ("tiny_zipf", 70),
                                    ("tiny_sig", 150)])
def test_block_small_shapes(gpu_backend, orc, name, T):
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, T)
    out = blk.moe(x)
    want = L.moe_block(x)
    err = rel_l2(out, want["out"])
    assert err <= REL_L2_TOL, err
    assert err <= 5e-3, f"small shapes should be well inside the bar, got {err}"
    blk.close()


@pytest.mark.parametrize("name,T", [("mid", 512), ("mid", 433), ("mid_ragged", 333), ("mid_ragged", 1000),
                                    ("mid_fp8", 512), ("mid_fp8", 97), ("mid_fp8_ragged", 333), ("mid_fp8_ragged", 1000),
                                    ("mid_fp8row", 100)])
def test_block_prefill_segments_tcgen05(gpu_backend, orc, name, T):
    """Segments of >= 8 rows on average take the tcgen05 path (TMA token tiles, TMEM accumulators):
    ragged segment lengths, K and feature counts that are not multiples of the tile, > 256 rows per
    expert; NVFP4 and both FP8 forms (block scales spread over orders of magnitude, per-row scales)."""
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, T)
    out, idx, w = blk.moe(x, want_routing=True)
    blk.check()
    want = L.moe_block(x)
    assert np.array_equal(idx, want["idx"]) and np.array_equal(w.view(np.uint32), want["w"].view(np.uint32))
    err = rel_l2(out, want["out"])
    assert err <= 5e-3, err
    # per-row agreement too: no row may be silently dropped or misplaced
    a = synth.bf16_bits_to_f32(out).astype(np.float64)
    b = synth.bf16_bits_to_f32(want["out"]).astype(np.float64)
    row_err = np.linalg.norm(a - b, axis=1) / np.maximum(np.linalg.norm(b, axis=1), 1e-30)
    assert row_err.max() <= 2e-2, (int(row_err.argmax()), float(row_err.max()))
    blk.close()


def test_block_empty_and_bounds(gpu_backend, orc):
    from speedycolibri_b200.backend import CudaError

    shape = CONFIGS["tiny"]
    _, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed), max_tokens=4)
    assert blk.moe(np.zeros((0, shape.H), np.uint16)).shape == (0, shape.H)
    with pytest.raises(CudaError, match="outside"):
        blk.moe(synth.host_tokens(shape, 5))
    assert blk.workspace_bytes() > 0
    blk.close()


def _tokens_covering_work_items(idx, n_total, n_segments=3, stride=128):
    """Tokens to check at full size: for each of the `n_segments` experts with the most rows, one
    token out of every `stride` consecutive rows of its segment (rows of a segment are its tokens in
    ascending order), so that every work item the expert kernels cut a long segment into (160 or 256
    rows each) contributes at least one checked row; topped up with evenly spaced tokens (which
    also walk the work items of the shared expert, whose rows are all tokens in order)."""
    T, k = idx.shape
    load = np.bincount(idx.reshape(-1))
    chosen = []
    for e in np.argsort(-load)[:n_segments]:
        toks = np.nonzero((idx == e).any(axis=1))[0]  # ascending = segment order
        chosen += toks[::stride].tolist() + [int(toks[-1])]
    chosen = sorted(set(chosen))
    if len(chosen) > n_total:  # keep the budget: thin out evenly
        chosen = [chosen[i] for i in np.linspace(0, len(chosen) - 1, n_total).astype(int)]
    extra = [t for t in np.linspace(0, T - 1, max(0, n_total - len(chosen)) + 2).astype(int).tolist() if t not in chosen]
    return np.array(sorted(set(chosen + extra[:max(0, n_total - len(chosen))])), dtype=int)


def _device_block_vs_oracle(shape, T_check, tokens_for_routing=None, cover_work_items=False):
    """Full-size run on the GPU with device-generated weights; the oracle recomputes a subset of
    the tokens (the block is row-independent) from the exported bytes of the same weights."""
    import torch
    from speedycolibri_b200.moe import Config, MoeBlock

    layer = synth.device_layer(shape)
    blk = MoeBlock(Config.from_shape(shape), layer, shape.T)
    x = synth.device_tokens(shape)
    out = blk.forward(x)
    torch.cuda.synchronize()
    idx, w = blk.last_routing(shape.T)
    out_h = out.view(torch.int16).cpu().numpy().view(np.uint16)
    x_h = x.view(torch.int16).cpu().numpy().view(np.uint16)
    sub = _tokens_covering_work_items(idx, T_check) if cover_work_items else np.linspace(0, shape.T - 1, T_check).astype(int)
    needed = set(idx[sub].reshape(-1).tolist())
    L = oracle_layer_from_device(shape, layer, needed)
    want = L.moe_block(x_h[sub])
    assert np.array_equal(idx[sub], want["idx"])
    assert np.array_equal(w[sub].view(np.uint32), want["w"].view(np.uint32))
    err = rel_l2(out_h[sub], want["out"])
    a = synth.bf16_bits_to_f32(out_h[sub]).astype(np.float64)
    b = synth.bf16_bits_to_f32(want["out"]).astype(np.float64)
    row_err = np.linalg.norm(a - b, axis=1) / np.maximum(np.linalg.norm(b, axis=1), 1e-30)
    assert row_err.max() <= 2e-2, (int(sub[row_err.argmax()]), float(row_err.max()))  # no row dropped or misplaced
    # routing of (many) more tokens, cheap on the CPU
    nr = min(shape.T, tokens_for_routing or shape.T)
    ridx, rw = L.route_tokens(x_h[:nr])
    assert np.array_equal(idx[:nr], ridx)
    assert np.array_equal(w[:nr].view(np.uint32), rw.view(np.uint32))
    # size-independent properties at full size
    assert np.isfinite(synth.bf16_bits_to_f32(out_h)).all()
    assert all(len(set(r)) == shape.k for r in idx[:: max(1, shape.T // 512)].tolist())
    blk.close()
    return err, idx


def test_block_c0_full(gpu_backend, orc):
    shape = CONFIGS["c0"]
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape)
    out, idx, w = blk.moe(x, want_routing=True)
    want = L.moe_block(x)
    assert np.array_equal(idx, want["idx"]) and np.array_equal(w.view(np.uint32), want["w"].view(np.uint32))
    assert rel_l2(out, want["out"]) <= REL_L2_TOL
    # device-pointer path gives the same bytes as the host-pointer path
    import torch
    xd = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16)
    od = blk.forward(xd)
    torch.cuda.synchronize()
    assert np.array_equal(od.view(torch.int16).cpu().numpy().view(np.uint16), out)
    blk.close()


@pytest.mark.parametrize("T", [1, 4, 8])
def test_block_c1_decode(gpu_backend, orc, T):
    err, _ = _device_block_vs_oracle(CONFIGS["c1"].with_tokens(T), T)
    assert err <= REL_L2_TOL, err


def test_block_c2_fp8_prefill(gpu_backend, orc):
    err, idx = _device_block_vs_oracle(CONFIGS["c2"], 24)
    assert err <= REL_L2_TOL, err
    load = np.bincount(idx.reshape(-1), minlength=128)
    assert load.min() > 0 and load.max() < 4 * load.mean()  # logits ~N(0,1): near-uniform load


def test_block_c3_group_limited_full_size(gpu_backend, orc):
    shape = CONFIGS["c3"]
    err, idx = _device_block_vs_oracle(shape, 48, tokens_for_routing=512, cover_work_items=True)
    assert err <= REL_L2_TOL, err
    groups = idx // (shape.E // shape.n_group)
    assert all(len(set(g)) <= shape.topk_group for g in groups[::16].tolist())


def test_block_c4_zipf_full_size(gpu_backend, orc):
    shape = CONFIGS["c4"]
    err, idx = _device_block_vs_oracle(shape, 320, tokens_for_routing=256, cover_work_items=True)
    assert err <= REL_L2_TOL, err
    load = np.sort(np.bincount(idx.reshape(-1), minlength=shape.E))[::-1]
    assert load[0] > 20 * max(1, load[-1])  # Zipf(1.2): heavy skew


def test_row_results_do_not_depend_on_batch(gpu_backend, orc):
    """A token's output must not change with the batch it travels in (the reference's `exact`
    contract, crates/colibri-engine/src/gpu.rs:122-146)."""
    shape = CONFIGS["tiny_sig"].with_tokens(200)
    _, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = synth.host_tokens(shape, 200)
    # kernel family is a function of (rows, segments, format) only: < 8 rows per segment on average
    # runs the register-level kernel, more the tcgen05 kernel; inside a family rows are bit-stable
    small = blk.moe(x[:24])
    for n in (1, 7, 16):
        assert np.array_equal(blk.moe(x[:n]), small[:n])
    big = blk.moe(x)
    for n in (40, 96, 150):
        assert np.array_equal(blk.moe(x[:n]), big[:n])
    assert rel_l2(small, big[:24]) < 2e-3  # across families only the f32 summation order differs
    blk.close()


# ---- the reference's host-pointer expert calls ------------------------------------------------------------
def test_expert_mlp_and_group_nvfp4(gpu_backend, orc):
    shape = CONFIGS["tiny_sig"]
    L, packed = host_layer(shape)
    layer = upload_layer(shape, packed)
    rng = np.random.default_rng(11)
    for S in (1, 4, 16, 32, 33):   # every kernel arm of the reference's own GPU test (gpu.rs:2291-2351)
        x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((S, shape.H)).astype(np.float32)))
        e = layer.experts[3]
        y = gpu_backend.expert_mlp_nvfp4(e.gate, e.up, e.down, x)
        want = L.expert_ffn(3, x)
        assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()
    rows = [3, 1, 9]
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((sum(rows), shape.H)).astype(np.float32)))
    es = [layer.experts[i] for i in (0, 5, 2)]
    y = gpu_backend.expert_group_nvfp4([e.gate for e in es], [e.up for e in es], [e.down for e in es], rows, x)
    off = 0
    for ei, r in zip((0, 5, 2), rows):
        want = L.expert_ffn(ei, x[off:off + r])
        assert np.abs(y[off:off + r] - want).max() <= 1e-2 * np.abs(want).max()
        off += r
    from speedycolibri_b200.backend import CudaError
    with pytest.raises(CudaError):  # shape mismatch is refused, as in backend_cuda.cu:3669-3671
        gpu_backend.expert_mlp_nvfp4(es[0].gate, es[0].down, es[0].down, x)


def test_expert_mlp_fp8_row_scaled(gpu_backend, orc):
    """fmt 4 (per-row scaled e4m3), the reference's resident fp8 expert format (linear.rs:93-109)."""
    rng = np.random.default_rng(2)
    H, I, S = 256, 128, 5
    mats = []
    for O, K in ((I, H), (I, H), (H, I)):
        w = (rng.standard_normal((O, K)) * 0.02).astype(np.float32)
        sc = (np.abs(w).max(axis=1) / 448.0).astype(np.float32)
        codes = np.array([[orc.lib().orc_f32_to_e4m3(float(v)) for v in row] for row in (w / sc[:, None])], np.uint8)
        mats.append((codes, sc))
    ts = [gpu_backend.CudaTensor.upload(c, s, FMT_E4M3_ROW, K, O) for (c, s), (O, K) in zip(mats, ((I, H), (I, H), (H, I)))]
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((S, H)).astype(np.float32)))
    y = gpu_backend.expert_mlp_fp8(ts[0], ts[1], ts[2], x)
    g = orc.matmul_qt(FMT_E4M3_ROW, mats[0][0], mats[0][1], 1.0, x, I)
    u = orc.matmul_qt(FMT_E4M3_ROW, mats[1][0], mats[1][1], 1.0, x, I)
    h = (g / (1 + np.exp(-g)) * u).astype(np.float32)
    want = orc.matmul_qt(FMT_E4M3_ROW, mats[2][0], mats[2][1], 1.0, h, H)
    assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()


# ---- stage calls (what expert parallelism is assembled from), emulated on one GPU -------------------------------
@pytest.mark.parametrize("world,name", [(1, "tiny_sig"), (2, "tiny_sig"), (4, "tiny_sig"), (2, "mid")])
def test_stage_calls_emulate_expert_parallel(gpu_backend, orc, world, name):
    """`world` handles on ONE GPU stand for the ranks (a single process, stages run one after the
    other, the all-gather done by concatenation and the reduce-scatter by a sum in rank order) —
    ranks never wait on one another on the device."""
    import torch
    from speedycolibri_b200.cluster import ExpertSharding
    from speedycolibri_b200.moe import Config, MoeBlock

    shape = CONFIGS[name].with_tokens((40 if name == "tiny_sig" else 160) * world)
    L, packed = host_layer(shape)
    x_all_h = synth.host_tokens(shape, shape.T)
    want = L.moe_block(x_all_h, world=world)
    sh = ExpertSharding.new(world, shape.E)
    T, Tl, k, H = shape.T, shape.T // world, shape.k, shape.H
    st = torch.cuda.current_stream().cuda_stream
    blks = []
    for r in range(world):
        layer = upload_layer(shape, packed, local=set(sh.local_experts(r)))
        blks.append(MoeBlock(Config.from_shape(shape), layer, T, ep_rank=r, ep_world=world))
        assert blks[r].local_experts() == sh.count_for(r)
    x_all = torch.from_numpy(x_all_h.view(np.int16)).cuda().view(torch.bfloat16)
    idx_all = torch.empty((T, k), dtype=torch.int32, device="cuda")
    w_all = torch.empty((T, k), dtype=torch.float32, device="cuda")
    for r in range(world):  # every rank routes its own tokens; "all-gather" = adjacent slices
        sl = slice(r * Tl, (r + 1) * Tl)
        blks[r].topk_dev(x_all[sl], idx_all[sl], w_all[sl], st)
    torch.cuda.synchronize()
    assert np.array_equal(idx_all.cpu().numpy(), want["idx"])
    assert np.array_equal(w_all.cpu().numpy().view(np.uint32), want["w"].view(np.uint32))
    total = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    rows_seen = 0
    for r in range(world):
        rows = torch.empty((T * k, H), dtype=torch.bfloat16, device="cuda")
        y = torch.empty_like(rows)
        seg = torch.zeros(max(1, sh.count_for(r)), dtype=torch.int32, device="cuda")
        slot = torch.empty(T * k, dtype=torch.int32, device="cuda")
        part = torch.empty((T, H), dtype=torch.float32, device="cuda")
        blks[r].gather_local_dev(x_all, idx_all, rows, seg, slot, st)
        blks[r].experts_dev(rows, seg, T * k // world, y, st)
        blks[r].combine_partial_dev(y, slot, w_all, part, st)
        total += part  # ascending rank order, as moe.rs:1725-1733 folds peer partials
        torch.cuda.synchronize()
        blks[r].check()
        # bookkeeping: this rank saw exactly the pairs routed to its experts
        local = set(sh.local_experts(r))
        n_local_pairs = int(np.isin(want["idx"], list(local)).sum())
        assert int(seg.sum()) == n_local_pairs and int((slot >= 0).sum()) == n_local_pairs
        rows_seen += n_local_pairs
    assert rows_seen == T * k
    outs = []
    for r in range(world):
        sl = slice(r * Tl, (r + 1) * Tl)
        sy = torch.empty((Tl, H), dtype=torch.bfloat16, device="cuda")
        blks[r].shared_dev(x_all[sl].contiguous(), sy, st)
        o = torch.empty((Tl, H), dtype=torch.bfloat16, device="cuda")
        blks[r].finish_dev(total[sl].contiguous(), sy, o, st)
        outs.append(o)
    torch.cuda.synchronize()
    got = torch.cat(outs).view(torch.int16).cpu().numpy().view(np.uint16)
    assert rel_l2(got, want["out"]) <= REL_L2_TOL
    layer = upload_layer(shape, packed)
    one = MoeBlock(Config.from_shape(shape), layer, T)
    assert rel_l2(got, one.moe(x_all_h)) <= 2e-3  # same kernels, one extra f32 fold
    one.close()
    for b in blks:
        b.close()


@pytest.mark.parametrize("transport", ["direct", "nccl"])
@pytest.mark.parametrize("world,name,T,balanced", [(2, "tiny_sig", 37, False), (4, "tiny_sig", 150, False), (3, "tiny_zipf", 70, True),
                                                    (2, "mid", 512, False), (8, "mid", 1000, True), (2, "tiny", 5, False)])
def test_expert_parallel_call_emulated_on_one_gpu(gpu_backend, orc, monkeypatch, world, name, T, balanced, transport):
    """The expert-parallel block call with `world` handles on ONE GPU (coli_b200_moe_block_ep_emulate:
    same kernels, same offsets; the peers' buffers are plain pointers, the barriers stream order):
    ragged token shards (one of them empty), contiguous and LPT expert maps, a rank that owns no
    expert of some tokens; both transports (rows stored straight into the peers' receive slabs, or
    packed and copied as the ncclSend / ncclRecv form lays them out).  Routing must be exact and
    every rank's output within the bar against the oracle."""
    import ctypes as C

    import torch

    monkeypatch.setenv("COLI_EP_TRANSPORT", transport)  # read when a handle's expert-parallel state is created

    from speedycolibri_b200 import _lib
    from speedycolibri_b200.cluster import ExpertSharding, ep_layout, rows_per_rank

    lib = _lib.load()
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    x_all = synth.host_tokens(shape, T)
    want = L.moe_block(x_all)
    load = np.bincount(want["idx"].reshape(-1), minlength=shape.E).tolist()
    sh = ExpertSharding.balanced(world, shape.E, load) if balanced else ExpertSharding.new(world, shape.E)
    # ragged shards; rank 1 gets nothing when there are more than two ranks
    cut = np.linspace(0, T, world + 1).astype(int)
    if world > 2:
        cut[2] = cut[1]
    blocks, xs, outs = [], [], []
    for r in range(world):
        layer = upload_layer(shape, packed, local=set(sh.local_experts(r)))
        blocks.append(make_block(shape, layer, max_tokens=T, ep_rank=r, ep_world=world,
                                 expert_owner=sh.owner_table() if balanced else None))
        xs.append(torch.from_numpy(x_all[cut[r]:cut[r + 1]].view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(-1, shape.H))
        outs.append(torch.zeros_like(xs[-1]))
    hp = (C.c_void_p * world)(*[b.handle for b in blocks])
    xp = (C.c_void_p * world)(*[t.data_ptr() if t.numel() else None for t in xs])
    op = (C.c_void_p * world)(*[t.data_ptr() if t.numel() else None for t in outs])
    tl = (C.c_int * world)(*[int(t.shape[0]) for t in xs])
    for rep in range(2):  # buffers are reused
        ok = lib.coli_b200_moe_block_ep_emulate(hp, world, xp, op, tl, None)
        assert ok == 1, lib.coli_cuda_last_error().decode()
    torch.cuda.synchronize()
    for r, b in enumerate(blocks):
        b.check()
        n = int(tl[r])
        if n == 0:
            continue
        idx, w = b.last_routing(n)
        assert np.array_equal(idx, want["idx"][cut[r]:cut[r + 1]])
        assert np.array_equal(w.view(np.uint32), want["w"][cut[r]:cut[r + 1]].view(np.uint32))
        got = outs[r].view(torch.int16).cpu().numpy().view(np.uint16)
        err = rel_l2(got, want["out"][cut[r]:cut[r + 1]])
        assert err <= 5e-3, (r, err)
    # the count table: every pair is computed exactly once, by the rank that owns its expert
    tab = blocks[0].ep_last_counts()
    assert tab[:, 1, :].sum() == T * shape.k
    own = np.array(sh.owner_table())
    assert rows_per_rank(tab).tolist() == [int((own[want["idx"]] == r).sum()) for r in range(world)]
    for r in range(world):
        lay = ep_layout(tab, r)
        assert lay["send_tok"].sum() <= int(tl[r]) * min(shape.k, world) and lay["recv_off"][r] == 0
    for b in blocks:
        b.close()


def test_expert_parallel_barrier_wait_is_bounded(gpu_backend, monkeypatch):
    """The barrier of the direct transport waits for its peers with a limit: when nothing ever sets the
    peers' counts the kernel returns, the context stays usable and the handle's check reports the
    abandoned barrier once; when the counts are there the barrier passes.  One handle, one kernel at
    a time: no kernel here waits for another launch."""
    import ctypes as C

    import torch

    monkeypatch.setenv("COLI_EP_TRANSPORT", "direct")
    from speedycolibri_b200 import _lib
    from speedycolibri_b200.backend import CudaError
    from speedycolibri_b200.cluster import ExpertSharding

    lib = _lib.load()
    world, shape = 2, CONFIGS["tiny_sig"].with_tokens(16)
    _, packed = host_layer(shape)
    sh = ExpertSharding.new(world, shape.E)
    blocks = [make_block(shape, upload_layer(shape, packed, local=set(sh.local_experts(r))), max_tokens=16, ep_rank=r, ep_world=world)
              for r in range(world)]
    x_all = synth.host_tokens(shape, 16)
    xs = [torch.from_numpy(x_all[8 * r:8 * r + 8].view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(-1, shape.H) for r in range(world)]
    outs = [torch.zeros_like(t) for t in xs]
    hp = (C.c_void_p * world)(*[b.handle for b in blocks])
    xp = (C.c_void_p * world)(*[t.data_ptr() for t in xs])
    op = (C.c_void_p * world)(*[t.data_ptr() for t in outs])
    tl = (C.c_int * world)(8, 8)
    assert lib.coli_b200_moe_block_ep_emulate(hp, world, xp, op, tl, None) == 1, lib.coli_cuda_last_error().decode()
    torch.cuda.synchronize()
    blocks[0].check()
    # peers present: passes
    assert lib.coli_b200_ep_barrier_probe(blocks[0].handle, 1, None) == 1, lib.coli_cuda_last_error().decode()
    torch.cuda.synchronize()
    blocks[0].check()
    # rank 1 never arrives: the wait runs out (about 13 ms), is reported once, and the handle keeps working
    assert lib.coli_b200_ep_barrier_probe(blocks[0].handle, 0, None) == 1
    torch.cuda.synchronize()
    with pytest.raises(CudaError, match="barrier"):
        blocks[0].check()
    blocks[0].check()
    assert lib.coli_b200_moe_block_ep_emulate(hp, world, xp, op, tl, None) == 1
    torch.cuda.synchronize()
    for b in blocks:
        b.check()
        b.close()


@pytest.mark.parametrize("name", ["tiny", "tiny_sig", "tiny_fp8", "tiny_mx", "tiny_zipf", "mid_ragged"])
def test_block_against_committed_fixture(gpu_backend, name):
    """The device block against the committed fixtures of tests/golden (made by make_golden.py from the
    pinned oracle): routing bits exact, output within the bar.  The digests tie the fixture to the inputs."""
    import hashlib
    import os

    want = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"block_{name}.npz"))
    shape = CONFIGS[name]
    _, packed = host_layer(shape)
    x = synth.host_tokens(shape)
    assert hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest() == str(want["x_sha"])
    blk = make_block(shape, upload_layer(shape, packed))
    out, idx, w = blk.moe(x, want_routing=True)
    blk.check()
    assert np.array_equal(idx, want["idx"]) and np.array_equal(w.view(np.uint32), want["w_bits"])
    assert rel_l2(np.asarray(out).view(np.uint16), want["out_bits"]) <= REL_L2_TOL
    blk.close()


def test_tracing_phases_and_launch_count(gpu_backend):
    import torch
    from speedycolibri_b200 import _lib

    shape = CONFIGS["tiny_sig"]
    _, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    x = torch.from_numpy(synth.host_tokens(shape).view(np.int16)).cuda().view(torch.bfloat16)
    n0 = _lib.load().coli_b200_launch_count()
    blk.forward(x)
    torch.cuda.synchronize()
    assert _lib.load().coli_b200_launch_count() - n0 == 6  # router 2, permute 1 (small batch), gate/up, down, combine
    blk.profile(True)
    for _ in range(3):
        blk.forward(x)
    ms, calls = blk.phase_ms()
    blk.profile(False)
    assert calls == 3 and all(v > 0 for v in ms.values())
    blk.close()


def test_decode_front_is_one_launch(gpu_backend):
    """T <= 8: router, top-k and permutation share one launch; repeated calls stay exact."""
    import torch
    from speedycolibri_b200 import _lib

    shape = CONFIGS["tiny"]
    layer, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    xh = synth.host_tokens(shape)
    x = torch.from_numpy(xh.view(np.int16)).cuda().view(torch.bfloat16)
    n0 = _lib.load().coli_b200_launch_count()
    blk.forward(x)
    torch.cuda.synchronize()
    assert _lib.load().coli_b200_launch_count() - n0 == 4  # front end, gate/up, down, combine
    want_idx, want_w = layer.route_tokens(xh)
    for _ in range(3):  # the ticket word returns to zero after every launch
        blk.forward(x)
        idx, w = blk.last_routing(shape.T)
        assert np.array_equal(idx, want_idx)
        assert np.array_equal(w.view(np.uint32), want_w.view(np.uint32))
    blk.close()


@pytest.mark.parametrize("act", [(1, 1.702, 0.2), (0, 0.0, 0.15)], ids=["swiglu_oai", "swiglu_clamped"])
@pytest.mark.parametrize("name,T", [("tiny", 5), ("tiny_fp8", 19), ("mid", 433)])
def test_block_other_activations(gpu_backend, orc, name, T, act):
    """The process-wide activation setting (coli_cuda_set_activation): clamped OpenAI-SwiGLU and
    the asymmetric-clamp SwiGLU, on the decode kernel (tiny*) and the tcgen05 kernel (mid).  The
    limits are small enough that about half of the gate/up values are clamped."""
    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    x = synth.host_tokens(shape, T)
    plain = L.moe_block(x)["out"]
    try:
        orc.set_activation(*act)
        gpu_backend.set_activation(*act)
        blk = make_block(shape, upload_layer(shape, packed))  # a handle keeps the setting it was created under
        out = blk.moe(x)
        blk.check()
        want = L.moe_block(x)["out"]
    finally:
        orc.set_activation(0, 1.702, 0.0)
        gpu_backend.set_activation(0, 0.0, 0.0)
    assert rel_l2(want, plain) > 0.05, "the activation setting must change the result"
    err = rel_l2(out, want)
    assert err <= 5e-3, err
    blk.close()


def test_generic_expert_calls_and_nvfp4_matmul(gpu_backend, orc):
    """coli_cuda_expert_mlp / coli_cuda_expert_group (format taken from the handles) and
    coli_cuda_matmul_nvfp4 (one matrix, slot reused between calls)."""
    shape = CONFIGS["tiny_sig"]
    L, packed = host_layer(shape)
    layer = upload_layer(shape, packed)
    rng = np.random.default_rng(5)
    rows = [2, 7]
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((sum(rows), shape.H)).astype(np.float32)))
    e = layer.experts[1]
    y = gpu_backend.expert_mlp(e.gate, e.up, e.down, x[:4])
    want = L.expert_ffn(1, x[:4])
    assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()
    es = [layer.experts[i] for i in (4, 1)]
    y = gpu_backend.expert_group([t.gate for t in es], [t.up for t in es], [t.down for t in es], rows, x)
    off = 0
    for ei, r in zip((4, 1), rows):
        want = L.expert_ffn(ei, x[off:off + r])
        assert np.abs(y[off:off + r] - want).max() <= 1e-2 * np.abs(want).max()
        off += r
    # a single NVFP4 matrix, ragged K and O, every row-count arm of the kernel
    O, I = 72, 200
    w = (rng.standard_normal((O, I)) * 0.05).astype(np.float32)
    nib, bs, g = orc.quantize_nvfp4(w)
    mm = gpu_backend.Nvfp4Matmul(nib, bs, g, O, I)
    for S in (1, 8, 9, 33, 70):
        xs = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((S, I)).astype(np.float32)))
        got = mm(xs)
        want = orc.matmul_qt(FMT_NVFP4, nib, bs, g, xs, O)
        assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max(), S
    mm.free()
    from speedycolibri_b200.backend import CudaError, F32Matmul
    f32 = F32Matmul(rng.standard_normal((8, 16)).astype(np.float32))
    f32(np.zeros((1, 16), np.float32))
    with pytest.raises(CudaError):  # an f32 tensor is not a resident expert format: declined, not computed
        import ctypes as C
        from speedycolibri_b200 import _lib
        from speedycolibri_b200.backend import _check
        yb = np.zeros((1, 16), np.float32)
        _check(_lib.load().coli_cuda_expert_mlp(f32.slot, f32.slot, f32.slot, yb.ctypes.data, yb.ctypes.data, 1), "coli_cuda_expert_mlp")
    f32.free()


def test_gateless_relu2_experts(gpu_backend, orc):
    """Gateless ReLU^2 experts, y = down(relu(up x)^2): moe.rs:1189-1199 restated with the oracle's
    matmul (the reference's own check is moe.rs:3386-3455: same composition, same tolerance class)."""
    shape = CONFIGS["tiny_sig"]
    L, packed = host_layer(shape)
    layer = upload_layer(shape, packed)
    rng = np.random.default_rng(17)

    def want_ffn(ei, x):
        _gate, up, down = packed["experts"][ei]  # each (codes, scales, tensor scale)
        u = orc.matmul_qt(FMT_NVFP4, up[0], up[1], up[2], x, shape.I)
        r = np.maximum(u, np.float32(0.0))
        return orc.matmul_qt(FMT_NVFP4, down[0], down[1], down[2], (r * r).astype(np.float32), shape.H)

    for S in (1, 9, 40):
        x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((S, shape.H)).astype(np.float32)))
        e = layer.experts[2]
        want = want_ffn(2, x)
        assert np.abs(want).max() > 0
        for exact in (False, True):
            y = gpu_backend.expert_mlp_relu2(e.up, e.down, x, exact)
            assert np.abs(y - want).max() <= 1e-2 * np.abs(want).max()
    rows = [5, 1, 12]
    ids = (6, 0, 3)
    x = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(rng.standard_normal((sum(rows), shape.H)).astype(np.float32)))
    es = [layer.experts[i] for i in ids]
    for seg in (False, True):
        y = gpu_backend.expert_group_relu2([t.up for t in es], [t.down for t in es], rows, x, seg=seg)
        off = 0
        for ei, r in zip(ids, rows):
            want = want_ffn(ei, x[off:off + r])
            assert np.abs(y[off:off + r] - want).max() <= 1e-2 * np.abs(want).max()
            off += r


def test_layer_loaded_from_container(gpu_backend, orc, tmp_path):
    """Experts written in the reference's container form (nibbles ++ scales blob + .g sidecar),
    loaded into HBM by name, give the same block output as the oracle on the same weights."""
    from speedycolibri_b200 import container
    from speedycolibri_b200.moe import Layer

    shape = CONFIGS["tiny"]
    L, packed = host_layer(shape)
    tensors = {}
    for e, p in enumerate(packed["experts"]):
        tensors.update(container.expert_tensors(2, e, p))
    tensors.update(container.expert_tensors(2, "shared", packed["shared"]))
    container.write_safetensors(str(tmp_path / "layer.safetensors"), tensors)
    experts, shared, _fmt = container.load_layer(container.Shards(str(tmp_path)), 2, shape.H, shape.I, shape.E, shared_id="shared")
    layer = Layer(router=packed["router"], experts=experts, router_bias=packed["select_bias"], logit_bias=packed["logit_bias"],
                  shared=shared)
    blk = make_block(shape, layer)
    x = synth.host_tokens(shape, shape.T)
    out, idx, w = blk.moe(x, want_routing=True)
    want = L.moe_block(x)
    assert np.array_equal(idx, want["idx"]) and np.array_equal(w.view(np.uint32), want["w"].view(np.uint32))
    assert rel_l2(out, want["out"]) <= 5e-3
    blk.close()


@pytest.mark.parametrize("name,T", [("tiny", 5), ("tiny_sig", 37), ("mid", 433)])
def test_layer_step_rmsnorm_block_residual(gpu_backend, orc, name, T):
    """coli_b200_moe_layer_step_dev against the reference's layer loop (forward.rs:376-393) restated
    with the oracle: nrm = rmsnorm(x) (math.rs:8-20), tmp = moe(bf16(nrm)), x += tmp."""
    import torch

    shape = CONFIGS[name].with_tokens(T)
    L, packed = host_layer(shape)
    blk = make_block(shape, upload_layer(shape, packed))
    rng = np.random.default_rng(T)
    resid = (rng.standard_normal((T, shape.H)) * 3.0).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(shape.H)).astype(np.float32)
    eps = 1e-5
    nrm_bits = synth.f32_to_bf16_bits(orc.rmsnorm(resid, w, eps))
    want = L.moe_block(nrm_bits)
    r = torch.from_numpy(resid.copy()).cuda()
    blk.layer_step(r, torch.from_numpy(w).cuda(), eps)
    blk.check()
    idx, rw = blk.last_routing(T)
    assert np.array_equal(idx, want["idx"]) and np.array_equal(rw.view(np.uint32), want["w"].view(np.uint32)), \
        "the normed rows must round to the same bf16 values, or the routing differs"
    delta = r.cpu().numpy().astype(np.float64) - resid.astype(np.float64)
    ref = synth.bf16_bits_to_f32(want["out"]).astype(np.float64)
    err = np.linalg.norm(delta - ref) / np.linalg.norm(ref)
    assert err <= 5e-3, err
    blk.close()
