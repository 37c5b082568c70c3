"""Pins the CPU oracle to the known-answer vectors the reference's own unit tests hold for this
path (values read from the reference's test source; cited per test)."""
import math

import numpy as np
import pytest

from speedycolibri_b200.configs import SCORE_SIGMOID, SCORE_SOFTMAX

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def f32(x):
    return float(np.float32(x))


def route_layer(orc, score, k, norm, scale, bias=None, E=4, n_group=1, topk_group=1):
    router = np.zeros((E, 4), np.uint16)
    return orc.Layer(4, E, k, 3, score, norm, scale, n_group, topk_group, 0, router, [None] * E, None, bias, None)


# crates/colibri-engine/src/convert.rs:2512-2535  float_to_e4m3_matches_hardware
E4M3_ENCODE = [(0.0, 0x00), (0.1, 0x1D), (0.5, 0x30), (1.0, 0x38), (1.5, 0x3C), (2.0, 0x40), (3.14159, 0x45),
               (7.0, 0x4E), (15.5, 0x58), (100.0, 0x6C), (448.0, 0x7E), (500.0, 0x7E), (-1.0, 0xB8), (-0.5, 0xB0),
               (-256.0, 0xF8), (0.015625, 0x08), (0.0078125, 0x04), (0.001, 0x01), (2.5, 0x42), (0.3, 0x2A),
               (0.017, 0x09), (255.9, 0x78)]


def test_float_to_e4m3_matches_hardware(orc):
    L = orc.lib()
    for x, want in E4M3_ENCODE:
        assert L.orc_f32_to_e4m3(x) == want, (x, hex(L.orc_f32_to_e4m3(x)), hex(want))


def test_float_to_e4m3_is_nearest_even_everywhere(orc):
    """Independent brute force: the nearest of the 127 finite magnitudes, ties to the even code."""
    L = orc.lib()
    vals = np.array([L.orc_e4m3_to_f32(c) for c in range(0x7F)], np.float64)  # codes 0..0x7E ascending
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.uniform(0, 460, 4000), rng.uniform(0, 0.05, 3000), 2.0 ** rng.uniform(-12, 9, 4000),
                         (vals[:-1] + vals[1:]) / 2]).astype(np.float32)
    for x in xs:
        a = float(x)
        d = np.abs(vals - min(a, 448.0))
        best = int(np.argmin(d))
        ties = np.flatnonzero(d == d[best])
        if len(ties) > 1:
            best = int([t for t in ties if t % 2 == 0][0])
        assert L.orc_f32_to_e4m3(a) == best, (a, L.orc_f32_to_e4m3(a), best)
        assert L.orc_f32_to_e4m3(-a) == (best | 0x80)


# crates/colibri-core/src/dtype.rs:297-310  f8e4m3_known_values
def test_e4m3_decode_known_values(orc):
    L = orc.lib()
    for code, want in [(0x00, 0.0), (0x38, 1.0), (0x40, 2.0), (0x30, 0.5), (0x3C, 1.5), (0xB8, -1.0), (0x7E, 448.0),
                       (0x01, 2.0 ** -9), (0x80, 0.0)]:
        assert L.orc_e4m3_to_f32(code) == want


# crates/colibri-engine/src/convert.rs:2583-2599  e2m1 grid, tie 5.0 -> 4.0, saturation, 0.2 -> 0
def test_e2m1_grid(orc):
    L = orc.lib()
    for i, v in enumerate(E2M1):
        assert L.orc_e2m1_code(v) == i and L.orc_e2m1_to_f32(i) == v
        if v:
            assert L.orc_e2m1_code(-v) == (i | 8) and L.orc_e2m1_to_f32(i | 8) == -v
    assert L.orc_e2m1_to_f32(L.orc_e2m1_code(5.0)) == 4.0
    assert L.orc_e2m1_to_f32(L.orc_e2m1_code(100.0)) == 6.0
    assert L.orc_e2m1_to_f32(L.orc_e2m1_code(0.2)) == 0.0


# crates/colibri-core/src/dtype.rs:237-251  bf16 exhaustive round trip
def test_bf16_roundtrip_exhaustive(orc):
    L = orc.lib()
    for h in range(0, 0x10000, 1):
        v = L.orc_bf16_to_f32(h)
        if math.isnan(v):
            continue
        assert L.orc_f32_to_bf16(v) == h


def test_bf16_rounds_to_nearest_even(orc):
    L = orc.lib()
    assert L.orc_f32_to_bf16(f32(1.0 + 2.0 ** -8)) == 0x3F80        # tie -> even (down)
    assert L.orc_f32_to_bf16(f32(1.0 + 3 * 2.0 ** -8)) == 0x3F82    # tie -> even (up)
    assert L.orc_f32_to_bf16(f32(1.0 + 2.0 ** -8 + 2.0 ** -20)) == 0x3F81


# crates/colibri-engine/src/convert.rs:2662-2700  nvfp4_encode_decode_matches_sim
def test_nvfp4_encode_decode_matches_sim(orc):
    o, i = 8, 128
    w = np.zeros((o, i), np.float32)
    for r in range(o):
        for c in range(i):
            w[r, c] = np.float32(10.0) ** (-((c // 16) % 4)) * (-1.0 if (r + c) % 3 == 0 else 1.0)
    nib, bs, g = orc.quantize_nvfp4(w)
    assert nib.shape == (o, i // 2) and bs.shape == (o, i // 16)
    L = orc.lib()
    dec = np.zeros_like(w)
    for r in range(o):
        for c in range(i):
            byte = int(nib[r, c >> 1])
            code = (byte >> 4) if c & 1 else (byte & 0xF)
            dec[r, c] = L.orc_e2m1_to_f32(code) * L.orc_e4m3_to_f32(int(bs[r, c // 16])) * g
    # the simulated reconstruction (convert.rs:1690-1715): nearest ue4m3 scale, nearest e2m1 value
    ue = np.array(sorted({L.orc_e4m3_to_f32(c) for c in range(0x7F)}), np.float64)
    lev = np.array(E2M1)
    amax = float(np.abs(w).max())
    glob = max(f32(amax / (6.0 * 448.0)), np.finfo(np.float32).tiny)
    sim = np.zeros_like(w)
    for r in range(o):
        for b in range(i // 16):
            blk = w[r, 16 * b:16 * b + 16].astype(np.float64)
            sf = ue[np.argmin(np.abs(ue - np.abs(blk).max() / 6.0 / glob))]
            eff = sf * glob
            q = np.array([lev[np.argmin(np.abs(lev - abs(v) / eff))] * np.sign(v) for v in blk]) if eff > 0 else 0 * blk
            sim[r, 16 * b:16 * b + 16] = q * eff
    rel = math.sqrt(((dec.astype(np.float64) - sim) ** 2).sum() / max((sim.astype(np.float64) ** 2).sum(), 1e-30))
    assert rel < 1e-4, rel
    # and the documented global: amax / (6 * 448)
    assert g == f32(f32(amax) / f32(6.0 * 448.0))


# crates/colibri-engine/src/linear.rs:449-485  one-hot probe: matmul output IS the weight column
def test_matmul_qt_onehot_is_dequant(orc):
    o, i = 3, 32
    w = np.sin(np.arange(o * i, dtype=np.float32) * np.float32(0.23)).reshape(o, i).astype(np.float32)
    nib, bs, g = orc.quantize_nvfp4(w)
    L = orc.lib()
    dense = orc.dequant(orc.FMT_NVFP4, nib, bs, g, o, i)
    for r in range(o):
        for c in range(i):
            byte = int(nib[r, c >> 1])
            code = (byte >> 4) if c & 1 else (byte & 0xF)
            want = L.orc_e2m1_to_f32(code) * L.orc_e4m3_to_f32(int(bs[r, c // 16])) * g
            assert abs(dense[r, c] - want) < 1e-5
    assert np.abs(dense - w).max() < 0.35 * np.abs(w).max()  # it is a 4-bit format, but it is this matrix


def test_expf_matches_libm(orc):
    """coli_expf (f64 evaluation, one rounding) against numpy's f64 exp rounded to f32."""
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.uniform(-104, 89, 400000), rng.normal(0, 3, 400000), [0.0, -0.0, 88.72, -103.9, 1e-8]]).astype(np.float32)
    y = np.empty_like(x)
    orc.lib().orc_expf_array(x.ctypes.data, y.ctypes.data, x.size)
    with np.errstate(over="ignore"):  # the last inputs round to +inf in f32, as they should
        want = np.exp(x.astype(np.float64)).astype(np.float32)
    assert np.array_equal(y, want)


# crates/colibri-engine/src/moe.rs:2252-2277  route_softmax_topk_renormalized
def test_route_softmax_topk_renormalized(orc):
    L = route_layer(orc, SCORE_SOFTMAX, 2, True, 1.0, bias=np.array([5, 0, 0, 0], np.float32))
    idx, w = L.route_logits(np.array([0.0, 2.0, -1.0, 0.3], np.float32))
    assert idx.tolist() == [1, 3]  # bias ignored by the softmax arm
    e1, e3 = math.exp(2.0), math.exp(0.3)
    assert abs(w[0] - e1 / (e1 + e3)) < 1e-6 and abs(w[1] - e3 / (e1 + e3)) < 1e-6
    assert abs(w[0] + w[1] - 1.0) < 1e-6
    sg = lambda z: 1 / (1 + math.exp(-z))
    assert abs(w[0] - sg(2.0) / (sg(2.0) + sg(0.3))) > 1e-3


# crates/colibri-engine/src/moe.rs:2282-2292  route_softmax_survives_large_logits
def test_route_softmax_survives_large_logits(orc):
    L = route_layer(orc, SCORE_SOFTMAX, 2, True, 1.0)
    idx, w = L.route_logits(np.array([200.0, 195.0, -300.0, 100.0], np.float32))
    assert idx.tolist() == [0, 1]
    assert np.isfinite(w).all() and abs(w.sum() - 1.0) < 1e-6
    assert abs(w[0] - 1.0 / (1.0 + math.exp(-5.0))) < 1e-6


# crates/colibri-engine/src/moe.rs:2296-2325  route_sigmoid_bias_topk_normalized_scaled
def test_route_sigmoid_bias_topk_normalized_scaled(orc):
    L = route_layer(orc, SCORE_SIGMOID, 2, True, 2.0, bias=np.array([5, 0, 0, 0], np.float32))
    idx, w = L.route_logits(np.array([0.0, 2.0, -1.0, 0.3], np.float32))
    assert sorted(idx.tolist()) == [0, 1]
    sg = lambda z: 1 / (1 + math.exp(-z))
    s0, s1 = sg(0.0), sg(2.0)
    wm = dict(zip(idx.tolist(), w.tolist()))
    assert abs(wm[0] - s0 / (s0 + s1) * 2.0) < 1e-5 and abs(wm[1] - s1 / (s0 + s1) * 2.0) < 1e-5


# crates/colibri-engine/src/moe.rs:2543-2555  route_selects_top_k_by_bias_augmented_score
def test_route_selects_top_k_by_bias_augmented_score(orc):
    L = route_layer(orc, SCORE_SIGMOID, 2, False, 1.0, bias=np.array([10, 0, 0, 0], np.float32))
    idx, w = L.route_logits(np.array([0.0, 1.0, 2.0, 3.0], np.float32))
    assert idx.tolist() == [0, 3]
    assert abs(w[0] - 0.5) < 1e-6 and abs(w[1] - 1 / (1 + math.exp(-3.0))) < 1e-6


# crates/colibri-engine/src/moe.rs:2557-2568  norm_topk_normalizes_weights
def test_norm_topk_normalizes_weights(orc):
    L = route_layer(orc, SCORE_SIGMOID, 2, True, 2.0, bias=np.zeros(4, np.float32))
    _, w = L.route_logits(np.array([3.0, 2.0, 1.0, 0.0], np.float32))
    assert abs(w.sum() - 2.0) < 1e-5


def test_route_ties_go_to_lowest_id(orc):
    L = route_layer(orc, SCORE_SOFTMAX, 3, False, 1.0, E=6)
    idx, _ = L.route_logits(np.array([1.0, 2.0, 2.0, 0.5, 2.0, 1.0], np.float32))
    assert idx.tolist() == [1, 2, 4]
    L = route_layer(orc, SCORE_SIGMOID, 2, False, 1.0, bias=np.zeros(6, np.float32), E=6)
    idx, _ = L.route_logits(np.zeros(6, np.float32))
    assert idx.tolist() == [0, 1]


def test_route_group_limited_definition(orc):
    """Not in the reference (config.rs:703-707 rejects n_group != 1): pins OUR definition —
    group score = sum of the two largest selection scores, best groups kept, ties -> lowest id."""
    E, G = 8, 4
    bias = np.zeros(E, np.float32)
    L = route_layer(orc, SCORE_SIGMOID, 2, False, 1.0, bias=bias, E=E, n_group=G, topk_group=2)
    # groups: (0,1) (2,3) (4,5) (6,7).  Expert 6 has the single largest score but its group loses on top-2 sum.
    z = np.array([1.0, 1.0, 0.9, 0.9, -5.0, -5.0, 3.0, -9.0], np.float32)
    idx, w = L.route_logits(z)
    sg = lambda v: 1 / (1 + math.exp(-v))
    sums = [sg(z[2 * g]) + sg(z[2 * g + 1]) for g in range(G)]
    keep = sorted(sorted(range(G), key=lambda g: (-sums[g], g))[:2])
    assert keep == [0, 1]
    assert idx.tolist() == [0, 1]
    assert abs(w[0] - sg(1.0)) < 1e-6
    # with one group allowed only, the choice moves with the group
    L1 = route_layer(orc, SCORE_SIGMOID, 2, False, 1.0, bias=bias, E=E, n_group=G, topk_group=1)
    z2 = np.array([0.0, 0.0, 0.0, 0.0, 2.0, 1.5, 4.0, -9.0], np.float32)
    idx, _ = L1.route_logits(z2)
    assert idx.tolist() == [4, 5]  # sg(2)+sg(1.5) > sg(4)+sg(-9)


def _expert_f32(seed, inter, d):
    # crates/colibri-engine/src/moe.rs:2327-2341  closed-form test expert
    def mk(o, i, s):
        k = np.arange(o * i)
        return ((((k * 3 + s * 7 + 1) % 9).astype(np.float32) - np.float32(4.0)) * np.float32(0.1)).reshape(o, i)
    return mk(inter, d, seed), mk(inter, d, seed + 1), mk(d, inter, seed + 2)


def _f32_layer(orc, k, experts, shared, router_f32, norm=False):
    from speedycolibri_b200.synth import f32_to_bf16_bits

    pack = lambda ex: None if ex is None else tuple((m.view(np.uint8), np.zeros(1, np.uint8), 1.0) for m in ex)
    L = orc.Layer(4, 4, k, 3, SCORE_SIGMOID, norm, 1.0, 1, 1, 0, f32_to_bf16_bits(router_f32),
                  [pack(e) for e in experts], pack(shared), np.zeros(4, np.float32), None)
    return L


# crates/colibri-engine/src/moe.rs:2570-2611  single_expert_moe_equals_weighted_ffn
def test_single_expert_moe_equals_weighted_ffn(orc):
    from speedycolibri_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits

    router = np.zeros((4, 4), np.float32)
    router[2, :] = 1.0
    ex2 = _expert_f32(20, 3, 4)
    L = _f32_layer(orc, 1, [None, None, ex2, None], None, router)
    xb = f32_to_bf16_bits(np.array([[0.3, 0.5, -0.2, 0.7]], np.float32))
    r = L.moe_block(xb)
    assert r["idx"].tolist() == [[2]]
    x = bf16_bits_to_f32(xb)
    logit = np.float32(0)
    for v in x[0]:
        logit = np.float32(logit + v)
    w = orc.lib().orc_sigmoidf(float(logit))
    assert r["w"][0, 0] == np.float32(w)
    ffn = L.expert_ffn(2, x)
    assert np.abs(r["out_f32"] - np.float32(w) * ffn).max() < 1e-5


# crates/colibri-engine/src/moe.rs:2613-2646  shared_expert_adds_its_ffn
def test_shared_expert_adds_its_ffn(orc):
    from speedycolibri_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits

    router = np.full((4, 4), 0.1, np.float32)
    experts = [_expert_f32(e * 5, 3, 4) for e in range(4)]
    sh = _expert_f32(50, 3, 4)
    xb = f32_to_bf16_bits(np.array([[0.2, -0.1, 0.4, 0.3]], np.float32))
    with_sh = _f32_layer(orc, 2, experts, sh, router).moe_block(xb)["out_f32"]
    Lw = _f32_layer(orc, 2, experts, None, router)
    without = Lw.moe_block(xb)["out_f32"]
    sh_out = _f32_layer(orc, 2, experts, sh, router).expert_ffn(4, bf16_bits_to_f32(xb))
    assert np.abs(with_sh - without - sh_out).max() < 1e-5


def test_block_matches_dense_numpy(orc):
    """The whole oracle block against a straightforward numpy evaluation on dequantised weights."""
    from speedycolibri_b200.configs import CONFIGS
    from speedycolibri_b200.synth import bf16_bits_to_f32, host_tokens
    from tests.helpers import host_layer

    for name in ("tiny", "tiny_sig", "tiny_fp8", "tiny_zipf"):
        shape = CONFIGS[name]
        L, packed = host_layer(shape)
        xb = host_tokens(shape)
        r = L.moe_block(xb)
        x = bf16_bits_to_f32(xb).astype(np.float64)
        deq = lambda ex, mi, O, K: orc.dequant(shape.fmt, ex[mi][0], ex[mi][1], ex[mi][2], O, K).astype(np.float64)
        def ffn(ex, v):
            g, u, d = deq(ex, 0, shape.I, shape.H), deq(ex, 1, shape.I, shape.H), deq(ex, 2, shape.H, shape.I)
            a, b = v @ g.T, v @ u.T
            return (a / (1 + np.exp(-a)) * b) @ d.T
        want = np.zeros((shape.T, shape.H))
        for t in range(shape.T):
            for kk in range(shape.k):
                want[t] += float(r["w"][t, kk]) * ffn(packed["experts"][int(r["idx"][t, kk])], x[t:t + 1])[0]
        if shape.shared:
            want += ffn(packed["shared"], x)
        err = np.linalg.norm(r["out_f32"] - want) / np.linalg.norm(want)
        assert err < 1e-5, (name, err)
        # routing weights: each token's experts are distinct and sorted by score
        assert all(len(set(row)) == shape.k for row in r["idx"].tolist())


def test_sharded_oracle_equals_single_node(orc):
    """crates/colibri-engine/src/moe.rs:2753-2850: sharded == single-node within 1e-5."""
    from speedycolibri_b200.configs import CONFIGS
    from speedycolibri_b200.synth import host_tokens
    from tests.helpers import host_layer

    shape = CONFIGS["tiny_sig"]
    L, _ = host_layer(shape)
    xb = host_tokens(shape)
    one = L.moe_block(xb)["out_f32"]
    for world in (2, 4):
        sh = L.moe_block(xb, world=world)["out_f32"]
        assert np.abs(sh - one).max() <= 1e-5 * max(1.0, np.abs(one).max())
    own = np.array([e % 2 for e in range(shape.E)], np.int32)
    sh = L.moe_block(xb, world=2, owner=own)["out_f32"]
    assert np.abs(sh - one).max() <= 1e-5 * max(1.0, np.abs(one).max())


def test_swiglu_oai_shape(orc):
    """crates/colibri-engine/src/math.rs:238-256 (swiglu_oai_shape)."""
    alpha, limit = 1.702, 7.0
    f = lambda g, u: orc.act_combine(g, u, 1, alpha, limit)
    assert abs(f(0.0, 3.0)) < 1e-6
    g, u = 1.5, 2.0
    assert abs(f(g, u) - (g / (1.0 + math.exp(-alpha * g))) * (u + 1.0)) < 1e-6
    clamped = (limit / (1.0 + math.exp(-alpha * limit))) * (limit + 1.0)
    assert abs(f(100.0, 100.0) - clamped) < 1e-4
    assert abs(f(2.0, -50.0) - (2.0 / (1.0 + math.exp(-alpha * 2.0))) * (-limit + 1.0)) < 1e-5


def test_swiglu_clamp_is_asymmetric_and_is_not_oai(orc):
    """crates/colibri-engine/src/dsv4.rs:752-764 (clamp_is_asymmetric_and_is_not_oai)."""
    lim = 10.0
    f = lambda g, u: orc.act_combine(g, u, 0, 0.0, lim)
    assert abs(f(-50.0, 1.0)) < 1e-6
    assert f(50.0, 1.0) == f(lim, 1.0)
    assert f(1.0, 50.0) == f(1.0, lim)
    assert f(1.0, -50.0) == f(1.0, -lim)
    assert abs(f(2.0, 0.0)) < 1e-6
    # limit = 0 and oai = 0 is the plain SiLU arm
    assert orc.act_combine(50.0, 50.0, 0, 0.0, 0.0) == orc.lib().orc_siluf(50.0) * 50.0


def test_rmsnorm_gives_unit_rms_with_unit_weight(orc):
    """crates/colibri-engine/src/math.rs:185-195."""
    out = orc.rmsnorm(np.array([[3.0, 4.0]], np.float32), np.array([1.0, 1.0], np.float32), 0.0)[0]
    rms = math.sqrt((out[0] * out[0] + out[1] * out[1]) / 2.0)
    assert abs(rms - 1.0) < 1e-5
    assert abs(out[1] / out[0] - 4.0 / 3.0) < 1e-5


# ---- MXFP4 (fmt 6): E2M1 nibbles with one E8M0 power-of-two scale per 32 inputs ---------------
# crates/colibri-core/src/dtype.rs:313-319  f8e8m0_known_values
def test_e8m0_known_values(orc):
    L = orc.lib()
    assert L.orc_e8m0_to_f32(127) == 1.0
    assert L.orc_e8m0_to_f32(128) == 2.0
    assert L.orc_e8m0_to_f32(126) == 0.5
    assert L.orc_e8m0_to_f32(0) == f32(2.0 ** -127)
    assert L.orc_e8m0_to_f32(254) == f32(2.0 ** 127)
    assert math.isnan(L.orc_e8m0_to_f32(255))  # dtype.rs:137-139


# crates/colibri-engine/src/gpubench.rs:552-597  quantize_mxfp4_round_trips_through_the_production_decode
def test_mxfp4_round_trips_through_the_decode(orc):
    o, i = 32, 64  # two blocks of 32 per row
    k = np.arange(o * i, dtype=np.float32)
    w = np.sin(k * np.float32(0.017)).astype(np.float32)
    w[1::2] *= np.float32(0.12)  # damped odd columns: a swapped nibble order becomes a large error
    w = w.reshape(o, i)
    nib, bs, g = orc.quantize_mxfp4(w)
    assert nib.shape == (o, i // 2) and bs.shape == (o, i // 32) and g == 1.0
    y = orc.matmul_qt(orc.FMT_MXFP4, nib, bs, g, np.eye(i, dtype=np.float32), o)  # y[k, r] = W[r, k]
    rel = math.sqrt(float(((y.T.astype(np.float64) - w) ** 2).sum() / (w.astype(np.float64) ** 2).sum()))
    assert rel < 0.25, rel  # the reference's bound: "quantized" lands near 0.1, "scrambled" near 1.0
    # the encoder's rule (gpubench.rs:95-105): smallest power of two that brings the block max to <= 6
    for r in (0, 7, 31):
        for b in range(2):
            bmax = float(np.abs(w[r, 32 * b:32 * b + 32]).max())
            e = int(bs[r, b]) - 127
            assert bmax / 2.0 ** e <= 6.0 < bmax / 2.0 ** (e - 1) + 1e-6


def test_mxfp4_decode_is_code_times_power_of_two(orc):
    """linear.rs:134-175 restated independently: W[o,k] = E2M1[nib] * 2^(bs[o, k/32] - 127) * g, low
    nibble = even k; checked through the one-hot probe of linear.rs:449-485."""
    rng = np.random.default_rng(5)
    o, i = 5, 96
    nib = rng.integers(0, 256, (o, i // 2), dtype=np.uint8)
    bs = rng.integers(110, 140, (o, i // 32), dtype=np.uint8)
    g = 0.75
    W = orc.dequant(orc.FMT_MXFP4, nib, bs, g, o, i)
    lut = np.array(E2M1 + [-v for v in E2M1], np.float32)
    for r in range(o):
        for k in range(i):
            byte = int(nib[r, k >> 1])
            code = (byte >> 4) if (k & 1) else (byte & 0x0F)
            want = f32(f32(lut[code] * np.float32(2.0 ** (int(bs[r, k >> 5]) - 127))) * np.float32(g))
            assert W[r, k] == want, (r, k, W[r, k], want)
