"""A lane-by-lane model of `tc_store_cols16` (speedycolibri_b200/csrc/tc_common.cuh): the byte
selectors and the two shuffle rounds that turn "one lane = one feature, 16 token columns" into
8-byte stores of four features of one column.  The model runs the same selectors on numpy arrays
and checks that every (column, feature) value lands at its token-major address exactly once."""
import numpy as np


def byte_perm(a: int, b: int, sel: int) -> int:
    src = [(a >> (8 * i)) & 0xFF for i in range(4)] + [(b >> (8 * i)) & 0xFF for i in range(4)]
    out = 0
    for i in range(4):
        out |= src[(sel >> (4 * i)) & 0x7] << (8 * i)
    return out


def store_cols16_model(vals: np.ndarray, ld: int):
    """vals[lane, col] = 16-bit value of feature `lane` at token column `col` (32 lanes, 16 columns).
    Returns {element offset: value} for a tile whose feature 0 / column 0 sits at offset 0."""
    lanes = 32
    pk = [[int(vals[l, 2 * i]) | (int(vals[l, 2 * i + 1]) << 16) for i in range(8)] for l in range(lanes)]
    mem = {}
    for g in range(4):
        p01 = [pk[l][2 * g] for l in range(lanes)]
        p23 = [pk[l][2 * g + 1] for l in range(lanes)]
        odd = [(l & 1) != 0 for l in range(lanes)]
        hi2 = [(l & 2) != 0 for l in range(lanes)]
        send1 = [byte_perm(p01[l], p23[l], 0x5410) if odd[l] else byte_perm(p01[l], p23[l], 0x7632) for l in range(lanes)]
        r1 = [send1[l ^ 1] for l in range(lanes)]
        xa = [byte_perm(p01[l], r1[l], 0x3254) if odd[l] else byte_perm(p01[l], r1[l], 0x5410) for l in range(lanes)]
        xb = [byte_perm(p23[l], r1[l], 0x3276) if odd[l] else byte_perm(p23[l], r1[l], 0x7610) for l in range(lanes)]
        send2 = [xa[l] if hi2[l] else xb[l] for l in range(lanes)]
        r2 = [send2[l ^ 2] for l in range(lanes)]
        for l in range(lanes):
            o0 = r2[l] if hi2[l] else xa[l]
            o1 = xb[l] if hi2[l] else r2[l]
            col = 4 * g + (1 if odd[l] else 0) + (2 if hi2[l] else 0)
            base = col * ld + (l & ~3)  # quad_base + col * ld, in 16-bit elements
            for j, word in enumerate((o0, o1)):
                for h in range(2):
                    off = base + 2 * j + h
                    assert off not in mem, "two lanes wrote the same element"
                    mem[off] = (word >> (16 * h)) & 0xFFFF
    return mem


def test_quad_transpose_lands_every_value_token_major():
    rng = np.random.default_rng(7)
    vals = rng.integers(0, 1 << 16, size=(32, 16), dtype=np.uint32)
    ld = 7168
    mem = store_cols16_model(vals, ld)
    assert len(mem) == 32 * 16
    for lane in range(32):
        for col in range(16):
            assert mem[col * ld + lane] == int(vals[lane, col]), (lane, col)


def test_byte_perm_model_matches_the_documented_selectors():
    a, b = 0x33221100, 0x77665544
    assert byte_perm(a, b, 0x3210) == a and byte_perm(a, b, 0x7654) == b
    assert byte_perm(a, b, 0x5410) == 0x55441100 and byte_perm(a, b, 0x7632) == 0x77663322
