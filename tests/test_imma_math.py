"""The arithmetic and the data flow of the integer tensor-core INT4 mat-vec (blok_b200/csrc/i4_imma.cuh), emulated in
numpy lane by lane: block-integer activations (two signed bytes per value relative to the scale group's largest
exponent), nibbles taken as bytes 16 (q + 8), the operand fragments of mma.m16n8k32 as the PTX ISA lays them out, the
per-group correction and scaling.  Checked against sum_c x_c q_c s (src/kimi_exec.cu:300-323 without its roundings).
Runs without a GPU; the kernel itself is checked on the GPU against the oracle."""
import numpy as np

import util

MASK = np.uint32(0xf0f0f0f0)


def stage(x_bits):
    """x bf16 bit patterns [cols] -> (xq bytes [cols * 2], meta_f [groups], meta_off [groups]) as stage_x_imma does."""
    cols = x_bits.size
    x = util.bf16_np_to_f32(x_bits).astype(np.float64)
    xq = np.zeros(cols * 2, np.uint8)
    f = np.zeros(cols // 32, np.float64)
    off = np.zeros(cols // 32, np.int64)
    for grp in range(cols // 32):
        seg = slice(grp * 32, grp * 32 + 32)
        e = int(((x_bits[seg].astype(np.uint32) >> 7) & 0xff).max())
        dead = e < 20
        e = min(e, 254)
        X = np.zeros(32, np.int64) if dead else np.clip(np.rint(x[seg] * 2.0 ** (140 - e)), -16383, 16383).astype(np.int64)
        h = (X + 128) >> 8
        l = X - (h << 8)
        assert np.all((-128 <= l) & (l <= 127)) and np.all((-64 <= h) & (h <= 64)) and np.all(256 * h + l == X)
        f[grp] = 0.0 if dead else 2.0 ** (e - 144)
        off[grp] = 128 * X.sum()
        kb, t = grp // 4, grp % 4
        for i in range(4):              # unit = word i of the group: 8 values
            for k in range(8):
                byte = (k & 1) * 4 + (k >> 1)       # b0 (even columns) then b1 (odd columns), byte = column pair
                base = kb * 256 + t * 64 + i * 8
                xq[base + byte] = np.uint8(h[i * 8 + k] & 0xff)
                xq[base + 32 + byte] = np.uint8(l[i * 8 + k] & 0xff)
    return xq, f, off


def _s8(byte):
    return byte - 256 if byte >= 128 else byte


def mma_u8s8_16832(a_regs, b_regs):
    """a_regs [32 lanes][4] uint32, b_regs [32][2] uint32 -> d [32][4] int64, per the PTX fragment layout of
    mma.m16n8k32 with 8-bit operands: a0 (row g, k 4t..), a1 (row g+8, k 4t..), a2 (row g, k 16+4t..), a3 (row g+8, ...);
    b0 (k 4t.., col g), b1 (k 16+4t.., col g); c0 (g, 2t), c1 (g, 2t+1), c2 (g+8, 2t), c3 (g+8, 2t+1)."""
    A = np.zeros((16, 32), np.int64)
    B = np.zeros((32, 8), np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for j in range(4):
            sh = 8 * j
            A[g, 4 * t + j] = (int(a_regs[lane][0]) >> sh) & 0xff              # unsigned bytes
            A[g + 8, 4 * t + j] = (int(a_regs[lane][1]) >> sh) & 0xff
            A[g, 16 + 4 * t + j] = (int(a_regs[lane][2]) >> sh) & 0xff
            A[g + 8, 16 + 4 * t + j] = (int(a_regs[lane][3]) >> sh) & 0xff
            B[4 * t + j, g] = _s8((int(b_regs[lane][0]) >> sh) & 0xff)         # signed bytes
            B[16 + 4 * t + j, g] = _s8((int(b_regs[lane][1]) >> sh) & 0xff)
    D = A @ B
    d = np.zeros((32, 4), np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        d[lane] = (D[g, 2 * t], D[g, 2 * t + 1], D[g + 8, 2 * t], D[g + 8, 2 * t + 1])
    return d


def gemv16(words, scales, x_bits):
    """One warp's 16 rows: words uint32 [16, cols / 8], scales bf16 bits [16, cols / 32] -> y float64 [16]."""
    cols = x_bits.size
    xq, f, off = stage(x_bits)
    xq32 = xq.view(np.uint32)
    acc = np.zeros((32, 2), np.float64)
    s = util.bf16_np_to_f32(scales).astype(np.float64)
    for kb in range(cols // 128):
        d = np.zeros((32, 4), np.int64)
        for i in range(4):
            a = np.zeros((32, 4), np.uint32)
            b = np.zeros((32, 2), np.uint32)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                wl = words[g, kb * 16 + t * 4 + i]
                wh = words[g + 8, kb * 16 + t * 4 + i]
                a[lane] = ((wl << np.uint32(4)) & MASK, (wh << np.uint32(4)) & MASK, wl & MASK, wh & MASK)
                if (g >> 1) == t:     # supplies limb g & 1 of its own group
                    at = (kb * 256 + t * 64 + (g & 1) * 32 + i * 8) // 4
                    b[lane] = (xq32[at], xq32[at + 1])
            d += mma_u8s8_16832(a, b)
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            grp = kb * 4 + t
            acc[lane, 0] += s[g, grp] * f[grp] * (256 * d[lane, 0] + d[lane, 1] - off[grp])
            acc[lane, 1] += s[g + 8, grp] * f[grp] * (256 * d[lane, 2] + d[lane, 3] - off[grp])
    y = np.zeros(16, np.float64)
    for lane in range(32):
        g = lane >> 2
        y[g] += acc[lane, 0]
        y[g + 8] += acc[lane, 1]
    return y


def _case(seed, cols, x_std, spread):
    rng = np.random.default_rng(seed)
    q, words = util.rand_i4(rng, 16, cols)
    scales = util.rand_scales(rng, 16, cols // 32, 0.01)
    x = rng.normal(0, x_std, cols) * np.exp(rng.normal(0, spread, cols))     # magnitudes spread over several octaves
    x_bits = util.f32_to_bf16_np(x.astype(np.float32))
    return q, words, scales, x_bits


def _rounding_bound(q, scales, x_bits):
    """What rounding the activations to integers can cost: half a unit 2^(E - 140) per element, E the biased exponent
    of its scale group's largest value, times |q| times the scale."""
    s = util.bf16_np_to_f32(scales).astype(np.float64)
    e = ((x_bits.astype(np.uint32) >> 7) & 0xff).reshape(-1, 32).max(axis=1).astype(np.float64)
    unit = np.where(e < 20, 0.0, 2.0 ** (e - 140))
    aq = np.abs(q).reshape(q.shape[0], -1, 32).sum(axis=2)
    return (aq * s * 0.5 * unit).sum(axis=1)


def test_integer_path_reproduces_the_dot_product():
    """Typical activations (a few octaves of spread inside a group) come out far more exactly than the bf16 rounding of
    the result; whatever the spread, the error stays inside half an integer unit per element: the integer form keeps
    14 bits below each group's largest value, smaller values lose precision and vanish below 2^-14 of it."""
    for seed, cols, std, spread, rel in ((0, 256, 1.0, 0.0, 2.0 ** -13), (1, 512, 1.0, 1.0, 2.0 ** -11), (2, 128, 1e-3, 1.0, 2.0 ** -11),
                                         (3, 256, 300.0, 3.0, None)):
        q, words, scales, x_bits = _case(seed, cols, std, spread)
        got = gemv16(words, scales, x_bits)
        x = util.bf16_np_to_f32(x_bits).astype(np.float64)
        s = np.repeat(util.bf16_np_to_f32(scales).astype(np.float64), 32, axis=1)
        want = (q.astype(np.float64) * s) @ x
        err = np.abs(got - want)
        assert np.all(err <= _rounding_bound(q, scales, x_bits) * (1 + 1e-9) + 1e-30), seed
        if rel is not None:
            assert np.all(err <= rel * ((np.abs(q) * s) @ np.abs(x))), (seed, np.max(err / ((np.abs(q) * s) @ np.abs(x))))


def test_values_within_six_octaves_of_the_group_maximum_are_exact():
    rng = np.random.default_rng(7)
    q, words = util.rand_i4(rng, 16, 128)
    scales = util.f32_to_bf16_np(np.full((16, 4), 0.0078125, np.float32))      # 2^-7: exact arithmetic throughout
    mant = rng.integers(128, 256, 128)
    expo = rng.integers(-6, 1, 128)
    expo[::32] = 0                                  # every group holds a value at the top exponent
    x = mant * 2.0 ** (expo - 7) * rng.choice([-1.0, 1.0], 128)
    x_bits = util.f32_to_bf16_np(x.astype(np.float32))
    assert np.array_equal(util.bf16_np_to_f32(x_bits).astype(np.float64), x)
    got = gemv16(words, scales, x_bits)
    want = (q.astype(np.float64) * 0.0078125) @ x
    assert np.array_equal(got, want)


def test_zero_and_tiny_groups_contribute_nothing_and_do_not_poison_the_rest():
    q, words, scales, x_bits = _case(5, 256, 1.0, 0.5)
    x_bits = x_bits.copy()
    x_bits[32:64] = 0                                              # an all-zero group
    x_bits[96:128] = util.f32_to_bf16_np(np.full(32, 1e-38, np.float32))   # below the staging floor of 2^-108
    got = gemv16(words, scales, x_bits)
    x = util.bf16_np_to_f32(x_bits).astype(np.float64)
    x[96:128] = 0
    s = np.repeat(util.bf16_np_to_f32(scales).astype(np.float64), 32, axis=1)
    want = (q.astype(np.float64) * s) @ x
    assert np.all(np.abs(got - want) <= _rounding_bound(q, scales, x_bits) * (1 + 1e-9))
