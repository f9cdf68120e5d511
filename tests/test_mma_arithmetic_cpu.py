"""The arithmetic of the persistent kernel's int4 path, restated in numpy and pinned against the oracle (no GPU).

The kernel never converts a nibble to a number: it masks a packed word into fp16 bit patterns whose values are the
nibbles plus a power-of-two offset, lets the tensor core multiply them by the inputs, and takes the offsets out with one
constant per quantisation group:

    (w & 0x000f000f) | 0x64006400          halves = 1024 + n0, 1024 + n4
    (w & 0x00f000f0) | 0x54005400          halves = 64 + n1, 64 + n5          (the nibble sits 4 bits up: unit 1/16 at 64)
    the same on w >> 8                      n2, n6 and n3, n7
    row sum of group G = scale * (acc - (1024 S_even + 64 S_odd) - zero * S_all)

where acc is the fp32 sum of the products, S_even / S_odd the sums of the group's inputs under even / odd nibbles.
This file checks the bit identities for every nibble value and the group formula against the oracle's dequantised
mat-vec (src/QWeight.cs:29-54 unpack, fp32 dot) on seeded weights of the model's value distributions.
"""
import numpy as np

import oracle


def halves(u32):
    """The two fp16 values a 32-bit register holds (low half first)."""
    return np.array([u32 & 0xFFFF, (u32 >> 16) & 0xFFFF], dtype=np.uint16).view(np.float16).astype(np.float32)


def test_masked_words_are_the_nibbles_plus_offsets():
    for n_lo in range(16):
        for n_hi in range(16):
            # one 16-bit half of a packed word: nibbles n0 n1 n2 n3 from bit 0 up; the same pattern in both halves
            half = n_lo | (n_hi << 4) | (((n_lo + 3) & 15) << 8) | (((n_hi + 5) & 15) << 12)
            w = half | (half << 16)
            a = (w & 0x000F000F) | 0x64006400
            b = (w & 0x00F000F0) | 0x54005400
            w8 = w >> 8
            c = (w8 & 0x000F000F) | 0x64006400
            d = (w8 & 0x00F000F0) | 0x54005400
            assert list(halves(a)) == [1024 + n_lo, 1024 + n_lo]
            assert list(halves(b)) == [64 + n_hi, 64 + n_hi]
            assert list(halves(c)) == [1024 + ((n_lo + 3) & 15)] * 2
            assert list(halves(d)) == [64 + ((n_hi + 5) & 15)] * 2


def emulate_row(words, zero_words, scales, x):
    """One output row the way the kernel computes it: per quantisation group of 128 inputs, offsets removed once."""
    x = x.astype(np.float32)
    total = np.float32(0.0)
    for g in range(x.size // 128):
        acc = np.float32(0.0)
        s_even = np.float32(0.0)
        s_odd = np.float32(0.0)
        for wi in range(16):
            w = int(words[g * 16 + wi])
            xs = x[g * 128 + wi * 8: g * 128 + wi * 8 + 8]
            w8 = w >> 8
            regs = [(w & 0x000F000F) | 0x64006400, (w & 0x00F000F0) | 0x54005400, (w8 & 0x000F000F) | 0x64006400, (w8 & 0x00F000F0) | 0x54005400]
            # register j holds nibbles j and j + 4 and meets the inputs j and j + 4 (the table's fp16 pairs)
            for j, r in enumerate(regs):
                lo, hi = halves(r)
                acc += np.float32(lo) * xs[j] + np.float32(hi) * xs[j + 4]
            s_even += xs[0] + xs[2] + xs[4] + xs[6]
            s_odd += xs[1] + xs[3] + xs[5] + xs[7]
        zero = (int(zero_words[g >> 3]) >> ((g & 7) * 4)) & 15
        corrected = acc - (np.float32(1024.0) * s_even + np.float32(64.0) * s_odd)
        total += np.float32(scales[g]) * (corrected - np.float32(zero) * (s_even + s_odd))
    return float(total)


def test_group_formula_matches_the_dequantised_matvec():
    rng = np.random.default_rng(7)
    rows, cols = 512, 6                       # 4 quantisation groups per row
    wsize, zsize, ssize = oracle.qweight_sizes(rows)
    w = rng.integers(0, 2 ** 32, size=cols * wsize, dtype=np.uint64).astype(np.uint32)
    z = np.zeros(cols * zsize, dtype=np.uint32)
    for c in range(cols):
        for g in range(ssize):
            z[c * zsize + (g >> 3)] |= int(rng.integers(5, 12)) << ((g & 7) * 4)
    s = (0.01 * (1.0 + 0.25 * rng.standard_normal(cols * ssize))).astype(np.float16)
    x = rng.standard_normal(rows).astype(np.float16)
    want = oracle.matvec_int4_f32(x, w, z, s, rows, cols, mode=1)      # fp32 accumulate over the dequantised fp16 weights
    got = np.array([emulate_row(w[c * wsize:(c + 1) * wsize], z[c * zsize:(c + 1) * zsize], s[c * ssize:(c + 1) * ssize], x)
                    for c in range(cols)])
    # the oracle rounds every dequantised weight to fp16 ((n - z) * scale, src/QWeight.cs:50); the kernel applies the scale
    # to the group sum in fp32: the two differ by that rounding, well inside the 1e-3 relative bound of the GPU tests
    scale = float(np.abs(want).max())
    assert np.abs(got - want).max() <= 1e-3 * scale
    # and the offsets must cancel: without them the sums are off by hundreds
    assert scale < 50
