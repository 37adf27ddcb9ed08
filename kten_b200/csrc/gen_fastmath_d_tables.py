"""Prints the two constant tables of ktc_fastmath_d.h (run: python gen_fastmath_d_tables.py).

kd_exp2_tab[j]   = 2^(j/16) rounded to double, j = 0..15
kd_log2_tab[j]   = {inv, -log2(inv)} for the 64 equal slices (in bit-pattern space) of
                   [sqrt(1/2), sqrt(2)): inv is 1/centre rounded to 13 significant bits (so the
                   product of a float mantissa with it is exact in double); the slice that holds
                   1.0 has inv = 1 and a zero logarithm, which keeps relative accuracy near 1.
Also prints the largest |m * inv - 1| over all slices (the polynomial's domain).
"""
import struct
from mpmath import mp, mpf, log

mp.prec = 200


def f32(bits):
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def round_bits(x, bits):
    m, e = mp.frexp(x)          # x = m * 2^e, 0.5 <= m < 1
    q = mp.nint(m * (1 << bits))
    return q / (1 << bits) * mpf(2) ** e


print("exp2 table")
for j in range(16):
    v = mpf(2) ** (mpf(j) / 16)
    print(f"    {float(v).hex()},   /* {float(v)!r} */")

print("log2 table (superseded by the 32-slice tables)")
LO = 0x3f3504f3
worst = mpf(0)
for j in range(64):
    b0 = LO + (j << 17)
    b1 = LO + ((j + 1) << 17) - 1
    m0, m1 = mpf(f32(b0)), mpf(f32(b1))
    if m0 >= 1:            # the patterns above 0x3f800000 belong to the next binade: halve them back into [1, sqrt2)
        pass
    # mantissa value m in [sqrt(1/2), sqrt(2)): patterns >= 0x3f800000 are already in [1, 2)
    if m0 <= 1 <= m1:
        inv = mpf(1)
    else:
        inv = round_bits(2 / (m0 + m1), 13)
    worst = max(worst, abs(m0 * inv - 1), abs(m1 * inv - 1))
    l = -log(inv) / log(2) if inv != 1 else mpf(0)
    print(f"    {{{float(inv).hex()}, {float(l).hex()}}},   /* 1/{float(1 / inv):.6f} */")
print("max |r| =", float(worst), "= 2^", float(log(worst) / log(2)))
