"""Prints the constant tables of ktc_fastmath_d.h (run: python gen_fastmath_d_tables.py [--check]).

kd_exp2_tab[j]     = 2^(j/16) rounded to double, high word lowered by j << 16, j = 0..15   (exp, pow)
kd_exp2_tab64[j]   = 2^(j/64) rounded to double, high word lowered by j << 14, j = 0..63   (sigmoid)
                     (the bias lets the code add k << 16 resp. k << 14 to the high word: the table index in the
                     low bits of k cancels against it and k's upper part lands in the exponent field)
kd_log2_inv_hi[j]  = high word of inv_j, kd_log2_lc[j] = -log2(inv_j) for the 32 equal slices (in bit-pattern
                     space) of [sqrt(1/2), sqrt(2)): inv_j is 1/centre rounded to 13 significant bits, so that
                     its low word is zero and the product of a float mantissa with it is exact in double; the
                     slice that holds 1.0 has inv = 1 and a zero logarithm, which keeps relative accuracy near 1.
Also prints the largest |m * inv - 1| over all slices (the logarithm polynomial's domain).
With --check the values are compared with the header next to this file instead.
"""
import os
import re
import struct
import sys

from mpmath import mp, mpf, log

mp.prec = 200
LO = 0x3f3504f3            # bit pattern of sqrt(1/2) rounded up: the first slice starts here


def f32(bits):
    return struct.unpack("<f", struct.pack("<I", bits & 0xffffffff))[0]


def round_bits(x, bits):
    m, e = mp.frexp(x)          # x = m * 2^e, 0.5 <= m < 1
    q = mp.nint(m * (1 << bits))
    return q / (1 << bits) * mpf(2) ** e


def hi_word(d):
    return struct.unpack("<q", struct.pack("<d", d))[0] >> 32


def biased(d, bias):
    bits = struct.unpack("<q", struct.pack("<d", d))[0] - (bias << 32)
    return struct.unpack("<d", struct.pack("<q", bits))[0]


def tables():
    exp16 = [biased(float(mpf(2) ** (mpf(j) / 16)), j << 16) for j in range(16)]
    exp64 = [biased(float(mpf(2) ** (mpf(j) / 64)), j << 14) for j in range(64)]
    inv_hi, lc, worst = [], [], mpf(0)
    for j in range(32):
        b0, b1 = LO + (j << 18), LO + ((j + 1) << 18) - 1
        # patterns at or above 0x3f800000 are mantissas in [1, sqrt 2); below, in [sqrt 1/2, 1)
        m0, m1 = mpf(f32(b0)), mpf(f32(b1))
        inv = mpf(1) if m0 <= 1 <= m1 else round_bits(2 / (m0 + m1), 13)
        worst = max(worst, abs(m0 * inv - 1), abs(m1 * inv - 1))
        d = float(inv)
        assert struct.unpack("<q", struct.pack("<d", d))[0] & 0xffffffff == 0
        inv_hi.append(hi_word(d))
        lc.append(float(-log(inv) / log(2)) if inv != 1 else 0.0)
    return exp16, exp64, inv_hi, lc, worst


def main():
    exp16, exp64, inv_hi, lc, worst = tables()
    if "--check" in sys.argv:
        text = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ktc_fastmath_d.h")).read()

        def block(name):
            body = re.search(name + r"\[\d+\] = \{(.*?)\};", text, flags=re.S).group(1)
            body = re.sub(r"/\*.*?\*/", "", body)
            return [t.strip() for t in body.split(",") if t.strip()]

        assert [float.fromhex(t) for t in block("kd_exp2_tab")] == exp16
        assert [float.fromhex(t) for t in block("kd_exp2_tab64")] == exp64
        assert [int(t, 16) for t in block("kd_log2_inv_hi")] == inv_hi
        assert [float.fromhex(t) for t in block("kd_log2_lc")] == lc
        print("tables of ktc_fastmath_d.h match")
        return
    for name, tab in (("kd_exp2_tab", exp16), ("kd_exp2_tab64", exp64)):
        print(name)
        for v in tab:
            print(f"    {v.hex()},   /* {v!r} */")
    print("kd_log2_inv_hi")
    print("    " + ", ".join(f"0x{v:08x}" for v in inv_hi))
    print("kd_log2_lc")
    print("    " + ", ".join(v.hex() for v in lc))
    print("max |r| =", float(worst), "= 2^", float(log(worst) / log(2)))


if __name__ == "__main__":
    main()
