"""Generates exp64_table.inc (the constants of exp64.cuh) with 400-bit arithmetic: python gen_exp64_table.py"""
import os
import mpmath as mp
mp.mp.prec = 400
def rn(x):  # nearest double
    return float(mp.mpf(x))
def hexd(d): return float.hex(d)
ln2_64 = mp.log(2)/64
# L1: ln2/64 truncated to 36 significant bits
e = mp.floor(mp.log(ln2_64, 2))
scale = mp.mpf(2)**(35 - e)
L1 = mp.floor(ln2_64*scale)/scale
L1d = float(L1); assert mp.mpf(L1d) == L1
L2d = rn(ln2_64 - L1); L3d = rn(ln2_64 - L1 - mp.mpf(L2d))
out = []
out.append("// Constants of exp64.cuh, generated with 400-bit arithmetic (mpmath): ln2/64 in three parts (the")
out.append("// first with 36 significant bits, so that k*L1 is exact for |k| < 2^17), 64/ln2, 1/n! as")
out.append("// double-double for n = 3..7, and 2^(j/64), j = 0..63, as double-double (hi = nearest double).")
out.append(f"#define KN_EXP64_L1 {hexd(L1d)}")
out.append(f"#define KN_EXP64_L2 {hexd(L2d)}")
out.append(f"#define KN_EXP64_L3 {hexd(L3d)}")
out.append(f"#define KN_EXP64_INV {hexd(rn(1/ln2_64))}")
for n in range(3, 8):
    c = 1/mp.factorial(n); h = rn(c); l = rn(c - mp.mpf(h))
    out.append(f"#define KN_EXP64_C{n}H {hexd(h)}")
    out.append(f"#define KN_EXP64_C{n}L {hexd(l)}")
for n in range(8, 14):
    out.append(f"#define KN_EXP64_C{n} {hexd(rn(1/mp.factorial(n)))}")
out.append("#define KN_EXP64_TABLE \\")
rows = []
for j in range(64):
    t = mp.mpf(2)**(mp.mpf(j)/64); h = rn(t); l = rn(t - mp.mpf(h))
    rows.append(f"  {hexd(h)}, {hexd(l)}")
out.append(", \\\n".join(rows))
open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "exp64_table.inc"), "w").write("\n".join(out) + "\n")
print("\n".join(out[:12]))
