"""Independent big-integer reference used to pin the C++ oracle.

Plain Python `int` arithmetic: nothing here shares code with the oracle or the
CUDA library, so agreement between them is meaningful.  Only for small cases.
"""
import random

R = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001
P = 0x1A0111EA397FE69A4B1BA7B6434BACD764774B84F38512BF6730D2A0F6B0F6241EABFFFEB153FFFFB9FEFFFFFFFFAAAB
GX = 0x17F1D3A73197D7942695638C4FA9AC0FC3688C4F9774B905A14E3A3F171BAC586C55E83FF97A1AEFFB3AF00ADB22C6BB
GY = 0x08B3F481E3AAA0F1A09E30ED741D8AE4FCF5E095D5D00AF600DB18CB2C04B3EDD03CC744A2888AE40CAA232946C5E7E1


def root_of_unity(n):
    assert n and n & (n - 1) == 0
    return pow(5, (R - 1) // n, R)


def fr_bytes(v):
    return int(v % R).to_bytes(32, "little")


def fr_array(vals):
    import numpy as np

    return np.frombuffer(b"".join(fr_bytes(v) for v in vals), dtype=np.uint8).reshape(len(vals), 32).copy()


def fr_ints(arr):
    import numpy as np

    a = np.ascontiguousarray(arr, dtype=np.uint8).reshape(-1, 32)
    return [int.from_bytes(a[i].tobytes(), "little") for i in range(a.shape[0])]


def rand_fr(rng, n):
    return [rng.randrange(R) for _ in range(n)]


def bary_weights(x, n):
    w = root_of_unity(n)
    z = (pow(x, n, R) - 1) % R
    ninv = pow(n, -1, R)
    out = []
    p = 1
    for _ in range(n):
        out.append(z * p % R * ninv % R * pow((x - p) % R, -1, R) % R)
        p = p * w % R
    return out


def g1_add(A, B):
    if A is None:
        return B
    if B is None:
        return A
    x1, y1 = A
    x2, y2 = B
    if x1 == x2:
        if (y1 + y2) % P == 0:
            return None
        lam = 3 * x1 * x1 * pow(2 * y1, -1, P) % P
    else:
        lam = (y2 - y1) * pow(x2 - x1, -1, P) % P
    x3 = (lam * lam - x1 - x2) % P
    return (x3, (lam * (x1 - x3) - y1) % P)


def g1_mul(k, A):
    k %= R
    acc = None
    while k:
        if k & 1:
            acc = g1_add(acc, A)
        A = g1_add(A, A)
        k >>= 1
    return acc


def g1_bytes(A):
    if A is None:
        return bytes(96)
    return A[0].to_bytes(48, "little") + A[1].to_bytes(48, "little")


def g1_from_bytes(b):
    b = bytes(b)
    if b == bytes(96):
        return None
    return (int.from_bytes(b[:48], "little"), int.from_bytes(b[48:], "little"))


def fnv1a(data: bytes):
    h = 1469598103934665603
    for ch in data:
        h ^= ch
        h = h * 1099511628211 % (1 << 64)
    return h
