"""Host-side conversions between Python integers and the library's wire form of BN254 field
elements (4 x u64 little-endian limbs, Montgomery form with R = 2^256)."""
from __future__ import annotations

import numpy as np

R_MOD = 0x30644E72E131A029B85045B68181585D2833E84879B9709143E1F593F0000001
Q_MOD = 0x30644E72E131A029B85045B68181585D97816A916871CA8D3C208C16D87CFD47
_R = 1 << 256
_RINV = {R_MOD: pow(_R, -1, R_MOD), Q_MOD: pow(_R, -1, Q_MOD)}
_M64 = (1 << 64) - 1


def to_mont_array(values, mod: int = R_MOD) -> np.ndarray:
    """ints (canonical, any sign) -> (n, 4) uint64 array of Montgomery limbs."""
    out = np.empty((len(values), 4), dtype=np.uint64)
    for i, v in enumerate(values):
        m = (int(v) % mod) * _R % mod
        out[i, 0] = m & _M64
        out[i, 1] = (m >> 64) & _M64
        out[i, 2] = (m >> 128) & _M64
        out[i, 3] = m >> 192
    return out


def from_mont_array(arr, mod: int = R_MOD):
    """(n, 4) uint64 Montgomery limbs -> list of canonical ints."""
    a = np.asarray(arr, dtype=np.uint64).reshape(-1, 4)
    rinv = _RINV[mod]
    return [((int(r[0]) | (int(r[1]) << 64) | (int(r[2]) << 128) | (int(r[3]) << 192)) * rinv) % mod for r in a]


def raw_ints(arr):
    """(n, 4) uint64 limbs -> list of the raw 256-bit integers (no Montgomery conversion)."""
    a = np.asarray(arr, dtype=np.uint64).reshape(-1, 4)
    return [int(r[0]) | (int(r[1]) << 64) | (int(r[2]) << 128) | (int(r[3]) << 192) for r in a]
