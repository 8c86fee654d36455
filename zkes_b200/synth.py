"""Seeded synthetic inputs that are produced on the host (benchmark and test data; no counterpart
in the reference, whose bins draw from StdRng).

The field elements of the workloads come from the device generators (zk_gen_uniform_fr,
zk_gen_small_fr, zk_gen_gauss_fr).  What has to be made on the host is the position list of a
sparse table: distinct indices need a sequential "skip duplicates" pass.  The list is defined
on the same ChaCha20 stream family (RFC 8439 block function, key = seed | stream as two
little-endian u64 followed by zeros, zero nonce, block counter from 0), so any harness can
regenerate it byte for byte:

    successive 32-bit little-endian keystream words, masked to `num_var` bits; a value that has
    appeared before is skipped; the first `count` values kept, then sorted ascending.
"""
from __future__ import annotations

import numpy as np

SPARSE_INDEX_STREAM = 3  # stream id of the position list (0: dense table, 2: sparse values)


def _rotl(x: np.ndarray, n: int) -> np.ndarray:
    return (x << np.uint32(n)) | (x >> np.uint32(32 - n))


def chacha20_words(seed: int, stream: int, first_block: int, n_blocks: int) -> np.ndarray:
    """Keystream words of blocks [first_block, first_block + n_blocks): uint32 array (n_blocks, 16)."""
    init = np.zeros((n_blocks, 16), dtype=np.uint32)
    init[:, 0:4] = np.array([0x61707865, 0x3320646E, 0x79622D32, 0x6B206574], dtype=np.uint32)
    init[:, 4] = seed & 0xFFFFFFFF
    init[:, 5] = (seed >> 32) & 0xFFFFFFFF
    init[:, 6] = stream & 0xFFFFFFFF
    init[:, 7] = (stream >> 32) & 0xFFFFFFFF
    init[:, 12] = (np.arange(n_blocks, dtype=np.uint64) + np.uint64(first_block)).astype(np.uint32)
    x = [init[:, i].copy() for i in range(16)]

    def qr(a, b, c, d):
        x[a] += x[b]; x[d] = _rotl(x[d] ^ x[a], 16)
        x[c] += x[d]; x[b] = _rotl(x[b] ^ x[c], 12)
        x[a] += x[b]; x[d] = _rotl(x[d] ^ x[a], 8)
        x[c] += x[d]; x[b] = _rotl(x[b] ^ x[c], 7)

    with np.errstate(over="ignore"):
        for _ in range(10):
            qr(0, 4, 8, 12); qr(1, 5, 9, 13); qr(2, 6, 10, 14); qr(3, 7, 11, 15)
            qr(0, 5, 10, 15); qr(1, 6, 11, 12); qr(2, 7, 8, 13); qr(3, 4, 9, 14)
        out = np.stack(x, axis=1) + init
    return out


def sparse_indices(seed: int, num_var: int, count: int, stream: int = SPARSE_INDEX_STREAM) -> np.ndarray:
    """`count` distinct positions below 2^num_var from the ChaCha20 stream (seed, stream), sorted
    ascending (uint64).  See the module docstring for the exact rule."""
    if not 0 <= count <= (1 << num_var):
        raise ValueError("more positions than the domain holds")
    if num_var > 32:
        raise ValueError("positions are 32-bit keystream words")
    mask = np.uint32((1 << num_var) - 1) if num_var < 32 else np.uint32(0xFFFFFFFF)
    kept = np.empty(0, dtype=np.uint32)
    block = 0
    while kept.size < count:
        want = count - kept.size
        n_blocks = max(64, (want + want // 8) // 16 + 1)
        words = chacha20_words(seed, stream, block, n_blocks).reshape(-1) & mask
        block += n_blocks
        cand = np.concatenate([kept, words])
        _, first = np.unique(cand, return_index=True)   # first occurrence of every value, stream order kept below
        first.sort()
        kept = cand[first][:count] if first.size >= count else cand[first]
    return np.sort(kept[:count]).astype(np.uint64)
