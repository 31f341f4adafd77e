"""Host restatement of the counter-based dropout masks.  TEST INFRASTRUCTURE ONLY.

Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed by a 64-bit
seed; the counter is (element index // 8, stream id, constant) and the four output words serve eight consecutive
elements with 16 bits each. An element is kept when its 16 bits are >= floor(p * 65536). The reference has no counterpart (its masks come
from triton.language.rand / torch.bernoulli), so these masks are pinned only to the Philox known-answer vectors
checked in tests/test_oracle_golden.py, not to the reference.
"""
from __future__ import annotations

import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
CTR3 = 0x50544A31
U32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter, key):
    """counter: 4 arrays (or ints) of uint32 values, key: 2 ints. Returns 4 uint32 arrays."""
    c = [np.asarray(x, dtype=np.uint64) & U32 for x in counter]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        n0 = ((p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0)) & U32
        n1 = p1 & U32
        n2 = ((p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1)) & U32
        n3 = p0 & U32
        c = [n0, n1, n2, n3]
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return [x.astype(np.uint32) for x in c]


def threshold16(p: float) -> int:
    return min(65535, max(0, int(float(np.float32(p)) * 65536.0)))


def keep_mask(seed: int, stream_id: int, n: int, p: float) -> np.ndarray:
    """float32 0/1 mask for element indices 0..n-1 of one site: 16 random bits per element, 8 elements per Philox call
    (element e of a call takes the low half of word e // 2 when e is even, the high half when odd); an element is
    dropped when its 16 bits are below floor(p * 65536)."""
    nblk = (n + 7) // 8
    ctr = np.arange(nblk, dtype=np.uint64)
    words = philox4x32_10([ctr & U32, ctr >> np.uint64(32), np.full(nblk, stream_id, np.uint64),
                           np.full(nblk, CTR3, np.uint64)], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    halves = []
    for w in words:
        halves += [w & np.uint32(0xFFFF), w >> np.uint32(16)]
    flat = np.stack(halves, axis=1).reshape(-1)[:n]
    return (flat >= np.uint32(threshold16(p))).astype(np.float32)
