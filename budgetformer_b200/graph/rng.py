"""Counter-based randomness shared bit-for-bit by the torch, C++ and CUDA edge builders.

Two primitives:

* ``philox4x32_10`` — the standard 10-round Philox-4x32 block.  A random walk step is
  addressed by ``counter = (walk_id_lo, walk_id_hi, step, PHILOX_TAG)`` under
  ``key = (seed_lo, seed_hi)``; the first output word ``r`` picks neighbour
  ``(r * degree) >> 32``.  Because the generator is stateless, a CPU thread, a CUDA
  thread and a vectorised numpy call all produce the same walk, which is what lets
  every rank build the attention graph locally instead of broadcasting it (the
  reference needs a broadcast whenever its walker is not reproducible:
  utils/fullgraph_sp_support.py:3262-3338).
* ``edge_hash31`` — the per-edge ranking key of the reference's per-query sampler,
  ``(src*1103515245 + dst*214013 + seed*2654435761 + 12345) mod 2**31``
  (utils/fullgraph_sp_support.py:982-989).  Kept verbatim so that the sampled sets
  coincide with the reference's up to hash ties.
"""
from __future__ import annotations

import numpy as np

PHILOX_M0 = 0xD2511F53
PHILOX_M1 = 0xCD9E8D57
PHILOX_W0 = 0x9E3779B9
PHILOX_W1 = 0xBB67AE85
PHILOX_TAG = 0x42554447  # fourth counter word, constant

REAL_SEED_OFFSET = 17  # utils/fullgraph_sp_support.py:970-972, 1250
RW_SEED_OFFSET = 37    # utils/fullgraph_sp_support.py:1260

_U32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox-4x32-10.  All inputs broadcastable uint64 arrays holding 32-bit values.

    Returns the four 32-bit output words as uint64 arrays.
    """
    c0 = np.asarray(c0, dtype=np.uint64) & _U32
    c1 = np.asarray(c1, dtype=np.uint64) & _U32
    c2 = np.asarray(c2, dtype=np.uint64) & _U32
    c3 = np.asarray(c3, dtype=np.uint64) & _U32
    k0 = np.asarray(k0, dtype=np.uint64) & _U32
    k1 = np.asarray(k1, dtype=np.uint64) & _U32
    m0 = np.uint64(PHILOX_M0)
    m1 = np.uint64(PHILOX_M1)
    sh = np.uint64(32)
    for _ in range(10):
        p0 = m0 * c0
        p1 = m1 * c2
        hi0, lo0 = p0 >> sh, p0 & _U32
        hi1, lo1 = p1 >> sh, p1 & _U32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _U32, lo1, (hi0 ^ c3 ^ k1) & _U32, lo0
        k0 = (k0 + np.uint64(PHILOX_W0)) & _U32
        k1 = (k1 + np.uint64(PHILOX_W1)) & _U32
    return c0, c1, c2, c3


def walk_uniform32(walk_id, step, seed):
    """First Philox word for (walk_id, step) under ``seed`` — uint64 array of 32-bit values."""
    walk_id = np.asarray(walk_id, dtype=np.uint64)
    seed = np.uint64(int(seed) & 0xFFFFFFFFFFFFFFFF)
    r, _, _, _ = philox4x32_10(
        walk_id & _U32, walk_id >> np.uint64(32), np.uint64(step), np.uint64(PHILOX_TAG),
        seed & _U32, seed >> np.uint64(32),
    )
    return r


def edge_hash31(src, dst, seed):
    """Reference ranking key; int64 numpy arrays in, uint64 array of 31-bit keys out."""
    src = np.asarray(src).astype(np.uint64)
    dst = np.asarray(dst).astype(np.uint64)
    c = np.uint64((int(seed) * 2654435761 + 12345) & 0xFFFFFFFFFFFFFFFF)
    with np.errstate(over="ignore"):
        k = src * np.uint64(1103515245) + dst * np.uint64(214013) + c
    return k & np.uint64(0x7FFFFFFF)
