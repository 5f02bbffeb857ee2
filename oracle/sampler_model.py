"""numpy restatement of the device id sampler (cuke_b200/csrc/train.cu).  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Philox4x32-10 as published (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11;
multipliers 0xD2511F53 / 0xCD9E8D57, Weyl constants 0x9E3779B9 / 0xBB67AE85), checked in tests/test_sampler.py against
the known-answer vectors of the Random123 distribution, then the same integer arithmetic the kernels use to turn the
64-bit word into an id.  The reference has no device sampler (apps/kge/data/data_init.py:47-63 draws on the host through
DGL), so there is no reference output to compare with: the contract is bit-equality between kernel and this model."""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised over the counter words (uint64 arrays holding 32-bit values); keys are Python ints."""
    c0, c1, c2, c3 = (np.asarray(x, dtype=np.uint64) & MASK for x in (c0, c1, c2, c3))
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & MASK, p1 >> np.uint64(32), p1 & MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def words(n, seed, stream_id):
    """The 64-bit word of elements 0..n-1 of a stream: x0 * 2^32 + x1."""
    i = np.arange(n, dtype=np.uint64)
    x0, x1, _, _ = philox4x32_10(i & MASK, i >> np.uint64(32), np.full(n, stream_id, dtype=np.uint64), np.zeros(n, dtype=np.uint64),
                                 seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return (x0 << np.uint64(32)) | x1


def mulhi64(w, m):
    """floor(w * m / 2^64) for uint64 arrays w and a Python int m < 2^63, in exact integer arithmetic."""
    m = int(m)
    wl, wh = w & MASK, w >> np.uint64(32)
    ml, mh = np.uint64(m & 0xFFFFFFFF), np.uint64(m >> 32)
    ll, lh, hl, hh = wl * ml, wl * mh, wh * ml, wh * mh
    mid = (ll >> np.uint64(32)) + (lh & MASK) + (hl & MASK)
    return hh + (lh >> np.uint64(32)) + (hl >> np.uint64(32)) + (mid >> np.uint64(32))


def sample_uniform(n, id_space, seed, stream_id):
    return mulhi64(words(n, seed, stream_id), id_space).astype(np.int64)


def sample_cdf(n, cdf, perm, seed, stream_id):
    u = (words(n, seed, stream_id) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    rank = np.minimum(np.searchsorted(cdf, u, side="left"), len(cdf) - 1)
    return (perm[rank] if perm is not None else rank).astype(np.int64)


def sample_triples(n, triples, seed, stream_id):
    row = mulhi64(words(n, seed, stream_id), len(triples)).astype(np.int64)
    return triples[row, 0], triples[row, 1], triples[row, 2]
