"""Shared synthetic inputs for the tests: seeded layer weights in the reference's blob layout."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def make_expert_blobs(rng, n, gu_type, d_type, H, I, sigma=0.02):
    """n expert blobs quantised from N(0, sigma^2) (IQ1_M: random valid blocks, there being no quantiser for it)."""
    L = O.Layout(gu_type, d_type, H, I)
    blobs = []
    for _ in range(n):
        unquantised = O.UNQUANTISED     # formats the oracle has no quantiser for: random valid blocks
        if gu_type in unquantised or d_type in unquantised:
            blob = np.zeros(L.bytes, np.uint8)
            for t, off, rows, cols in ((gu_type, 0, 2 * I, H), (d_type, L.down_off, H, I)):
                if t == O.T_IQ1_M:
                    raw = O.random_iq1m_rows(rng, rows, cols)
                elif t in unquantised:
                    raw = O.random_rows(t, rng, rows, cols)
                else:
                    raw = O.quantize(t, (rng.standard_normal((rows, cols)) * sigma).astype(np.float32))
                blob[off:off + raw.size] = raw
        else:
            G = (rng.standard_normal((I, H)) * sigma).astype(np.float32)
            U = (rng.standard_normal((I, H)) * sigma).astype(np.float32)
            D = (rng.standard_normal((H, I)) * sigma).astype(np.float32)
            blob = O.make_blob(L, G, U, D)
        blobs.append(blob)
    return L, blobs


def pad16(n: int) -> int:
    return (n + 15) // 16 * 16


def stack_blobs(blobs):
    """[n][stride] uint8 with a 16-byte-aligned stride."""
    stride = pad16(blobs[0].size)
    out = np.zeros((len(blobs), stride), np.uint8)
    for i, b in enumerate(blobs):
        out[i, :b.size] = b
    return out
