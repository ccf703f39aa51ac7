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


def near_tie_ok(ids, want_ids, b):
    """rows whose ids differ may differ only by experts whose biased scores are within 1e-5 of the k-th
    (the reference's own allowance, src/models/deepseek41/kernels/router_parity.cpp:96-107)"""
    for t in range(ids.shape[0]):
        if np.array_equal(ids[t], want_ids[t]):
            continue
        kth = b[t, want_ids[t, -1]]
        for e in set(ids[t].tolist()) ^ set(want_ids[t].tolist()):
            assert abs(b[t, e] - kth) < 1e-5, (t, e)
        if set(ids[t].tolist()) == set(want_ids[t].tolist()):   # an order swap: equal-score neighbours
            for a_, w_ in zip(ids[t], want_ids[t]):
                assert abs(b[t, a_] - b[t, w_]) < 1e-5


def group_near_tie_ok(ids, want_ids, b, n_group, topk_group, tol=1e-5):
    """Group-limited rows that differ from the oracle: recompute in fp64 which groups could have been kept once scores within
    `tol` count as tied, and require that the device's experts all lie in keepable groups and that, inside the union of kept
    groups it implies, they differ from the best k only by experts within `tol` of the k-th."""
    E = b.shape[1]
    gs = E // n_group
    k = ids.shape[1]
    for t in range(ids.shape[0]):
        if np.array_equal(ids[t], want_ids[t]):
            continue
        grp = b[t].reshape(n_group, gs)
        top2 = np.sort(grp, axis=1)[:, -2:].sum(1) if gs > 1 else grp[:, 0]
        cut = np.sort(top2)[::-1][topk_group - 1]
        sure = set(np.nonzero(top2 > cut + tol)[0].tolist())
        maybe = set(np.nonzero(np.abs(top2 - cut) <= tol)[0].tolist())
        got_groups = set((ids[t] // gs).tolist())
        assert got_groups <= (sure | maybe), (t, got_groups, sure, maybe)
        # the kept set the device must have used: the sure groups plus the tied ones it drew from, filled up with tied ones
        kept = set(sure) | (got_groups & maybe)
        for g in sorted(maybe - kept):
            if len(kept) < topk_group:
                kept.add(g)
        assert len(kept) == topk_group, (t, kept)
        live = np.concatenate([np.arange(g * gs, (g + 1) * gs) for g in sorted(kept)])
        order = live[np.argsort(-b[t, live], kind="stable")]
        kth = b[t, order[k - 1]]
        best = set(order[:k].tolist())
        for e in set(ids[t].tolist()) ^ best:
            assert abs(b[t, e] - kth) < tol, (t, e)
