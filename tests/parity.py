"""Acceptance rule shared by the GPU parity tests.

Distances must agree with the oracle within 1e-4 relative.  Top-k id sets must be
identical, except that an id may differ where the oracle's own distance for it
lies within that tolerance of the oracle's k-th distance (a tolerance tie at the
k-th / (k+1)-th boundary).
"""
import numpy as np

RTOL = 1e-4


def assert_distances_close(got, want, what=""):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    both_inf = np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want))
    err = np.abs(got - want)
    ok = both_inf | (err <= RTOL * np.abs(want) + 1e-30)
    assert ok.all(), (f"{what}: {int((~ok).sum())} distances off by more than {RTOL} relative; worst "
                      f"{np.nanmax(np.where(both_inf, 0, err / np.maximum(np.abs(want), 1e-30)))}")


def assert_topk_matches(oracle, xb, xq, metric, D, I, Dref, Iref, what="", candidates=None):
    """candidates: optional per-query arrays of admissible row ids (IVF probe union)."""
    nq, k = Iref.shape
    assert D.shape == Dref.shape and I.shape == Iref.shape, what
    for q in range(nq):
        valid_ref = Iref[q] >= 0
        nvalid = int(valid_ref.sum())
        assert (I[q, nvalid:] == -1).all(), f"{what}: query {q} should have {k - nvalid} missing slots"
        got, want = I[q, :nvalid], Iref[q, :nvalid]
        assert len(set(got.tolist())) == nvalid, f"{what}: query {q} returned duplicate or missing labels"
        # sorted best first
        dq = D[q, :nvalid].astype(np.float64)
        sgn = 1.0 if metric == oracle.METRIC_L2 else -1.0
        assert (np.diff(sgn * dq) >= 0).all(), f"{what}: query {q} not sorted best first"
        if set(got.tolist()) != set(want.tolist()):
            # every swapped-in id must be a tolerance tie with the oracle's k-th distance
            alld = oracle.all_distances(xb, xq[q], metric)
            kth = float(Dref[q, nvalid - 1])
            band = RTOL * abs(kth) + 1e-30
            for i in set(got.tolist()) ^ set(want.tolist()):
                assert abs(alld[i] - kth) <= 2 * band, (f"{what}: query {q} id {i} (distance {alld[i]}) differs from "
                                                        f"the oracle and is not a tie with the k-th ({kth})")
                if candidates is not None:
                    assert i in candidates[q], f"{what}: query {q} id {i} is outside the probed lists"
            # distances still have to match position by position
        assert_distances_close(D[q, :nvalid], Dref[q, :nvalid], f"{what} query {q}")
        # each reported distance must be the true distance of the reported id
        if nvalid:
            rows = xb[got].astype(np.float64)
            qq = xq[q].astype(np.float64)
            true = ((rows - qq) ** 2).sum(1) if metric == oracle.METRIC_L2 else rows @ qq
            assert_distances_close(D[q, :nvalid], true, f"{what} query {q} (distance of returned id)")
