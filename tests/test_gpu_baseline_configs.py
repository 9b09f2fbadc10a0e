"""The engine against upstream cuLSH's own CUDA build, run live on the same device tensors,
on the benchmark configurations themselves (their value laws, table / hash counts and seeds;
the two largest at reduced row counts so that the comparison takes seconds).

What must hold (the tolerance is the benchmark specification's):
  * hash parameters bit-equal (same cuRAND calls in the same order);
  * MinHash: all four index arrays and both candidate CSRs array-equal;
  * dense families: the signature elements stored by the two indexes are equal except where
    a float64 recomputation puts the projection within REL_BAND of the sign / floor boundary;
    the number of such elements is printed and bounded; the index arrays are array-equal when
    no element differs, and the candidate lists are equal once the rows whose signature
    differs are set aside (queries with an element inside the band are set aside too, since
    upstream's query signatures cannot be read back).
Skipped only when upstream's module (oracle/_ref, built by oracle/Makefile) is not loadable.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
from oracle import oracle  # noqa: E402

pytestmark = pytest.mark.gpu

REL_BAND = 1e-5          # relative distance from the boundary inside which a bit may differ
MAX_BAND_FRACTION = 2e-4  # of all signature elements; measured: a few 1e-5 on these laws

# workload id -> (rows, queries) used here; None keeps the benchmark's own size
SIZES = {"c1": (None, None), "c2": (200_000, 2_000), "c3": (100_000, 1_000), "c4": (500_000, 2_000),
         "c5": (200_000, None)}


@pytest.fixture(scope="module")
def ref():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    mod = bench.load_reference_module()
    if mod is None:
        pytest.skip("upstream's CUDA build (oracle/_ref) is not loadable")
    return mod


def _setup(wl):
    import torch
    spec = dict(bench.WORKLOADS[wl])
    rows, queries = SIZES[wl]
    if rows:
        spec["n"] = rows
    if queries:
        spec["nq"] = queries
    device = torch.device("cuda:0")
    X, Q = bench.make_inputs(torch, device, 0, wl, spec)
    torch.cuda.synchronize()
    return torch, device, spec, X, Q


def _csr_pairs(indices, offsets, keep_query, drop_row):
    """(query, id) pairs of a CSR restricted to kept queries and to ids not in drop_row."""
    off = offsets.astype(np.int64)
    q = np.repeat(np.arange(len(off) - 1), np.diff(off))
    keep = keep_query[q] & ~drop_row[indices]
    return q[keep], indices[keep]


def _assert_csr_equal_modulo(a, b, keep_query, drop_row, what):
    qa, ia = _csr_pairs(a.get_indices(), a.get_offsets(), keep_query, drop_row)
    qb, ib = _csr_pairs(b.get_indices(), b.get_offsets(), keep_query, drop_row)
    assert np.array_equal(qa, qb) and np.array_equal(ia, ib), f"{what}: candidate lists differ"


def _index_arrays_equal(a, b):
    return (a.n_total_buckets == b.n_total_buckets
            and np.array_equal(a.get_table_bucket_offsets(), b.get_table_bucket_offsets())
            and np.array_equal(a.get_bucket_candidate_offsets(), b.get_bucket_candidate_offsets())
            and np.array_equal(a.get_bucket_signatures(), b.get_bucket_signatures())
            and np.array_equal(a.get_candidate_indices(), b.get_candidate_indices()))


def _dense_case(ref, wl):
    from culsh_b200 import _culsh_core
    torch, device, spec, X, Q = _setup(wl)
    n, nq, L, k, d, fam = spec["n"], spec["nq"], spec["L"], spec["k"], spec["d"], spec["family"]
    ours_core, ref_core = bench.make_core(_culsh_core, spec), bench.make_core(ref, spec)
    ours = bench.core_fit(ours_core, spec, X)
    theirs = bench.core_fit(ref_core, spec, X)
    # parameters: same seed, same numbers
    P = theirs.get_projection_matrix()
    assert np.array_equal(ours.get_projection_matrix(), P)
    bias = None
    if fam == "pslsh":
        bias = theirs.get_bias()
        assert np.array_equal(ours.get_bias(), bias)
    Pd = torch.from_numpy(P).to(device).view(L * k, d)
    bd = torch.from_numpy(bias).to(device) if bias is not None else None
    # stored signatures, element by element
    mm = bench.signature_mismatch(torch, fam, bench.row_signatures(torch, device, theirs, n, L),
                                  bench.row_signatures(torch, device, ours, n, L), X, Pd, bd, k, REL_BAND)
    print(f"{wl}: {mm['mismatch']} of {mm['elements']} signature elements differ from upstream's "
          f"({mm['in_band']} inside the {REL_BAND:g} band, {mm['out_of_band']} outside), "
          f"{int(mm['rows'].numel())} rows affected")
    assert mm["out_of_band"] == 0, "a signature element differs outside the rounding band"
    assert mm["mismatch"] <= MAX_BAND_FRACTION * mm["elements"]
    bad = np.zeros(n, dtype=bool)
    bad[mm["rows"].cpu().numpy()] = True
    if not bad.any():
        assert _index_arrays_equal(ours, theirs), "index arrays differ although every signature is equal"
    return torch, spec, X, Q, ours_core, ref_core, ours, theirs, P, bias, bad


def _query_clean(fam, Q, P, bias, L, k, d):
    Qh = Q.cpu().numpy()
    Pm = P.reshape(L * k, d)
    near = (oracle.rplsh_near_boundary(Qh, Pm, REL_BAND) if fam == "rplsh"
            else oracle.pslsh_near_boundary(Qh, Pm, bias, REL_BAND))
    return ~near.any(axis=1)


@pytest.mark.parametrize("wl", ["c1", "c2", "c4"])
def test_dense_fit_and_query_equal_upstream(ref, wl):
    torch, spec, X, Q, ours_core, ref_core, ours, theirs, P, bias, bad = _dense_case(ref, wl)
    nq = spec["nq"]
    batch = nq if wl == "c2" else None
    a = bench.core_query(ours_core, spec, Q, ours, batch)
    b = bench.core_query(ref_core, spec, Q, theirs, batch)
    clean = _query_clean(spec["family"], Q, P, bias, spec["L"], spec["k"], spec["d"])
    assert clean.mean() > 0.5
    if not bad.any() and clean.all():
        assert np.array_equal(a.get_indices(), b.get_indices())
        assert np.array_equal(a.get_offsets(), b.get_offsets())
        assert np.array_equal(a.get_counts(), b.get_counts())
    _assert_csr_equal_modulo(a, b, clean, bad, wl)
    print(f"{wl}: {a.n_total_candidates} candidates here, {b.n_total_candidates} upstream, "
          f"{int((~clean).sum())} of {nq} queries set aside, {int(bad.sum())} rows set aside")


def test_self_join_equals_upstream_c5(ref):
    torch, spec, X, Q, ours_core, ref_core, ours, theirs, P, bias, bad = _dense_case(ref, "c5")
    n, d = spec["n"], spec["d"]
    a = ours_core.fit_query_float(X, n, d)
    b = ref_core.fit_query_float(X, n, d)
    assert a.n_queries == b.n_queries == n
    if not bad.any():
        assert np.array_equal(a.get_indices(), b.get_indices())
        assert np.array_equal(a.get_offsets(), b.get_offsets())
    _assert_csr_equal_modulo(a, b, ~bad, bad, "c5")
    print(f"c5: {a.n_total_candidates} candidates here, {b.n_total_candidates} upstream, "
          f"{int(bad.sum())} rows set aside")


def test_minhash_equals_upstream_c3(ref):
    from culsh_b200 import _culsh_core
    torch, device, spec, X, Q = _setup("c3")
    ours_core, ref_core = bench.make_core(_culsh_core, spec), bench.make_core(ref, spec)
    ours = bench.core_fit(ours_core, spec, X)
    theirs = bench.core_fit(ref_core, spec, X)
    assert np.array_equal(ours.get_hash_a(), theirs.get_hash_a())
    assert np.array_equal(ours.get_hash_b(), theirs.get_hash_b())
    assert _index_arrays_equal(ours, theirs)
    a = bench.core_query(ours_core, spec, Q, ours, None)
    b = bench.core_query(ref_core, spec, Q, theirs, None)
    for g in ("get_indices", "get_offsets", "get_counts"):
        assert np.array_equal(getattr(a, g)(), getattr(b, g)()), g
    a = ours_core.fit_query(X[0], X[1], spec["n"], spec["d"])
    b = ref_core.fit_query(X[0], X[1], spec["n"], spec["d"])
    for g in ("get_indices", "get_offsets", "get_counts"):
        assert np.array_equal(getattr(a, g)(), getattr(b, g)()), g
    print(f"c3: {ours.n_total_buckets} buckets, {a.n_total_candidates} self-join candidates, all arrays equal")
