"""The CUDA path against arrays captured from upstream's own CUDA build on a B200
(tests/golden/ref_cuda_*.npz): same seeds must give the same hash parameters (same cuRAND
calls in the same order), the same index arrays and the same candidates."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from cases import CASES, PARAM_SEEDS, PARAM_SHAPE, csr_inputs, dense_inputs  # noqa: E402
from test_oracle_vs_ref_cuda import _csr_lists, _ref_row_signatures  # noqa: E402

from oracle import oracle  # noqa: E402

pytestmark = pytest.mark.gpu


def _index_arrays_equal(ix, g):
    return (ix.n_total_buckets == int(g["n_total_buckets"])
            and np.array_equal(ix.get_table_bucket_offsets(), g["table_bucket_offsets"])
            and np.array_equal(ix.get_bucket_candidate_offsets(), g["bucket_candidate_offsets"])
            and np.array_equal(ix.get_bucket_signatures(), g["bucket_signatures"])
            and np.array_equal(ix.get_candidate_indices(), g["candidate_indices"]))


def test_hash_parameters_equal_reference_for_benchmark_seeds(golden_dir):
    import culsh_b200
    g = np.load(os.path.join(golden_dir, "ref_cuda_params.npz"))
    ps = PARAM_SHAPE
    ones = np.ones((4, ps["d"]), np.float32)
    import scipy.sparse as sp
    tiny = sp.csr_matrix(np.array([[1, 1, 0, 0]], dtype=np.float32))
    for seed in PARAM_SEEDS:
        ix = culsh_b200.RPLSH(ps["L"], ps["k"], seed=seed).fit(ones).index
        assert np.array_equal(ix.get_projection_matrix(), g[f"rplsh_P_seed{seed}"])
        ix = culsh_b200.PStableLSH(ps["L"], ps["k"], window_size=ps["w"], seed=seed).fit(ones).index
        assert np.array_equal(ix.get_projection_matrix(), g[f"pslsh_P_seed{seed}"])
        assert np.array_equal(ix.get_bias(), g[f"pslsh_b_seed{seed}"])
        ix = culsh_b200.MinHashLSH(ps["L"], ps["k"], seed=seed).fit(tiny).index
        assert np.array_equal(ix.get_hash_a(), g[f"minhash_A_seed{seed}"])
        assert np.array_equal(ix.get_hash_b(), g[f"minhash_B_seed{seed}"])


def test_minhash_equals_reference_cuda(golden_dir):
    import culsh_b200
    c = CASES["minhash"]
    g = np.load(os.path.join(golden_dir, "ref_cuda_minhash.npz"))
    X, Q = csr_inputs(c)
    lsh = culsh_b200.MinHashLSH(c["L"], c["k"], seed=c["seed"])
    model = lsh.fit(X)
    assert np.array_equal(model.index.get_hash_a(), g["hash_a"])
    assert np.array_equal(model.index.get_hash_b(), g["hash_b"])
    assert _index_arrays_equal(model.index, g)
    r = model.query(Q)
    assert np.array_equal(r.get_indices(), g["query_indices"])
    assert np.array_equal(r.get_offsets(), g["query_offsets"])
    assert np.array_equal(r.get_counts(), g["query_counts"])
    r = lsh.fit_query(X)
    assert np.array_equal(r.get_indices(), g["fit_query_indices"])
    assert np.array_equal(r.get_offsets(), g["fit_query_offsets"])


@pytest.mark.parametrize("fam", ["rplsh", "pslsh"])
@pytest.mark.parametrize("path", [1, 0])  # 1 = CUDA-core projection, 0 = automatic (tensor cores)
def test_dense_equals_reference_cuda(golden_dir, fam, path):
    import culsh_b200
    from culsh_b200 import _culsh_core
    c = CASES[fam]
    g = np.load(os.path.join(golden_dir, f"ref_cuda_{fam}.npz"))
    X, Q = dense_inputs(c)
    n, L, k, d = c["n"], c["L"], c["k"], c["d"]
    if fam == "rplsh":
        lsh = culsh_b200.RPLSH(L, k, seed=c["seed"])
        core = _culsh_core.RPLSHCore(L, k, c["seed"])
        s, elem = k, np.uint8
    else:
        lsh = culsh_b200.PStableLSH(L, k, window_size=c["w"], seed=c["seed"])
        core = _culsh_core.PSLSHCore(L, k, c["w"], c["seed"])
        s, elem = 4 * k, np.int32
    core.set_projection_path(path)
    try:
        model = lsh.fit(X)
        ix = model.index
        assert np.array_equal(ix.get_projection_matrix(), g["projection"])  # cuRAND parity
        P = g["projection"].reshape(L * k, d)
        if fam == "rplsh":
            near, qnear = oracle.rplsh_near_boundary(X, P), oracle.rplsh_near_boundary(Q, P)
        else:
            assert np.array_equal(ix.get_bias(), g["bias"])
            near = oracle.pslsh_near_boundary(X, P, g["bias"])
            qnear = oracle.pslsh_near_boundary(Q, P, g["bias"])
        ref_raw = _ref_row_signatures(g, n, L, s)
        ours_raw = np.ascontiguousarray(core.hash(X, ix)).view(np.uint8).reshape(L, n, s)
        differ = np.any(ref_raw != ours_raw, axis=2)
        near_tr = near.reshape(n, L, k).any(axis=2).T
        assert not np.any(differ & ~near_tr), "signature differs from the reference outside the band"
        print(f"{fam}: {int(differ.sum())} of {differ.size} (table,row) signatures differ inside the band")
        if not differ.any():
            assert _index_arrays_equal(ix, g)
        r = model.query(Q)
        ours = _csr_lists(r.get_indices(), r.get_offsets())
        theirs = _csr_lists(g["query_indices"], g["query_offsets"])
        clean = ~qnear.any(axis=1)
        if differ.any():  # a flipped row may enter or leave a candidate list: compare modulo those rows
            bad = set(np.flatnonzero(differ.any(axis=0)).tolist())
            for q in np.flatnonzero(clean):
                assert set(ours[q].tolist()) - bad == set(theirs[q].tolist()) - bad
        else:
            for q in np.flatnonzero(clean):
                assert np.array_equal(ours[q], theirs[q])
    finally:
        core.set_projection_path(0)
