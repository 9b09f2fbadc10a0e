"""fit -> query -> evaluate_recall -> make_report on candidates that come from the GPU, on the
shapes of upstream's recall tests (python/tests/test_rplsh.py:27-73, test_pslsh.py:26-85,
test_minhash.py:36-82: 1000 rows, 100 features, 8 / 32 / 64 tables, recall@20).

Two comparisons per case:
  * exact: the recall of the engine's candidates equals the recall of the CPU oracle's
    candidates built from the same signatures (the candidate sets are equal, so every
    per-query figure must be equal);
  * statistical, as upstream does it: the mean recall@20 is close to that of an independent
    CPU LSH of the same family and size whose hash parameters come from NumPy's generator.
    Upstream allows 0.05 between its two single draws; on these shapes the recall of
    independent draws of the CPU LSH alone spreads by up to 0.07 (MinHash, 32 tables, density
    0.5), so the bound here is 0.1 - the exact comparison above is the strict one.
"""
import numpy as np
import pytest
import scipy.sparse as sp

from oracle import oracle

pytestmark = pytest.mark.gpu

N, D, K_EVAL, N_EVAL, THRESHOLD = 1000, 100, 20, 50, 0.1


class _OracleCandidates:
    def __init__(self, ind, off):
        self._ind, self._off, self.n_queries = ind, off, len(off) - 1

    def get_indices(self):
        return self._ind

    def get_offsets(self):
        return self._off


def _dense(seed=42):
    rng = np.random.RandomState(seed)
    return rng.randn(N, D).astype(np.float32)


def _sparse(density, seed=42):
    X = sp.random(N, D, density=density, format="csr", dtype=np.float32, random_state=np.random.RandomState(seed))
    X.data[:] = 1.0
    X.sort_indices()
    return X


def _evaluate(ev, X, cand, metric):
    return ev.evaluate_recall(X, X, cand, [K_EVAL], metric, n_eval=N_EVAL)


def _check(ev, name, X, cand, oracle_same, oracle_indep, metric, L, k, seed):
    got = _evaluate(ev, X, cand, metric)
    same = _evaluate(ev, X, oracle_same, metric)
    indep = _evaluate(ev, X, oracle_indep, metric)
    assert got["per_query_recall_at_k"] == same["per_query_recall_at_k"]
    assert got["mean_candidates"] == same["mean_candidates"]
    assert got["queries_with_candidates"] == N_EVAL  # every row is a candidate of itself
    diff = abs(got["recall_at_k"][K_EVAL] - indep["recall_at_k"][K_EVAL])
    print(f"{name} {L}x{k}: recall@{K_EVAL} {got['recall_at_k'][K_EVAL]:.4f} (independent CPU LSH "
          f"{indep['recall_at_k'][K_EVAL]:.4f}), mean candidates {got['mean_candidates']:.1f}")
    assert diff < THRESHOLD
    rep = ev.make_report(name, L, k, seed, cand.n_queries, got, fit_query_time=0.0)
    assert rep["params"]["mode"] == "fit_query" and rep["recall_evaluation"]["n_eval_queries"] == N_EVAL
    assert rep["params"]["recall_k"] == [K_EVAL]


@pytest.mark.parametrize("L", [8, 32, 64])
@pytest.mark.parametrize("k", [8, 16])
def test_rplsh_harness(L, k):
    import culsh_b200
    from culsh_b200 import _culsh_core, evaluate as ev
    X = _dense()
    lsh = culsh_b200.RPLSH(L, k, seed=42)
    cand = lsh.fit_query(X)
    model = lsh.fit(X)
    sig = _culsh_core.RPLSHCore(L, k, 42).hash(X, model.index).transpose(1, 0, 2).reshape(N, L * k)
    same = _OracleCandidates(*oracle.fit_query(sig, L, k)[:2])
    P = np.random.RandomState(7).randn(L * k, D).astype(np.float32)
    indep = _OracleCandidates(*oracle.fit_query(oracle.rplsh_signatures(X, P), L, k)[:2])
    _check(ev, "RPLSH", X, cand, same, indep, "cosine", L, k, 42)


@pytest.mark.parametrize("L", [8, 32])
@pytest.mark.parametrize("k,w", [(8, 8), (4, 4)])
def test_pslsh_harness(L, k, w):
    import culsh_b200
    from culsh_b200 import _culsh_core, evaluate as ev
    X = _dense()
    lsh = culsh_b200.PStableLSH(L, k, window_size=w, seed=42)
    cand = lsh.fit_query(X)
    model = lsh.fit(X)
    sig = _culsh_core.PSLSHCore(L, k, w, 42).hash(X, model.index).transpose(1, 0, 2).reshape(N, L * k)
    same = _OracleCandidates(*oracle.fit_query(sig, L, k)[:2])
    rng = np.random.RandomState(7)
    P = (rng.randn(L * k, D) / w).astype(np.float32)
    b = rng.uniform(0, 1, L * k).astype(np.float32)
    indep = _OracleCandidates(*oracle.fit_query(oracle.pslsh_signatures(X, P, b), L, k)[:2])
    _check(ev, "PStableLSH", X, cand, same, indep, "euclidean", L, k, 42)


@pytest.mark.parametrize("L", [8, 32])
@pytest.mark.parametrize("density", [0.1, 0.5])
def test_minhash_harness(L, density):
    import culsh_b200
    from culsh_b200 import _culsh_core, evaluate as ev
    k = 4
    X = _sparse(density)
    lsh = culsh_b200.MinHashLSH(L, k, seed=42)
    cand = lsh.fit_query(X)
    model = lsh.fit(X)
    sig = oracle.minhash_signatures(X.indices, X.indptr, model.index.get_hash_a(), model.index.get_hash_b())
    same = _OracleCandidates(*oracle.fit_query(sig, L, k)[:2])
    rng = np.random.RandomState(7)
    A, B = oracle.minhash_normalize(rng.randint(0, 2 ** 32, L * k, dtype=np.uint64),
                                    rng.randint(0, 2 ** 32, L * k, dtype=np.uint64))
    indep_sig = oracle.minhash_signatures(X.indices, X.indptr, A, B)
    indep = _OracleCandidates(*oracle.fit_query(indep_sig, L, k)[:2])
    _check(ev, "MinHashLSH", X, cand, same, indep, "jaccard", L, k, 42)
