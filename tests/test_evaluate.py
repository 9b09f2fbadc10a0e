"""Recall evaluation (host side): exact neighbours under the three metrics and the report keys of
upstream's harness (python/benchmark/bench_base.py:154-213, :301-351)."""
import importlib.util
import os
import sys
import types

import numpy as np
import scipy.sparse as sp


def _load_evaluate():
    """Import culsh_b200/evaluate.py without the package's import-time load of the CUDA library,
    so the check runs on machines without a GPU build as well."""
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "culsh_b200")
    pkg = types.ModuleType("_culsh_eval_pkg")
    pkg.__path__ = [root]
    sys.modules["_culsh_eval_pkg"] = pkg
    for name in ("utils", "evaluate"):
        spec = importlib.util.spec_from_file_location(f"_culsh_eval_pkg.{name}", os.path.join(root, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
    return sys.modules["_culsh_eval_pkg.evaluate"]


class _Cand:
    def __init__(self, lists):
        self.n_queries = len(lists)
        self._idx = np.concatenate([np.asarray(x, dtype=np.int32) for x in lists]) if lists else np.zeros(0, np.int32)
        self._off = np.concatenate([[0], np.cumsum([len(x) for x in lists])]).astype(np.uint64)

    def get_indices(self):
        return self._idx

    def get_offsets(self):
        return self._off


def test_ground_truth_and_recall_report():
    ev = _load_evaluate()
    rng = np.random.RandomState(0)
    X = rng.randn(200, 16)
    Q = X[:5] + 0.01 * rng.randn(5, 16)
    # exact neighbours: brute force by definition
    for i in range(5):
        cos = (X @ Q[i]) / (np.linalg.norm(X, axis=1) * np.linalg.norm(Q[i]))
        assert np.array_equal(ev.ground_truth_top_k(X, Q[i], 7, "cosine"), np.argsort(-cos, kind="stable")[:7])
        dist = np.linalg.norm(X - Q[i], axis=1)
        assert np.array_equal(ev.ground_truth_top_k(X, Q[i], 7, "euclidean"), np.argsort(dist, kind="stable")[:7])
    S = sp.random(50, 40, density=0.2, random_state=1, format="csr")
    q = S[3:4]
    A = (S.toarray() != 0)
    jac = (A & A[3]).sum(1) / np.maximum((A | A[3]).sum(1), 1)
    got = ev.ground_truth_top_k(S, q, 5, "jaccard")
    assert got[0] == 3 and np.allclose(np.sort(jac[got])[::-1], np.sort(jac)[::-1][:5])
    # perfect candidates, half candidates, none
    full = [ev.ground_truth_top_k(X, Q[i], 10, "cosine") for i in range(3)]
    cand = _Cand([np.sort(full[0]), np.sort(full[1][:5]), []])
    r = ev.evaluate_recall(X, Q, cand, [5, 10], "cosine", n_eval=10)
    assert r["n_eval_queries"] == 3 and r["queries_with_candidates"] == 2
    assert r["per_query_recall_at_k"][10] == [1.0, 0.5, 0.0]
    assert r["per_query_recall_at_k"][5] == [1.0, 1.0, 0.0]
    assert abs(r["mean_candidates"] - 5.0) < 1e-12
    rep = ev.make_report("RPLSH", 16, 4, 42, 3, r, fit_time=0.1, query_time=0.2)
    assert set(rep) == {"algorithm", "params", "runtimes", "recall_evaluation"}
    assert rep["params"]["mode"] == "fit+query" and set(rep["runtimes"]) == {"fit_time", "query_time"}
    assert ev.make_report("RPLSH", 16, 4, 42, 3, r, fit_query_time=0.3)["params"]["mode"] == "fit_query"
