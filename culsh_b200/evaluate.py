"""Recall evaluation of LSH candidates against exact neighbours (host side, NumPy / SciPy).

Mirrors what upstream's benchmark harness reports (python/benchmark/bench_base.py:154-213,
the `recall_evaluation` block of its JSON report, :301-351) so that results of the two
implementations can be laid side by side: recall@k of the first `n_eval` queries, the number of
queries with at least one candidate and the mean candidate count.  Exact neighbours are found
by brute force under the metric the family approximates: cosine similarity (RPLSH,
bench_rplsh.py:65-71), Euclidean distance (PStableLSH) or Jaccard similarity of the sets of
non-zero columns (MinHashLSH).
"""
from __future__ import annotations

from typing import Dict, Iterable, List

import numpy as np

from .utils import compute_recall

METRICS = ("cosine", "euclidean", "jaccard")


def ground_truth_top_k(X, q, k: int, metric: str) -> np.ndarray:
    """Indices of the k rows of X nearest to the single query q, best first."""
    if metric == "cosine":
        X = np.asarray(X, dtype=np.float64)
        q = np.asarray(q, dtype=np.float64).ravel()
        score = (X @ q) / np.maximum(np.linalg.norm(X, axis=1) * np.linalg.norm(q), 1e-300)
    elif metric == "euclidean":
        X = np.asarray(X, dtype=np.float64)
        q = np.asarray(q, dtype=np.float64).ravel()
        score = -(np.einsum("ij,ij->i", X, X) - 2.0 * (X @ q))
    elif metric == "jaccard":
        import scipy.sparse as sp
        Xb = sp.csr_matrix(X).astype(bool).astype(np.float64)
        qb = sp.csr_matrix(q).astype(bool).astype(np.float64)
        inter = np.asarray((Xb @ qb.T).todense()).ravel()
        union = np.asarray(Xb.sum(axis=1)).ravel() + qb.sum() - inter
        score = np.where(union > 0, inter / np.maximum(union, 1.0), 0.0)
    else:
        raise ValueError(f"metric must be one of {METRICS}")
    k = min(int(k), score.shape[0])
    top = np.argpartition(-score, k - 1)[:k] if k < score.shape[0] else np.arange(score.shape[0])
    return top[np.argsort(-score[top], kind="stable")]


def evaluate_recall(X, Q, candidates, recall_k_values: Iterable[int], metric: str,
                    n_eval: int = 10) -> Dict:
    """Recall@k of `candidates` (anything with n_queries, get_indices(), get_offsets()) for the
    first n_eval queries of Q.  Same keys as upstream's report block."""
    ks: List[int] = [int(k) for k in recall_k_values]
    n_eval = min(int(n_eval), Q.shape[0], candidates.n_queries)
    indices = np.asarray(candidates.get_indices())
    offsets = np.asarray(candidates.get_offsets()).astype(np.int64)
    per_query = {k: [] for k in ks}
    counts, with_candidates = [], 0
    for i in range(n_eval):
        mine = indices[offsets[i]:offsets[i + 1]]
        counts.append(int(mine.shape[0]))
        if mine.shape[0] == 0:
            for k in ks:
                per_query[k].append(0.0)
            continue
        with_candidates += 1
        qi = Q[i] if metric != "jaccard" else Q[i:i + 1]
        best = ground_truth_top_k(X, qi, max(ks), metric)
        for k in ks:
            per_query[k].append(float(compute_recall(mine, best[:k])))
    return {
        "n_eval_queries": n_eval,
        "queries_with_candidates": with_candidates,
        "recall_at_k": {k: float(np.mean(v)) if v else 0.0 for k, v in per_query.items()},
        "mean_candidates": float(np.mean(counts)) if counts else 0.0,
        "per_query_recall_at_k": per_query,
    }


def make_report(algorithm: str, n_hash_tables: int, n_hashes: int, seed: int, n_queries: int,
                recall_results: Dict, fit_time: float = None, query_time: float = None,
                fit_query_time: float = None) -> Dict:
    """The JSON report upstream's harness writes (bench_base.py:301-351), as a dict."""
    fused = fit_query_time is not None
    return {
        "algorithm": algorithm,
        "params": {"n_hash_tables": int(n_hash_tables), "n_hashes": int(n_hashes), "seed": int(seed),
                   "n_queries": int(n_queries), "recall_k": list(recall_results["recall_at_k"].keys()),
                   "mode": "fit_query" if fused else "fit+query"},
        "runtimes": ({"fit_query_time": fit_query_time} if fused
                     else {"fit_time": fit_time, "query_time": query_time}),
        "recall_evaluation": recall_results,
    }
