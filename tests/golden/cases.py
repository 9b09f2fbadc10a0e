"""Seeded inputs shared by capture_ref_cuda.py (which ran upstream's CUDA build on them)
and by the tests that compare against the captured arrays."""
import numpy as np
import scipy.sparse as sp

CASES = {
    "rplsh": dict(n=1200, nq=100, d=32, L=8, k=10, seed=42),
    "pslsh": dict(n=1200, nq=100, d=32, L=8, k=4, w=4, seed=0),
    "minhash": dict(n=800, nq=80, d=300, density=0.05, L=8, k=3, seed=1),
}
PARAM_SEEDS = (42, 0, 1, 2, 3)
PARAM_SHAPE = dict(L=4, k=8, d=16, w=3)


def dense_inputs(c):
    rng = np.random.RandomState(c["seed"] + 1000)
    X = rng.randn(c["n"], c["d"]).astype(np.float32)
    Q = np.concatenate([X[:50] + 0.01 * rng.randn(50, c["d"]).astype(np.float32),
                        rng.randn(c["nq"] - 50, c["d"]).astype(np.float32)])
    return X, Q


def csr_inputs(c):
    rng = np.random.RandomState(c["seed"] + 1000)
    X = sp.random(c["n"], c["d"], density=c["density"], format="csr", dtype=np.float32, random_state=rng)
    X.sort_indices()
    Q = sp.vstack([X[:40], sp.random(c["nq"] - 40, c["d"], density=c["density"], format="csr",
                                     dtype=np.float32, random_state=rng)]).tocsr()
    Q.sort_indices()
    return X, Q
