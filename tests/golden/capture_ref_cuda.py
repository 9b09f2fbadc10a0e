"""Capture golden arrays from upstream cuLSH's own CUDA build (run on a GPU box).

    make -C oracle ref REF=/path/to/cuLSH        # builds oracle/_ref/_culsh_core*.so
    python tests/golden/capture_ref_cuda.py [out_dir]

Drives upstream's pybind11 module directly with torch CUDA tensors (it only reads the raw
pointer from ``__cuda_array_interface__``), on small seeded inputs that the tests rebuild
with the same NumPy seeds, and stores hash parameters, the four index arrays and the
candidates CSR per family in ``ref_cuda_<family>.npz``.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(0, HERE)
import _culsh_core as ref  # noqa: E402  (upstream's module, unmodified)

OUT = sys.argv[1] if len(sys.argv) > 1 else HERE

from cases import CASES, PARAM_SEEDS, PARAM_SHAPE, csr_inputs, dense_inputs  # noqa: E402


def dev(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    torch.cuda.synchronize()
    return t


def index_arrays(ix):
    return dict(candidate_indices=ix.get_candidate_indices(), bucket_signatures=ix.get_bucket_signatures(),
                bucket_candidate_offsets=ix.get_bucket_candidate_offsets(),
                table_bucket_offsets=ix.get_table_bucket_offsets(),
                n_total_buckets=ix.n_total_buckets, sig_nbytes=ix.sig_nbytes)


def cand_arrays(c, prefix):
    return {f"{prefix}_indices": c.get_indices(), f"{prefix}_offsets": c.get_offsets(),
            f"{prefix}_counts": c.get_counts()}


def main():
    c = CASES["rplsh"]
    X, Q = dense_inputs(c)
    core = ref.RPLSHCore(c["L"], c["k"], c["seed"])
    Xd, Qd = dev(X), dev(Q)
    ix = core.fit_float(Xd, c["n"], c["d"])
    out = dict(index_arrays(ix), projection=ix.get_projection_matrix())
    out.update(cand_arrays(core.query_float(Qd, c["nq"], ix), "query"))
    out.update(cand_arrays(core.fit_query_float(Xd, c["n"], c["d"]), "fit_query"))
    np.savez_compressed(os.path.join(OUT, "ref_cuda_rplsh.npz"), **out)

    c = CASES["pslsh"]
    X, Q = dense_inputs(c)
    core = ref.PSLSHCore(c["L"], c["k"], c["w"], c["seed"])
    Xd, Qd = dev(X), dev(Q)
    ix = core.fit_float(Xd, c["n"], c["d"])
    out = dict(index_arrays(ix), projection=ix.get_projection_matrix(), bias=ix.get_bias())
    out.update(cand_arrays(core.query_float(Qd, c["nq"], ix), "query"))
    np.savez_compressed(os.path.join(OUT, "ref_cuda_pslsh.npz"), **out)

    c = CASES["minhash"]
    X, Q = csr_inputs(c)
    core = ref.MinHashCore(c["L"], c["k"], c["seed"])
    xi, xp = dev(X.indices.astype(np.int32)), dev(X.indptr.astype(np.int32))
    qi, qp = dev(Q.indices.astype(np.int32)), dev(Q.indptr.astype(np.int32))
    ix = core.fit(xi, xp, c["n"], c["d"])
    out = dict(index_arrays(ix), hash_a=ix.get_hash_a(), hash_b=ix.get_hash_b())
    out.update(cand_arrays(core.query(qi, qp, c["nq"], ix), "query"))
    out.update(cand_arrays(core.fit_query(xi, xp, c["n"], c["d"]), "fit_query"))
    np.savez_compressed(os.path.join(OUT, "ref_cuda_minhash.npz"), **out)

    # hash parameters for the seeds of the benchmark configurations (small shapes)
    params = {}
    ps = PARAM_SHAPE
    assert (ps["L"], ps["k"], ps["d"], ps["w"]) == (4, 8, 16, 3)
    for seed in PARAM_SEEDS:
        ix = ref.RPLSHCore(4, 8, seed).fit_float(dev(np.ones((4, 16), np.float32)), 4, 16)
        params[f"rplsh_P_seed{seed}"] = ix.get_projection_matrix()
        ix = ref.PSLSHCore(4, 8, 3, seed).fit_float(dev(np.ones((4, 16), np.float32)), 4, 16)
        params[f"pslsh_P_seed{seed}"] = ix.get_projection_matrix()
        params[f"pslsh_b_seed{seed}"] = ix.get_bias()
        ix = ref.MinHashCore(4, 8, seed).fit(dev(np.array([0, 1], np.int32)), dev(np.array([0, 2], np.int32)), 1, 4)
        params[f"minhash_A_seed{seed}"] = ix.get_hash_a()
        params[f"minhash_B_seed{seed}"] = ix.get_hash_b()
    np.savez_compressed(os.path.join(OUT, "ref_cuda_params.npz"), **params)
    print("captured reference CUDA goldens into", OUT)


if __name__ == "__main__":
    main()
