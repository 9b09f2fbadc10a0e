"""The C-ABI library loads and exports every entry point that include/culsh_b200.h declares;
the Python layer mirrors upstream's class surface; nothing falls back to the CPU."""
import ctypes
import inspect
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "culsh_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(culsh_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from culsh_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.ALL_SYMBOLS) == names, "ctypes table and header disagree"


def test_struct_layouts_match_header():
    from culsh_b200 import _lib
    assert ctypes.sizeof(_lib.IndexMeta) == 12 * 4 + 2 * 8
    assert ctypes.sizeof(_lib.Stats) == 10 * 4 + 4 * 8 + 6 * 4


def test_python_layer_mirrors_upstream_surface():
    import culsh_b200
    from culsh_b200 import _culsh_core as cc
    for cls, methods in [
        (cc.RPLSHCore, ["fit_float", "fit_double", "query_float", "query_double", "fit_query_float", "fit_query_double"]),
        (cc.PSLSHCore, ["fit_float", "fit_double", "query_float", "query_double", "fit_query_float", "fit_query_double"]),
        (cc.MinHashCore, ["fit", "query", "fit_query"]),
        (cc.Candidates, ["empty", "get_indices", "get_counts", "get_offsets"]),
        (cc.RPLSHIndex, ["get_candidate_indices", "get_bucket_signatures", "get_bucket_candidate_offsets",
                         "get_table_bucket_offsets", "get_projection_matrix", "load_float", "load_double",
                         "empty", "size_bytes"]),
        (cc.PSLSHIndex, ["get_bias", "get_projection_matrix", "load_float", "load_double"]),
        (cc.MinHashIndex, ["get_hash_a", "get_hash_b", "load"]),
    ]:
        for m in methods:
            assert callable(getattr(cls, m)), f"{cls.__name__}.{m} missing"
    assert "as_cupy" in inspect.signature(cc.Candidates.get_indices).parameters
    assert inspect.signature(cc.RPLSHCore.__init__).parameters["seed"].default == 42
    for name in ["RPLSH", "RPLSHModel", "PStableLSH", "PStableLSHModel", "MinHashLSH", "MinHashLSHModel"]:
        assert hasattr(culsh_b200, name)
    for model in (culsh_b200.RPLSHModel, culsh_b200.PStableLSHModel, culsh_b200.MinHashLSHModel):
        for m in ("query", "save", "load"):
            assert callable(getattr(model, m))


def test_argument_validation_happens_before_any_gpu_work():
    import culsh_b200
    with pytest.raises(ValueError):
        culsh_b200.RPLSH(0, 4)
    with pytest.raises(ValueError):
        culsh_b200.PStableLSH(4, 0)
    with pytest.raises(ValueError):
        culsh_b200.PStableLSH(4, 4, window_size=0)
    with pytest.raises(ValueError):
        culsh_b200.MinHashLSH(-1, 4)
    assert culsh_b200.RPLSH(2, 2).seed >= 0  # seed=None draws one
    assert culsh_b200.PStableLSH(2, 2).window_size == "auto"


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import culsh_b200
    with pytest.raises(RuntimeError):
        culsh_b200.RPLSH(2, 4, seed=1).fit(np.zeros((8, 4), dtype=np.float32))


def test_product_code_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "culsh_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"


def test_every_entry_point_that_runs_the_gather_reads_the_device_error_word():
    """The gather's look-back waits are bounded and report through the handle's error word; a
    call that returns a result without reading that word could hand back a CSR written at
    wrong offsets.  Source-level check: between a call of the gather and the release of its
    result the error word is read and checked."""
    text = open(os.path.join(ROOT, "culsh_b200", "csrc", "culsh_b200.cu")).read()
    sites = [m.start() for m in re.finditer(r"\bquery_from_matched\(\*ix|\brun\(Q, n_q, \*res\)|\bquery_batch\(\*ix, n_q", text)]
    assert len(sites) >= 4
    for pos in sites:
        end = text.index("*out = res.release();", pos)
        assert "check_error_word(read_error_word(" in text[pos:end], text[pos:pos + 80]
