"""culsh_b200: B200-native LSH engine with cuLSH's public API.

    from culsh_b200 import RPLSH, PStableLSH, MinHashLSH

The CUDA library (libculsh_b200.so, built by ``python -m culsh_b200.build``) is loaded on
import; there is no CPU fallback.
"""
import sys as _sys

__version__ = "0.1.0"

# `python -m culsh_b200.build` must be able to replace a missing or outdated library, so the
# build entry point alone skips loading it.
_building = any(str(a).endswith("culsh_b200.build") for a in getattr(_sys, "orig_argv", []))

if not _building:
    from . import _lib

    _lib.load()  # fail loudly if the CUDA library is missing

    from ._culsh_core import Candidates  # noqa: E402
    from .minhash_lsh import MinHashLSH, MinHashLSHModel  # noqa: E402
    from .pstable_lsh import PStableLSH, PStableLSHModel  # noqa: E402
    from .rp_lsh import RPLSH, RPLSHModel  # noqa: E402

    __all__ = ["RPLSH", "RPLSHModel", "MinHashLSH", "MinHashLSHModel", "PStableLSH", "PStableLSHModel",
               "Candidates"]
