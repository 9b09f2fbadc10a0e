"""Helpers of the user-facing layer (mirrors python/culsh/utils.py:15-80 without the hard
CuPy dependency: NumPy / SciPy inputs are passed to the engine as host memory, CuPy / torch
CUDA arrays as device memory)."""
from __future__ import annotations

import logging
import random
from typing import Optional

import numpy as np
import scipy.sparse


def resolve_seed(seed: Optional[int]) -> int:
    """A given seed is used as is; None draws a fresh one (python/culsh/utils.py:15-19)."""
    return random.randint(0, 2**63 - 1) if seed is None else seed


def is_device_array(arr) -> bool:
    if hasattr(arr, "__cuda_array_interface__"):
        return True
    return type(arr).__module__.startswith("torch") and bool(getattr(arr, "is_cuda", False))


def is_sparse(arr) -> bool:
    if scipy.sparse.issparse(arr):
        return True
    return type(arr).__module__.startswith("cupyx.scipy.sparse")


def get_array_info(arr):
    """(n_rows, n_cols, dtype) of a 2-D dense or CSR array (python/culsh/utils.py:22-31)."""
    if arr.ndim != 2:
        raise ValueError(f"Expected 2D array, got {arr.ndim}D")
    dtype = arr.dtype
    if type(arr).__module__.startswith("torch"):
        import torch
        dtype = {torch.float32: np.dtype(np.float32), torch.float64: np.dtype(np.float64)}.get(dtype, dtype)
    return int(arr.shape[0]), int(arr.shape[1]), dtype


def ensure_engine_array(arr):
    """Dense input as something the engine can read: a C-contiguous NumPy array (host) or a
    C-contiguous device array.  Counterpart of ensure_device_array
    (python/culsh/utils.py:34-53); the host-to-device copy happens inside the engine."""
    if is_device_array(arr):
        if type(arr).__module__.startswith("torch"):
            return arr if arr.is_contiguous() else arr.contiguous()
        if not arr.flags.c_contiguous:
            import cupy as cp
            return cp.ascontiguousarray(arr)
        return arr
    if type(arr).__module__.startswith("torch"):
        arr = arr.detach().numpy()
    return np.ascontiguousarray(arr)


def compute_recall(lsh_indices, gt_indices) -> float:
    """|candidates ∩ ground truth| / |ground truth| (python/culsh/utils.py:56-67)."""
    if len(gt_indices) == 0:
        return 0.0
    return len(np.intersect1d(np.asarray(lsh_indices), np.asarray(gt_indices))) / len(gt_indices)


def get_logger(instance: object) -> logging.Logger:
    logger = logging.getLogger(instance.__class__.__name__)
    logger.setLevel(logging.INFO)
    if not logger.handlers:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter(
            "%(asctime)s [%(name)s] %(levelname)s: %(message)s", datefmt="%Y-%m-%d %H:%M:%S"))
        logger.addHandler(handler)
    return logger
