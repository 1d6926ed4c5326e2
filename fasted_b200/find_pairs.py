"""Host-side mirror of the reference's Python entry to its shared library
(results/scripts/experiment/find_pairs.py): same names, same ctypes layout, same
call signatures, so the reference's experiment driver can import this module in
place of its own and run unchanged against the B200 library.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable

from . import _lib


def compute_selectivity(result_set_size: int, dataset_size: int) -> float:
    """(|R| - |D|) / |D|, clamped at 0 -- results/scripts/experiment/find_pairs.py:9-21."""
    return max(0, result_set_size * 1.0 - dataset_size * 1.0) / dataset_size * 1.0


class mmaShape(ctypes.Structure):
    """results/scripts/experiment/find_pairs.py:24-32."""
    _fields_ = [("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int)]

    def __repr__(self):
        return f"mmaShape(m={self.m}, n={self.n}, k={self.k})"


class Results(ctypes.Structure):
    """results/scripts/experiment/find_pairs.py:35-54."""
    _fields_ = [
        ("totalTime", ctypes.c_double),
        ("TFLOPS", ctypes.c_double),
        ("pairsFound", ctypes.c_ulonglong),
        ("pairsStored", ctypes.c_ulonglong),
        ("inputProblemShape", mmaShape),
        ("paddedProblemShape", mmaShape),
    ]

    def __repr__(self):
        return (f"Results(totalTime={self.totalTime}, TFLOPS={self.TFLOPS}, pairsFound={self.pairsFound}, "
                f"pairsStored={self.pairsStored}, inputProblemShape={self.inputProblemShape}, "
                f"paddedProblemShape={self.paddedProblemShape})")

    def get_selectivity(self) -> float:
        return compute_selectivity(self.pairsFound, self.inputProblemShape.m)


class RerunnablePairsFinder:
    """First call runs the full routine (dataset build + upload + join), later calls only re-join
    with a new epsilon -- results/scripts/experiment/find_pairs.py:57-89."""

    def __init__(self, first_find_pairs: Callable[[float, bool], Results],
                 rerun_find_pairs: Callable[[float, bool], Results]):
        self._first_find_pairs = first_find_pairs
        self._rerun_find_pairs = rerun_find_pairs
        self._first_run = True

    def __call__(self, epsilon: float, save_pairs: bool = False) -> Results:
        if self._first_run:
            self._first_run = False
            print("First time running find_pairs, running full method")
            return self._first_find_pairs(epsilon, save_pairs)
        print("Rerunning find_pairs")
        return self._rerun_find_pairs(epsilon, save_pairs)


def load_findpairs(path: str | None = None):
    """ctypes handle with the four entry points typed as the reference types them
    (results/scripts/experiment/find_pairs.py:93-127).  The reference hard-wires
    "../../source/main.so"; here the default is the in-tree build."""
    path = path or _lib.LEGACY_LIB_PATH
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is missing: build it with `python -m fasted_b200.build`")
    find_pairs = ctypes.CDLL(path)
    find_pairs.runFromExponentialDataset.restype = Results
    find_pairs.runFromExponentialDataset.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_double,
                                                     ctypes.c_double, ctypes.c_bool]
    find_pairs.runFromFile.restype = Results
    find_pairs.runFromFile.argtypes = [ctypes.c_char_p, ctypes.c_double, ctypes.c_bool]
    find_pairs.reRun.restype = Results
    find_pairs.reRun.argtypes = [ctypes.c_double, ctypes.c_bool]
    find_pairs.releaseResources.argtypes = []
    find_pairs.releaseResources.restype = None
    return find_pairs
