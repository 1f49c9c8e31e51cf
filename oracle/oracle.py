"""TEST INFRASTRUCTURE — Python face of the CPU oracle (oracle/gguf_oracle.c).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the shipped
package never does.  It builds the C restatement with gcc, loads it through ctypes, hands it the two
format tables from the installed gguf package (the reference does the same:
gguf-plugin/gluon/iq3s.py:41-52, gguf-plugin/gluon/iq4xs.py:190-206) and exposes

    dequantize(raw, type)            fp32 [n, K]      — the format reference restated in C
    matmul_f64(x, raw, type)         fp64 [M, n]      — x . dequantize(raw)^T, the GEMM oracle
    matmul_c(x, raw, type)           fp32 [M, n]      — fused multi-threaded C version (timed baseline)
    rel_err(y, y_ref)                max|y - y_ref| / max_row|y_ref|  (the reference's own error
                                     metric, gguf-plugin/test_gluon_kq_gpu.py:81-86)
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "gguf_oracle.c")
_SO = os.path.join(_HERE, "libgguf_oracle.so")

TYPES = {"Q4_0": 2, "Q5_0": 6, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14,
         "IQ4_NL": 20, "IQ3_S": 21, "IQ4_XS": 23}
BYTES_PER_256 = {2: 144, 6: 176, 8: 272, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210, 20: 144, 21: 110, 23: 136, 18: 98, 16: 66, 17: 74, 22: 82, 29: 56}

_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle (gcc -O2 -ffp-contract=off -fopenmp) next to its source."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", _SO, _SRC])
    return _SO


def iq3s_grid_bytes() -> np.ndarray:
    """The 512 x 4 magnitude bytes of the IQ3_S grid, from the gguf package."""
    from gguf.quants import IQ3_S

    IQ3_S.init_grid()
    return np.ascontiguousarray(IQ3_S.grid.reshape(512, 4).astype(np.uint8))


def iq_grids() -> list[np.ndarray]:
    """The magnitude bytes of the IQ3_XXS (256 x 4), IQ2_XXS (256 x 8), IQ2_XS (512 x 8) and IQ2_S (1024 x 8) grids, from
    the gguf package."""
    import gguf.quants as q

    out = []
    for cls, shape in ((q.IQ3_XXS, (256, 4)), (q.IQ2_XXS, (256, 8)), (q.IQ2_XS, (512, 8)), (q.IQ2_S, (1024, 8))):
        cls.init_grid()
        out.append(np.ascontiguousarray(cls.grid.reshape(shape).astype(np.uint8)))
    return out


def iq1_grid() -> np.ndarray:
    """The 2048 x 8 entries (-1, 0, 1) of the IQ1 grid, from the gguf package."""
    from gguf.quants import IQ1_M

    IQ1_M.init_grid()
    return np.ascontiguousarray(IQ1_M.grid.reshape(2048, 8).astype(np.int8))


def iq4_kvalues() -> np.ndarray:
    from gguf.quants import IQ4_NL

    return np.array(IQ4_NL.kvalues, dtype=np.int8)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        L.oracle_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
        L.oracle_dequantize.restype = ctypes.c_int
        L.oracle_matmul.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                    ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64]
        L.oracle_matmul.restype = ctypes.c_int
        L.oracle_bytes_per_256.argtypes = [ctypes.c_int]
        L.oracle_bytes_per_256.restype = ctypes.c_int
        L.oracle_num_threads.restype = ctypes.c_int
        g, kv = iq3s_grid_bytes(), iq4_kvalues()
        L.oracle_set_tables(g.ctypes.data_as(ctypes.c_void_p), kv.ctypes.data_as(ctypes.c_void_p))
        L.oracle_set_iq_grids(*[a.ctypes.data_as(ctypes.c_void_p) for a in iq_grids()])
        L.oracle_set_iq1_grid(iq1_grid().ctypes.data_as(ctypes.c_void_p))
        _lib = L
    return _lib


def _raw2d(raw, wtype: int):
    raw = np.ascontiguousarray(np.asarray(raw, dtype=np.uint8))
    assert raw.ndim == 2, raw.shape
    bb = BYTES_PER_256[int(wtype)]
    assert raw.shape[1] % bb == 0, (raw.shape, bb)
    return raw, raw.shape[1] // bb * 256


def dequantize(raw, wtype: int) -> np.ndarray:
    """raw uint8 [n, (K/256) * bytes_per_256] -> fp32 [n, K]."""
    raw, K = _raw2d(raw, wtype)
    out = np.empty((raw.shape[0], K), dtype=np.float32)
    rc = lib().oracle_dequantize(int(wtype), raw.ctypes.data_as(ctypes.c_void_p), raw.shape[0], K,
                                 out.ctypes.data_as(ctypes.c_void_p))
    if rc:
        raise ValueError(f"oracle_dequantize failed: {rc}")
    return out


def matmul_f64(x, raw, wtype: int) -> np.ndarray:
    """x [M, K] (any float dtype, taken to fp64) times the dequantised weights, in fp64 -> [M, n]."""
    w = dequantize(raw, wtype).astype(np.float64)
    return np.asarray(x, dtype=np.float64) @ w.T


def matmul_c(x, raw, wtype: int) -> np.ndarray:
    """The fused multi-threaded C dequantise-and-dot (fp32 accumulate).  x fp32 [M, K] -> fp32 [M, n]."""
    raw, K = _raw2d(raw, wtype)
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    assert x.shape[1] == K
    y = np.empty((x.shape[0], raw.shape[0]), dtype=np.float32)
    rc = lib().oracle_matmul(int(wtype), raw.ctypes.data_as(ctypes.c_void_p), raw.shape[0], K,
                             x.ctypes.data_as(ctypes.c_void_p), x.shape[0], y.ctypes.data_as(ctypes.c_void_p), raw.shape[0])
    if rc:
        raise ValueError(f"oracle_matmul failed: {rc}")
    return y


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Let the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says (torchrun
    exports OMP_NUM_THREADS=1 to its workers); returns the thread count now in force."""
    import os

    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    L = lib()
    L.oracle_set_num_threads.argtypes = [ctypes.c_int]
    L.oracle_set_num_threads.restype = None
    L.oracle_set_num_threads(int(n))
    return num_threads()


def rel_err(y, y_ref) -> float:
    """max over rows and columns of |y - y_ref| / (that row's max |y_ref|) for y [M, n] — the
    reference's error metric."""
    y = np.atleast_2d(np.asarray(y, dtype=np.float64))
    y_ref = np.atleast_2d(np.asarray(y_ref, dtype=np.float64))
    if y.size == 0:
        return 0.0
    scale = np.maximum(np.abs(y_ref).max(axis=1, keepdims=True), 1e-30)
    return float((np.abs(y - y_ref) / scale).max())
